# surogate-b200: Blackwell (sm_100a) native LLM training.
#
#   docker build -t surogate-b200:latest .
#   docker run --gpus all --ipc=host -v $PWD/cfg.yaml:/cfg.yaml -v $PWD/out:/out surogate-b200:latest sft /cfg.yaml
#
# The image carries the CUDA toolkit because the native parts are compiled in-tree at build time (nvcc cross-compiles for
# sm_100a without a GPU) and run-time kernels are compiled on first use.
FROM nvidia/cuda:12.9.1-devel-ubuntu24.04

ENV DEBIAN_FRONTEND=noninteractive PIP_NO_CACHE_DIR=1 SUROGATE_NO_BANNER=0
RUN apt-get update && apt-get install -y --no-install-recommends python3 python3-dev python3-venv python3-pip build-essential ninja-build git openssh-client tmux ca-certificates \
    && rm -rf /var/lib/apt/lists/*
RUN python3 -m venv /opt/venv
ENV PATH=/opt/venv/bin:$PATH
RUN pip install --index-url https://download.pytorch.org/whl/cu128 torch \
    && pip install numpy pyyaml safetensors pybind11 ninja jinja2 regex psutil nvidia-ml-py cuda-python transformers huggingface_hub datasets pyarrow rich

WORKDIR /opt/surogate-b200
COPY . .
RUN python -c "import __graft_entry__ as g; g.build()" && pip install -e . --no-build-isolation --no-deps

# one process per GPU talks over NCCL and CUDA IPC: run with --ipc=host (or a large --shm-size)
ENTRYPOINT ["surogate"]
CMD ["--help"]
