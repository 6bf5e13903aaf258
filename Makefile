# Developer entry points.  `make help` lists them.
PYTHON ?= python
GPUS   ?= 1

.PHONY: all build install wheel test test-gpu test-multi regression-smoke regression-update-baseline bench bench-moe kernels sanitize docs-check clean info help

all: build

build:            ## compile the CUDA extension (sm_100a), the C++ host runtime and the run-time kernels, in-tree
	$(PYTHON) -c "import __graft_entry__ as g; g.build()"

install: build    ## editable install: the `surogate` command
	$(PYTHON) -m pip install -e . --no-build-isolation

wheel: build      ## wheel with the built native parts inside
	$(PYTHON) -m pip wheel . --no-deps --no-build-isolation -w dist

test:             ## CPU suite
	$(PYTHON) -m pytest tests -x -q -m "not gpu"

test-gpu:         ## kernels against fp32 references and end-to-end runs on a B200
	$(PYTHON) -m pytest tests -x -q -m gpu

test-multi:       ## multi-GPU tests (2+ B200s)
	$(PYTHON) -m pytest tests/test_multigpu.py -x -q -m gpu

regression-smoke: ## the regression matrix against the locked artifacts
	$(PYTHON) -m surogate_b200.regression.runner --baselines regression_baselines/locked

regression-update-baseline: ## re-run the matrix and overwrite regression_baselines/locked
	$(PYTHON) -m surogate_b200.regression.runner --baselines regression_baselines/locked --update

bench:            ## flagship benchmark (Qwen3-8B FP8-hybrid) on $(GPUS) GPU(s)
ifeq ($(GPUS),1)
	$(PYTHON) bench.py --steps 10 --warmup 3
else
	$(PYTHON) -m torch.distributed.run --nnodes=1 --nproc-per-node $(GPUS) --master-addr 127.0.0.1 bench.py --gpus $(GPUS) --steps 10 --warmup 3
endif

bench-moe:        ## Qwen3-30B-A3B NVFP4, expert parallel over $(GPUS) GPUs
	$(PYTHON) -m torch.distributed.run --nnodes=1 --nproc-per-node $(GPUS) --master-addr 127.0.0.1 bench.py --gpus $(GPUS) --model qwen3-30b-a3b --steps 10 --warmup 3

kernels:          ## per-kernel time and roofline fractions
	$(PYTHON) -m surogate_b200.utils.kernel_bench all

sanitize:         ## C++ host runtime under AddressSanitizer + UBSan
	$(PYTHON) -m surogate_b200.debug.sanitize

docs-check:       ## every example config parses
	$(PYTHON) -m pytest tests/test_cli_and_tools_cpu.py -x -q -k example

info:             ## system report
	$(PYTHON) -m surogate_b200.cli.main info

clean:            ## remove built native parts and caches
	$(PYTHON) -c "import shutil, glob; [shutil.rmtree(p, ignore_errors=True) for p in ['surogate_b200/_ext', 'build', 'dist'] + glob.glob('**/__pycache__', recursive=True)]"

help:
	@grep -E '^[a-z-]+: .*##' $(MAKEFILE_LIST) | sed -E 's/:[^#]*## /\t/' | expand -t 28
