"""surogate_b200: a Blackwell (sm_100a) native LLM training framework.

PyTorch is the tensor / stream / process-group layer; the model is described in a
Python DSL traced to an explicit graph with ahead-of-time autodiff; the hot ops
are hand-written sm_100a CUDA kernels (tcgen05 + TMEM + TMA) and the
communication-bound paths are kernels that move data over NVLink themselves.
"""
__version__ = "0.1.0"
