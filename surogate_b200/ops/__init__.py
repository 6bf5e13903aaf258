"""Python entry points of the hand-written sm_100a kernels (see ``csrc/``)."""
from __future__ import annotations


def ext():
    """The compiled extension module.  Raises with a clear message when it cannot be loaded."""
    from . import _build

    try:
        return _build.load()
    except Exception as e:  # noqa: BLE001
        raise RuntimeError(
            "surogate_b200 CUDA extension (sm_100a) is not available: build it with "
            "`python -c 'import __graft_entry__ as g; g.build()'` — GPU ops do not fall back to PyTorch") from e


def host():
    """The CUDA-free native host runtime (tokenizer, token loader, safetensors I/O, CPU AdamW, LPT planner, telemetry)."""
    from . import _build

    return _build.load_host()


def host_available() -> bool:
    from . import _build

    return _build.host_available()


def check_device_errors(reset: bool = True) -> None:
    """Raise if any kernel reported a pipeline time-out (bounded waits) since the last check. Synchronises."""
    flag = ext().read_error_flag(reset)
    if flag:
        what = {1: "a bounded device-side wait timed out", 2: "a token id outside [0, vocab_size) reached the embedding"}.get(flag, "a kernel reported an error")
        raise RuntimeError(f"surogate_b200 device error flag = {flag}: {what}")
