"""Run the C++ host runtime under AddressSanitizer + UndefinedBehaviorSanitizer.

``python -m surogate_b200.debug.sanitize [pytest arguments]`` builds a sanitized copy of the host library and runs a workload
against it in a child process that has the sanitizer runtime preloaded: the host-runtime tests when a ``tests`` directory is
next to the package (tokenizer, token loader, safetensors I/O, CPU AdamW, expert-placement planner), otherwise a built-in
exercise of the same entry points.  Exit code 0 means the sanitizers saw nothing; their reports go to stderr otherwise.
CUDA code is not covered: device-side checks are the kernels' own error flags and the numerics tests.

Parity: the reference's ENABLE_SANITIZERS CMake option (ASan + UBSan on the C++ translation units, csrc/CMakeLists.txt).
"""
from __future__ import annotations

import os
import subprocess
import sys
from typing import List, Optional


def sanitizer_runtime() -> Optional[str]:
    out = subprocess.run(["gcc", "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
    return out if out and os.path.isabs(out) and os.path.exists(out) else None


def builtin_workload() -> None:
    """Touches every host entry point with small inputs (runs inside the sanitized child)."""
    import tempfile

    import numpy as np

    from ..ops import host

    h = host()
    with tempfile.TemporaryDirectory() as d:
        from ..data.loader import write_synthetic_tokens
        from ..io import safetensors_native as st

        path = os.path.join(d, "train-000.bin")
        write_synthetic_tokens(path, 16, 32, 1000, seed=1)
        from ..data.loader import DataLoader

        dl = DataLoader([path], 4, 32, seed=3, native=True)
        for _ in range(6):
            dl.next_batch()
        import torch

        tensors = {"a": torch.arange(1024, dtype=torch.float32).reshape(32, 32), "b": torch.ones(7, 3, dtype=torch.float16)}
        st.save_file_native(tensors, os.path.join(d, "t.safetensors"))
        f = st.NativeSafetensors(os.path.join(d, "t.safetensors"))
        assert torch.equal(f.get_tensor("a"), tensors["a"]) and torch.equal(f.get_rows("a", 4, 9), tensors["a"][4:9])
    counts = [5, 0, 9, 1, 3, 3, 8, 2]
    placement, moved = h.balanced_placement(counts, 4, list(range(8)), 0.05)
    assert sorted(placement) == list(range(8)) and moved >= 0
    import torch

    p = torch.randn(4096)
    g, m, v = torch.ones(4096), torch.zeros(4096), torch.zeros(4096)
    h.cpu_adamw_step(p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), False, 0, 4096, 1e-3, 0.9, 0.999, 1e-8, 0.1, 1.0, 1, 0)
    assert float(h.cpu_sum_squares(g.data_ptr(), False, 4096)) == 4096.0
    print("host workload ok")


def run(pytest_args: Optional[List[str]] = None) -> int:
    from ..ops import _build

    rt = sanitizer_runtime()
    if rt is None:
        print("no libasan.so next to gcc: cannot run the sanitized build", file=sys.stderr)
        return 2
    so = _build.build_host_sanitized()
    env = dict(os.environ, LD_PRELOAD=rt, SUROGATE_HOST_SO=so, ASAN_OPTIONS="detect_leaks=0:abort_on_error=0:halt_on_error=1",
               UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=1", OMP_NUM_THREADS="2")
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    tests = os.path.join(root, "tests", "test_host_runtime.py")
    if os.path.exists(tests):
        cmd = [sys.executable, "-m", "pytest", tests, "-q", "-x"] + list(pytest_args or [])
        offload = os.path.join(root, "tests", "test_offload_cpu.py")
        if os.path.exists(offload) and not pytest_args:  # the optimizer worker thread: buffer ownership with an update in flight
            # (tests that make the worker throw are left out: a preloaded ASan cannot intercept __cxa_throw)
            cmd += [offload + "::test_dropping_a_trainer_with_an_update_in_flight_frees_nothing_the_worker_writes"]
    else:
        cmd = [sys.executable, "-c", "from surogate_b200.debug.sanitize import builtin_workload; builtin_workload()"]
    return subprocess.run(cmd, env=env, cwd=root).returncode


if __name__ == "__main__":
    sys.exit(run(sys.argv[1:]))
