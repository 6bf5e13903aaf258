"""Run-time compiled kernels: compile + cache + manifest work without a GPU (nvcc cross-compiles for sm_100a)."""
import json
import os

import pytest
import torch

from surogate_b200.ops import jit


def test_cubins_are_compiled_once_and_described_by_a_manifest(tmp_path, monkeypatch):
    monkeypatch.setenv("SUROGATE_JIT_CACHE", str(tmp_path))
    op = jit.ElementwiseOp("leaky", ("x",), "y = x > 0.f ? x : slope * x;", {"x": "dx = x > 0.f ? dy : slope * dy;"}, consts=("slope",))
    man = op.compile()
    assert set(man.entries) == {"leaky_fwd_bf16", "leaky_bwd_bf16", "leaky_fwd_f32", "leaky_bwd_f32"} and man.arch == "sm_100a"
    assert all(man.resources[e]["registers"] > 0 and man.resources[e].get("spill_store_bytes", 0) == 0 for e in man.entries)
    files = sorted(os.listdir(tmp_path))
    assert len(files) == 2 and files[0].endswith(".cubin") and os.path.getsize(tmp_path / files[0]) > 1000
    with open(tmp_path / files[1]) as f:
        assert json.load(f)["source_sha256"] == man.source_sha256
    stamp = os.path.getmtime(tmp_path / files[0])
    assert op.compile().cubin == man.cubin and os.path.getmtime(tmp_path / files[0]) == stamp          # cache hit: nothing rebuilt
    other = jit.ElementwiseOp("leaky", ("x",), "y = x > 0.f ? x : 2.f * slope * x;", {"x": "dx = dy;"}, consts=("slope",)).compile()
    assert other.cubin != man.cubin                                                                   # the hash follows the source
    with pytest.raises(RuntimeError, match="nvcc failed"):
        jit.compile_cubin("broken", 'extern "C" __global__ void k() { this is not CUDA }')


def test_cpu_tensors_take_the_pytorch_statement():
    x = torch.randn(4, 16)
    assert torch.equal(jit.RELU2(x), torch.relu(x) ** 2)
    assert torch.allclose(jit.SOFTCAP(x, cap=5.0), 5 * torch.tanh(x / 5))
    from surogate_b200.runtime.torch_fns import geglu, relu2, softcap

    assert torch.equal(relu2(x), torch.relu(x) ** 2) and softcap(x, cap=3.0).shape == x.shape and geglu(x).shape == (4, 8)
