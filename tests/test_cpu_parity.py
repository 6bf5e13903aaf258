"""fp32 CPU plumbing test: DSL model + AOT autodiff + executor vs torch autograd (loss and every gradient)."""
import numpy as np
import pytest
import torch

from surogate_b200.dsl.compiler import compile_model
from surogate_b200.dsl.models import Qwen3Model, Qwen3MoEModel, LlamaModel, Qwen2Model
from surogate_b200.runtime.executor import ExecOptions, Executor
from surogate_b200.runtime.ops_ref import RefOps
from surogate_b200.runtime.params import ParamStore

from surogate_b200.runtime.trainer import Trainer, TrainerConfig
from torch_reference import model_loss


def _run(model, cfg, recompute=False, mask_frac=0.0):
    torch.manual_seed(0)
    cm = compile_model(model)
    store = ParamStore(cm, device="cpu", param_dtype=torch.float32)
    store.init_weights(seed=0)
    # perturb norm weights so their gradients are exercised away from the all-ones point
    g = torch.Generator().manual_seed(5)
    for b in store.buckets.values():
        for s in b.slots:
            if s.entry.spec.init == "ones":
                b.master[s.offset:s.offset + s.numel] += 0.1 * torch.randn(s.numel, generator=g)
    ex = Executor(cm, store, RefOps(lmhead_chunk_rows=50), options=ExecOptions(recompute=recompute))
    B, T, V = 2, 64, cfg["V"]
    gen = torch.Generator().manual_seed(1)
    tokens = torch.randint(0, V, (B, T + 1), generator=gen)
    inp, tgt = tokens[:, :-1].to(torch.int32), tokens[:, 1:].to(torch.int32).clone()
    if mask_frac:
        tgt[:, : int(T * mask_frac)] = -100
    pos = torch.arange(T, dtype=torch.int32)[None].expand(B, T).contiguous()
    store.begin_step()
    ctx, outs = ex.forward_backward(inp, pos, tgt)
    store.finish_reduce()

    p = {n: t.detach().clone().requires_grad_(True) for n, t in store.named_full_tensors()}
    loss_ref, aux_ref = model_loss(p, inp.long(), pos, tgt, cfg)
    (loss_ref + aux_ref).backward()
    assert torch.allclose(outs[0], loss_ref.detach(), rtol=1e-5, atol=1e-4), (outs[0], loss_ref)
    if len(outs) > 1:
        assert torch.allclose(outs[1], aux_ref.detach(), rtol=1e-5, atol=1e-6)
    n_checked = 0
    for name, t in p.items():
        g = store.grad_of(name)
        assert g is not None, name
        ref = t.grad if t.grad is not None else torch.zeros_like(t)
        err = (g - ref).abs().max().item()
        scale = max(ref.abs().max().item(), 1.0)
        assert err <= 1e-5 * scale + 2e-5, f"{name}: max err {err} (ref max {ref.abs().max().item()})"
        n_checked += 1
    assert n_checked == len(p)


TINY = dict(vocab_size=1024, d_model=128, n_layers=2, num_query_heads=4, num_kv_heads=2, head_size=32, d_ff=384,
            eps=1e-6, rope_theta=1e6, tie_word_embeddings=True)
TINY_CFG = dict(V=1024, n_layers=2, Hq=4, Hkv=2, D=32, eps=1e-6, theta=1e6)


def test_qwen3_tiny_matches_autograd():
    _run(Qwen3Model(**TINY), TINY_CFG)


def test_qwen3_tiny_recompute_and_masked_targets():
    _run(Qwen3Model(**TINY), TINY_CFG, recompute=True, mask_frac=0.25)


def test_qwen3_untied():
    _run(Qwen3Model(**{**TINY, "tie_word_embeddings": False}), TINY_CFG)


def test_llama_tiny():
    _run(LlamaModel(**{**TINY, "rope_theta": 10000.0}), {**TINY_CFG, "theta": 10000.0, "qk_norm": False})


def test_qwen2_bias():
    _run(Qwen2Model(**TINY), {**TINY_CFG, "qk_norm": False})


def test_qwen3_moe_tiny():
    m = Qwen3MoEModel(vocab_size=512, d_model=64, n_layers=2, num_query_heads=4, num_kv_heads=2, head_size=16, moe_d_ff=32,
                      num_experts=8, num_experts_per_tok=2, aux_loss_coef=1e-2, tie_word_embeddings=False)
    _run(m, dict(V=512, n_layers=2, Hq=4, Hkv=2, D=16, eps=1e-6, theta=1e6, E=8, K=2, aux_coef=1e-2))


def test_tiled_mlp_matches_autograd_and_the_untiled_model():
    """long_context: the MLP runs over row tiles and recomputes them in backward; results equal the ordinary path."""
    _run(Qwen3Model(**TINY, mlp_tile_rows=48), TINY_CFG)


@pytest.mark.parametrize("arch", ["dense", "moe"])
def test_sequence_chunks_match_the_unchunked_step(arch):
    """Training a row in 4 pieces against a key/value prefix (pass A fills it, pass B walks backwards accumulating dK / dV)
    gives the loss and gradients of the ordinary step; sliding-window attention and recompute included."""
    if arch == "dense":
        model = dict(architecture="Qwen3ForCausalLM", vocab_size=200, d_model=64, n_layers=2, num_query_heads=4, num_kv_heads=2, head_size=16, d_ff=96,
                     tie_word_embeddings=True)
    else:
        model = dict(architecture="Qwen3MoeForCausalLM", vocab_size=200, d_model=64, n_layers=2, num_query_heads=4, num_kv_heads=2, head_size=16, moe_d_ff=32,
                     num_experts=4, num_experts_per_tok=2, aux_loss_coef=0.0, tie_word_embeddings=False)
    rng = np.random.default_rng(0)
    tok = rng.integers(0, 200, (2, 65)).astype(np.int32)
    x, y = tok[:, :-1].copy(), tok[:, 1:].copy()
    y[0, :7] = -100

    def run(chunks, recompute=False):
        tr = Trainer(TrainerConfig(model=model, batch_size=1, grad_accum=2, seq_len=64, zero_level=0, sequence_chunks=chunks, recompute=recompute), device=torch.device("cpu"))
        tr.init_weights(seed=3)
        r = tr.forward_backward(x, y)
        grads = {n: tr.store.grad_of(n).clone() for n in list(tr.store.where)[:40] if tr.store.grad_of(n) is not None}
        return float(r["loss_sum"] / r["n_valid"]), float(tr.grad_norm()), grads

    l1, n1, g1 = run(1)
    for rec in (False, True):
        l4, n4, g4 = run(4, rec)
        assert abs(l1 - l4) < 1e-5 and abs(n1 - n4) < 1e-4 * n1, (l1, l4, n1, n4)
        for k in g1:
            assert torch.allclose(g1[k], g4[k], atol=2e-5, rtol=1e-3), k


def test_dropping_ignored_rows_before_the_lm_head_changes_nothing():
    model = dict(architecture="Qwen3ForCausalLM", vocab_size=200, d_model=64, n_layers=1, num_query_heads=4, num_kv_heads=2, head_size=16, d_ff=96,
                 tie_word_embeddings=False)
    rng = np.random.default_rng(0)
    tok = rng.integers(0, 200, (2, 33)).astype(np.int32)
    x, y = tok[:, :-1].copy(), tok[:, 1:].copy()
    y[0, :19] = -100
    y[1, 5:9] = -100

    def run(drop):
        tr = Trainer(TrainerConfig(model=model, batch_size=2, seq_len=32, zero_level=0, lmhead_drop_ignored_rows=drop, lmhead_chunk_rows=16), device=torch.device("cpu"))
        tr.init_weights(seed=3)
        r = tr.forward_backward(x, y)
        return float(r["loss_sum"]), float(tr.grad_norm()), tr.store.grad_of("lm_head").clone()

    a, b = run(False), run(True)
    assert abs(a[0] - b[0]) < 1e-4 and abs(a[1] - b[1]) < 1e-5 * a[1] and torch.allclose(a[2], b[2], atol=1e-6)


def test_chunked_gated_delta_rule_equals_the_recurrence():
    """The chunk-wise evaluation (triangular solve inside chunks of 64, state carried between chunks) reproduces the
    step-by-step recurrence and its gradients, including a ragged last chunk."""
    from surogate_b200.runtime.torch_fns import gated_delta_rule, gated_delta_rule_recurrent

    torch.manual_seed(0)
    B, T, H, Dk, Dv = 2, 150, 3, 16, 24
    ins = [torch.randn(B, T, H, Dk), torch.randn(B, T, H, Dk), torch.randn(B, T, H, Dv), -torch.rand(B, T, H) * 0.5, torch.rand(B, T, H)]
    for t in ins:
        t.requires_grad_(True)
    a, b = gated_delta_rule(*ins), gated_delta_rule_recurrent(*ins)
    assert torch.allclose(a, b, atol=1e-5)
    ga = torch.autograd.grad(a.square().sum(), ins)
    gb = torch.autograd.grad(b.square().sum(), ins)
    for x, y in zip(ga, gb):
        assert torch.allclose(x, y, atol=1e-4 * float(y.abs().max()))


def test_expert_of_each_row_is_read_from_every_plan_layout():
    """Per-expert bias rows are found from device-side range starts / counts: plain plans ([E + 1] starts + counts), kernel plans
    with padded ranges, and expert-parallel receive plans ([El + 1 starts, overflow, El counts] in one tensor)."""
    from types import SimpleNamespace

    from surogate_b200.runtime.ops_ref import RefOps

    plain = SimpleNamespace(offsets=torch.tensor([0, 2, 2, 5]), counts=torch.tensor([2, 0, 3]), local=None)
    eid, valid = RefOps._row_experts(plain, 5, torch.device("cpu"))
    assert eid.tolist() == [0, 0, 2, 2, 2] and valid.all()
    padded = SimpleNamespace(offsets=torch.tensor([0, 4, 8, 12]), counts=torch.tensor([2, 0, 3]), local=None)  # ranges padded to 4 rows
    eid, valid = RefOps._row_experts(padded, 12, torch.device("cpu"))
    assert eid.tolist() == [0] * 4 + [1] * 4 + [2] * 4 and valid.tolist() == [True, True, False, False] + [False] * 4 + [True, True, True, False]
    ep = SimpleNamespace(offsets=torch.tensor([0, 4, 8, 0, 3, 1]), local=None)  # El = 2: starts [0, 4, 8], overflow 0, counts [3, 1]
    eid, valid = RefOps._row_experts(ep, 8, torch.device("cpu"))
    assert eid.tolist() == [0] * 4 + [1] * 4 and valid.tolist() == [True, True, True, False, True, False, False, False]
