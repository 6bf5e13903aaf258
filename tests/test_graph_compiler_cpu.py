"""Graph compiler passes: fusion rules rewrite primitive graphs into the fused ops (same numbers), consumer annotations, the static
buffer plan (no live tensors alias; reuse shrinks the arena), baked programs (the executor's results do not change)."""
import pytest
import torch

from surogate_b200.dsl.compiler import compile_model, model_from_hf_config
from surogate_b200.dsl.graph_compiler import FUSION_RULES, apply_fusion_rules, bake_program, plan_buffers, plan_model, register_fusion_rule
from surogate_b200.dsl.ir import Graph, ParamSpec

QWEN = dict(model_type="qwen3", hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
            vocab_size=256, max_position_embeddings=128, rms_norm_eps=1e-6, rope_theta=1e4, tie_word_embeddings=False)


def _primitive_graph():
    g = Graph("prim", inputs=["x", "res"])
    g.params["w"] = ParamSpec("w", (32,), init="ones")
    g.params["proj"] = ParamSpec("proj", (48, 32))
    g.params["bias"] = ParamSpec("bias", (48,), init="zeros")
    for n, shape in (("x", ("B", "T", 32)), ("res", ("B", "T", 32))):
        g.add_tensor(n, shape, kind="input")
    g.add_tensor("sum", ("B", "T", 32)); g.add_tensor("y", ("B", "T", 32)); g.add_tensor("rstd", ("B", "T"), "fp32")
    g.add_tensor("s1", ("B", "T", 32)); g.add_tensor("s2", ("B", "T", 32)); g.add_tensor("mm", ("B", "T", 48)); g.add_tensor("out", ("B", "T", 48))
    g.add_tensor("unused", ("B", "T", 32))
    g.add_op("add", ["res", "x"], ["sum"])
    g.add_op("rmsnorm", ["sum", "w"], ["y", "rstd"], eps=1e-6)
    g.add_op("scale", ["y"], ["s1"], factor=2.0)
    g.add_op("scale", ["s1"], ["s2"], factor=0.25)
    g.add_op("scale", ["y"], ["unused"], factor=3.0)
    g.add_op("matmul", ["s2", "proj", None], ["mm"], transpose="NT", role="qkv")
    g.add_op("add", ["mm", "bias"], ["out"])
    g.outputs = ["out", "sum"]
    g.validate()
    return g


def test_fusion_rules_rewrite_a_primitive_graph_and_keep_its_numbers():
    from surogate_b200.runtime.ops_ref import RefOps

    g = _primitive_graph()
    before = [o.kind for o in g.ops]
    fired = apply_fusion_rules(g)
    kinds = [o.kind for o in g.ops]
    assert before == ["add", "rmsnorm", "scale", "scale", "scale", "matmul", "add"]
    assert kinds == ["fused_residual_rmsnorm", "scale", "matmul"], kinds
    assert fired == {"residual_add_rmsnorm": 1, "scale_folding": 1, "matmul_bias": 1, "dead_ops": 1}
    assert g.ops[1].attrs["factor"] == 0.5 and g.ops[2].inputs[2] == "bias" and "unused" not in g.tensors and "s1" not in g.tensors
    # numbers: run both forms through the reference backend's ops by hand
    torch.manual_seed(0)
    x, res = torch.randn(2, 5, 32), torch.randn(2, 5, 32)
    w, proj, bias = torch.rand(32) + 0.5, torch.randn(48, 32) * 0.1, torch.randn(48)
    s = x + res
    y = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6) * w
    want = (y * 0.5) @ proj.t() + bias
    be = RefOps()

    class Ctx:
        graph, layer, lora, recipe, training = g, None, None, None, False
    env = {"x": x, "res": res}
    vals = {"w": w, "proj": proj, "bias": bias}
    for op in g.ops:
        ins = [None if n is None else vals.get(n, env.get(n)) for n in op.inputs]
        outs = getattr(be, op.kind)(Ctx, op, *ins)
        env.update({n: v for n, v in zip(op.outputs, outs) if n is not None})
    assert torch.allclose(env["out"], want, atol=1e-5) and torch.allclose(env["sum"], s)


def test_a_registered_rule_takes_part_and_the_traced_models_are_already_fused():
    n = len(FUSION_RULES)

    @register_fusion_rule("double_view_noop")
    def _never(g, i, readers):
        return None
    try:
        cm = compile_model(model_from_hf_config(QWEN))
        assert len(FUSION_RULES) == n + 1 and cm.fwd.meta["fusion_report"] == {}       # modules emit the fused ops themselves
    finally:
        FUSION_RULES.pop()
    kinds = [o.kind for o in next(iter(cm.block_fwd.values())).ops]
    assert "fused_residual_rmsnorm" in kinds and "add" not in kinds


def test_consumer_annotations_say_which_activations_may_leave_their_kernel_quantised():
    cm = compile_model(model_from_hf_config(QWEN))
    (bt, g), = cm.block_fwd.items()
    info = g.meta["consumers"]
    assert info["ln1"]["quant_only"] and info["ln2"]["quant_only"] and info["swiglu"]["quant_only"] and info["att"]["quant_only"]
    assert not info["qkv"]["quant_only"] and not info["res_ffn"]["quant_only"]
    b = cm.block_bwd[bt].meta["consumers"]
    assert b["d_mlp_up"]["sole_backward_matmul"] == "mlp_up" and b["d_swiglu"]["sole_backward_matmul"] is None
    moe = compile_model(model_from_hf_config(dict(QWEN, model_type="qwen3_moe", num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, norm_topk_prob=True)))
    (_, gm), = moe.block_fwd.items()
    assert not gm.meta["consumers"]["ln2"]["quant_only"]           # the router and the permutation read it in bf16


def test_buffer_plan_reuses_dead_buffers_and_never_aliases_live_ones():
    cm = compile_model(model_from_hf_config(QWEN))
    (bt, g), = cm.block_fwd.items()
    bwd = cm.block_bwd[bt]
    dims = {"B": 2, "T": 128}
    pf = plan_buffers(g, dims, saved=bwd.meta["saved"])
    pb = plan_buffers(bwd, dims, saved=[])
    for p in (pf, pb):
        p.validate()
    assert pf.tensors["ln1"].region == "saved" and pf.tensors["ln1"].nbytes == 2 * 128 * 64 * 2 and pf.tensors["ln1_rstd"].nbytes == 2 * 128 * 4
    assert pb.region_bytes["temp"] < pb.unpacked_bytes["temp"] and pb.aliases()        # backward temporaries share bytes
    assert "live [" in pb.table()
    # a plan that is made to alias two live tensors is caught
    a, b = [t for t in pb.tensors.values() if t.region == "temp" and t.nbytes][:2]
    a.first, a.last, b.first, b.last, b.offset = 0, 5, 3, 8, a.offset
    with pytest.raises(AssertionError, match="alias"):
        pb.validate()
    m = plan_model(cm, batch=2, seq_len=128)
    r = plan_model(cm, batch=2, seq_len=128, recompute=True)
    assert m.saved_bytes == 2 * pf.region_bytes["saved"] and r.saved_bytes < m.saved_bytes + 1 and m.temp_bytes >= pb.region_bytes["temp"]
    assert m.summary()["layers"] == 2.0 and m.activation_bytes == m.saved_bytes + m.temp_bytes


def test_the_plan_predicts_what_the_interpreter_keeps_alive():
    """Saved-region size of the plan == bytes the executor actually holds for backward after a forward pass (fp32 reference backend)."""
    from surogate_b200.runtime.trainer import Trainer, TrainerConfig

    tr = Trainer(TrainerConfig(model=QWEN, batch_size=2, seq_len=32, recipe="bf16", backend="ref"), device=torch.device("cpu"))
    tr.init_weights(seed=0)
    x = torch.randint(0, 256, (2, 32))
    pos = torch.arange(32).expand(2, 32).contiguous()
    ctx, _ = tr.executor.forward(x, pos, x, training=True)
    held = 0
    for saved in tr.executor._layer_saved:
        seen = set()
        for v in saved.values():
            if torch.is_tensor(v) and v.data_ptr() not in seen and v.dtype != torch.int64:
                seen.add(v.data_ptr())
                held += v.numel() * v.element_size()
    act_bytes = tr.executor._layer_saved[0]["ln1"].element_size()
    plan = plan_model(tr.cm, batch=2, seq_len=32, act_bytes=act_bytes)
    names = set(next(iter(plan.per_block.values()))["fwd"].tensors)
    planned = sum(t.nbytes for p in [plan.per_block[bt]["fwd"] for bt in plan.layer_types] for t in p.tensors.values() if t.region == "saved")
    assert "ln1" in names and abs(planned - held) <= 0.05 * held, (planned, held)
    tr.executor.backward(ctx)


def test_baked_programs_resolve_names_once_and_free_what_is_dead():
    from surogate_b200.runtime.ops_ref import RefOps

    cm = compile_model(model_from_hf_config(QWEN))
    (bt, g), = cm.block_fwd.items()
    keep = set(cm.block_bwd[bt].meta["saved"])
    prog = bake_program(g, RefOps(), keep)
    assert [b.op.kind for b in prog] == [o.kind for o in g.ops]
    assert prog[1].sources[1] == (1, "qkv_weight") and prog[1].sources[0] == (2, "ln1") and prog[1].sources[2] == (0, None)
    freed = {n for b in prog for n in b.frees}
    assert "att_out" in freed and not (freed & keep) and "x" not in freed
    with pytest.raises(NotImplementedError, match="E030"):
        bad = Graph("bad", inputs=["x"])
        bad.add_tensor("x", ("B",), kind="input"); bad.add_tensor("y", ("B",))
        bad.add_op("no_such_op", ["x"], ["y"])
        bake_program(bad, RefOps(), set())


def test_tensor_debug_commands(tmp_path, capsys):
    import json

    from surogate_b200.cli.main import cli_main
    from surogate_b200.debug import tensor_tools as tt

    cfgp = tmp_path / "config.json"
    cfgp.write_text(json.dumps(dict(QWEN, architectures=["Qwen3ForCausalLM"])))
    arena = tt.tensor_arena(str(cfgp), batch=2, seq_len=64, out=str(tmp_path / "arena.jsonl"))
    tags = [r["tag"] for r in arena]
    assert tags.count("TENSOR_ARENA") == 2 and tags[-1] == "SUMMARY" and arena[-1]["layers"] == 2 and (tmp_path / "arena.jsonl").exists()
    fwd = next(r for r in arena if r["tag"] == "TENSOR_ARENA" and r["graph"] == "forward")
    assert fwd["coverage"] == 1.0 and len(fwd["layout_hash"]) == 16
    assert tt.tensor_arena(str(cfgp), batch=2, seq_len=64)[0]["layout_hash"] == arena[0]["layout_hash"]         # deterministic
    layout = tt.tensor_layout(str(cfgp), batch=2, seq_len=64)
    ln1 = next(r for r in layout if r["name"] == "ln1" and r["graph"] == "forward")
    assert ln1["region"] == "saved" and ln1["bytes"] == 2 * 64 * 64 * 2 and ln1["retain_through_forward"]
    static = tt.tensor_aliasing(str(cfgp), batch=2, seq_len=64)
    assert all(r["valid"] for r in static) and any(r["legal_sharing_pairs"] > 0 for r in static)
    runtime = tt.tensor_aliasing(str(cfgp), batch=1, seq_len=16, mode="runtime")
    assert runtime == [{"tag": "TENSOR_ALIAS_RUNTIME", "events": 0}], runtime[:3]
    res = tt.tensor_resolve(str(cfgp), "qkv", batch=2, seq_len=64)
    f = next(r for r in res if r["graph"] == "forward")
    assert f["producer"]["op"] == "matmul" and f["readers"][0]["op"] == "qkv_qk_norm_rope" and f["saved_for_backward"] and f["plan"]["region"] == "saved"
    assert tt.tensor_resolve(str(cfgp), "nope")[0]["error"]
    assert cli_main(["debug", "tensor-resolve", str(cfgp), "--name", "ln2", "--seq-len", "64"]) == 0
    assert "TENSOR_RESOLVE" in capsys.readouterr().out


def test_native_buffer_planner_equals_the_python_statement_and_validates_plans():
    import random

    from surogate_b200.dsl.graph_compiler import PlannedTensor, _pack
    from surogate_b200.ops import host

    h = host()
    rnd = random.Random(0)
    for trial in range(20):
        n = rnd.randint(1, 60)
        specs = []
        for i in range(n):
            a = rnd.randint(0, 40)
            specs.append((rnd.choice([0, 64, 256, 1000, 4096, 70000]), a, a + rnd.randint(0, 12)))
        py = [PlannedTensor(f"t{i}", "temp", nb, f, l) for i, (nb, f, l) in enumerate(specs)]
        nat = [PlannedTensor(f"t{i}", "temp", nb, f, l) for i, (nb, f, l) in enumerate(specs)]
        total_py, total_nat = _pack(py, use_native=False), _pack(nat, use_native=True)
        assert total_py == total_nat and [t.offset for t in py] == [t.offset for t in nat], trial
        nb, fi, la = [s[0] for s in specs], [s[1] for s in specs], [s[2] for s in specs]
        assert h.validate_buffer_plan(nb, fi, la, [t.offset for t in nat], total_nat) == ""
        assert total_nat <= sum((x + 255) // 256 * 256 for x in nb)
    # two tensors alive together at the same offset are reported
    assert "alias" in h.validate_buffer_plan([512, 512], [0, 1], [5, 3], [0, 256], 1024)
    assert "aligned" in h.validate_buffer_plan([512], [0], [1], [8], 1024) and "outside" in h.validate_buffer_plan([512], [0], [1], [768], 1024)


def test_row_to_expert_lookup_for_the_three_plan_kinds():
    """Which expert slot a permuted row belongs to, and whether it is a real row: local plans ([E + 1] starts + counts), portable
    expert-parallel receive plans (their own offsets, not the sender's), kernel expert-parallel plans (padded layout tensor)."""
    from types import SimpleNamespace

    from surogate_b200.runtime.ops_ref import RefOps

    local = SimpleNamespace(offsets=torch.tensor([0, 2, 2, 5], dtype=torch.int32), counts=torch.tensor([2, 0, 3], dtype=torch.int32), local=None)
    eid, valid = RefOps._row_experts(local, 5, torch.device("cpu"))
    assert eid.tolist() == [0, 0, 2, 2, 2] and valid.all()
    sender = SimpleNamespace(offsets=torch.tensor([0, 1, 2, 3, 4], dtype=torch.int32), counts=torch.tensor([1, 1, 1, 1], dtype=torch.int32), local=None)
    recv = SimpleNamespace(offsets=torch.tensor([0, 3, 4], dtype=torch.int32), counts=torch.tensor([3, 1], dtype=torch.int32), local=sender, recv_splits=[2, 2])
    eid, valid = RefOps._row_experts(recv, 4, torch.device("cpu"))
    assert eid.tolist() == [0, 0, 0, 1] and valid.all()
    # kernel plan: 2 local experts, padded starts 0 / 128 / 256, real rows 3 and 5: rows 3..127 and 133..255 are padding
    layout = torch.tensor([0, 128, 256, 0, 3, 5], dtype=torch.int32)
    kernel = SimpleNamespace(offsets=layout[:3], layout=layout, local=None)
    eid, valid = RefOps._row_experts(kernel, 256, torch.device("cpu"))
    assert eid[:128].eq(0).all() and eid[128:].eq(1).all() and valid.nonzero().flatten().tolist() == [0, 1, 2, 128, 129, 130, 131, 132]
