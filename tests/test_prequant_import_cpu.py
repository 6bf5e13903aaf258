"""Pre-quantised HuggingFace checkpoints (block FP8, ModelOpt NVFP4, gpt-oss MXFP4, bitsandbytes NF4) import as dequantised weights."""
import json
import os

import numpy as np
import torch
from safetensors.torch import save_file

from surogate_b200.io.hf_checkpoint import LazyCheckpoint
from surogate_b200.io.prequant import E2M1, DequantizingCheckpoint, wrap_if_quantized


def _fp4_codes(x):
    """Nearest E2M1 code of every element of ``x`` (already divided by its scale)."""
    d = (x.unsqueeze(-1) - E2M1).abs()
    d[..., 8] = 1e9   # never emit -0
    return d.argmin(-1).to(torch.uint8)


def _enc_fp8_block(w, bn=128, bk=128):
    N, K = w.shape
    s = torch.zeros((N + bn - 1) // bn, (K + bk - 1) // bk)
    q = torch.empty(N, K, dtype=torch.float8_e4m3fn)
    for i in range(s.shape[0]):
        for j in range(s.shape[1]):
            blk = w[i * bn:(i + 1) * bn, j * bk:(j + 1) * bk]
            s[i, j] = blk.abs().max() / 448.0
            q[i * bn:(i + 1) * bn, j * bk:(j + 1) * bk] = (blk / s[i, j]).to(torch.float8_e4m3fn)
    return q, s


def _enc_nvfp4(w):
    N, K = w.shape
    ts = w.abs().max() / (448.0 * 6.0)
    blocks = w.reshape(N, K // 16, 16)
    bs = (blocks.abs().amax(-1) / 6.0 / ts).to(torch.float8_e4m3fn)
    codes = _fp4_codes(blocks / (bs.float().unsqueeze(-1) * ts + 1e-30)).reshape(N, K)
    return (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous(), bs, ts.reshape(())


def _enc_mxfp4(w_t):
    """``w_t``: [..., R, K] (the stored, transposed layout) -> blocks [..., R, K/32, 16], scales [..., R, K/32]."""
    b = w_t.reshape(*w_t.shape[:-1], w_t.shape[-1] // 32, 32)
    e = torch.ceil(torch.log2(b.abs().amax(-1).clamp_min(2.0 ** -120) / 6.0)).to(torch.int32)
    codes = _fp4_codes(b / torch.exp2(e.float()).unsqueeze(-1))
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).contiguous(), (e + 127).to(torch.uint8)


NF4 = torch.tensor([-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
                    0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0])


def _enc_bnb(w, double_quant):
    flat = w.reshape(-1)
    blocks = flat.reshape(-1, 64)
    absmax = blocks.abs().amax(-1)
    codes = (blocks / absmax.unsqueeze(-1)).unsqueeze(-1).sub(NF4).abs().argmin(-1).to(torch.uint8).reshape(-1)
    packed = ((codes[0::2] << 4) | codes[1::2]).reshape(-1, 1)
    state = {"shape": list(w.shape), "blocksize": 64, "quant_type": "nf4", "dtype": "bfloat16"}
    out = {"packed": packed, "quant_map": NF4.clone()}
    if double_quant:
        offset = absmax.mean()
        a = absmax - offset
        nb = a.reshape(-1, 256) if a.numel() % 256 == 0 else torch.nn.functional.pad(a, (0, 256 - a.numel() % 256)).reshape(-1, 256)
        nmax = nb.abs().amax(-1)
        nmap = torch.linspace(-1, 1, 256)
        qa = (nb / nmax.unsqueeze(-1)).unsqueeze(-1).sub(nmap).abs().argmin(-1).to(torch.uint8).reshape(-1)[: a.numel()]
        out.update(absmax=qa, nested_absmax=nmax, nested_quant_map=nmap)
        state.update(nested_blocksize=256, nested_offset=float(offset))
    else:
        out["absmax"] = absmax
    out["state"] = torch.tensor(list(json.dumps(state).encode()), dtype=torch.uint8)
    return out


def test_each_format_dequantises_close_to_the_original(tmp_path):
    g = torch.Generator().manual_seed(0)
    w_fp8, w_fp4, w_nf4, w_nf4d = (torch.randn(s, generator=g) * 0.05 for s in ((200, 256), (64, 128), (96, 128), (128, 256)))
    w_mx = torch.randn(2, 64, 96, generator=g) * 0.05                     # bf16 layout [E, hidden, 2*inter]
    tensors = {"plain.weight": torch.randn(8, 8, generator=g).bfloat16()}
    tensors["a.weight"], tensors["a.weight_scale_inv"] = _enc_fp8_block(w_fp8)
    tensors["s.weight"], tensors["s.weight_scale"] = (w_fp8 / (w_fp8.abs().max() / 448)).to(torch.float8_e4m3fn), (w_fp8.abs().max() / 448).reshape(())
    tensors["b.weight"], tensors["b.weight_scale"], tensors["b.weight_scale_2"] = _enc_nvfp4(w_fp4)
    tensors["e.gate_up_proj_blocks"], tensors["e.gate_up_proj_scales"] = _enc_mxfp4(w_mx.transpose(1, 2).contiguous())
    for key, w, dq in (("c", w_nf4, False), ("d", w_nf4d, True)):
        enc = _enc_bnb(w, dq)
        tensors[f"{key}.weight"], tensors[f"{key}.weight.absmax"], tensors[f"{key}.weight.quant_map"] = enc["packed"], enc["absmax"], enc["quant_map"]
        tensors[f"{key}.weight.quant_state.bitsandbytes__nf4"] = enc["state"]
        if dq:
            tensors[f"{key}.weight.nested_absmax"], tensors[f"{key}.weight.nested_quant_map"] = enc["nested_absmax"], enc["nested_quant_map"]
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / "model.safetensors"))
    raw = LazyCheckpoint(str(tmp_path))
    ck = wrap_if_quantized(raw, None)                                      # detected from the companion tensors alone
    assert isinstance(ck, DequantizingCheckpoint)
    assert sorted(ck.names()) == ["a.weight", "b.weight", "c.weight", "d.weight", "e.gate_up_proj", "plain.weight", "s.weight"]
    assert "e.gate_up_proj" in ck and "zzz" not in ck

    def rel(a, b):
        return ((a.float() - b).norm() / b.norm()).item()
    assert rel(ck.get("a.weight"), w_fp8) < 0.04 and rel(ck.get("s.weight"), w_fp8) < 0.05
    assert rel(ck.get("b.weight"), w_fp4) < 0.15
    got = ck.get("e.gate_up_proj")
    assert got.shape == w_mx.shape and rel(got, w_mx) < 0.15
    assert rel(ck.get("c.weight"), w_nf4) < 0.12 and rel(ck.get("d.weight"), w_nf4d) < 0.13
    assert torch.equal(ck.get("plain.weight"), tensors["plain.weight"])
    assert ck.stats == {"fp8": 2, "nvfp4": 1, "mxfp4": 1, "bnb_nf4": 2, "plain": 1}
    assert wrap_if_quantized(LazyCheckpoint(str(tmp_path)), {"quantization_config": {"quant_method": "fp8", "weight_block_size": [128, 128]}}).fp8_block == (128, 128)


def test_a_block_fp8_checkpoint_imports_into_a_trainer_and_feeds_qlora(tmp_path):
    """End to end: export a tiny model, rewrite its projections as block FP8 + scale_inv, import: logits stay close, the report says so."""
    from surogate_b200.runtime.trainer import Trainer, TrainerConfig

    model = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                 num_key_value_heads=2, head_dim=32, vocab_size=256, max_position_embeddings=128, rms_norm_eps=1e-6, rope_theta=1e4, tie_word_embeddings=False)
    a = Trainer(TrainerConfig(model=model, batch_size=1, seq_len=16, backend="ref"), device=torch.device("cpu"))
    a.init_weights(seed=0)
    a.export_model(str(tmp_path / "bf16"), model)
    from safetensors.torch import load_file

    sd = load_file(str(tmp_path / "bf16" / "model.safetensors"))
    out = {}
    for k, v in sd.items():
        if k.endswith("proj.weight"):
            out[k], out[k + "_scale_inv"] = _enc_fp8_block(v.float(), 128, 128)
        else:
            out[k] = v
    os.makedirs(tmp_path / "fp8")
    save_file(out, str(tmp_path / "fp8" / "model.safetensors"))
    with open(tmp_path / "fp8" / "config.json", "w") as f:
        json.dump(dict(model, quantization_config={"quant_method": "fp8", "weight_block_size": [128, 128], "fmt": "e4m3"}), f)
    b = Trainer(TrainerConfig(model=model, batch_size=1, seq_len=16, backend="ref"), device=torch.device("cpu"))
    b.import_weights(str(tmp_path / "fp8"))
    x = np.random.default_rng(0).integers(0, 256, (1, 16)).astype(np.int32)
    la, lb = a.logits(x), b.logits(x)
    assert ((la - lb).norm() / la.norm()).item() < 0.06
