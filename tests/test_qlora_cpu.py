"""QLoRA storage codecs and training over a block-quantised frozen base."""
import numpy as np
import pytest
import torch

from surogate_b200.quant.codecs import BlockFP8, BnbNF4, MXFP4, NVFP4Storage
from surogate_b200.runtime.trainer import Trainer, TrainerConfig


@pytest.mark.parametrize("codec,tol,bits", [(BnbNF4(64, True), 0.11, 4.13), (BnbNF4(64, False), 0.11, 4.5), (BlockFP8(128), 0.04, 8.25),
                                            (NVFP4Storage(True), 0.10, 4.5), (MXFP4(), 0.14, 4.25)])
def test_codec_round_trip(codec, tol, bits):
    torch.manual_seed(0)
    x = torch.randn(1 << 14) * 0.02
    st = codec.quantize(x)
    y = codec.dequantize(st, torch.float32)
    assert ((y - x).norm() / x.norm()).item() < tol
    assert abs(sum(t.numel() * t.element_size() for t in st.values()) * 8 / x.numel() - bits) < 0.05
    again = codec.dequantize(codec.quantize(y), torch.float32)  # values already on the grid survive a second pass
    assert ((again - y).norm() / y.norm()).item() < 0.03


def test_nvfp4_four_over_six_never_hurts():
    torch.manual_seed(1)
    x = torch.randn(1 << 14)
    e6 = (NVFP4Storage(False).dequantize(NVFP4Storage(False).quantize(x), torch.float32) - x).norm()
    e46 = (NVFP4Storage(True).dequantize(NVFP4Storage(True).quantize(x), torch.float32) - x).norm()
    assert e46 <= e6


def test_block_fp8_2d_prequantised_layout():
    torch.manual_seed(2)
    w = torch.randn(256, 384) * 0.05
    s = w.reshape(2, 128, 3, 128).abs().amax((1, 3)) / 448.0
    q = (w / s.repeat_interleave(128, 0).repeat_interleave(128, 1)).to(torch.float8_e4m3fn)
    back = BlockFP8.dequantize_2d(q, s, dtype=torch.float32)
    assert ((back - w).norm() / w.norm()).item() < 0.04


MODEL = dict(architecture="Qwen3ForCausalLM", vocab_size=256, d_model=64, n_layers=2, num_query_heads=4, num_kv_heads=2, head_size=16, d_ff=128,
             tie_word_embeddings=True)
LORA = dict(rank=4, alpha=8, dropout=0.0, dtype="fp32", targets=["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"],
            rslora=False, train_router=False)


@pytest.mark.parametrize("kind", ["bnb_nf4", "fp8_block", "nvfp4"])
def test_qlora_training(kind):
    def make(q):
        tr = Trainer(TrainerConfig(model=MODEL, batch_size=2, seq_len=32, recipe="bf16", optimizer="adamw", learning_rate=2e-2, zero_level=0, lora=LORA,
                                   qlora=q), device=torch.device("cpu"))
        tr.init_weights(seed=0)
        return tr

    q, ref = make(kind), make(None)
    assert q.qlora_bytes_saved > 0
    assert all(b.master.numel() == 0 for b in q.store.buckets.values() if b.layer is not None)
    rng = np.random.default_rng(0)
    tok = rng.integers(0, 256, (2, 33)).astype(np.int32)
    lq = [q.step(tok[:, :-1], tok[:, 1:])["loss"] for _ in range(6)]
    lr = [ref.step(tok[:, :-1], tok[:, 1:])["loss"] for _ in range(6)]
    assert abs(lq[0] - lr[0]) < 0.05 * lr[0]  # the quantised base is close to the original
    assert lq[-1] < lq[0] - 0.2
    assert all(b.work is None for b in q.store.buckets.values() if getattr(b, "qstate", None) is not None)  # bf16 copies are transient
    w = q.store.full_tensor("blocks.0.qkv_weight")
    w0 = ref.store.full_tensor("blocks.0.qkv_weight")
    assert ((w.float() - w0.float()).norm() / w0.float().norm()).item() < 0.12
