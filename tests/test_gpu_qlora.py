"""CUDA dequantisers of the QLoRA storage formats against the PyTorch statements of the same formats (quant/codecs.py)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("kind,kw", [("bnb_nf4", dict(double_quant=True)), ("bnb_nf4", dict(double_quant=False)), ("fp8_block", dict(block=128)),
                                     ("fp8_block", dict(block=64)), ("nvfp4", dict(four_over_six=True)), ("nvfp4", dict(four_over_six=False)), ("mxfp4", {})])
def test_dequantisers_match_the_pytorch_statements(kind, kw):
    from surogate_b200.quant.codecs import make_codec

    torch.manual_seed(0)
    codec = make_codec(kind, **kw)
    x = (torch.randn(3 * 256 * 257, device=DEV) * torch.rand(3 * 256 * 257, device=DEV).pow(3)).bfloat16()
    x = x[: x.numel() // 65536 * 65536]
    st = codec.quantize(x)
    fast = codec.dequantize(st)
    ref = codec.dequantize_reference(st)
    assert fast.dtype == torch.bfloat16 and fast.shape == ref.shape
    assert torch.equal(fast, ref), (fast.float() - ref.float()).abs().max()
    # and the format itself reconstructs the tensor to its precision
    err = ((fast.float() - x.float()).norm() / x.float().norm()).item()
    assert err < {"bnb_nf4": 0.12, "fp8_block": 0.04, "nvfp4": 0.14, "mxfp4": 0.2}[kind], err


def test_qlora_step_runs_on_the_cuda_dequantisers():
    """A QLoRA step on the GPU (NF4 base, LoRA adapters): the frozen layers are rebuilt by the kernels, the loss falls."""
    import numpy as np

    from surogate_b200.ops import ext
    from surogate_b200.runtime.trainer import Trainer, TrainerConfig

    model = dict(architecture="Qwen3ForCausalLM", vocab_size=1024, d_model=256, n_layers=2, num_query_heads=2, num_kv_heads=1, head_size=128, d_ff=512,
                 tie_word_embeddings=False)
    lora = dict(rank=8, alpha=16, dropout=0.0, dtype="fp32", targets=["q_proj", "v_proj", "down_proj"], rslora=False, train_router=False)
    cfg = TrainerConfig(model=model, batch_size=2, seq_len=128, recipe="bf16", optimizer="adamw", learning_rate=5e-3, lora=lora, qlora="bnb_nf4")
    tr = Trainer(cfg, device=torch.device("cuda:0"))
    tr.init_weights(seed=0)
    rng = np.random.default_rng(0)
    tok = rng.integers(0, 1024, (2, 129)).astype(np.int32)
    before = ext().launch_count()
    losses = [tr.step(tok[:, :-1], tok[:, 1:])["loss"] for _ in range(6)]
    assert losses[-1] < losses[0] - 0.05, losses
    assert ext().launch_count() > before
