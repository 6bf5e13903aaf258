"""Checkpoint compatibility with HuggingFace transformers: a randomly initialised HF model is saved, imported through the
DSL's weight mappings and must produce the same logits; exporting back must reproduce the HF tensors."""
import os

import numpy as np
import pytest
import torch

transformers = pytest.importorskip("transformers")

from surogate_b200.dsl.compiler import load_hf_config  # noqa: E402
from surogate_b200.runtime.trainer import Trainer, TrainerConfig  # noqa: E402

COMMON = dict(vocab_size=320, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=96,
              max_position_embeddings=128, rms_norm_eps=1e-6)


def _cases():
    from transformers import Gemma4TextConfig, Qwen3_5MoeTextConfig, GptOssConfig, Lfm2Config, LlamaConfig, NemotronHConfig, Qwen3_5TextConfig, MistralConfig, Qwen2Config, Qwen3Config, Qwen3MoeConfig

    yield "qwen3", Qwen3Config(**COMMON, head_dim=16, rope_theta=1e6, tie_word_embeddings=True)
    yield "qwen3-untied", Qwen3Config(**COMMON, head_dim=32, rope_theta=1e6, tie_word_embeddings=False)
    yield "qwen2", Qwen2Config(**COMMON, rope_theta=1e6, tie_word_embeddings=False)
    yield "llama", LlamaConfig(**COMMON, rope_theta=10000.0, tie_word_embeddings=False)
    yield "mistral", MistralConfig(**COMMON, head_dim=16, rope_theta=10000.0, sliding_window=None, tie_word_embeddings=False)
    yield "qwen3-moe", Qwen3MoeConfig(**COMMON, head_dim=16, rope_theta=1e6, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=48,
                                      norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[], tie_word_embeddings=False)
    yield "lfm2", Lfm2Config(vocab_size=320, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, intermediate_size=96,
                             conv_L_cache=3, block_auto_adjust_ff_dim=False, layer_types=["conv", "full_attention", "conv", "full_attention"],
                             max_position_embeddings=256, tie_word_embeddings=True)
    yield "nemotron-h", NemotronHConfig(vocab_size=320, hidden_size=64, layers_block_type=["mamba", "moe", "attention", "moe"], num_attention_heads=4,
                                        num_key_value_heads=2, head_dim=16, intermediate_size=96, ssm_state_size=16, mamba_num_heads=8, mamba_head_dim=16,
                                        n_groups=2, conv_kernel=4, chunk_size=8, max_position_embeddings=128, n_routed_experts=4, num_experts_per_tok=2,
                                        moe_intermediate_size=32, moe_shared_expert_intermediate_size=48, tie_word_embeddings=False)
    yield "qwen3.5", Qwen3_5TextConfig(vocab_size=320, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                                       intermediate_size=96, linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=8, linear_value_head_dim=8,
                                       linear_conv_kernel_dim=4, max_position_embeddings=256, tie_word_embeddings=False)
    yield "qwen3.5-moe", Qwen3_5MoeTextConfig(vocab_size=320, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                                              moe_intermediate_size=32, shared_expert_intermediate_size=48, num_experts=4, num_experts_per_tok=2,
                                              linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=8, linear_value_head_dim=8,
                                              linear_conv_kernel_dim=4, max_position_embeddings=256, tie_word_embeddings=False)
    g4 = dict(vocab_size=320, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=16, global_head_dim=32,
              intermediate_size=96, sliding_window=8, max_position_embeddings=256, hidden_size_per_layer_input=0, num_kv_shared_layers=0,
              layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"], final_logit_softcapping=30.0, tie_word_embeddings=True)
    yield "gemma4", Gemma4TextConfig(**g4)
    yield "gemma4-moe-keqv", Gemma4TextConfig(**{**g4, "tie_word_embeddings": True}, attention_k_eq_v=True, num_global_key_value_heads=1, enable_moe_block=True,
                                               num_experts=4, top_k_experts=2, moe_intermediate_size=32)
    yield "gemma4-pli-kvshare", Gemma4TextConfig(**{**g4, "num_hidden_layers": 6, "hidden_size_per_layer_input": 8, "vocab_size_per_layer_input": 320,
                                                    "num_kv_shared_layers": 2, "use_double_wide_mlp": True,
                                                    "layer_types": ["sliding_attention", "full_attention", "sliding_attention", "full_attention",
                                                                    "sliding_attention", "full_attention"]})
    yield "gpt-oss", GptOssConfig(vocab_size=320, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                                  intermediate_size=32, num_local_experts=4, num_experts_per_tok=2, sliding_window=8, max_position_embeddings=256,
                                  rope_parameters={"rope_type": "yarn", "rope_theta": 150000.0, "factor": 4.0, "beta_fast": 32.0, "beta_slow": 1.0,
                                                   "truncate": False, "original_max_position_embeddings": 64}, tie_word_embeddings=False)


@pytest.mark.parametrize("name,config", list(_cases()), ids=[n for n, _ in _cases()])
def test_logits_match_transformers_and_export_round_trips(tmp_path, name, config):
    from transformers import AutoModelForCausalLM

    torch.manual_seed(0)
    hf = AutoModelForCausalLM.from_config(config).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():  # make norms / biases non-trivial
            if p.dim() == 1 or "bias" in n:
                p.add_(0.1 * torch.randn_like(p))
    src = os.path.join(tmp_path, "hf")
    hf.save_pretrained(src, safe_serialization=True)
    tok = np.random.default_rng(0).integers(0, 320, (2, 24)).astype(np.int32)
    with torch.no_grad():
        want = hf(torch.from_numpy(tok).long()).logits
    cfg = load_hf_config(src)
    tr = Trainer(TrainerConfig(model=cfg, batch_size=2, seq_len=24, zero_level=0), device=torch.device("cpu"))
    tr.import_weights(src)
    got = tr.logits(tok)
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), (name, float((got - want).abs().max()))
    # backward: same loss and same global gradient norm as autograd through the transformers model
    tgt = np.roll(tok, -1, axis=1).astype(np.int32)
    tgt[:, -1] = -100
    r = tr.forward_backward(tok, tgt)
    lg = hf(torch.from_numpy(tok).long()).logits
    loss = torch.nn.functional.cross_entropy(lg.reshape(-1, lg.shape[-1]), torch.from_numpy(tgt).long().reshape(-1), ignore_index=-100, reduction="mean")
    hf.zero_grad()
    loss.backward()
    want_norm = torch.sqrt(sum((p.grad.float() ** 2).sum() for p in hf.parameters() if p.grad is not None))
    assert abs(float(r["loss_sum"] / r["n_valid"]) - float(loss)) < 1e-4
    got_norm = float(tr.grad_norm())
    if name not in ("qwen3-moe", "qwen3.5-moe"):  # the MoE model adds its load-balancing loss to the gradient
        assert abs(got_norm - float(want_norm)) < 2e-3 * float(want_norm), (name, got_norm, float(want_norm))
    tr.store.release_grads()
    out = os.path.join(tmp_path, "export")
    tr.export_model(out, cfg)
    from safetensors.torch import load_file

    a, b = load_file(os.path.join(src, "model.safetensors")), load_file(os.path.join(out, "model.safetensors"))
    for k, v in a.items():
        assert k in b, k
        assert torch.allclose(b[k].float(), v.float(), atol=1e-2, rtol=1e-2), k  # export writes bf16
    # the export holds bfloat16 weights: reloaded, it must behave like the original model with its weights rounded the same way
    import copy

    rounded = copy.deepcopy(hf)
    with torch.no_grad():
        for t in rounded.state_dict().values():  # parameters and saved buffers, not derived tables such as rotary frequencies
            if t.is_floating_point():
                t.copy_(t.bfloat16().float())
        want_rounded = rounded(torch.from_numpy(tok).long()).logits
    back = AutoModelForCausalLM.from_pretrained(out, torch_dtype=torch.float32).eval()
    with torch.no_grad():
        again = back(torch.from_numpy(tok).long()).logits
    assert torch.allclose(again, want_rounded, atol=1e-4, rtol=1e-3), float((again - want_rounded).abs().max())

def test_fused_expert_tensor_mapping_swaps_gate_and_up_and_inverts():
    """Checkpoints that store a layer's experts as one [E, 2F, C] tensor with the gate rows first load into the [up; gate] layout
    and export back unchanged."""
    from surogate_b200.dsl import hf as hfmap

    m = hfmap.transform("layers.{L}.mlp.experts.gate_up_proj", fn="swap_row_halves")
    t = torch.arange(2 * 6 * 3, dtype=torch.float32).reshape(2, 6, 3)
    got = m.load(lambda name: {"layers.1.mlp.experts.gate_up_proj": t}[name], 1)
    assert torch.equal(got[:, :3], t[:, 3:]) and torch.equal(got[:, 3:], t[:, :3])
    assert torch.equal(m.export(got, 1)["layers.1.mlp.experts.gate_up_proj"], t)


def test_qwen3_vl_text_decoder_with_visual_side_inputs_matches_transformers(tmp_path):
    """Multi-axis rotary positions, scatter of vision features into the embeddings and deepstack injection: the decoder fed
    with synthetic vision-tower outputs gives the logits of transformers' Qwen3-VL language model fed with the same."""
    from transformers import Qwen3VLConfig, Qwen3VLForConditionalGeneration

    text = dict(vocab_size=320, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=96,
                max_position_embeddings=256, rms_norm_eps=1e-6, rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [4, 2, 2], "mrope_interleaved": True},
                tie_word_embeddings=False)
    vision = dict(depth=2, hidden_size=32, intermediate_size=48, num_heads=2, out_hidden_size=64, patch_size=4, spatial_merge_size=2, temporal_patch_size=2,
                  deepstack_visual_indexes=[0, 1], num_position_embeddings=16)
    torch.manual_seed(0)
    hf = Qwen3VLForConditionalGeneration(Qwen3VLConfig(text_config=text, vision_config=vision, tie_word_embeddings=False)).float().eval()
    src = os.path.join(tmp_path, "hf")
    hf.save_pretrained(src, safe_serialization=True)
    rows, T, C = 2, 24, 64
    rng = np.random.default_rng(0)
    tok = rng.integers(0, 320, (rows, T)).astype(np.int32)
    mask = np.zeros((rows, T), bool)
    mask[0, 3:11] = True
    mask[1, 5:9] = True
    n_vis = int(mask.sum())
    vis = torch.randn(n_vis, C)
    deep = [0.5 * torch.randn(n_vis, C) for _ in range(2)]
    pos3 = np.tile(np.arange(T, dtype=np.int64), (3, rows, 1))
    pos3[1, 0, 3:11] = 3 + np.repeat(np.arange(2), 4)  # a 2 x 4 grid of patches: height index
    pos3[2, 0, 3:11] = 3 + np.tile(np.arange(4), 2)    # width index
    pos3[0, 0, 3:11] = 3
    pos3[:, 0, 11:] = pos3[:, 0, 11:] - 4              # text resumes after max(grid) + 1
    lm = hf.model.language_model
    with torch.no_grad():
        emb = lm.embed_tokens(torch.from_numpy(tok).long())
        emb = emb.masked_scatter(torch.from_numpy(mask)[..., None], vis)
        hidden = lm(inputs_embeds=emb, position_ids=torch.from_numpy(pos3), visual_pos_masks=torch.from_numpy(mask), deepstack_visual_embeds=deep).last_hidden_state
        want = hf.lm_head(hidden)
        want_text = hf.lm_head(lm(inputs_embeds=lm.embed_tokens(torch.from_numpy(tok).long())).last_hidden_state)
    cfg = load_hf_config(src)
    tr = Trainer(TrainerConfig(model=cfg, batch_size=1, seq_len=T, grad_accum=2, zero_level=0), device=torch.device("cpu"))
    tr.import_weights(src)
    assert torch.allclose(tr.logits(tok), want_text, atol=2e-4, rtol=1e-3)  # text-only batch: plain rotary positions
    tr.set_visual_inputs(mask, vis, deep, pos3)
    got = tr.logits(tok)
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), float((got - want).abs().max())
    # a training step with two micro-batches slices the packed vision features per row; embedding rows under the mask get no gradient
    tgt = np.roll(tok, -1, axis=1).astype(np.int32)
    tgt[:, -1] = -100
    r = tr.forward_backward(tok, tgt)
    loss = torch.nn.functional.cross_entropy(want.reshape(-1, 320), torch.from_numpy(tgt).long().reshape(-1), ignore_index=-100)
    assert abs(float(r["loss_sum"] / r["n_valid"]) - float(loss)) < 1e-4
    tr.set_visual_inputs()
    assert torch.allclose(tr.logits(tok), want_text, atol=2e-4, rtol=1e-3)
    # export keeps the vision tower of the imported checkpoint, so the directory loads as the full model again
    tr.store.release_grads()
    out = os.path.join(tmp_path, "export")
    tr.export_model(out, cfg)
    back = Qwen3VLForConditionalGeneration.from_pretrained(out, torch_dtype=torch.float32)
    assert any(k.startswith("model.visual.") for k in back.state_dict())
    for (ka, va), (kb, vb) in zip(sorted(hf.state_dict().items()), sorted(back.state_dict().items())):
        assert ka == kb and torch.allclose(va.float(), vb.float(), atol=1e-2, rtol=1e-2), ka
