"""Vision-language batches: rotary position rule, frozen vision tower, batcher -> trainer side inputs, against transformers."""
import os

import numpy as np
import pytest
import torch

transformers = pytest.importorskip("transformers")

from surogate_b200.dsl.compiler import load_hf_config  # noqa: E402
from surogate_b200.runtime.trainer import Trainer, TrainerConfig  # noqa: E402
from surogate_b200.train import vision  # noqa: E402

IMG, VID, VSTART = 300, 301, 302


def _tiny_model():
    from transformers import Qwen3VLConfig, Qwen3VLForConditionalGeneration

    text = dict(vocab_size=320, hidden_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=96,
                max_position_embeddings=256, rms_norm_eps=1e-6, rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [4, 2, 2]},
                tie_word_embeddings=False)
    vis = dict(depth=2, hidden_size=32, intermediate_size=48, num_heads=2, out_hidden_size=64, patch_size=4, spatial_merge_size=2, temporal_patch_size=2,
               deepstack_visual_indexes=[0, 1], num_position_embeddings=16, in_channels=3)
    torch.manual_seed(0)
    cfg = Qwen3VLConfig(text_config=text, vision_config=vis, image_token_id=IMG, video_token_id=VID, vision_start_token_id=VSTART, tie_word_embeddings=False)
    return Qwen3VLForConditionalGeneration(cfg).float().eval()


def _row(rng, grid, n_before, n_after):
    """token ids with one image of patch grid (t, h, w); pixel_values are flattened patches [t*h*w, C*tp*p*p]."""
    t, h, w = grid
    n_img = t * h * w // 4
    ids = np.concatenate([rng.integers(0, 290, n_before), [VSTART], np.full(n_img, IMG), rng.integers(0, 290, n_after)]).astype(np.int64)
    labels = ids.copy()
    labels[:n_before + 1 + n_img] = -100
    px = rng.standard_normal((t * h * w, 3 * 2 * 4 * 4)).astype(np.float32)
    return {"input_ids": ids, "labels": labels, "pixel_values": px, "image_grid_thw": np.asarray([grid])}


def test_rotary_positions_follow_the_reference_rule():
    hf = _tiny_model()
    rng = np.random.default_rng(0)
    r = _row(rng, (1, 4, 8), 5, 7)
    ids = torch.from_numpy(r["input_ids"])[None]
    types = (ids == IMG).int()
    want, _ = hf.model.get_rope_index(ids, types, image_grid_thw=torch.from_numpy(r["image_grid_thw"]))
    got = vision.mrope_positions(types[0].tolist(), r["image_grid_thw"].tolist(), spatial_merge=2)
    assert np.array_equal(got, want[:, 0].numpy())
    assert got[:, -1].tolist() == [5 + 1 + 4 + 6] * 3  # text resumes after max(h, w) / merge = 4 positions
    with pytest.raises(ValueError):
        vision.mrope_positions([0, 1, 1, 0], [[1, 4, 4]], 2)  # 2 placeholders for a 4-token grid


def test_batches_through_the_frozen_tower_match_the_full_transformers_model(tmp_path):
    hf = _tiny_model()
    src = os.path.join(tmp_path, "hf")
    hf.save_pretrained(src, safe_serialization=True)
    rng = np.random.default_rng(1)
    rows = [_row(rng, (1, 4, 8), 5, 9), _row(rng, (1, 4, 4), 3, 12), {"input_ids": np.arange(500), "labels": np.arange(500)}]  # the last one is too long
    T = 26
    tower = vision.VisionTower(hf.model.visual, torch.device("cpu"), torch.float32)
    b = vision.OnTheFlyMultimodalBatcher(rows, lambda r: r, tower, batch_rows=2, seq_len=T, image_token_id=IMG, video_token_id=VID)
    batch = b.next_batch()
    assert batch["inputs"].shape == (2, T) and int(batch["visual_pos_masks"].sum()) == 8 + 4 == batch["visual_embeds"].shape[0]
    assert len(batch["deepstack_visual_embeds"]) == 2
    tr = Trainer(TrainerConfig(model=load_hf_config(src), batch_size=2, seq_len=T, zero_level=0), device=torch.device("cpu"))
    tr.import_weights(src)
    vision.apply(tr, batch)
    got = tr.logits(batch["inputs"])
    for r in range(2):
        n = len(rows[r]["input_ids"]) - 1
        ids = torch.from_numpy(rows[r]["input_ids"][:n])[None]
        with torch.no_grad():
            want = hf(input_ids=ids, pixel_values=torch.from_numpy(rows[r]["pixel_values"]), image_grid_thw=torch.from_numpy(rows[r]["image_grid_thw"]),
                      mm_token_type_ids=(ids == IMG).int()).logits[0]
        assert torch.allclose(got[r, :n], want, atol=3e-4, rtol=1e-3), (r, float((got[r, :n] - want).abs().max()))
    res = tr.step(batch["inputs"], batch["targets"], lr=1e-3)
    assert np.isfinite(res["loss"])
    b2 = vision.OnTheFlyMultimodalBatcher(rows, lambda r: r, tower, batch_rows=2, seq_len=T, image_token_id=IMG)
    b2.next_batch(), b2.next_batch(), b2.next_batch()
    assert b2.skipped == 2 and b2.epoch == 2  # the over-long row is skipped on every pass
