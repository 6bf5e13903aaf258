"""On-the-fly multimodal batches for vision-language fine-tuning (Qwen3-VL family).

The text decoder is the trained model; the vision tower stays a frozen HuggingFace module that runs once per batch, outside
the training graph.  A batch is ordinary ``inputs`` / ``targets`` plus the decoder's side inputs:

* ``visual_pos_masks`` [rows, T]: which tokens are image / video placeholders,
* ``visual_embeds`` [n_visual, C]: the tower's merged patch embeddings, in row-major mask order,
* ``deepstack_visual_embeds``: a list of [n_visual, C] intermediate features added by the first decoder layers,
* ``mrope_position_ids`` [3, rows, T]: temporal / height / width rotary positions.

``OnTheFlyMultimodalBatcher.next_batch()`` returns that dict; ``apply(trainer, batch)`` hands the side inputs to
``Trainer.set_visual_inputs``.

Parity: surogate/train/vision.py (MultimodalEncoder, OnTheFlyMultimodalBatcher, init_mm_helpers).
"""
from __future__ import annotations

import itertools
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence

import numpy as np
import torch

IGNORE = -100


# --------------------------------------------------------------------------------------------- rotary positions
def mrope_positions(token_types: Sequence[int], grids: Iterable[Sequence[int]], spatial_merge: int = 2) -> np.ndarray:
    """(t, h, w) rotary positions [3, T] of one sequence.

    ``token_types[i]`` is 0 for text and non-zero for an image / video-frame placeholder token; every maximal run of non-zero
    types consumes the next ``(t, h, w)`` patch grid from ``grids``.  Text advances all three axes together.  A vision run
    keeps the temporal axis at the run's start and counts rows / columns of the merged grid on the other two; the text after
    it resumes at start + max(h, w) / spatial_merge, so later tokens never share a position with a patch.
    """
    out: List[np.ndarray] = []
    cur = 0
    grids = iter(grids)
    for kind, run in itertools.groupby(token_types, key=lambda v: int(v) != 0):
        n = sum(1 for _ in run)
        if not kind:
            out.append(np.tile(np.arange(cur, cur + n, dtype=np.int64), (3, 1)))
            cur += n
            continue
        t, h, w = (int(v) for v in next(grids))
        gh, gw = h // spatial_merge, w // spatial_merge
        if t * gh * gw != n:
            raise ValueError(f"placeholder run of {n} tokens does not match its patch grid {t}x{h}x{w} (merge {spatial_merge})")
        hh = np.repeat(np.arange(cur, cur + gh, dtype=np.int64), gw * t)
        ww = np.tile(np.arange(cur, cur + gw, dtype=np.int64), gh * t)
        out.append(np.stack([np.full(n, cur, np.int64), hh, ww]))
        cur += max(h, w) // spatial_merge
    return np.concatenate(out, axis=1) if out else np.zeros((3, 0), np.int64)


def split_video_grids(video_grid_thw: Optional[np.ndarray]) -> List[List[int]]:
    """Videos are laid out frame by frame (a timestamp and a placeholder run per frame): a (t, h, w) video becomes t grids of
    (1, h, w)."""
    out: List[List[int]] = []
    for t, h, w in (np.asarray(video_grid_thw).tolist() if video_grid_thw is not None else []):
        out.extend([[1, h, w]] * int(t))
    return out


# --------------------------------------------------------------------------------------------- frozen vision tower
class VisionTower:
    """The frozen HuggingFace vision module of a vision-language checkpoint.

    ``encode(pixel_values, grid_thw)`` returns (embeds [n_visual, C], [deepstack features [n_visual, C], ...])."""

    def __init__(self, visual: torch.nn.Module, device: Optional[torch.device] = None, dtype: torch.dtype = torch.bfloat16):
        self.visual = visual.to(device=device, dtype=dtype).eval().requires_grad_(False)
        self.device, self.dtype = device, dtype
        self.spatial_merge = int(getattr(visual, "spatial_merge_size", 2))

    @classmethod
    def from_pretrained(cls, model_dir: str, device: Optional[torch.device] = None, dtype: torch.dtype = torch.bfloat16) -> "VisionTower":
        from transformers import AutoModelForImageTextToText

        full = AutoModelForImageTextToText.from_pretrained(model_dir, torch_dtype=dtype)
        visual = find_visual(full)
        del full
        return cls(visual, device, dtype)

    @torch.no_grad()
    def encode(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor):
        out = self.visual(pixel_values.to(self.device, self.dtype), grid_thw=grid_thw.to(self.device), return_dict=True)
        deep = list(getattr(out, "deepstack_features", None) or [])
        return out.pooler_output, deep


def find_visual(hf_model) -> torch.nn.Module:
    for path in ("model.visual", "visual", "model.vision_tower", "vision_tower"):
        node = hf_model
        try:
            for part in path.split("."):
                node = getattr(node, part)
            return node
        except AttributeError:
            continue
    raise AttributeError("no vision tower found on this model (looked for model.visual, visual, model.vision_tower, vision_tower)")


# --------------------------------------------------------------------------------------------- row encoder
class MultimodalEncoder:
    """One dataset row ({"messages": [...], "images": [...]} in the chat format of HF processors) -> token ids, training labels,
    pixel values and patch grids.  Labels cover assistant turns only (everything up to and including each assistant header is
    ignored), found by re-encoding the conversation prefix before each assistant turn."""

    def __init__(self, processor, image_token_id: int, video_token_id: Optional[int] = None):
        self.processor, self.image_token_id, self.video_token_id = processor, int(image_token_id), video_token_id

    def _ids(self, messages, images, add_generation_prompt=False) -> Dict[str, Any]:
        text = self.processor.apply_chat_template(messages, tokenize=False, add_generation_prompt=add_generation_prompt)
        return self.processor(text=[text], images=images or None, return_tensors="np")

    def encode(self, row: Dict[str, Any]) -> Optional[Dict[str, Any]]:
        messages, images = row["messages"], row.get("images") or []
        full = self._ids(messages, images)
        ids = np.asarray(full["input_ids"][0], np.int64)
        labels = np.full_like(ids, IGNORE)
        used = 0
        for i, m in enumerate(messages):
            if m.get("role") != "assistant":
                continue
            n_img = sum(1 for mm in messages[:i] for c in (mm["content"] if isinstance(mm["content"], list) else []) if c.get("type") == "image")
            prefix = np.asarray(self._ids(messages[:i], images[:n_img], add_generation_prompt=True)["input_ids"][0])
            upto = np.asarray(self._ids(messages[:i + 1], images[:n_img])["input_ids"][0])
            a, b = len(prefix), len(upto)
            if b <= a or b > len(ids):
                return None  # template did not nest as expected: skip the row rather than train on wrong labels
            labels[a:b] = ids[a:b]
            used += b - a
        if used == 0:
            return None
        return {"input_ids": ids, "labels": labels, "pixel_values": full.get("pixel_values"), "image_grid_thw": full.get("image_grid_thw"),
                "pixel_values_videos": full.get("pixel_values_videos"), "video_grid_thw": full.get("video_grid_thw")}


# --------------------------------------------------------------------------------------------- batcher
class OnTheFlyMultimodalBatcher:
    """Pulls raw rows, encodes them, runs the frozen vision tower and pads to fixed [rows, seq_len] arrays.

    ``rows``: an iterable of dataset rows (restarted at the end: one pass is one epoch); ``encode``: row -> dict with
    ``input_ids``, ``labels`` and optionally ``pixel_values`` / ``image_grid_thw`` / ``pixel_values_videos`` /
    ``video_grid_thw`` (``MultimodalEncoder.encode``), or None to skip; ``tower``: object with
    ``encode(pixel_values, grid_thw)`` and ``spatial_merge``.  Rows that do not fit ``seq_len`` or whose placeholder count
    disagrees with their patch grids are skipped and counted in ``skipped``.
    """

    def __init__(self, rows: Iterable[Dict[str, Any]], encode: Callable[[Dict[str, Any]], Optional[Dict[str, Any]]], tower, batch_rows: int, seq_len: int,
                 image_token_id: int, video_token_id: Optional[int] = None, pad_token_id: int = 0, d_model: Optional[int] = None):
        self._rows, self._encode, self.tower = rows, encode, tower
        self.batch_rows, self.seq_len = int(batch_rows), int(seq_len)
        self.image_token_id, self.video_token_id, self.pad_token_id = int(image_token_id), video_token_id, int(pad_token_id)
        self.d_model = d_model
        self.epoch, self.skipped, self.rows_seen = 0, 0, 0
        self._it: Iterator[Dict[str, Any]] = iter(self._rows)

    def _next_row(self) -> Dict[str, Any]:
        for _ in range(2):
            try:
                self.rows_seen += 1
                return next(self._it)
            except StopIteration:
                self.epoch += 1
                self._it = iter(self._rows)
        raise RuntimeError("multimodal dataset is empty")

    def _usable(self, enc: Optional[Dict[str, Any]]) -> bool:
        if enc is None or len(enc["input_ids"]) > self.seq_len + 1 or len(enc["input_ids"]) < 2:
            return False
        m = self.tower.spatial_merge ** 2
        ids = np.asarray(enc["input_ids"])
        want_img = int(sum(int(np.prod(g)) // m for g in (np.asarray(enc["image_grid_thw"]).tolist() if enc.get("image_grid_thw") is not None else [])))
        want_vid = int(sum(int(np.prod(g)) // m for g in (np.asarray(enc["video_grid_thw"]).tolist() if enc.get("video_grid_thw") is not None else [])))
        have_img = int((ids == self.image_token_id).sum())
        have_vid = int((ids == self.video_token_id).sum()) if self.video_token_id is not None else 0
        return want_img == have_img and want_vid == have_vid

    def next_batch(self) -> Dict[str, Any]:
        picked: List[Dict[str, Any]] = []
        tries = 0
        while len(picked) < self.batch_rows:
            tries += 1
            if tries > 64 * self.batch_rows:
                raise RuntimeError("no usable multimodal rows: every row was skipped (too long for seq_len, or placeholder / grid mismatch)")
            enc = self._encode(self._next_row())
            if self._usable(enc):
                picked.append(enc)
            else:
                self.skipped += 1
        return self._build(picked)

    def _build(self, encs: List[Dict[str, Any]]) -> Dict[str, Any]:
        R, T = len(encs), self.seq_len
        inputs = np.full((R, T), self.pad_token_id, np.int32)
        targets = np.full((R, T), IGNORE, np.int32)
        mask = np.zeros((R, T), bool)
        pos3 = np.zeros((3, R, T), np.int32)
        embeds: List[torch.Tensor] = []
        deep: List[List[torch.Tensor]] = []
        for r, e in enumerate(encs):
            ids, labels = np.asarray(e["input_ids"]), np.asarray(e["labels"])
            n = min(len(ids) - 1, T)
            inputs[r, :n] = ids[:n]
            targets[r, :n] = labels[1:n + 1]  # next-token targets
            is_img = ids == self.image_token_id
            is_vid = (ids == self.video_token_id) if self.video_token_id is not None else np.zeros_like(is_img)
            types = np.where(is_img, 1, np.where(is_vid, 2, 0))
            # grids in order of appearance: images and video frames interleave as their placeholder runs do
            img = iter(np.asarray(e["image_grid_thw"]).tolist() if e.get("image_grid_thw") is not None else [])
            vid = iter(split_video_grids(e.get("video_grid_thw")))
            grids = [next(img) if kind == 1 else next(vid) for kind, _ in itertools.groupby(types.tolist()) if kind != 0]
            p = mrope_positions(types.tolist(), grids, self.tower.spatial_merge)
            pos3[:, r, :n] = p[:, :n]
            if n < T:  # padding continues the text positions (never attended to by real tokens, never a target)
                last = int(p[:, :n].max()) + 1 if n else 0
                pos3[:, r, n:] = np.arange(last, last + T - n, dtype=np.int32)
            mask[r, :n] = (types != 0)[:n]
            row_embeds, row_deep = [], []
            for px, grid in ((e.get("pixel_values"), e.get("image_grid_thw")), (e.get("pixel_values_videos"), e.get("video_grid_thw"))):
                if px is None or grid is None or len(grid) == 0:
                    continue
                emb, ds = self.tower.encode(torch.as_tensor(px), torch.as_tensor(np.asarray(grid)))
                row_embeds.append(emb)
                row_deep.append(ds)
            if row_embeds:
                emb = torch.cat(row_embeds, 0)
                kept = int(mask[r].sum())  # a placeholder run cut by seq_len keeps its first rows
                embeds.append(emb[:kept])
                deep.append([torch.cat([d[i] for d in row_deep], 0)[:kept] for i in range(len(row_deep[0]))])
        out: Dict[str, Any] = {"inputs": inputs, "targets": targets, "position_ids": pos3[0].copy(), "mrope_position_ids": pos3, "visual_pos_masks": mask}
        if embeds:
            out["visual_embeds"] = torch.cat(embeds, 0)
            out["deepstack_visual_embeds"] = [torch.cat([d[i] for d in deep], 0) for i in range(len(deep[0]))]
        else:
            out["visual_embeds"], out["deepstack_visual_embeds"] = None, []
        return out


def apply(trainer, batch: Dict[str, Any]) -> None:
    """Hand a batch's side inputs to the trainer (clears them for a text-only batch)."""
    if batch.get("visual_embeds") is None:
        trainer.set_visual_inputs(mrope_position_ids=batch.get("mrope_position_ids"))
    else:
        trainer.set_visual_inputs(batch["visual_pos_masks"], batch["visual_embeds"], batch["deepstack_visual_embeds"], batch["mrope_position_ids"])


def init_mm_helpers(model_dir: str, device: Optional[torch.device] = None, dtype: torch.dtype = torch.bfloat16):
    """(processor, encoder, tower) for a vision-language checkpoint directory."""
    import json
    import os

    from transformers import AutoProcessor

    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    processor = AutoProcessor.from_pretrained(model_dir)
    enc = MultimodalEncoder(processor, cfg["image_token_id"], cfg.get("video_token_id"))
    return processor, enc, VisionTower.from_pretrained(model_dir, device, dtype)


def load_multimodal_rows(paths: Sequence[str]) -> List[Dict[str, Any]]:
    """Rows of JSON-lines files: {"messages": [...], "images": ["path" | already-decoded image, ...]}.  Image paths are opened
    with PIL relative to the file's directory."""
    import json
    import os

    rows: List[Dict[str, Any]] = []
    for path in paths:
        base = os.path.dirname(os.path.abspath(path))
        with open(path) as f:
            for line in f:
                if not line.strip():
                    continue
                row = json.loads(line)
                imgs = []
                for im in row.get("images") or []:
                    if isinstance(im, str):
                        from PIL import Image

                        im = Image.open(im if os.path.isabs(im) else os.path.join(base, im)).convert("RGB")
                    imgs.append(im)
                row["images"] = imgs
                rows.append(row)
    return rows


class VisionTrainLoader:
    """Adapter with the token loader's interface (``next_batch() -> (inputs, targets, position_ids)``) over a multimodal
    batcher: each call also installs the batch's side inputs on the trainer.  Every rank reads the rows ``rank::world``."""

    def __init__(self, batcher: OnTheFlyMultimodalBatcher, trainer):
        self.batcher, self.trainer = batcher, trainer

    def next_batch(self):
        b = self.batcher.next_batch()
        apply(self.trainer, b)
        return b["inputs"], b["targets"], b["position_ids"]

    def steps_per_epoch(self) -> int:
        n = len(self.batcher._rows) if hasattr(self.batcher._rows, "__len__") else 0
        return max(1, n // max(1, self.batcher.batch_rows))

    def state_dict(self) -> Dict[str, Any]:
        return {"rows_seen": self.batcher.rows_seen, "epoch": self.batcher.epoch}

    def load_state_dict(self, state: Dict[str, Any]) -> None:
        seen = int(state.get("rows_seen", 0))
        for _ in range(seen - self.batcher.rows_seen):  # replay the row cursor (rows are cheap to skip: nothing is encoded)
            self.batcher._next_row()
