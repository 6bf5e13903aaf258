"""Tokenising a dataset through a pool of processes gives the same documents, in the same order, as one process."""
import json
import os

import numpy as np
import pytest

from surogate_b200.ops import host_available

pytestmark = pytest.mark.skipif(not host_available(), reason="host runtime not built")


def test_process_count_sources(monkeypatch):
    import types

    from surogate_b200.train.tokenize import dataset_processes

    monkeypatch.delenv("SUROGATE_DATASET_PROCESSES", raising=False)
    monkeypatch.delenv("RUNPOD_CPU_COUNT", raising=False)
    assert 1 <= dataset_processes() <= 8
    monkeypatch.setenv("RUNPOD_CPU_COUNT", "3")
    assert dataset_processes() == 3
    monkeypatch.setenv("SUROGATE_DATASET_PROCESSES", "64")
    assert dataset_processes() == 8  # capped
    assert dataset_processes(types.SimpleNamespace(dataloader_num_workers=2)) == 2
    monkeypatch.setenv("SUROGATE_DATASET_PROCESSES", "1")
    assert dataset_processes(types.SimpleNamespace(dataloader_num_workers=0)) == 1


def test_pool_equals_one_process(tmp_path, monkeypatch):
    pytest.importorskip("tokenizers")
    from test_host_runtime import QWEN_PATTERN, _train_tokenizer

    import surogate_b200.train.tokenize as tz
    from surogate_b200.config.sft_config import SFTConfig

    _, mdir = _train_tokenizer(QWEN_PATTERN, str(tmp_path), "model")
    with open(os.path.join(mdir, "tokenizer_config.json"), "w") as f:
        json.dump({"eos_token": "<|im_end|>", "pad_token": "<|endoftext|>"}, f)
    data = os.path.join(tmp_path, "chat.jsonl")
    with open(data, "w") as f:
        for i in range(300):
            if i % 50 == 7:
                f.write(json.dumps({"unknown": i}) + "\n")  # a row that encodes to nothing is dropped in both paths
            else:
                f.write(json.dumps({"messages": [{"role": "user", "content": f"Hello world {i}"}, {"role": "assistant", "content": "It's a test " * (1 + i % 5)}]}) + "\n")
    cfg = SFTConfig.from_dict(dict(model=mdir, datasets=[{"path": data}], sequence_len=40, truncation_strategy="delete", output_dir=str(tmp_path / "out")))
    from surogate_b200.data.datasets import load_dataset_rows

    rows = load_dataset_rows(cfg.datasets[0])
    monkeypatch.setenv("SUROGATE_DATASET_PROCESSES", "1")
    serial = tz.TokenizeDatasets(cfg, {"vocab_size": 600}, "").encode_rows(rows)
    monkeypatch.setenv("SUROGATE_DATASET_PROCESSES", "2")
    monkeypatch.setattr(tz, "PARALLEL_MIN_ROWS", 100)
    pooled = tz.TokenizeDatasets(cfg, {"vocab_size": 600}, "").encode_rows(rows)
    assert 0 < len(serial) < len(rows) and len(pooled) == len(serial)
    for (a, am), (b, bm) in zip(serial, pooled):
        assert np.array_equal(a, b) and np.array_equal(am, bm) and a.dtype == b.dtype
    # a tokenizer object handed in by the caller stays in this process whatever the size
    from surogate_b200.data.tokenizer import Tokenizer

    own = tz.TokenizeDatasets(cfg, {"vocab_size": 600}, "", tokenizer=Tokenizer.from_pretrained(mdir))
    assert len(own.encode_rows(rows)) == len(serial)


def test_tokenizer_profile(tmp_path, monkeypatch):
    import io

    pytest.importorskip("tokenizers")
    from test_host_runtime import QWEN_PATTERN, _train_tokenizer

    from surogate_b200.data import tok_profile
    from surogate_b200.data.tokenizer import Tokenizer

    _, mdir = _train_tokenizer(QWEN_PATTERN, str(tmp_path), "model")
    with open(os.path.join(mdir, "tokenizer_config.json"), "w") as f:
        json.dump({"eos_token": "<|im_end|>", "pad_token": "<|endoftext|>"}, f)
    plain = Tokenizer.from_pretrained(mdir)
    assert "encode" not in vars(plain)  # nothing wrapped without the variable
    monkeypatch.setenv("SUROGATE_TOK_PROFILE", "1")
    tok = Tokenizer.from_pretrained(mdir)
    tok_profile.profile().reset()
    msgs = [{"role": "user", "content": "Hello world"}, {"role": "assistant", "content": "It's a test"}]
    want = plain.encode_for_training(msgs)
    assert tok.encode_for_training(msgs) == want and tok.encode_for_training(msgs) == want
    s = tok_profile.profile().summary()
    assert s["calls"]["encode_for_training"] == 2 and s["calls"]["render"] >= 2 and s["calls"]["encode"] >= 2 and s["tokens"] == 2 * len(want[0])
    assert s["ms"]["encode_for_training"] >= s["ms"]["render"] and s["align_and_label_ms"] >= 0 and s["tokens_per_second"] > 0
    buf = io.StringIO()
    tok_profile.profile().report(buf)
    assert "[tok-profile]" in buf.getvalue() and "align + labels" in buf.getvalue()
    tok_profile.profile().reset()
    empty = io.StringIO()
    tok_profile.profile().report(empty)
    assert empty.getvalue() == ""
