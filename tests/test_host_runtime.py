"""Native host runtime (CUDA-free C++): tokenizer, token loader, safetensors I/O, CPU AdamW, LPT planner, telemetry."""
import json
import os

import numpy as np
import pytest
import torch

from surogate_b200.ops import host, host_available

pytestmark = pytest.mark.skipif(not host_available(), reason="host runtime not built")

CORPUS = [
    "Hello world! It's a test, isn't it? We'll see what they've done.",
    "def f(x):\n    return x**2 + 12345  # comment\n\n\nclass A:  pass",
    "Ünïcödé tèxt — 中文字符 和 日本語 テキスト 1234567 ٣٤٥",
    "   leading spaces\tand\ttabs \n trailing  \r\n windows line   ",
    "I'M SHOUTING, DON'T YOU'RE — emojis 🙂🙃 and symbols ###$$$ ...",
]


def _train_tokenizer(pattern, tmp_path, name):
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers

    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(pattern), behavior="isolated"),
                                                 pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=600, special_tokens=["<|endoftext|>", "<|im_start|>", "<|im_end|>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(CORPUS * 4, trainer)
    path = os.path.join(tmp_path, name)
    os.makedirs(path, exist_ok=True)
    tok.save(os.path.join(path, "tokenizer.json"))
    return tok, path


QWEN_PATTERN = r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"
LLAMA3_PATTERN = r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"
GPT2_PATTERN = r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"


@pytest.mark.parametrize("pattern,name", [(QWEN_PATTERN, "qwen"), (LLAMA3_PATTERN, "llama3"), (GPT2_PATTERN, "gpt2")])
def test_bpe_matches_hf_tokenizers(tmp_path, pattern, name):
    ref, path = _train_tokenizer(pattern, str(tmp_path), name)
    from surogate_b200.data.tokenizer import Tokenizer

    tok = Tokenizer.from_pretrained(path)
    extra = ["", " ", "a", "x  y   z", "12 345 6789012", "tail space ", "\n\n\nthree", "<|im_start|>user\nhi<|im_end|>\n<|endoftext|>",
             "mixed<|im_end|>inline 's 'S 'Re", "🙂" * 5]
    for text in CORPUS + extra:
        want = ref.encode(text).ids
        got = tok.encode(text)
        assert got == want, (name, text, got, want)
        assert tok.decode(got) == text
    assert tok.encode_batch(CORPUS, threads=3) == [ref.encode(t).ids for t in CORPUS]
    assert tok.is_special_token(tok.core.token_to_id(b"<|im_end|>"))


def test_chat_template_training_mask(tmp_path):
    _, path = _train_tokenizer(QWEN_PATTERN, str(tmp_path), "chat")
    with open(os.path.join(path, "tokenizer_config.json"), "w") as f:
        json.dump({"eos_token": "<|im_end|>", "pad_token": "<|endoftext|>"}, f)
    from surogate_b200.data.tokenizer import IGNORE, Tokenizer

    tok = Tokenizer.from_pretrained(path)
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "Hello world"}, {"role": "assistant", "content": "It's a test"},
            {"role": "user", "content": "more"}, {"role": "assistant", "content": "done"}]
    ids, labels = tok.encode_for_training(msgs)
    assert len(ids) == len(labels)
    trained = tok.decode([l for l in labels if l != IGNORE])
    assert trained == "It's a test<|im_end|>\ndone<|im_end|>\n"
    _, last = tok.encode_for_training(msgs, train_on="last")
    assert tok.decode([l for l in last if l != IGNORE]) == "done<|im_end|>\n"
    assert tok.eos_token_id == tok.core.token_to_id(b"<|im_end|>")
    # a message's own ``loss`` field overrides the mode for that turn
    off = [dict(m, loss=0) if m["content"] == "It's a test" else m for m in msgs]
    assert tok.decode([l for l in tok.encode_for_training(off)[1] if l != IGNORE]) == "done<|im_end|>\n"
    on = [dict(m, loss=1) if m["content"] == "It's a test" else m for m in msgs]
    assert tok.decode([l for l in tok.encode_for_training(on, train_on="last")[1] if l != IGNORE]) == "It's a test<|im_end|>\ndone<|im_end|>\n"
    all_ids, all_labels = tok.encode_for_training(off, train_on="all")
    assert "It's a test" not in tok.decode([l for l in all_labels if l != IGNORE]) and "Hello world" in tok.decode([l for l in all_labels if l != IGNORE])
    # two assistant turns after the last user message are both "the last round"
    tail = msgs[:4] + [{"role": "assistant", "content": "one"}, {"role": "tool", "content": "r"}, {"role": "assistant", "content": "two"}]
    got = tok.decode([l for l in tok.encode_for_training(tail, train_on="last")[1] if l != IGNORE])
    assert "one" in got and "two" in got and "It's a test" not in got
    from surogate_b200.train.tokenize import loss_scale_mode

    assert [loss_scale_mode(x) for x in ("default", "all", "last_round", "last_round+-", "-", "default+default")] == ["assistant", "all", "last", "last", "assistant", "assistant"]
    with pytest.raises(ValueError):
        loss_scale_mode("react")


def test_token_loader_native_matches_python_and_resumes(tmp_path):
    from surogate_b200.data.loader import DataLoader
    from surogate_b200.data.tokfile import TokenFileWriter

    rng = np.random.default_rng(0)
    files = []
    for i, rows in enumerate([9, 14]):
        p = os.path.join(tmp_path, f"train-{i:03d}.bin")
        w = TokenFileWriter(p, 1000, has_masks=True, non_overlapping=True)
        for _ in range(rows):
            t = rng.integers(0, 1000, 16).astype(np.int32)
            pos = np.concatenate([np.arange(7), np.arange(9)]).astype(np.int32)
            w.add(t, pos, (rng.random(16) > 0.3).astype(np.uint8))
        w.close()
        files.append(p)
    for rank in range(2):
        nat = DataLoader(files, 3, 16, seed=7, rank=rank, world=2, native=True)
        ref = DataLoader(files, 3, 16, seed=7, rank=rank, world=2, native=False)
        assert nat.steps_per_epoch() == ref.steps_per_epoch()
        for step in range(9):  # crosses file and epoch boundaries
            a, b = nat.next_batch(), ref.next_batch()
            for u, v in zip(a, b):
                np.testing.assert_array_equal(u, v)
            assert nat.state_dict() == ref.state_dict()
            if step == 4:
                saved = nat.state_dict()
        resumed = DataLoader(files, 3, 16, seed=7, rank=rank, world=2, native=True)
        resumed.load_state_dict(saved)
        again = DataLoader(files, 3, 16, seed=7, rank=rank, world=2, native=False)
        again.load_state_dict(saved)
        for _ in range(3):
            for u, v in zip(resumed.next_batch(), again.next_batch()):
                np.testing.assert_array_equal(u, v)
    x, y, p = ref.next_batch()
    assert (y[:, -1] == -100).all() and (y[:, 6] == -100).all()  # row end and document boundary carry no target


def test_safetensors_native_roundtrip(tmp_path):
    from safetensors.torch import load_file, save_file

    from surogate_b200.io.safetensors_native import NativeSafetensors, save_file_native

    torch.manual_seed(0)
    tensors = {"a.weight": torch.randn(64, 32).bfloat16(), "b": torch.arange(10, dtype=torch.int32), "c": torch.randn(3, 5, 7),
               "big": torch.randn(3000, 1024)}
    p1, p2 = os.path.join(tmp_path, "lib.safetensors"), os.path.join(tmp_path, "native.safetensors")
    save_file(tensors, p1, metadata={"format": "pt"})
    f = NativeSafetensors(p1, threads=4)
    assert sorted(f.keys()) == sorted(tensors) and f.metadata() == {"format": "pt"}
    for k, t in tensors.items():
        assert torch.equal(f.get_tensor(k), t)
    assert torch.equal(f.get_rows("big", 1000, 2500), tensors["big"][1000:2500])
    save_file_native(tensors, p2, metadata={"format": "pt"}, threads=4)
    back = load_file(p2)
    for k, t in tensors.items():
        assert torch.equal(back[k], t)


def test_cpu_adamw_matches_torch():
    h = host()
    torch.manual_seed(0)
    n = 10007
    p = torch.randn(n)
    ref = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v, work = torch.zeros(n), torch.zeros(n), torch.zeros(n, dtype=torch.bfloat16)
    for step in range(1, 4):
        g = torch.randn(n)
        ref.grad = g.clone()
        opt.step()
        gb = g.bfloat16() if step == 3 else g
        if step == 3:
            ref.data.copy_(p)  # redo the reference with the rounded gradient
            opt.state[ref]["exp_avg"].copy_(m)
            opt.state[ref]["exp_avg_sq"].copy_(v)
            opt.state[ref]["step"].fill_(2)
            ref.grad = gb.float()
            opt.step()
        h.cpu_adamw_step(p.data_ptr(), m.data_ptr(), v.data_ptr(), gb.data_ptr(), gb.dtype == torch.bfloat16, work.data_ptr(), n, 1e-2, 0.9, 0.95, 1e-8,
                         0.1, 1.0, step)
        torch.testing.assert_close(p, ref.detach(), rtol=1e-5, atol=1e-6)
    assert torch.equal(work, p.bfloat16())
    assert abs(h.cpu_sum_squares(p.data_ptr(), False, n) - float((p.double() ** 2).sum())) < 1e-6 * n


def test_lpt_plan_balances_and_conserves_tokens():
    h = host()
    counts = [9000, 200, 100, 300, 500, 400, 300, 200, 250, 250, 250, 250, 100, 100, 100, 100]
    assert h.compute_lpt_plan(counts, 4, 100.0, 1.1, 64)["uses_lpt"] is False
    plan = h.compute_lpt_plan(counts, 4, 1.3, 1.1, 64)
    assert plan["uses_lpt"] and plan["imbalance"] > 1.3
    for e, chunks in enumerate(plan["assignments"]):
        assert sum(b - a for _, a, b in chunks) == counts[e]
        assert chunks[0][1] == 0 and all(chunks[i][2] == chunks[i + 1][1] for i in range(len(chunks) - 1))
    assert sum(plan["gpu_loads"]) == sum(counts)
    assert max(plan["gpu_loads"]) < 0.5 * 9000 + 2000  # the hot expert was spread
    assert all(src == e // 4 for e, src, _ in plan["moves"])


def test_crash_handler_and_telemetry_are_safe_without_gpu():
    h = host()
    h.install_crash_handler("test")
    info = h.query_gpu(0)
    assert "ok" in info and (info["ok"] or info["error"])


def test_expert_replacement_moves_only_when_it_pays():
    """Placement decisions: a stable skew is corrected, balanced or noisy counts and hot single experts leave the placement alone."""
    from surogate_b200.parallel.ep import decide_placement

    cur = list(range(8))
    new, moved = decide_placement([100, 100, 100, 100, 10, 10, 10, 10], cur, 2)
    per_rank = [sum(c for e, c in enumerate([100, 100, 100, 100, 10, 10, 10, 10]) if new[e] // 4 == r) for r in range(2)]
    assert moved > 0 and sorted(new) == cur and max(per_rank) <= 1.1 * (sum(per_rank) / 2)
    assert decide_placement([100, 90, 110, 100, 95, 105, 100, 100], cur, 2) == (cur, 0)   # within the threshold
    assert decide_placement([400, 0, 0, 0, 100, 100, 100, 100], cur, 2) == (cur, 0)       # one hot expert: no placement helps
    assert decide_placement([100, 100, 100, 100, 10, 10, 10, 10], cur, 2, max_moved_fraction=0.1) == (cur, 0)  # too many moves at once


def test_device_stack_frames_and_memory_registry():
    """Stack-ordered transients: 4 KiB-aligned views of one buffer, a frame releases what it took, the same request gets the same
    address again, an over-full stack names its live blocks, an empty one grows; the registry sums long-lived tensors by
    category and memory kind without counting shared storage twice."""
    import torch

    from surogate_b200.runtime.memory import DeviceStack, registry_for
    from surogate_b200.runtime.trainer import Trainer, TrainerConfig

    st = DeviceStack("cpu", 64 * 1024)
    with st.frame():
        a = st.alloc((100,), torch.float32, "a")
        b = st.alloc((3, 5), torch.bfloat16, "b")
        assert a.data_ptr() % 4096 == 0 and b.data_ptr() - a.data_ptr() == 4096 and b.shape == (3, 5)
        a.fill_(1.0), b.fill_(2.0)
        assert float(a.sum()) == 100.0 and st.used == 8192
        first = a.data_ptr()
        with pytest.raises(RuntimeError, match=r"live: \[\('a', 4096\)"):
            st.alloc((1 << 20,), torch.float32, "too big")
    assert st.used == 0 and st.high_water == 8192
    with st.frame():
        assert st.alloc((100,), torch.float32, "a").data_ptr() == first
    big = st.alloc((1 << 20,), torch.uint8, "grown")   # empty stack: replaced by a larger one
    assert st.capacity >= 1 << 20 and big.numel() == 1 << 20
    assert st.stats()["peak_by_name"]["grown"] == 1 << 20

    model = dict(architecture="Qwen3ForCausalLM", vocab_size=128, d_model=32, n_layers=2, num_query_heads=2, num_kv_heads=1, head_size=16, d_ff=64)
    tr = Trainer(TrainerConfig(model=model, batch_size=2, seq_len=16, zero_level=0, optimizer="adamw"), device=torch.device("cpu"))
    tr.init_weights(0)
    tok = torch.randint(0, 128, (2, 17)).numpy()
    tr.step(tok[:, :-1], tok[:, 1:])
    reg = registry_for(tr)
    cats = reg.by_category()
    n = sum(b.master.numel() for b in tr.store.buckets.values())
    assert cats["weights_master"] == 4 * n and cats["optimizer_state"] == 8 * n
    mb = tr.memory_breakdown()
    assert mb["category.weights_master"] == 4 * n and mb["kind.host"] >= 12 * n


def test_placement_backoff_pauses_layers_whose_moves_do_not_help():
    from surogate_b200.parallel.ep import PlacementBackoff

    b = PlacementBackoff()
    assert not b.sits_out(0, 1.9)            # never moved: free to decide
    b.moved(0, 1.9)
    assert b.sits_out(0, 1.85)               # the move did not lower the imbalance by a tenth: pause 1 refresh (this one)
    assert not b.sits_out(0, 1.9)            # pause over: may decide again
    b.moved(0, 1.9)
    assert [b.sits_out(0, 1.88) for _ in range(3)] == [True, True, False]          # failed again: 2 refreshes
    b.moved(0, 1.9)
    assert [b.sits_out(0, 1.9) for _ in range(5)] == [True] * 4 + [False]          # 4
    b.moved(0, 1.9)
    assert sum(b.sits_out(0, 1.9) for _ in range(12)) == 8                         # capped at 8
    b.moved(0, 1.9)
    assert not b.sits_out(0, 1.2)            # this one helped: no pause, and the next failure starts at 1 again
    b.moved(0, 1.5)
    assert [b.sits_out(0, 1.5) for _ in range(2)] == [True, False]
    assert not b.sits_out(7, 3.0)            # layers are independent
