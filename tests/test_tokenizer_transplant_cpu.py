"""Tokenizer transplant (``utils/tokenizer_transplant.py``): the sparse fit recovers new rows through the shared tokens, model
directories are rewritten consistently, the manifest drives the way back, the external engine's command line is as documented."""
import json
import os

import pytest
import torch
from safetensors import safe_open
from safetensors.torch import save_file

from surogate_b200.utils import tokenizer_transplant as tt


def _bytes_vocab():
    """GPT-2 style byte alphabet: every byte has a printable stand-in character, in id order 0..255."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    order = sorted(zip(bs, cs))
    return [chr(c) for _, c in order]


def _model_dir(path, tokens, merges, embed, head=None, extra_cfg=None, added=()):
    os.makedirs(path, exist_ok=True)
    vocab = {t: i for i, t in enumerate(tokens)}
    tj = {"version": "1.0", "added_tokens": [{"id": len(tokens) + i, "content": a, "special": True} for i, a in enumerate(added)],
          "pre_tokenizer": {"type": "ByteLevel", "add_prefix_space": False, "use_regex": True}, "decoder": {"type": "ByteLevel"},
          "model": {"type": "BPE", "vocab": vocab, "merges": merges}}
    json.dump(tj, open(os.path.join(path, "tokenizer.json"), "w"))
    json.dump({"chat_template": f"template of {os.path.basename(path)}"}, open(os.path.join(path, "tokenizer_config.json"), "w"))
    cfg = dict(architectures=["Qwen3ForCausalLM"], vocab_size=embed.shape[0], hidden_size=embed.shape[1], eos_token_id=1, **(extra_cfg or {}))
    json.dump(cfg, open(os.path.join(path, "config.json"), "w"))
    tensors = {"model.embed_tokens.weight": embed.contiguous(), "model.layers.0.mlp.up_proj.weight": torch.full((4, embed.shape[1]), 0.5)}
    if head is not None:
        tensors["lm_head.weight"] = head.contiguous()
    save_file(tensors, os.path.join(path, "model.safetensors"), metadata={"format": "pt"})
    return path


def test_omp_recovers_a_sparse_combination_through_the_shared_tokens():
    torch.manual_seed(0)
    S, d_ref, d_out = 200, 128, 96
    atoms_out = torch.randn(S, d_out)
    Q = torch.linalg.qr(torch.randn(d_ref, d_ref)).Q[:d_out]   # the reference space is a rotated, zero-padded copy of the output space
    atoms_ref = atoms_out @ Q
    coef = torch.zeros(5, S)
    for r in range(5):
        coef[r, torch.randperm(S)[:3]] = torch.tensor([1.0, -0.9, 0.8])
    fit = tt.omp_rows(coef @ atoms_ref, atoms_ref, atoms_out, k=3, candidates=S)
    assert torch.allclose(fit, coef @ atoms_out, atol=1e-3)
    # pruning the candidates to the most correlated atoms still finds them; more atoms than needed do not hurt
    fit2 = tt.omp_rows(coef @ atoms_ref, atoms_ref, atoms_out, k=8, candidates=64)
    assert torch.allclose(fit2, coef @ atoms_out, atol=5e-3)
    assert tt.omp_rows(torch.zeros(0, d_ref), atoms_ref, atoms_out).shape == (0, d_out)


def test_transplant_rewrites_the_model_directory_and_restores(tmp_path):
    torch.manual_seed(1)
    alphabet = _bytes_vocab()
    d_s, d_t = 16, 24
    # student: bytes + "ab"; teacher: bytes + "ab" + "abc" + "zz" and one special token; ids differ between the two
    s_tokens = alphabet + ["ab"]
    t_tokens = ["ab", "abc"] + alphabet + ["zz"]
    E_s = torch.randn(len(s_tokens), d_s)
    Q = torch.linalg.qr(torch.randn(d_t, d_t)).Q[:d_s]
    E_t = torch.zeros(len(t_tokens) + 1 + 3, d_t)  # + special token + 3 padding rows, as configs pad their vocabularies
    s_id = {t: i for i, t in enumerate(s_tokens)}
    for i, tok in enumerate(t_tokens):
        if tok in s_id:
            E_t[i] = E_s[s_id[tok]] @ Q
    E_t[1] = 0.6 * E_t[0] + 0.4 * E_t[t_tokens.index("c")]           # "abc" = 0.6 "ab" + 0.4 "c" in the teacher's space
    E_t[t_tokens.index("zz")] = 2.0 * E_t[t_tokens.index("z")]
    student = _model_dir(str(tmp_path / "student"), s_tokens, ["a b"], E_s.to(torch.bfloat16), head=(E_s * 2).to(torch.bfloat16))
    teacher = _model_dir(str(tmp_path / "teacher"), t_tokens, ["a b", "ab c", "z z"], E_t, head=E_t * 3, extra_cfg=dict(bos_token_id=7, pad_token_id=9), added=["<|special|>"])
    out = str(tmp_path / "out")
    res = tt.run_transplant(student, teacher, out, method="omp", k=2, engine="builtin")
    assert res["engine"] == "builtin" and res["shared"] == 257 and res["new"] == 3 + 3 and res["rows"] == len(t_tokens) + 4
    cfg = json.load(open(os.path.join(out, "config.json")))
    assert cfg["vocab_size"] == len(t_tokens) + 4 and cfg["bos_token_id"] == 7 and cfg["pad_token_id"] == 9 and cfg["hidden_size"] == d_s
    assert json.load(open(os.path.join(out, "tokenizer_config.json")))["chat_template"] == "template of teacher"
    assert tt.load_vocab(out) == tt.load_vocab(teacher)
    with safe_open(os.path.join(out, "model.safetensors"), framework="pt") as f:
        E, H, other = f.get_tensor("model.embed_tokens.weight"), f.get_tensor("lm_head.weight"), f.get_tensor("model.layers.0.mlp.up_proj.weight")
    assert E.shape == (len(t_tokens) + 4, d_s) and E.dtype == torch.bfloat16 and torch.equal(other, torch.full((4, d_s), 0.5))
    Eb = E_s.to(torch.bfloat16)
    for tok in ("ab", "c", "z", "!"):   # shared tokens keep their rows exactly, at the teacher's ids
        assert torch.equal(E[t_tokens.index(tok)], Eb[s_id[tok]]) and torch.equal(H[t_tokens.index(tok)], (E_s * 2).to(torch.bfloat16)[s_id[tok]])
    want = 0.6 * Eb[s_id["ab"]].float() + 0.4 * Eb[s_id["c"]].float()
    assert torch.allclose(E[1].float(), want, atol=3e-2) and torch.allclose(H[1].float(), 2 * want, atol=6e-2)
    assert torch.allclose(E[t_tokens.index("zz")].float(), 2 * Eb[s_id["z"]].float(), atol=3e-2)
    man = json.load(open(res["manifest"]))
    assert man["method"] == "omp" and man["k"] == 2 and man["student_dir"] == os.path.abspath(student) and man["engine"] == "builtin"

    # the way back: the distilled model (teacher vocabulary) returns to the student's tokenizer; shared rows survive the round trip
    back = str(tmp_path / "back")
    tt.run_transplant_back(out, res["manifest"], back, engine="builtin")
    with safe_open(os.path.join(back, "model.safetensors"), framework="pt") as f:
        Eb2 = f.get_tensor("model.embed_tokens.weight")
    assert Eb2.shape == Eb.shape and torch.equal(Eb2, Eb) and tt.load_vocab(back) == tt.load_vocab(student)
    assert json.load(open(os.path.join(back, "tokenizer_config.json")))["chat_template"] == "template of student"


def test_simple_methods_and_validation(tmp_path):
    torch.manual_seed(2)
    alphabet = _bytes_vocab()
    E_s = torch.randn(len(alphabet) + 1, 8)
    student = _model_dir(str(tmp_path / "s"), alphabet + ["ab"], ["a b"], E_s)          # tied: no lm_head
    teacher = _model_dir(str(tmp_path / "t"), alphabet + ["bc"], ["b c"], torch.randn(len(alphabet) + 1, 12))
    new = len(alphabet)
    out = {}
    for m in ("mean", "zero", "subword"):
        tt.run_transplant(student, teacher, str(tmp_path / m), method=m, engine="builtin")
        with safe_open(os.path.join(str(tmp_path / m), "model.safetensors"), framework="pt") as f:
            assert "lm_head.weight" not in f.keys()
            out[m] = f.get_tensor("model.embed_tokens.weight")
        assert torch.equal(out[m][:new], E_s[:new])
    assert torch.allclose(out["mean"][new], E_s.mean(0), atol=1e-6) and torch.count_nonzero(out["zero"][new]) == 0
    # "bc" is cut by the student's tokenizer into "b", "c": the new row is the mean of those two
    assert torch.allclose(out["subword"][new], (E_s[alphabet.index("b")] + E_s[alphabet.index("c")]) / 2, atol=1e-6)
    with pytest.raises(ValueError, match="unknown method"):
        tt.run_transplant(student, teacher, str(tmp_path / "x"), method="john_hewitt", engine="builtin")
    with pytest.raises(ValueError, match="k must be"):
        tt.run_transplant(student, teacher, str(tmp_path / "x"), k=0, engine="builtin")
    os.remove(os.path.join(str(tmp_path / "mean"), "tokenizer.json"))
    with pytest.raises(RuntimeError, match="lacks tokenizer.json"):
        tt.validate_output_model(str(tmp_path / "mean"))


def test_external_engine_command_and_cli(tmp_path, monkeypatch, capsys):
    cmd = tt.mergekit_command("S", "T", "O", "omp", 32, device="cuda", trust_remote_code=True, extra=["--x"])
    assert cmd == ["mergekit-tokensurgeon", "S", "T", "O", "--approximation-method", "omp", "--k", "32", "--device", "cuda", "--trust-remote-code", "--x"]
    with pytest.raises(ValueError):
        tt.mergekit_command("S", "T", "O", "nope")
    monkeypatch.setattr(tt, "find_tokensurgeon", lambda: None)
    with pytest.raises(RuntimeError, match="not found on PATH"):
        tt._run("S", "T", "O", "omp", 64, None, False, None, "mergekit")
    # with the tool present, methods the built-in engine lacks go to it; its failure surfaces with the tail of its output
    monkeypatch.setattr(tt, "find_tokensurgeon", lambda: ["mergekit-tokensurgeon"])
    calls = []

    class R:
        returncode, stdout, stderr = 1, "", "a\nboom"

    with pytest.raises(RuntimeError, match="boom"):
        tt._run("S", "T", "O", "mp_rope", 64, None, False, None, "auto", runner=lambda c, **k: calls.append(c) or R())
    assert calls[0][:4] == ["mergekit-tokensurgeon", "S", "T", "O"]

    from surogate_b200.cli import transplant as cli

    alphabet = _bytes_vocab()
    student = _model_dir(str(tmp_path / "s"), alphabet, [], torch.randn(256, 8))
    teacher = _model_dir(str(tmp_path / "t"), alphabet + ["ab"], ["a b"], torch.randn(257, 8))
    assert cli.main(["--student", student, "--teacher", teacher, "--output", str(tmp_path / "o"), "--engine", "builtin", "--k", "4"]) == 0
    res = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert res["new"] == 1 and os.path.exists(res["manifest"])
    assert cli.main(["--restore", res["manifest"], "--student", str(tmp_path / "o"), "--output", str(tmp_path / "b"), "--engine", "builtin"]) == 0
    assert cli.main(["--student", student, "--teacher", teacher, "--output", str(tmp_path / "o2"), "--engine", "builtin", "--method", "randn"]) == 3
    with pytest.raises(SystemExit):
        cli.main(["--output", str(tmp_path / "o3")])
