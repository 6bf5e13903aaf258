"""Host-resident state (offload_master / offload_optimizer / cpu_training) follows the same trajectory as the plain path."""
import numpy as np
import pytest
import torch

from surogate_b200.runtime.trainer import Trainer, TrainerConfig

MODEL = dict(architecture="Qwen3ForCausalLM", vocab_size=256, d_model=64, n_layers=2, num_query_heads=4, num_kv_heads=2, head_size=16, d_ff=128,
             tie_word_embeddings=True)


def _run(steps=3, **kw):
    cfg = TrainerConfig(model=MODEL, batch_size=2, seq_len=32, recipe="bf16", learning_rate=1e-2, weight_decay=0.1, zero_level=0, **kw)
    tr = Trainer(cfg, device=torch.device("cpu"))
    tr.init_weights(seed=3)
    rng = np.random.default_rng(0)
    out = []
    for _ in range(steps):
        tok = rng.integers(0, 256, (2, 33)).astype(np.int32)
        out.append(tr.step(tok[:, :-1], tok[:, 1:]))
    return tr, out


@pytest.mark.parametrize("opt", ["adamw", "adamw_8bit"])
def test_streamed_optimizer_matches_plain(opt):
    _, base = _run(optimizer=opt)
    tr, off = _run(optimizer=opt, offload_master=True, offload_optimizer=True)
    for a, b in zip(base, off):
        assert abs(a["loss"] - b["loss"]) < 1e-6 and abs(a["norm"] - b["norm"]) < 1e-6
    assert tr.streamed is not None


def test_cpu_training_matches_adamw():
    _, base = _run(optimizer="adamw")
    tr, cpu = _run(optimizer="adamw", cpu_training=True)
    for a, b in zip(base, cpu):
        assert abs(a["loss"] - b["loss"]) < 2e-5, (a, b)
    assert type(tr.optimizer).__name__ == "CpuAdamW"
    assert all(b.master.dtype == torch.float32 for b in tr.store.buckets.values())


def test_lora_with_host_resident_base():
    lora = dict(rank=4, alpha=8, dropout=0.0, dtype="fp32", targets=["q_proj", "v_proj", "down_proj"], rslora=False, train_router=False)
    _, base = _run(optimizer="adamw", lora=lora)
    _, off = _run(optimizer="adamw", lora=lora, offload_master=True, offload_optimizer=True)
    for a, b in zip(base, off):
        assert abs(a["loss"] - b["loss"]) < 1e-6


def test_resident_layers_keep_frozen_weights_on_the_device_side():
    """With offloaded masters the first N layers' frozen weights can stay resident: same trajectory, and the flag only applies to
    frozen layer buckets."""
    lora = dict(rank=4, alpha=8, dropout=0.0, dtype="fp32", targets=["q_proj", "v_proj", "down_proj"], rslora=False, train_router=False)
    tr_a, a = _run(optimizer="adamw", lora=lora, offload_master=True, offload_optimizer=True)
    tr_b, b = _run(optimizer="adamw", lora=lora, offload_master=True, offload_optimizer=True, resident_layers=1)
    assert a == b
    st = tr_b.store
    assert st._resident(st.buckets["layer0"]) and not st._resident(st.buckets["layer1"]) and not st._resident(st.buckets["embedding"])



def test_stale_optimizer_worker_matches_the_inline_update_and_reports_errors():
    """The native depth-1 worker: two queued updates give exactly the buffers of two direct kernel calls; a bad job raises at
    the next drain and the worker keeps working afterwards."""
    from surogate_b200.ops import host

    h = host()
    n = 50_000

    def buffers():
        g = torch.Generator().manual_seed(0)
        return [torch.randn(n, generator=g), torch.zeros(n), torch.zeros(n), torch.randn(n, generator=g).bfloat16(), torch.zeros(n, dtype=torch.bfloat16),
                torch.ones(n, dtype=torch.uint8)]

    a, b = buffers(), buffers()
    w = h.AsyncAdamW(True)
    for step in (1, 2):
        h.cpu_adamw_step(a[0].data_ptr(), a[1].data_ptr(), a[2].data_ptr(), a[3].data_ptr(), True, a[4].data_ptr(), n, 1e-3, 0.9, 0.999, 1e-8, 0.1, 0.5, step, a[5].data_ptr())
        w.submit([(b[0].data_ptr(), b[1].data_ptr(), b[2].data_ptr(), b[3].data_ptr(), True, b[4].data_ptr(), True, n, b[5].data_ptr())], 1e-3, 0.9, 0.999, 1e-8, 0.1, 0.5, step)
    w.drain()
    assert w.completed() == 2 and all(torch.equal(x, y) for x, y in zip(a, b))
    w.submit([(0, 0, 0, 0, False, 0, False, 4, 0)], 1e-3, 0.9, 0.999, 1e-8, 0.1, 0.5, 1)
    with pytest.raises(Exception, match="null buffer"):
        w.drain()
    w.submit([], 1e-3, 0.9, 0.999, 1e-8, 0.1, 0.5, 1)
    w.drain()
    assert w.completed() == 4


@pytest.mark.parametrize("zero", [0, 3])
def test_one_step_stale_optimizer(tmp_path, zero):
    """``async_optimizer``: the host update of step N runs while step N+1 computes with the weights of update N-1.  On a repeated
    batch the first two losses are therefore equal and the third is the plain optimizer's second; the overlapped run reproduces the
    inline run bit for bit; draining publishes the last update (evaluation and a checkpoint see it) and a resumed run continues."""
    tok = np.random.default_rng(1).integers(0, 256, (2, 33)).astype(np.int32)

    def run(mode, steps=4):
        cfg = TrainerConfig(model=MODEL, batch_size=2, seq_len=32, recipe="bf16", learning_rate=1e-2, weight_decay=0.1, zero_level=zero, optimizer="adamw",
                            cpu_training=True, async_optimizer=mode)
        tr = Trainer(cfg, device=torch.device("cpu"))
        tr.init_weights(seed=3)
        return tr, [tr.step(tok[:, :-1], tok[:, 1:])["loss"] for _ in range(steps)]

    _, plain = run(None)
    tr_i, inline = run("inline")
    tr_o, over = run("overlap")
    assert over == inline
    assert over[0] == over[1] == plain[0] and abs(over[2] - plain[1]) < 1e-6
    v = tr_o.validate(tok[:, :-1], tok[:, 1:])["loss"]
    assert v == tr_i.validate(tok[:, :-1], tok[:, 1:])["loss"] and v < over[-1]
    assert not tr_o.optimizer._pending
    for b in tr_o.store.trainable_buckets():
        assert torch.equal(b.work_host, b.master.to(b.work_host.dtype))
    path = tr_o.save_checkpoint(str(tmp_path), step=4)
    tr_r, _ = run("overlap", steps=0)
    tr_r.load_checkpoint(str(tmp_path))
    a = tr_o.step(tok[:, :-1], tok[:, 1:])["loss"]
    assert tr_r.step(tok[:, :-1], tok[:, 1:])["loss"] == a == v


def test_dropping_a_trainer_with_an_update_in_flight_frees_nothing_the_worker_writes():
    """The worker owns references to every buffer of its job: a trainer dropped right after a step (one update queued on the worker
    thread) is collected without the worker touching freed memory, and the worker object reports when it still holds buffers."""
    import gc

    from surogate_b200.ops import host

    h = host()
    tok = np.random.default_rng(1).integers(0, 256, (2, 33)).astype(np.int32)
    for _ in range(6):
        cfg = TrainerConfig(model=MODEL, batch_size=2, seq_len=32, recipe="bf16", learning_rate=1e-2, zero_level=0, optimizer="adamw", cpu_training=True,
                            async_optimizer="overlap")
        tr = Trainer(cfg, device=torch.device("cpu"))
        tr.init_weights(seed=3)
        tr.step(tok[:, :-1], tok[:, 1:])
        worker = tr.optimizer.worker
        assert worker.holds_buffers
        del tr
        gc.collect()
        junk = [torch.full((100_000,), 7.0) for _ in range(8)]  # recycle the allocator's blocks while the update may still run
        worker.drain()
        assert not worker.holds_buffers and all(bool((j == 7.0).all()) for j in junk)
        del worker
    # stand-alone: the buffers behind a queued job are dropped by the caller at once and live on inside the worker
    n = 400_000
    w = h.AsyncAdamW(True)
    bufs = [torch.randn(n), torch.zeros(n), torch.zeros(n), torch.randn(n), torch.zeros(n), torch.ones(n, dtype=torch.uint8)]
    job = [(bufs[0].data_ptr(), bufs[1].data_ptr(), bufs[2].data_ptr(), bufs[3].data_ptr(), False, bufs[4].data_ptr(), False, n, bufs[5].data_ptr())]
    w.submit(job, 1e-3, 0.9, 0.999, 1e-8, 0.1, 1.0, 1, bufs)
    del bufs, job
    gc.collect()
    del w  # the destructor waits for the update before the references go
    gc.collect()


def test_non_finite_gradient_skips_the_update():
    """An Inf in the gradient makes the norm non-finite: weights, moments and the adapter stay bit-equal and finite, and the next
    clean step trains again (fp32 and 8-bit state, CPU optimizer, LoRA)."""
    tok = np.random.default_rng(1).integers(0, 256, (2, 33)).astype(np.int32)
    lora = dict(rank=4, alpha=8, dropout=0.0, dtype="fp32", targets=["q_proj", "v_proj"], rslora=False, train_router=False)
    for kw in (dict(optimizer="adamw"), dict(optimizer="adamw_8bit"), dict(optimizer="adamw", cpu_training=True), dict(optimizer="adamw", lora=lora)):
        cfg = TrainerConfig(model=MODEL, batch_size=2, seq_len=32, recipe="bf16", learning_rate=1e-2, weight_decay=0.1, zero_level=0, **kw)
        tr = Trainer(cfg, device=torch.device("cpu"))
        tr.init_weights(seed=3)
        tr.step(tok[:, :-1], tok[:, 1:])

        def snapshot():
            out = [b.master.clone() for b in tr.store.buckets.values()]
            out += [t.clone() for st in tr.optimizer.state.values() for t in st.values()]
            if tr.lora is not None:
                out += [tr.lora.master.clone()] + [t.clone() for t in (tr.lora.opt_state or {}).values()]
            return out

        before = snapshot()
        tr.forward_backward(tok[:, :-1], tok[:, 1:])
        if tr.lora is not None:
            tr.lora.grad[3] = float("inf")
        else:
            next(b for b in tr.store.trainable_buckets() if b.grad_shard is not None).grad_shard[5] = float("inf")
        norm = tr.optimizer_step()
        assert not bool(torch.isfinite(norm)), kw
        after = snapshot()
        assert len(before) == len(after) and all(torch.equal(a, b) and bool(torch.isfinite(b.float()).all()) for a, b in zip(before, after)), kw
        out = tr.step(tok[:, :-1], tok[:, 1:])
        assert np.isfinite(out["loss"]) and np.isfinite(out["norm"])
        assert any(not torch.equal(a, b) for a, b in zip(after, snapshot())), kw
