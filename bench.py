#!/usr/bin/env python
"""Headline benchmark: training tokens/s of the flagship configuration on N GPUs of one node.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Default model: Qwen3-8B pre-training, FP8-hybrid recipe (E4M3 forward / E5M2 gradients, per-tensor delayed
scaling, history 16), ZeRO-3 sharding of weights, gradients and 8-bit AdamW state over the N ranks,
sequence 4096, micro-batch 2 per GPU, synthetic uniform token ids, random-init weights N(0, 0.02).
Every step is a full forward + backward + gradient reduction + clipping + optimizer update.

Two timings are taken after the warm-up (every step of either sees a batch it has not seen before):
* ``value``: K steps timed with CUDA events on the device (inputs already resident), max over ranks;
* ``e2e``:  K steps through the public ``Trainer.step`` API including the pinned-host -> device copy of each
  step's tokens/targets and the device -> host read of loss and gradient norm.

``--impl reference`` would run the unmodified reference; it cannot be installed offline in this image, so that
arm prints an ``unavailable`` line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

MODELS = {
    # name: (architecture kwargs, seq_len, micro_batch, recipe, optimizer, zero_level, extra)
    "qwen3-8b": dict(model=dict(architecture="Qwen3ForCausalLM", vocab_size=151936, d_model=4096, n_layers=36, num_query_heads=32,
                                num_kv_heads=8, head_size=128, d_ff=12288, tie_word_embeddings=False),
                     seq_len=4096, batch=2, recipe="fp8_hybrid", optimizer="adamw_8bit", zero=3, label="Qwen3-8B",
                     metric="tokens/sec Qwen3-8B FP8-hybrid pretrain (ZeRO-3, 8-bit AdamW)"),
    "qwen3-0.6b": dict(model=dict(architecture="Qwen3ForCausalLM", vocab_size=151936, d_model=1024, n_layers=28, num_query_heads=16,
                                  num_kv_heads=8, head_size=128, d_ff=3072, tie_word_embeddings=True),
                       seq_len=2048, batch=8, recipe="bf16", optimizer="adamw", zero=1, label="Qwen3-0.6B",
                       metric="tokens/sec Qwen3-0.6B BF16 full fine-tune (DP)"),
    "qwen3-30b-a3b": dict(model=dict(architecture="Qwen3MoeForCausalLM", vocab_size=151936, d_model=2048, n_layers=48, num_query_heads=32,
                                     num_kv_heads=4, head_size=128, moe_d_ff=768, num_experts=128, num_experts_per_tok=8,
                                     aux_loss_coef=1e-3, tie_word_embeddings=False),
                          seq_len=4096, batch=1, recipe="nvfp4", optimizer="adamw_8bit", zero=1, label="Qwen3-30B-A3B",
                          metric="tokens/sec Qwen3-30B-A3B NVFP4 (EP)"),
    "qwen3-14b-lora": dict(model=dict(architecture="Qwen3ForCausalLM", vocab_size=151936, d_model=5120, n_layers=40, num_query_heads=40,
                                      num_kv_heads=8, head_size=128, d_ff=17408, tie_word_embeddings=False),
                           seq_len=8192, batch=1, recipe="bf16", optimizer="adamw_8bit", zero=3, label="Qwen3-14B-LoRA-r16",
                           metric="tokens/sec Qwen3-14B LoRA SFT (BF16 base in pinned host memory, ZeRO-3 gather per layer)",
                           lora=dict(rank=16, alpha=32, dropout=0.0, dtype="fp32", rslora=False, train_router=False,
                                     targets=["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]),
                           offload=True, recompute=True, mask_first_fraction=0.25),
    "tiny": dict(model=dict(architecture="Qwen3ForCausalLM", vocab_size=4096, d_model=512, n_layers=2, num_query_heads=4, num_kv_heads=2,
                            head_size=128, d_ff=1536, tie_word_embeddings=True),
                 seq_len=512, batch=2, recipe="bf16", optimizer="adamw_8bit", zero=1, label="tiny", metric="tokens/sec tiny"),
}

# the reference publishes no B200 number for this metric (its B200 table is all TODO): no vs_baseline denominator
PUBLISHED_BASELINE = None


class ClockSampler:
    """Samples SM clock and throttle reasons of this rank's GPU with nvidia-smi while the timed region runs."""

    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu_index: int):
        self.rows = []
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.gpu)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:  # noqa: BLE001
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()  # our own child, by handle
            try:
                self.proc.wait(timeout=5)
            except Exception:  # noqa: BLE001
                pass
        sm, mx, reasons = [], 0.0, set()
        for r in self.rows:
            f = [x.strip() for x in r.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx = max(mx, float(f[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = sorted(sm)[len(sm) // 4:] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args):
    print(json.dumps({"impl": "reference", "unavailable": "reference cannot be installed offline: pip build of the reference source tree fails "
                      "(scikit-build metadata needs setuptools_scm; CMake FetchContent needs network for CUTLASS 4.6.1, "
                      "flash-attention, cudnn-frontend, nanobind)"}))
    return 0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference", "library"])
    ap.add_argument("--ep-refresh", type=int, default=0, dest="ep_refresh",
                    help="steps between expert re-placement decisions (expert parallel); 0 = experts stay where they are")
    ap.add_argument("--model", default="qwen3-8b", choices=sorted(MODELS))
    ap.add_argument("--recipe", default=None)
    ap.add_argument("--optimizer", default=None)
    ap.add_argument("--zero", type=int, default=None)
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--recompute", action="store_true")
    ap.add_argument("--collectives", default="auto", choices=["auto", "nccl", "symm"])
    ap.add_argument("--ep", type=int, default=None)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-offload", action="store_true", help="keep weights and optimizer state on the device for configs that offload by default")
    ap.add_argument("--attention", default="auto", choices=["auto", "native", "library"], help="native = tcgen05 flash attention of this repo")
    ap.add_argument("--profile", default=None, help="write a per-kernel time table of one extra step (torch.profiler, rank 0) to this path; not a timed run")
    ap.add_argument("--resident-layers", type=int, default=0, help="offload configs: keep the frozen weights of the first N layers in device memory")
    ap.add_argument("--graphs", action="store_true", help="replay forward + backward from CUDA graphs (one GPU, dense models)")
    ap.add_argument("--drop-ignored-rows", action="store_true", help="compact rows without a target away before the LM head")
    ap.add_argument("--layers", type=int, default=None, help="profiling only: truncate the layer stack (the JSON line names the reduced model)")
    ap.add_argument("--no-secondary", action="store_true",
                    help="with the default model on 2 or more GPUs the second half of the headline metric (Qwen3-30B-A3B NVFP4, EP = N) is measured "
                         "after the first and attached to the same JSON line as `secondary`; this flag leaves it out")
    return ap.parse_args()


def measure(args, model_key, info, comm, dev):
    """Build the trainer of one configuration, run warm-up + timed steps (device-timed and end to end) and return the JSON record
    (rank 0; None elsewhere).  Every step of both timed regions gets a batch it has not seen before."""
    import numpy as np
    import torch

    from surogate_b200.runtime.trainer import Trainer, TrainerConfig

    world = info.world
    spec = dict(MODELS[model_key])
    if args.layers:
        spec["model"] = dict(spec["model"], n_layers=args.layers)
        spec["label"] = f"{spec['label']}-truncated-{args.layers}-layers"
        spec["metric"] += f" [TRUNCATED to {args.layers} layers: profiling run, not a benchmark value]"
    primary = model_key == args.model
    seq = (args.seq_len if primary else None) or spec["seq_len"]
    mb = (args.batch if primary else None) or spec["batch"]
    recipe = (args.recipe if primary else None) or spec["recipe"]
    zero = args.zero if (primary and args.zero is not None) else spec["zero"]
    ep = args.ep if (primary and args.ep is not None) else (world if model_key == "qwen3-30b-a3b" else 1)
    cfg = TrainerConfig(model=spec["model"], batch_size=mb, seq_len=seq, grad_accum=1, recipe=recipe, optimizer=(args.optimizer if primary else None) or spec["optimizer"],
                        learning_rate=1e-4, weight_decay=0.1, zero_level=zero, recompute=args.recompute,
                        backend="ref" if args.impl == "library" else "cuda", collectives=args.collectives, ep_size=ep, attention=args.attention,
                        lora=spec.get("lora"), offload_master=bool(spec.get("offload")) and not args.no_offload,
                        offload_optimizer=bool(spec.get("offload")) and not args.no_offload, keep_gathered=not spec.get("offload"),
                        # receive room for 3x the mean load of a rank (all of it when ep <= 3); the busiest rank of a randomly initialised
                        # router stays below 2x, and rows that would not fit are counted and reported in the JSON line (expected: 0)
                        ep_capacity_factor=float(max(1, min(ep, 3))),
                        resident_layers=args.resident_layers, use_cuda_graphs=args.graphs, lmhead_drop_ignored_rows=args.drop_ignored_rows,
                        ep_plan_refresh_interval=args.ep_refresh)   # 0: no expert re-placement.  A decision costs about 250 ms at EP=2, does not
                                                                     # lower the imbalance of randomly initialised routers, and a 4-GPU run stalled in its moves
    if spec.get("recompute"):
        cfg.recompute = True
    trace = os.environ.get("SUROGATE_BENCH_TRACE") == "1"     # progress marks on stderr from every rank (where does a stalled run stop?)

    def mark(what):
        if trace:
            print(f"[trace r{info.rank} {time.strftime('%H:%M:%S')}] {model_key}: {what}", file=sys.stderr, flush=True)

    mark("building the trainer")
    tr = Trainer(cfg, device=dev, comm=comm)
    mark("initialising weights")
    tr.init_weights(seed=0)
    mark("weights ready")
    V = spec["model"]["vocab_size"]
    rng = np.random.default_rng(1234 + info.rank)
    n_dev = args.warmup + args.steps          # device-timed region: one fresh batch per step, resident before the clock starts
    n_host = args.steps + 1                   # end-to-end region: one fresh batch per step, copied from pinned host memory inside the clock

    def draw():
        b = rng.integers(0, V, size=(mb, seq + 1), dtype=np.int64).astype(np.int32)
        x, y = b[:, :-1].copy(), b[:, 1:].copy()   # copies: the target mask below must not touch the inputs
        if spec.get("mask_first_fraction"):        # supervised fine-tuning shape: no loss on the prompt part of each sequence
            y[:, : int(seq * spec["mask_first_fraction"])] = -100
        return x, y

    dev_batches = [tuple(torch.from_numpy(t).to(dev) for t in draw()) for _ in range(n_dev)]
    host_batches = [draw() for _ in range(n_host)]

    def barrier():
        if world > 1:
            comm.barrier()
        torch.cuda.synchronize()

    def device_step(i):
        x, y = dev_batches[i]
        tr.forward_backward(x, y)
        tr.optimizer_step()

    ext = tr.backend.ext if tr.backend.name == "cuda" else None
    for i in range(args.warmup):
        device_step(i)
        if trace:      # a step at a time: synchronise, report, and fail at the first bounded wait that ran out
            torch.cuda.synchronize()
            mark(f"warm-up step {i} done")
            if ext is not None:
                from surogate_b200.ops import check_device_errors

                check_device_errors()
    barrier()
    mark("timed region starts")
    sampler = ClockSampler(info.local_rank)
    sampler.start()
    launches0 = ext.launch_count() if ext is not None else 0
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for i in range(args.steps):
        device_step(args.warmup + i)
    ev1.record()
    barrier()
    mark("timed region done")
    ms = ev0.elapsed_time(ev1)
    if ext is not None:
        from surogate_b200.ops import check_device_errors

        check_device_errors()  # a kernel that timed out on a wait or met an invalid token id invalidates the run
    launches = (ext.launch_count() - launches0) if ext is not None else 0
    clocks = sampler.stop()

    if args.profile and primary:
        from torch.profiler import ProfilerActivity, profile

        barrier()
        with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
            device_step(0)
            torch.cuda.synchronize()
        if info.rank == 0:
            os.makedirs(os.path.dirname(os.path.abspath(args.profile)), exist_ok=True)
            with open(args.profile, "w") as f:
                f.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=45, max_name_column_width=70))
        barrier()

    # end to end through the public API: numpy batches from host memory in, python floats out, every step
    e2e = None
    if not args.no_e2e:
        tr.h2d_bytes = tr.d2h_bytes = 0
        out = tr.step(*host_batches[0])  # one warm step through this path (allocates the pinned buffers)
        tr.h2d_bytes = tr.d2h_bytes = 0
        barrier()
        sampler2 = ClockSampler(info.local_rank)
        sampler2.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for i in range(args.steps):
            out = tr.step(*host_batches[1 + i])
        e1.record()
        barrier()
        wall_ms = (time.perf_counter() - t0) * 1e3
        e2e_ms = max(e0.elapsed_time(e1), wall_ms)
        e2e = (e2e_ms, tr.h2d_bytes // args.steps, tr.d2h_bytes // args.steps, out, sampler2.stop())

    t = torch.tensor([ms, e2e[0] if e2e else 0.0], dtype=torch.float64, device=dev)
    if world > 1:
        comm.all_reduce(t, "max")
    ms, e2e_ms = float(t[0]), float(t[1])
    line = None
    if info.rank == 0:
        tokens_per_step = world * mb * seq
        value = tokens_per_step * args.steps / (ms / 1e3)
        par = f"zero{zero}-dp{world}" if ep <= 1 else f"ep{ep}-zero{zero}"
        line = {
            "metric": spec["metric"], "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms / args.steps, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / PUBLISHED_BASELINE) if PUBLISHED_BASELINE else None, "dtype": "fp8" if recipe.startswith("fp8") else recipe,
            "data": "synthetic uniform token ids (a fresh batch every step), random-init weights N(0,0.02)", "impl": args.impl,
            "config": {"model": spec["label"], "global_batch": world * mb, "seq_len": seq, "parallelism": par, "recipe": recipe,
                       "optimizer": cfg.optimizer, "attention": args.attention, "recompute": bool(cfg.recompute), "micro_batch_per_gpu": mb,
                       "lora_rank": (spec.get("lora") or {}).get("rank"), "offload": bool(cfg.offload_master),
                       "ep_plan_refresh_interval": int(cfg.ep_plan_refresh_interval) if ep > 1 else None,
                       "keep_gathered": bool(cfg.keep_gathered and zero >= 3),   # ZeRO-3: gathered layer weights stay from forward to backward (one gather per step, not two)
                       "cuda_graphs": bool(getattr(tr, "graph_replays", 0)), "drop_ignored_rows": bool(cfg.lmhead_drop_ignored_rows), "resident_layers": int(args.resident_layers),
                       "weight_h2d_bytes_per_step": int(tr.store.h2d_bytes // max(1, args.steps + args.warmup + (0 if args.no_e2e else args.steps + 1))),
                       "l2_policy": "per-step working set (weights+activations, tens of GB) far exceeds the 126 MB L2; no explicit flush",
                       "timing": "CUDA events on the launching stream, barrier+synchronize on both sides, max over ranks"},
            "clocks": clocks, "gpu_launches": int(launches),
            **({"ep_dropped_rows_rank0": tr.ep.dropped_rows(), "ep_rank_imbalance": round(tr.ep.imbalance(), 3), "ep_experts_moved": tr.ep.moves_done}
               if tr.ep is not None else {}),
            "peak_mem_gb": round(torch.cuda.max_memory_allocated(dev) / 2 ** 30, 2),
        }
        if e2e:
            line["e2e"] = {"value": round(tokens_per_step * args.steps / (e2e_ms / 1e3), 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms / args.steps, 3),
                           "h2d_bytes_per_step": int(e2e[1]), "d2h_bytes_per_step": int(e2e[2]), "last_loss": e2e[3]["loss"], "clocks": e2e[4]}
    # give the memory back before another configuration is built in this process
    del tr, dev_batches
    import gc

    gc.collect()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats(dev)
    return line


def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3

    import torch

    from surogate_b200.parallel.dist import TorchComm, init_distributed

    info = init_distributed()
    world = info.world
    if world != args.gpus and info.rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}; using {world}", file=sys.stderr)
    dev = torch.device("cuda", info.local_rank)
    torch.cuda.set_device(dev)
    comm = TorchComm() if world > 1 else None

    sec = None
    if args.model == "qwen3-8b" and world >= 2 and not args.no_secondary and args.impl == "native" and not args.layers:
        # The second half of the headline metric (Qwen3-30B-A3B, EP = N) runs FIRST: at EP = 2 it needs 147 GB per GPU and only fits
        # while nothing else is allocated; the 8B model afterwards needs far less than what is left.  Peer-mapped buffers of the first
        # trainer stay allocated (see parallel/symm_comm.py), everything else returns to the caching allocator when it goes out of scope.
        # A failure here must not lose the headline.
        try:
            sec = measure(args, "qwen3-30b-a3b", info, comm, dev)
        except Exception as e:  # noqa: BLE001
            sec = {"error": f"{type(e).__name__}: {e}"[:400]}
            import gc

            gc.collect()     # the failed trainer's ordinary tensors return to the caching allocator; symmetric arenas are kept alive on purpose
    line = measure(args, args.model, info, comm, dev)
    if sec is not None and info.rank == 0:
        line["secondary"] = sec
    if info.rank == 0:
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
