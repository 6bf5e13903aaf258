"""Worker for multi-process tests: trains a tiny model for a few steps and prints one JSON line from rank 0.

Launched with ``python -m torch.distributed.run --nproc-per-node N tests/mp_worker.py <json-args>`` (or directly for N=1).
Every rank sees the same global batch and takes its slice, so runs at different world sizes are comparable.
"""
import json
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from surogate_b200.parallel.dist import TorchComm, init_distributed  # noqa: E402
from surogate_b200.runtime.trainer import Trainer, TrainerConfig  # noqa: E402


def main():
    a = json.loads(sys.argv[1]) if len(sys.argv) > 1 else {}
    use_gpu = a.get("device", "cuda") == "cuda" and torch.cuda.is_available()
    info = init_distributed(backend="nccl" if use_gpu else "gloo", timeout_s=a.get("timeout_s", 120))
    dev = torch.device("cuda", info.local_rank) if use_gpu else torch.device("cpu")
    if use_gpu:
        torch.cuda.set_device(dev)
    comm = TorchComm() if info.world > 1 else None
    gb, T = a.get("global_batch", 4), a.get("seq_len", 128)
    model = a.get("model") or dict(architecture="Qwen3ForCausalLM", vocab_size=1024, d_model=256, n_layers=2, num_query_heads=2,
                                   num_kv_heads=1, head_size=128, d_ff=512, tie_word_embeddings=True)
    cfg = TrainerConfig(model=model, batch_size=gb // info.world // a.get("grad_accum", 1), seq_len=T, grad_accum=a.get("grad_accum", 1),
                        recipe=a.get("recipe", "bf16"), optimizer=a.get("optimizer", "adamw"), learning_rate=1e-3, zero_level=a.get("zero", 1),
                        collectives=a.get("collectives", "auto"), keep_gathered=a.get("keep_gathered", True), ep_size=a.get("ep", 1),
                        lora=a.get("lora"), offload_master=a.get("offload_master", False), offload_optimizer=a.get("offload_optimizer", False),
                        cpu_training=a.get("cpu_training", False), ep_capacity_factor=a.get("ep_capacity_factor", 1.5),
                        ep_spill_threshold=a.get("ep_spill", 0.0), ep_spill_min_rows=a.get("ep_spill_min_rows", 64),
                        qlora=a.get("qlora"), qlora_experts=a.get("qlora_experts", True), qlora_offload_experts=a.get("qlora_offload_experts", False),
                        use_cuda_graphs=a.get("graphs", False), ep_plan_refresh_interval=a.get("ep_refresh", 16), ep_load_balance_threshold=a.get("ep_threshold", 1.3))
    pp = a.get("pp", False)
    if pp:  # pipeline stages: every rank gets the whole global batch and cuts it into world * grad_accum micro-batches
        from surogate_b200.parallel.dispatch_pp import PipelineTrainer

        cfg.zero_level = 0
        tr = PipelineTrainer(cfg, device=dev, stage_layers=a.get("stage_layers", 0))
    else:
        tr = Trainer(cfg, device=dev, comm=comm)
    tr.init_weights(seed=0)
    rng = np.random.default_rng(7)
    V = model["vocab_size"]
    losses, norms = [], []
    per_rank = gb // info.world
    for step in range(a.get("steps", 4)):
        tok = rng.integers(0, V, (gb, T + 1)).astype(np.int32)
        x, y = tok[:, :-1], tok[:, 1:]
        sl = slice(info.rank * per_rank, (info.rank + 1) * per_rank)
        out = tr.step(x, y) if pp else tr.step(x[sl], y[sl])
        losses.append(out["loss"])
        norms.append(out["norm"])
    extra = {}
    if getattr(tr.store, "expert_offload", None) is not None:
        extra["expert_offload"] = tr.store.expert_offload.stats()
        extra["expert_master_elems"] = sum(b.master.numel() for b in tr.store.buckets.values() if b.expert)
        extra["exported_expert_shape"] = list(tr.store.full_tensor("blocks.0.experts_down").shape)
    if pp:
        if a.get("export_dir"):
            tr.export_model(a["export_dir"])
        if info.rank == 0:
            print("RESULT " + json.dumps({"losses": losses, "norms": norms, "world": info.world, "stages": [[s.first_layer, s.last_layer, s.gpu] for s in tr.stages],
                                          "held_params": len(tr.inner.store.where)}), flush=True)
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
        return
    if a.get("checkpoint_dir"):
        fail_rank = a.get("checkpoint_fail_rank")
        if fail_rank is not None and info.rank == fail_rank:  # this rank's shard cannot be written (a full disk, a lost mount)
            import surogate_b200.io.checkpoint as ck

            def refuse(*_a, **_k):
                raise OSError(28, "No space left on device")

            ck.save_file = refuse
        try:
            tr.save_checkpoint(a["checkpoint_dir"], step=len(losses))
            extra["checkpoint"] = "written"
        except OSError as e:
            extra["checkpoint"] = type(e).__name__
        if fail_rank is not None:  # every rank is still on the same collective sequence: one more step must work and agree
            tok = rng.integers(0, V, (gb, T + 1)).astype(np.int32)
            sl = slice(info.rank * per_rank, (info.rank + 1) * per_rank)
            extra["loss_after"] = tr.step(tok[:, :-1][sl], tok[:, 1:][sl])["loss"]
            flags = [None] * info.world
            import torch.distributed as dist

            dist.all_gather_object(flags, extra["checkpoint"])
            extra["checkpoint_all_ranks"] = flags
    if info.rank == 0:
        print("RESULT " + json.dumps({"losses": losses, "norms": norms, "world": info.world, "comm": type(tr.comm).__name__,
                                      "fused_norm": bool(tr.store.fused_sumsq is not None and tr.store.sumsq_valid),
                                      "fp8_gather": bool(tr.store.fp8_gather), "fp8_shards": bool(getattr(tr.store, "fp8_arena", None) is not None), "graph_replays": getattr(tr, "graph_replays", 0), "h2d_weight_bytes": int(tr.store.h2d_bytes),
                                      "stage_slots": len(tr.store.stage_slots),
                                      "ep_dropped": tr.ep.dropped_rows() if tr.ep is not None else 0, "fp8_dispatches": int(getattr(tr.ep, "fp8_dispatches", 0)) if tr.ep is not None else 0,
                                      "ep_moves": tr.ep.moves_done if tr.ep is not None else 0, "ep_spilled_layers": int(getattr(tr.ep, "spilled_layers", 0)) if tr.ep is not None else 0,
                                      "ep_imbalance": tr.ep.imbalance() if tr.ep is not None else 1.0, **extra}), flush=True)
    if info.world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
