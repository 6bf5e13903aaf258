"""Multi-node training: one process per GPU on every node, a single global NCCL communicator.

The reference runs one Ray actor per node that owns a thread per GPU, creates an NCCL id on the head and uses a barrier
actor so that all nodes enter communicator creation together.  With one process per GPU the same job is done by the
``torch.distributed`` rendezvous: node ``i`` starts ``gpus_per_node`` ranks whose global rank is
``i * gpus_per_node + local_rank`` and all of them meet at ``master_addr:master_port``.  This module

* plans the per-node launch commands (``plan_launch``) and runs this node's share (``run_multinode``), picking the node
  index from ``SUROGATE_NODE_RANK`` / ``NODE_RANK`` / ``SLURM_NODEID``;
* detects the network interface NCCL should use for inter-node traffic and exports ``NCCL_SOCKET_IFNAME``;
* optionally drives all nodes from one place over SSH (``launch_over_ssh``) or through Ray when it is installed
  (``launch_with_ray``: one remote task per node that runs that node's command).

Data: every node tokenises (or reads) the same shards; the loader's rank/world striding gives each global rank its
share, and only global rank 0 writes checkpoints and exports.

Parity: surogate/train/distributed.py (NodeTrainer :156, RayDistributedTrainer :881, _detect_nccl_interface :118).
"""
from __future__ import annotations

import os
import shlex
import socket
import subprocess
import sys
from dataclasses import dataclass
from typing import Dict, List, Optional


@dataclass
class NodeLaunch:
    node_rank: int
    command: List[str]
    env: Dict[str, str]


def detect_nccl_interface(master_addr: Optional[str] = None) -> Optional[str]:
    """Name of the interface that routes to ``master_addr`` (or the first non-loopback interface that is up)."""
    try:
        import psutil
    except ImportError:
        return None
    addrs, stats = psutil.net_if_addrs(), psutil.net_if_stats()
    local_ip = None
    if master_addr and master_addr not in ("127.0.0.1", "localhost"):
        try:
            s = socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
            s.connect((master_addr, 9))  # no packet is sent for a UDP connect; it only selects the route
            local_ip = s.getsockname()[0]
            s.close()
        except OSError:
            local_ip = None
    candidates = []
    for name, lst in addrs.items():
        st = stats.get(name)
        if st is None or not st.isup or name == "lo" or name.startswith(("docker", "veth", "br-", "virbr")):
            continue
        ips = [a.address for a in lst if a.family == socket.AF_INET]
        if not ips:
            continue
        if local_ip and local_ip in ips:
            return name
        candidates.append((0 if name.startswith(("ib", "bond")) else 1 if name.startswith(("en", "eth")) else 2, name))
    return sorted(candidates)[0][1] if candidates else None


def plan_launch(config_path: str, command: str, num_nodes: int, gpus_per_node: int, master_addr: str, master_port: int,
                extra_args: Optional[List[str]] = None) -> List[NodeLaunch]:
    out = []
    for node in range(num_nodes):
        cmd = [sys.executable, "-m", "torch.distributed.run", f"--nnodes={num_nodes}", f"--node-rank={node}", f"--nproc-per-node={gpus_per_node}",
               "--master-addr", master_addr, "--master-port", str(master_port), "-m", "surogate_b200.cli.main", command, config_path] + list(extra_args or [])
        env = {"SUROGATE_NODE_RANK": str(node), "SUROGATE_MULTINODE_CHILD": "1"}
        out.append(NodeLaunch(node, cmd, env))
    return out


def node_rank_from_env() -> Optional[int]:
    for k in ("SUROGATE_NODE_RANK", "NODE_RANK", "SLURM_NODEID", "GROUP_RANK"):
        if os.environ.get(k) not in (None, ""):
            return int(os.environ[k])
    return None


def run_multinode(cfg, workflow_cls=None, command: str = "sft", config_path: Optional[str] = None):
    """Called by the workflow when ``distributed.num_nodes > 1``.  Inside a rank started by the launcher it simply trains;
    otherwise it starts this node's ranks (the node index must come from the environment)."""
    d = cfg.distributed
    if os.environ.get("SUROGATE_MULTINODE_CHILD") == "1" or "RANK" in os.environ:
        from .sft import train_with_oom_recovery

        return train_with_oom_recovery(cfg)
    node = node_rank_from_env()
    if node is None:
        raise RuntimeError("multi-node run: set SUROGATE_NODE_RANK (0..num_nodes-1) on every node, or start the job with "
                           "`surogate_b200.train.distributed.launch_over_ssh` / `launch_with_ray`")
    gpn = d.gpus_per_node or cfg.gpus
    ifname = os.environ.get("NCCL_SOCKET_IFNAME") or detect_nccl_interface(d.master_addr)
    plan = plan_launch(config_path or os.environ.get("SUROGATE_CONFIG_PATH", ""), command, d.num_nodes, gpn, d.master_addr, d.master_port)[node]
    env = dict(os.environ, **plan.env)
    if ifname:
        env["NCCL_SOCKET_IFNAME"] = ifname
    rc = subprocess.call(plan.command, env=env)
    if rc != 0:
        raise RuntimeError(f"node {node}: training ranks exited with code {rc}")
    return {"steps": None, "final": None, "node": node}


def launch_over_ssh(hosts: List[str], config_path: str, command: str, gpus_per_node: int, master_port: int = 29500, workdir: Optional[str] = None,
                    dry_run: bool = False):
    """Start every node's ranks from here: ``ssh host 'cd workdir && env ... python -m torch.distributed.run ...'``."""
    plan = plan_launch(config_path, command, len(hosts), gpus_per_node, hosts[0], master_port)
    cmds, procs = [], []
    for host, p in zip(hosts, plan):
        envs = " ".join(f"{k}={shlex.quote(v)}" for k, v in p.env.items())
        remote = f"cd {shlex.quote(workdir or os.getcwd())} && env {envs} " + " ".join(shlex.quote(c) for c in p.command)
        cmds.append(["ssh", "-o", "BatchMode=yes", host, remote])
    if dry_run:
        return cmds
    for c in cmds:
        procs.append(subprocess.Popen(c))
    return [p.wait() for p in procs]


def launch_with_ray(config_path: str, command: str, num_nodes: int, gpus_per_node: int, master_port: int = 29500, ray_address: Optional[str] = None,
                    extra_args: Optional[List[str]] = None):
    """One Ray task per node: a placement group with one bundle of ``gpus_per_node`` GPUs per node (strict spread, so no two bundles
    share a node), node 0's address becomes the rendezvous address, every task runs its node's launcher command.  Returns the exit
    codes in node order; the placement group is removed afterwards."""
    try:
        import ray
        from ray.util.placement_group import placement_group, remove_placement_group
        from ray.util.scheduling_strategies import PlacementGroupSchedulingStrategy
    except ImportError as e:
        raise RuntimeError("Ray is not installed: use torchrun on every node (plan_launch) or launch_over_ssh") from e
    ray.init(address=ray_address or "auto", ignore_reinit_error=True)
    pg = placement_group([{"GPU": gpus_per_node, "CPU": 1} for _ in range(num_nodes)], strategy="STRICT_SPREAD" if num_nodes > 1 else "PACK")
    ray.get(pg.ready())

    @ray.remote(num_gpus=gpus_per_node)
    def node_task(cmd, env):
        import subprocess as sp

        return sp.call(cmd, env=dict(os.environ, **env))

    @ray.remote(num_gpus=gpus_per_node)
    def node_ip():
        return ray.util.get_node_ip_address()

    def on(bundle):
        return PlacementGroupSchedulingStrategy(placement_group=pg, placement_group_bundle_index=bundle)

    try:
        head_ip = ray.get(node_ip.options(scheduling_strategy=on(0)).remote())
        plan = plan_launch(config_path, command, num_nodes, gpus_per_node, head_ip, master_port, extra_args)
        return ray.get([node_task.options(scheduling_strategy=on(p.node_rank)).remote(p.command, p.env) for p in plan])
    finally:
        remove_placement_group(pg)
