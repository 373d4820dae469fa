"""One tensor-parallel replica: a leader process (HTTP + scheduler) and follower rank processes.

``python -m b200serve.api.server --gpus-per-replica N`` makes the calling process rank 0 and
starts ranks 1..N-1 with ``python -m b200serve.parallel.replica``; every rank loads its shard of
the checkpoint onto its own GPU (``LOCAL_RANK``), joins one ``torch.distributed`` group (NCCL for
tensors, an extra gloo group for the lockstep messages) and runs the same engine
(``parallel.lockstep``). On a machine without GPUs the ranks are CPU processes over gloo, which
is how the plumbing is tested.
"""

from __future__ import annotations

import argparse
import os
import signal
import socket
import subprocess
import sys
from datetime import timedelta

import torch


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def init_rank(rank: int, world: int, port: int, cuda: bool):
    import torch.distributed as dist

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ["MASTER_PORT"] = str(port)
    if cuda:
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=timedelta(minutes=30))
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(days=7))
    cpu_group = dist.new_group(backend="gloo", timeout=timedelta(days=7))
    return dev, cpu_group


def build_engine(model_dir: str, rank: int, world: int, dev: torch.device, cpu_group, engine_cfg, split: str = "tensor"):
    """One rank's engine of a replica over ``world`` devices. ``split``: "tensor" shards every layer (heads, experts,
    vocabulary) across the ranks; "layers" gives each rank a run of whole layers (parallel/pp.py)."""
    import torch.distributed as dist

    from ..models.checkpoint import load_checkpoint
    from ..sched.engine import Engine
    from .lockstep import Coordinator
    from .tp import DistComm, FusedComm, TPContext

    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    if split == "layers":
        from .pp import PPContext

        weights = load_checkpoint(model_dir, device=dev, dtype=dtype, layers=(rank, world))
        engine = Engine(weights, engine_cfg, pp=PPContext(rank, world))
        engine.coordinator = Coordinator(cpu_group, rank)
        return engine
    weights = load_checkpoint(model_dir, device=dev, dtype=dtype, shard=(rank, world))
    if dev.type == "cuda" and engine_cfg.fused_collectives:
        comm = FusedComm(dev, dist.group.WORLD)
    else:
        comm = DistComm(dist.group.WORLD)
    engine = Engine(weights, engine_cfg, tp=TPContext(rank, world, comm))
    engine.coordinator = Coordinator(cpu_group, rank)
    return engine


def start_followers(model_dir: str, world: int, port: int, cuda: bool, cfg_args: list[str],
                    split: str = "tensor") -> list[subprocess.Popen]:
    procs = []
    for r in range(1, world):
        cmd = [sys.executable, "-m", "b200serve.parallel.replica", "--model", model_dir, "--rank", str(r), "--world",
               str(world), "--port", str(port), "--device", "cuda" if cuda else "cpu", "--split", split, *cfg_args]
        env = dict(os.environ)
        import b200serve

        root = os.path.dirname(os.path.dirname(os.path.abspath(b200serve.__file__)))
        env["PYTHONPATH"] = root + (os.pathsep + env["PYTHONPATH"] if env.get("PYTHONPATH") else "")
        procs.append(subprocess.Popen(cmd, env=env))
    return procs


def follower_main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--rank", type=int, required=True)
    ap.add_argument("--world", type=int, required=True)
    ap.add_argument("--port", type=int, required=True)
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--split", default="tensor", choices=["tensor", "layers"])
    ap.add_argument("--max-model-len", type=int, default=262144)
    ap.add_argument("--prefill-chunk-tokens", type=int, default=2048)
    ap.add_argument("--prefix-cache-tokens", type=int, default=4194304)
    ap.add_argument("--prefix-cache-entries", type=int, default=128)
    ap.add_argument("--prefix-cache-gib", type=float, default=16.0)
    ap.add_argument("--max-seqs", type=int, default=128)
    args = ap.parse_args(argv)
    try:  # leave with the leader
        import ctypes

        ctypes.CDLL("libc.so.6", use_errno=True).prctl(1, signal.SIGTERM)
    except OSError:
        pass
    from ..config import EngineConfig

    dev, cpu_group = init_rank(args.rank, args.world, args.port, args.device == "cuda")
    cfg = EngineConfig.from_env(
        model=args.model, max_model_len=args.max_model_len, prefill_chunk_tokens=args.prefill_chunk_tokens,
        prefix_cache_tokens=args.prefix_cache_tokens, prefix_cache_entries=args.prefix_cache_entries,
        prefix_cache_gib=args.prefix_cache_gib, max_seqs=args.max_seqs,
    )
    engine = build_engine(args.model, args.rank, args.world, dev, cpu_group, cfg, split=args.split)
    print(f"engine: rank {args.rank}/{args.world} ready on {dev}", flush=True)
    engine.coordinator.follow(engine)


def leader_engine(model_dir: str, world: int, cuda: bool, engine_cfg, cfg_args: list[str], split: str = "tensor"):
    """Start the followers, build rank 0's engine; returns ``(engine, follower processes)``."""
    port = _free_port()
    followers = start_followers(model_dir, world, port, cuda, cfg_args, split)
    try:
        dev, cpu_group = init_rank(0, world, port, cuda)
        engine = build_engine(model_dir, 0, world, dev, cpu_group, engine_cfg, split=split)
    except BaseException:
        for p in followers:
            p.terminate()
        raise
    return engine, followers


if __name__ == "__main__":
    follower_main()
