"""Serving with data-parallel attention and expert-parallel MoE: N replicas, one process and one GPU each.

Every replica is a full server (its own HTTP port behind the data-parallel front, its own requests, scheduler,
KV pool and prefix cache) with all dense weights, but only ``E / N`` of the routed experts; inside every MoE block
the rows of all replicas meet their experts through the dispatch / combine kernels of ``parallel/ep.py``. Those
kernels rendezvous on the device, so the replicas must issue the same sequence of passes. ``TickCoordinator``
arranges that: before a prefill pass and before a decode pass every replica says whether it has rows for it (one
small all-reduce over a CPU group); the pass runs everywhere as soon as one replica wants it, and a replica without
rows joins with an empty pass (``Model.forward_empty``), in which it still serves as a host of experts. The same
message carries "a device-side failure was seen" and "shutting down", so that all replicas tear down or leave
together instead of waiting for a peer that is gone.

The reference has neither expert parallelism nor shared passes between its replicas (``engine/router.py:1-27``:
independent replicas behind a front); this is the serving form of data-parallel attention over expert-parallel MoE
blocks (``parallel/ep.py``).
``GlooEpMoE`` is the CPU stand-in of the NVLink kernels (object all-gathers over gloo, same arithmetic as the
single-process block) with which the scheduling is tested without GPUs.
"""

from __future__ import annotations

import os
from datetime import timedelta

import torch

from ..ops import torch_ops


class TickStop(Exception):
    pass


class TickCoordinator:
    """Per-pass agreement of the replicas' schedulers over a CPU process group."""

    def __init__(self, group) -> None:
        import torch.distributed as dist

        self.dist, self.group = dist, group
        self.stopping = False
        self.stopped = False
        self.ticks = 0
        self.trace = os.environ.get("ENGINE_TICK_TRACE", "0") == "1"  # log every agreement that leads to a pass
        self._last_traced = False

    def any(self, engine, want: bool, what: str = "") -> bool:
        """True when at least one replica has rows for the pass about to run. Also spreads failure and shutdown."""
        if self.stopped:
            return False
        if self.trace and (want or self._last_traced):
            print(f"tick {self.ticks} {what}: want={int(want)} running={len(engine.running)} "
                  f"prefilling={len(engine.prefilling)}", flush=True)
        msg = torch.tensor([1 if want else 0, 1 if engine.device_error_pending else 0, 1 if self.stopping else 0],
                           dtype=torch.int32)
        try:
            self.dist.all_reduce(msg, op=self.dist.ReduceOp.MAX, group=self.group)
        except Exception as e:  # noqa: BLE001 - a peer process is gone (the group timeout ran out)
            self.stopped = True
            engine.tear_down(f"lost the other replicas of the expert-parallel group: {e!r}")
            return False
        self.ticks += 1
        if int(msg[1]):
            engine.device_error_pending = False
            self.stopped = True
            engine.tear_down("a device-side failure or an escaped exception on one replica of the expert-parallel group")
            return False
        if int(msg[2]):
            self.stopped = True
            engine.tear_down("the expert-parallel group is shutting down")
            return False
        if self.trace and (int(msg[0]) or self._last_traced):
            print(f"tick {self.ticks - 1} {what}: agreed={int(msg[0])}", flush=True)
        self._last_traced = bool(int(msg[0]))
        return bool(int(msg[0]))

    def rendezvous(self, engine) -> None:
        """All replicas meet here with idle devices. Used between the graph captures of the warm-up: capturing and
        instantiating a graph takes a replica anything from tens of milliseconds to over a second, and the eager run
        that precedes the next capture contains peer waits that give up after about a second."""
        if self.stopped:
            return
        if engine.device.type == "cuda":
            torch.cuda.synchronize(engine.device)
        try:
            self.dist.barrier(group=self.group)
        except Exception as e:  # noqa: BLE001
            self.stopped = True
            engine.tear_down(f"lost the other replicas of the expert-parallel group: {e!r}")

    def stop(self, engine) -> None:
        """Tell the other replicas that this one leaves (they tear down at their next agreement)."""
        self.stopping = True
        if not self.stopped:
            self.any(engine, False)


class GlooEpMoE:
    """CPU stand-in of ``parallel.ep.EpMoE``: the same routing, per-pair arithmetic and pair-order combine as the
    single-process block (``ops.torch_ops.moe_block``), with the rows exchanged by object all-gathers."""

    def __init__(self, group, n_experts: int, top_k: int) -> None:
        import torch.distributed as dist

        self.dist, self.group = dist, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.E, self.top_k, self.per = n_experts, top_k, n_experts // self.world

    def forward(self, x, router, w_gate_up_local, w_down_local, residual=None, norm_w=None, eps: float = 1e-6):
        E, k, me = self.E, self.top_k, self.rank
        inter = w_down_local.shape[2]
        logits = torch_ops.linear(x, router, out_dtype=torch.float32)
        wts, idx = torch_ops.router_topk(logits[:, :E], k)
        wts = torch.cat([wts, torch.sigmoid(logits[:, E:E + 1])], dim=1).to(x.dtype)
        idx = torch.cat([idx, torch.full_like(idx[:, :1], E)], dim=1)
        rows: list = [None] * self.world
        self.dist.all_gather_object(rows, (x, idx), group=self.group)
        outs = []
        for r, (xr, ir) in enumerate(rows):  # my experts' outputs for every replica's pairs
            T, P = ir.shape
            pair = torch.zeros(T, P, xr.shape[1], dtype=xr.dtype)
            flat = ir.reshape(-1).long()
            for e in torch.unique(flat).tolist():
                if e == E:
                    if r != me:
                        continue  # the shared expert is served where the row lives
                    local = self.per
                elif e // self.per == me:
                    local = e - me * self.per
                else:
                    continue
                sel = (flat == e).nonzero(as_tuple=True)[0]
                gu = torch_ops.linear(xr[sel // P], w_gate_up_local[local])
                act = torch.nn.functional.silu(gu[:, :inter].float()).to(xr.dtype) * gu[:, inter:]
                pair.view(T * P, -1)[sel] = torch_ops.linear(act, w_down_local[local])
            outs.append(pair)
        back: list = [None] * self.world
        self.dist.all_gather_object(back, outs, group=self.group)
        pair_out = back[0][me].clone()
        for h in range(1, self.world):
            pair_out += back[h][me]  # exactly one host wrote each pair, the others hold zeros
        out = (pair_out.float() * wts.float()[:, :, None]).sum(1).to(x.dtype)
        if norm_w is not None:
            return torch_ops.add_rmsnorm(out, residual, norm_w, eps)
        return out

    def close(self) -> None:
        return None


def env_group() -> tuple[int, int, int, int] | None:
    """(rank, world, port, local device index) of this replica's expert-parallel group, from the environment the
    data-parallel front sets for its children; None when the replica stands alone."""
    world = int(os.environ.get("ENGINE_EP_WORLD", "1") or 1)
    if world <= 1:
        return None
    return (int(os.environ["ENGINE_EP_RANK"]), world, int(os.environ["ENGINE_EP_PORT"]),
            int(os.environ.get("ENGINE_EP_LOCAL", os.environ["ENGINE_EP_RANK"])))


def build_engine(model: str, engine_cfg, use_cuda: bool, weights=None):
    """This replica's engine inside its expert-parallel group (see ``env_group``): joins the process group, loads the
    dense weights and its share of the experts, sets up the peer-memory MoE block and the pass agreement."""
    import dataclasses

    import torch.distributed as dist

    from ..models.checkpoint import load_checkpoint
    from ..sched.engine import Engine
    from .ep import EpMoE, shard_experts

    rank, world, port, local = env_group()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ["MASTER_PORT"] = str(port)
    wait = timedelta(seconds=float(os.environ.get("ENGINE_EP_TIMEOUT_S", "120")))
    if use_cuda:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")  # a replica that dies must not fault its peers' GPUs
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=timedelta(minutes=30))
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(minutes=30))
    cpu_group = dist.new_group(backend="gloo", timeout=wait)
    dtype = torch.bfloat16 if use_cuda else torch.float32
    if weights is None:
        weights = load_checkpoint(model, device=dev, dtype=dtype, experts=(rank, world))
    else:
        weights = shard_experts(weights, rank, world)
    mcfg = weights.config
    cfg = dataclasses.replace(engine_cfg, mtp=False)  # drafts would make the replicas' pass sequences differ
    if use_cuda:
        # Each replica launches its passes from its own process, next to its own request threads: between the
        # agreement on a pass and the launch of its kernels the interpreter lock may go to those threads for a while,
        # so the peer waits get seconds, not the one second of ranks driven by one program.
        ep = EpMoE(dev, dist.group.WORLD, mcfg.num_experts, mcfg.hidden_size, mcfg.num_experts_per_tok,
                   max_rows=max(cfg.prefill_pack_tokens, cfg.max_seqs),
                   wait_s=float(os.environ.get("ENGINE_EP_WAIT_S", "20")))
        # the block's work buffers (activations of the received rows, their expert-sorted copy, tile tables) are
        # made now, before the engine sizes its KV pool from the memory that is left; the captured decode graphs and
        # a prefill pass of the packed size still need their share afterwards
        ep.reserve(mcfg.moe_intermediate_size, dtype)
        cfg = dataclasses.replace(cfg, reserve_gb=cfg.reserve_gb + float(os.environ.get("ENGINE_EP_RESERVE_GB", "4")))
    else:
        ep = GlooEpMoE(dist.group.WORLD, mcfg.num_experts, mcfg.num_experts_per_tok)
    engine = Engine(weights, cfg, ep=ep)
    engine.tick = TickCoordinator(cpu_group)
    return engine
