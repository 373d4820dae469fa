"""Lockstep execution of one engine per rank inside a tensor-parallel replica.

Rank 0 (the leader) owns the HTTP side and the only source of nondeterminism: which requests
arrive and which are cancelled between two scheduler iterations. Before every iteration it
broadcasts exactly that (new requests with their ids, prompts, sampling and seeds; ids of
requests to cancel; a stop flag) over a CPU (gloo) group; every rank then runs the same
``Engine.step()``. All scheduling decisions are functions of the engine state and of these
messages, page and slot allocation is deterministic, and sampled tokens come from all-reduced
picks or identically seeded generators, so the ranks stay in step without further traffic
(the reference runs its two ranks as threads of one process that share the host-side scheduler
state, ``engine/fast/tp.py:816-883``; processes need the explicit message).
"""

from __future__ import annotations

import dataclasses
import time

from ..sched.request import Generation, Sampling


class Coordinator:
    def __init__(self, group, rank: int, leader: int = 0) -> None:
        import torch.distributed as dist

        self.dist = dist
        self.group = group
        self.rank = rank
        self.leader = leader
        self.is_leader = rank == leader
        self.live: dict[int, Generation] = {}
        self._cancel_sent: set[int] = set()
        self.stopped = False

    # ------------------------------------------------------------------ leader side
    def _collect(self, engine) -> dict:
        new = []
        while True:
            try:
                g = engine._inbox.get_nowait()
            except Exception:  # queue.Empty
                break
            if g.sampling.seed is None and not g.sampling.greedy:
                g.sampling.seed = (g.id * 7919 + int(time.time() * 1e3)) % (2**31)
            self.live[g.id] = g
            new.append((g.id, g.prompt, dataclasses.asdict(g.sampling)))
            engine.waiting.append(g)
        cancel = [i for i, g in self.live.items() if g.cancelled.is_set() and i not in self._cancel_sent and not g.done]
        self._cancel_sent.update(cancel)
        return {"new": new, "cancel": cancel, "stop": self.stopped}

    # ------------------------------------------------------------------ both sides
    def sync(self, engine) -> bool:
        """Exchange this iteration's events; returns False when the replica is shutting down."""
        # Did any rank see a device-side failure (a peer wait that ran out, an index check) or an escaped exception in
        # the last iteration? Such a rank skipped stores the others made: the group is out of step for good. All ranks
        # learn of it here, before the next launch, and every one of them tears its engine down (fails what is in
        # flight, refuses new work, reports it on /health).
        import torch

        flag = torch.tensor([1 if engine.device_error_pending else 0], dtype=torch.int32)
        self.dist.all_reduce(flag, op=self.dist.ReduceOp.MAX, group=self.group)
        if int(flag.item()):
            engine.device_error_pending = False
            engine.tear_down("a device-side failure or an escaped exception on one rank of the group")
        msg = [self._collect(engine) if self.is_leader else None]
        self.dist.broadcast_object_list(msg, src=self.leader, group=self.group)
        m = msg[0]
        if not self.is_leader:
            for gid, prompt, sampling in m["new"]:
                g = Generation(prompt, Sampling(**sampling))
                g.id = gid
                self.live[gid] = g
                engine.waiting.append(g)
        for gid in m["cancel"]:
            g = self.live.get(gid)
            if g is not None:
                g.cancel_now = True
        for gid in [i for i, g in self.live.items() if g.done]:
            self.live.pop(gid, None)
            self._cancel_sent.discard(gid)
        return not m["stop"]

    def follow(self, engine) -> None:
        """Follower main loop: mirror the leader until it stops."""
        while self.sync(engine):
            engine.step(synced=True)

    def stop(self, engine) -> None:
        """Leader: tell the followers to leave their loop."""
        self.stopped = True
        self.sync(engine)
