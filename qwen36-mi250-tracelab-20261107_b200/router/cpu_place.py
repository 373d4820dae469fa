"""CPU placement for replica and rank processes.

Reads the machine's topology from sysfs (allowed CPUs, NUMA nodes, SMT siblings, L3 groups, the
NUMA node of each GPU's PCI function) and hands every replica a disjoint slice of physical cores
near its GPUs, keeping clear of the L3 group of CPU 0 where the kernel's housekeeping lands, with
one dedicated core per rank's engine thread; it also caps the OpenMP / Rayon pools so that
tokenizer threads of neighbouring replicas do not oversubscribe (reference:
``engine/cpu_place.py:93-321``, which reads the GPU nodes from AMD's KFD; here they come from the
PCI devices' ``numa_node``). Everything takes a ``root`` so tests can run on synthetic trees.
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field
from pathlib import Path


def parse_cpu_list(text: str) -> list[int]:
    out: list[int] = []
    for part in text.strip().split(","):
        part = part.strip()
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-")
            out.extend(range(int(a), int(b) + 1))
        else:
            out.append(int(part))
    return sorted(set(out))


def format_cpu_list(cpus: list[int]) -> str:
    cpus = sorted(set(cpus))
    parts, i = [], 0
    while i < len(cpus):
        j = i
        while j + 1 < len(cpus) and cpus[j + 1] == cpus[j] + 1:
            j += 1
        parts.append(str(cpus[i]) if i == j else f"{cpus[i]}-{cpus[j]}")
        i = j + 1
    return ",".join(parts)


def _read(path: Path) -> str | None:
    try:
        return path.read_text()
    except OSError:
        return None


@dataclass
class Topology:
    allowed: list[int]
    node_of: dict[int, int] = field(default_factory=dict)  # cpu -> NUMA node
    core_of: dict[int, int] = field(default_factory=dict)  # cpu -> id of its physical core (lowest sibling)
    l3_of: dict[int, int] = field(default_factory=dict)  # cpu -> id of its L3 group (lowest cpu sharing it)
    gpu_nodes: list[int] = field(default_factory=list)  # NUMA node per GPU index (-1 unknown)

    @classmethod
    def read(cls, root: str | Path = "/", allowed: list[int] | None = None, gpu_bdfs: list[str] | None = None) -> "Topology":
        root = Path(root)
        if allowed is None:
            try:
                allowed = sorted(os.sched_getaffinity(0))
            except (AttributeError, OSError):
                allowed = list(range(os.cpu_count() or 1))
        topo = cls(allowed=list(allowed))
        nodes = root / "sys/devices/system/node"
        if nodes.is_dir():
            for d in sorted(nodes.glob("node[0-9]*")):
                txt = _read(d / "cpulist")
                if txt:
                    for c in parse_cpu_list(txt):
                        topo.node_of[c] = int(d.name[4:])
        for c in allowed:
            base = root / f"sys/devices/system/cpu/cpu{c}"
            sib = _read(base / "topology/thread_siblings_list")
            topo.core_of[c] = min(parse_cpu_list(sib)) if sib else c
            l3 = _read(base / "cache/index3/shared_cpu_list")
            topo.l3_of[c] = min(parse_cpu_list(l3)) if l3 else topo.node_of.get(c, 0) * 100000
            topo.node_of.setdefault(c, 0)
        for bdf in gpu_bdfs or []:
            txt = _read(root / f"sys/bus/pci/devices/{bdf.lower()}/numa_node")
            try:
                topo.gpu_nodes.append(int(txt.strip()) if txt else -1)
            except ValueError:
                topo.gpu_nodes.append(-1)
        return topo

    def physical_cores(self) -> list[int]:
        """One CPU per physical core (its lowest allowed sibling), in id order."""
        seen, out = set(), []
        for c in self.allowed:
            core = self.core_of.get(c, c)
            if core not in seen:
                seen.add(core)
                out.append(c)
        return out


@dataclass
class ReplicaCpus:
    cpus: list[int]  # everything the replica's processes may run on
    rank_cpus: list[int]  # one dedicated CPU per rank engine thread


def replica_slices(topo: Topology, replicas: list[list[int]], min_per_replica: int = 2) -> list[ReplicaCpus]:
    """Disjoint CPU slices, one per replica (``replicas[i]`` = GPU indices of replica i)."""
    cores = topo.physical_cores()
    zero_l3 = topo.l3_of.get(0, topo.l3_of.get(cores[0], 0)) if cores else 0
    preferred = [c for c in cores if topo.l3_of.get(c) != zero_l3]
    need = max(min_per_replica, max((len(r) for r in replicas), default=1) + 1) * len(replicas)
    pool = preferred if len(preferred) >= need else cores  # avoid CPU 0's L3 group only when affordable
    by_node: dict[int, list[int]] = {}
    for c in pool:
        by_node.setdefault(topo.node_of.get(c, 0), []).append(c)
    # replicas ask for the node of their first GPU; unknown nodes are spread round-robin
    node_ids = sorted(by_node) or [0]
    wants = []
    for i, gpus in enumerate(replicas):
        n = topo.gpu_nodes[gpus[0]] if gpus and gpus[0] < len(topo.gpu_nodes) else -1
        wants.append(n if n in by_node else node_ids[i % len(node_ids)])
    share: dict[int, int] = {}
    for n in wants:
        share[n] = share.get(n, 0) + 1
    out: list[ReplicaCpus] = []
    taken: dict[int, int] = {n: 0 for n in node_ids}
    for i, gpus in enumerate(replicas):
        n = wants[i]
        avail = by_node.get(n, [])
        per = max(1, len(avail) // share[n])
        lo = taken[n]
        mine = avail[lo : lo + per] or (avail[-per:] if avail else cores[:1])
        taken[n] = lo + per
        siblings = [c for c in topo.allowed if topo.core_of.get(c, c) in {topo.core_of.get(m, m) for m in mine}]
        ranks = max(1, len(gpus))
        rank_cpus = [mine[j % len(mine)] for j in range(ranks)]
        out.append(ReplicaCpus(sorted(set(siblings) | set(mine)), rank_cpus))
    return out


def pin_rank(cpu: int | None) -> bool:
    """Pin the calling thread to one CPU (engine threads must not migrate)."""
    if cpu is None:
        return False
    try:
        os.sched_setaffinity(0, {cpu})
        return True
    except (AttributeError, OSError):
        return False


def thread_caps(n_cpus: int) -> dict[str, str]:
    """Environment for a replica process: bound the implicit thread pools to its slice."""
    n = str(max(1, n_cpus))
    return {"OMP_NUM_THREADS": n, "MKL_NUM_THREADS": n, "RAYON_NUM_THREADS": n, "TOKENIZERS_PARALLELISM": "true"}


def gpu_bdfs() -> list[str]:
    """PCI addresses of the visible GPUs via NVML (empty when there is none)."""
    try:
        import pynvml

        pynvml.nvmlInit()
        out = []
        for i in range(pynvml.nvmlDeviceGetCount()):
            info = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(i))
            bus = info.busId.decode() if isinstance(info.busId, bytes) else info.busId
            out.append(bus[-12:] if len(bus) > 12 else bus)
        return out
    except Exception:  # noqa: BLE001 - no driver / no NVML: placement falls back to an even split
        return []
