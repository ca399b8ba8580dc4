"""Which GPU serves which session.

Sessions are independent (src/core/batch.c:6-8), so a batch larger than one
GPU's share is split by session with no data-path collective.  A decode step
streams every cached key of every session once, so a GPU's step time follows
the SUM of its sessions' context lengths, and the step of the whole job is the
slowest GPU's: the split has to balance that sum, under the reference's cap of
WR_BATCH_MAX sessions per batched step (include/wayruntime/wayruntime.h:423).
"""
from __future__ import annotations

BATCH_MAX = 16


def assign_sessions(lens, world: int, per_gpu: int = BATCH_MAX) -> list[list[int]]:
    """Indices of `lens` for each of `world` GPUs, at most `per_gpu` each.

    Longest-first greedy onto the least-loaded GPU that still has a free slot,
    then pairwise swaps between the heaviest GPU and the others while they
    lower its load.  Deterministic (ties go to the lower index)."""
    n = len(lens)
    if world < 1 or per_gpu < 1:
        raise ValueError("world and per_gpu must be positive")
    if n > world * per_gpu:
        raise ValueError(f"{n} sessions do not fit {world} GPUs x {per_gpu}")
    order = sorted(range(n), key=lambda i: (-int(lens[i]), i))
    bins: list[list[int]] = [[] for _ in range(world)]
    load = [0] * world
    for i in order:
        g = min((g for g in range(world) if len(bins[g]) < per_gpu), key=lambda g: (load[g], g))
        bins[g].append(i)
        load[g] += int(lens[i])
    for _ in range(4 * n):
        hi = max(range(world), key=lambda g: (load[g], -g))
        best = None
        for lo in range(world):
            if lo == hi:
                continue
            gap = load[hi] - load[lo]
            for a in bins[hi]:
                for b in bins[lo]:
                    d = int(lens[a]) - int(lens[b])
                    if 0 < d < gap and (best is None or abs(gap - 2 * d) < best[0]):
                        best = (abs(gap - 2 * d), lo, a, b, d)
        if best is None:
            break
        _, lo, a, b, d = best
        new_peak = max(load[hi] - d, load[lo] + d)
        if new_peak >= load[hi]:
            break
        bins[hi].remove(a), bins[lo].remove(b)
        bins[hi].append(b), bins[lo].append(a)
        load[hi] -= d
        load[lo] += d
    return [sorted(b) for b in bins]


def imbalance(lens, bins) -> float:
    """max over GPUs of the summed length, over the mean (1.0 = perfectly even)."""
    loads = [sum(int(lens[i]) for i in b) for b in bins]
    mean = sum(loads) / max(len(loads), 1)
    return max(loads) / mean if mean else 1.0
