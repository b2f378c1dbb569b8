"""One process per GPU: sharding of chunk tasks over ranks and reassembly on rank 0.

Mirrors the reference's worker pool (src/long_form.rs:266-342): workers share nothing, each takes a
block of tasks, results are put back in task order and merged by one consumer.  There is no
data-path collective; `torch.distributed` only carries the small per-task token streams."""
from __future__ import annotations

from .pipeline import RawTranscription, longform_finish


def shard_bounds(n_tasks: int, rank: int, world: int):
    """Contiguous block of rank `rank` (so that a rank needs one contiguous PCM span)."""
    return n_tasks * rank // world, n_tasks * (rank + 1) // world


def gather_raws(raws, rank: int, world: int, group=None):
    """Rank 0 returns all ranks' RawTranscription lists concatenated in rank (= task) order; others None."""
    if world == 1:
        return list(raws)
    import torch.distributed as dist

    payload = [(r.token_ids, r.frame_indices, r.durations, r.confidences) for r in raws]
    parts = [None] * world if rank == 0 else None
    dist.gather_object(payload, parts, dst=0, group=group)
    if rank != 0:
        return None
    return [RawTranscription(*t) for part in parts for t in part]


def gather_and_finish(vocab, audio_len: int, raws, rank: int, world: int, group=None):
    """Gather, then merge + decode + build the long-form result on rank 0 (None elsewhere)."""
    allr = gather_raws(raws, rank, world, group)
    if allr is None:
        return None
    return longform_finish(vocab, audio_len, allr)
