"""One process per GPU: sharding of chunk tasks over ranks and reassembly on rank 0.

Mirrors the reference's worker pool (src/long_form.rs:266-342): workers share nothing, each takes a
block of tasks, results are put back in task order and merged by one consumer.  There is no
data-path collective; `torch.distributed` only carries the small per-task token streams."""
from __future__ import annotations

from .pipeline import RawBatch, RawTranscription, longform_finish


def shard_bounds(n_tasks: int, rank: int, world: int):
    """Contiguous block of rank `rank` (so that a rank needs one contiguous PCM span)."""
    return n_tasks * rank // world, n_tasks * (rank + 1) // world


def gather_raws(raws, rank: int, world: int, group=None):
    """Rank 0 returns all ranks' token streams concatenated in rank (= task) order; others None."""
    if world == 1:
        return raws
    import torch.distributed as dist

    if not isinstance(raws, RawBatch):
        raws = RawBatch.concat([_as_batch(raws)])
    parts = [None] * world if rank == 0 else None
    dist.gather_object(raws.flat(), parts, dst=0, group=group)
    if rank != 0:
        return None
    return RawBatch.concat([RawBatch(p[4], p[0], p[1], p[2], p[3]) for p in parts])


def _as_batch(raws) -> RawBatch:
    import numpy as np

    offs = np.zeros(len(raws) + 1, np.int64)
    for i, r in enumerate(raws):
        offs[i + 1] = offs[i] + len(r.token_ids)
    cat = lambda attr, dt: (np.concatenate([np.asarray(getattr(r, attr), dt) for r in raws]) if len(raws)
                            else np.zeros(0, dt))
    return RawBatch(offs, cat("token_ids", np.uint32), cat("frame_indices", np.int64), cat("durations", np.int64),
                    cat("confidences", np.float32))


def gather_and_finish(vocab, audio_len: int, raws, rank: int, world: int, group=None):
    """Gather, then merge + decode + build the long-form result on rank 0 (None elsewhere)."""
    allr = gather_raws(raws, rank, world, group)
    if allr is None:
        return None
    return longform_finish(vocab, audio_len, allr)
