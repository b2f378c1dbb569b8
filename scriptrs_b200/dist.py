"""One process per GPU: sharding of chunk tasks over ranks and reassembly on rank 0.

Mirrors the reference's worker pool (src/long_form.rs:266-342): workers share nothing, each takes a
block of tasks, results are put back in task order and merged by one consumer.  There is no
data-path collective; `torch.distributed` only carries the small per-task token streams."""
from __future__ import annotations

from .pipeline import RawBatch, RawTranscription, longform_finish, longform_finish_regions


def shard_bounds(n_tasks: int, rank: int, world: int):
    """Contiguous block of rank `rank` (so that a rank needs one contiguous PCM span)."""
    return n_tasks * rank // world, n_tasks * (rank + 1) // world


def _pack(b: RawBatch):
    """One byte buffer per rank: offsets (int64, n + 1) | frames (int64) | durations (int64) | token ids (uint32) |
    confidences (float32); its length follows from the task and token counts."""
    import numpy as np

    parts = [np.ascontiguousarray(b.offsets, np.int64), np.ascontiguousarray(b.frame_indices, np.int64),
             np.ascontiguousarray(b.durations, np.int64), np.ascontiguousarray(b.token_ids, np.uint32),
             np.ascontiguousarray(b.confidences, np.float32)]
    return np.concatenate([p.view(np.uint8) for p in parts]) if parts else np.zeros(0, np.uint8)


def _packed_bytes(n_tasks: int, n_tokens: int) -> int:
    return 8 * (n_tasks + 1) + n_tokens * (8 + 8 + 4 + 4)


def _unpack(buf, n_tasks: int, n_tokens: int) -> RawBatch:
    import numpy as np

    o = 0

    def take(dt, count):
        nonlocal o
        nb = np.dtype(dt).itemsize * count
        a = buf[o:o + nb].view(dt).copy()
        o += nb
        return a

    offs = take(np.int64, n_tasks + 1)
    frm = take(np.int64, n_tokens)
    dur = take(np.int64, n_tokens)
    tok = take(np.uint32, n_tokens)
    conf = take(np.float32, n_tokens)
    return RawBatch(offs, tok, frm, dur, conf)


def gather_raws(raws, rank: int, world: int, group=None):
    """Rank 0 returns all ranks' token streams concatenated in rank (= task) order; others None.
    Two fixed-layout collectives (no pickling): the (tasks, tokens) counts of every rank, then one padded byte
    buffer per rank gathered to rank 0.  On the NCCL backend the buffers pass through device memory."""
    if world == 1:
        return raws
    import numpy as np
    import torch
    import torch.distributed as dist

    if not isinstance(raws, RawBatch):
        raws = RawBatch.concat([_as_batch(raws)])
    on_gpu = dist.get_backend(group) == "nccl"
    dev = torch.device("cuda", torch.cuda.current_device()) if on_gpu else torch.device("cpu")
    n_tasks, n_tokens = len(raws), int(raws.offsets[-1])
    counts = torch.tensor([n_tasks, n_tokens], dtype=torch.int64, device=dev)
    all_counts = torch.empty(world * 2, dtype=torch.int64, device=dev)
    dist.all_gather_into_tensor(all_counts, counts, group=group)
    all_counts = all_counts.cpu().numpy().reshape(world, 2)
    sizes = [_packed_bytes(int(a), int(b)) for a, b in all_counts]
    cap = max(sizes)
    mine = torch.zeros(cap, dtype=torch.uint8)
    payload = _pack(raws)
    mine[: payload.size] = torch.from_numpy(payload)
    mine = mine.to(dev)
    parts = [torch.empty(cap, dtype=torch.uint8, device=dev) for _ in range(world)] if rank == 0 else None
    dist.gather(mine, parts, dst=0, group=group)
    if rank != 0:
        return None
    out = []
    for r in range(world):
        buf = parts[r].cpu().numpy()
        out.append(_unpack(buf[: sizes[r]], int(all_counts[r][0]), int(all_counts[r][1])))
    return RawBatch.concat(out)


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


def gather_and_finish_regions(vocab, audio_len: int, tasks, region_tasks, raws, rank: int, world: int, group=None):
    """The same for a plan of region tasks (the VAD mode): every rank builds the same plan from the same
    probabilities (the planner is deterministic host logic, so no plan is sent), transcribes its block
    `shard_bounds(len(tasks), rank, world)` of the tasks, and rank 0 joins the regions
    (build_parallel_result, src/long_form.rs:344-374).  None on the other ranks."""
    allr = gather_raws(raws, rank, world, group)
    if allr is None:
        return None
    return longform_finish_regions(vocab, audio_len, tasks, region_tasks, allr)
