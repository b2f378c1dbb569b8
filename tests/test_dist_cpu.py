"""world_size-2 gloo test of the rank sharding + reassembly used by the multi-GPU bench (CPU only)."""
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def fake_transcribe(task):
    """Deterministic stand-in for a GPU shard: tokens derived from the global frame grid, so that
    neighbouring windows agree on their overlap exactly like real re-decodes do."""
    import scriptrs_b200 as sb

    a, b, off, cs = task
    f0, f1 = off // 1280, (b + 1279) // 1280
    frames = np.arange(f0, f1, 3, dtype=np.int64)
    frames = frames[frames % 7 != 0]
    toks = (frames * 2654435761 % 1000).astype(np.uint32)
    return sb.RawTranscription(toks, frames, np.ones(frames.size, np.int64), np.full(frames.size, 0.5, np.float32))


def worker(rank, world, port, n, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist

    import scriptrs_b200 as sb
    from scriptrs_b200 import dist as sbd

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    tasks = sb.plan_fast(n)
    lo, hi = sbd.shard_bounds(len(tasks), rank, world)
    raws = [fake_transcribe(t) for t in tasks[lo:hi]]
    vocab = sb.Vocabulary.from_tokens([f"▁t{i}" for i in range(1000)] + ["<blk>"])
    res = sbd.gather_and_finish(vocab, n, raws, rank, world)
    if rank == 0:
        q.put((res.text, [(t.token_id, t.start, t.end) for t in res.tokens], len(tasks)))
    else:
        assert res is None
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_run_equals_single_process(world):
    import scriptrs_b200 as sb

    n = 16000 * 200
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + world
    procs = [ctx.Process(target=worker, args=(r, world, port, n, q)) for r in range(world)]
    for p in procs:
        p.start()
    text, tokens, n_tasks = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    tasks = sb.plan_fast(n)
    assert n_tasks == len(tasks) and len(tasks) > world
    vocab = sb.Vocabulary.from_tokens([f"▁t{i}" for i in range(1000)] + ["<blk>"])
    single = sb.longform_finish(vocab, n, [fake_transcribe(t) for t in tasks])
    assert text == single.text
    assert tokens == [(t.token_id, t.start, t.end) for t in single.tokens]
    # the merge removed the duplicated overlap: frames strictly increase
    starts = [s for _, s, _ in tokens]
    assert all(a < b for a, b in zip(starts[:-1], starts[1:]))


def test_shard_bounds_cover_all_tasks_once():
    from scriptrs_b200 import dist as sbd

    for n in (0, 1, 5, 2236):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                lo, hi = sbd.shard_bounds(n, r, world)
                seen.extend(range(lo, hi))
            assert seen == list(range(n))


# ---------------------------------------------------------------- VAD mode: a plan of region tasks over ranks
def vad_plan_for_test(n):
    import scriptrs_b200 as sb

    rng = np.random.default_rng(11)
    probs = np.full(sb.vad_num_windows(n), 0.95, np.float32)
    w = 0
    while w < probs.size:                      # speech of 3..40 s, silences of 1..5 s
        w += int(rng.uniform(3, 40) * 31.25)
        gap = int(rng.uniform(1, 5) * 31.25)
        probs[w:w + gap] = 0.02
        w += gap
    regions = sb.detect_speech_regions(probs, n)
    tasks, region_tasks = sb.plan_vad(regions, probs)
    return tasks, region_tasks


def fake_transcribe_segment(task):
    """Tokens on the task's own frame grid (segment tasks carry no global offset)."""
    import scriptrs_b200 as sb

    a, b, off, cs = task
    if off or cs:
        return fake_transcribe(task)
    frames = np.arange(0, (b - a) // 1280, 4, dtype=np.int64)
    toks = ((frames + a // 1280) * 40503 % 1000).astype(np.uint32)
    return sb.RawTranscription(toks, frames, np.ones(frames.size, np.int64), np.full(frames.size, 0.5, np.float32))


def vad_worker(rank, world, port, n, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist

    import scriptrs_b200 as sb
    from scriptrs_b200 import dist as sbd

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    tasks, region_tasks = vad_plan_for_test(n)
    lo, hi = sbd.shard_bounds(len(tasks), rank, world)
    raws = [fake_transcribe_segment(t) for t in tasks[lo:hi]]
    vocab = sb.Vocabulary.from_tokens([f"▁t{i}" for i in range(1000)] + ["<blk>"])
    res = sbd.gather_and_finish_regions(vocab, n, tasks, region_tasks, raws, rank, world)
    if rank == 0:
        q.put((res.text, [(t.token_id, t.start, t.end) for t in res.tokens], [(c.start, c.end) for c in res.chunks]))
    else:
        assert res is None
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_vad_plan_equals_single_process():
    import scriptrs_b200 as sb

    n, world = 16000 * 400, 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=vad_worker, args=(r, world, 29671, n, q)) for r in range(world)]
    for p in procs:
        p.start()
    text, tokens, chunks = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    tasks, region_tasks = vad_plan_for_test(n)
    assert {k for k, _, _ in region_tasks} == {0, 1} and len(tasks) > len(region_tasks) > 4
    vocab = sb.Vocabulary.from_tokens([f"▁t{i}" for i in range(1000)] + ["<blk>"])
    single = sb.longform_finish_regions(vocab, n, tasks, region_tasks, [fake_transcribe_segment(t) for t in tasks])
    assert text == single.text and len(chunks) == len(region_tasks)
    assert tokens == [(t.token_id, t.start, t.end) for t in single.tokens]
    assert chunks == [(c.start, c.end) for c in single.chunks]
