"""Pins the long-form oracle (oracle/longform_oracle.c, oracle/text_oracle.py) against the
reference's own known-answer tests, carried over as data."""
import numpy as np

import oracle
from oracle import text_oracle


def test_overlap_plan_advances_with_stride():
    # src/long_form/planner.rs:376-385
    chunks = oracle.plan_fast(600_000)
    assert len(chunks) > 1
    assert chunks[1][2] < chunks[0][1]  # chunk[1].start < chunk[0].end


def test_default_chunk_geometry():
    # src/long_form/planner.rs:104-122 evaluated for the defaults
    assert oracle.chunk_samples() == 238_080
    assert oracle.overlap_samples() == 32_000
    assert oracle.stride_samples() == 206_080


def test_eight_hour_plan():
    tasks = oracle.plan_fast(460_800_000)
    assert len(tasks) == 2236
    assert tasks[0] == (0, 238_080, 0, 0)
    assert tasks[1][1] - tasks[1][0] == 239_360 and tasks[1][3] == 1280
    assert tasks[-1][1] == 460_800_000 and tasks[-1][1] - tasks[-1][0] == 212_480


def test_parallel_worker_count_respects_requested_workers():
    # src/long_form.rs:738-745
    assert oracle.parallel_worker_count(0, 4) == 1
    assert oracle.parallel_worker_count(1, 4) == 1
    assert oracle.parallel_worker_count(3, 0) == 1
    assert oracle.parallel_worker_count(3, 2) == 2
    assert oracle.parallel_worker_count(3, 8) == 3


def test_fast_plan_is_one_region_over_all_tasks():
    # src/long_form.rs:757-769: 96000 samples -> a non-empty plan
    assert len(oracle.plan_fast(96_000)) == 1


def test_contiguous_tokens_are_deduplicated():
    # src/long_form/merge.rs:208-224
    left = ([1, 2, 3], [0, 10, 20], [1, 1, 1], [0.9] * 3)
    right = ([2, 3, 4], [10, 20, 30], [1, 1, 1], [0.9] * 3)
    tok, frm, dur, conf = oracle.merge_windows([left, right])
    assert list(tok) == [1, 2, 3, 4]


def test_midpoint_fallback_keeps_monotonic_frames():
    # src/long_form/merge.rs:226-247
    left = ([1, 2], [0, 10], [1, 1], [0.9] * 2)
    right = ([9, 10], [8, 18], [1, 1], [0.9] * 2)
    tok, frm, dur, conf = oracle.merge_windows([left, right])
    assert all(a <= b for a, b in zip(frm[:-1], frm[1:]))


def test_time_offsets():
    # src/pipeline.rs:219-252
    tok, frm, dur, conf = oracle.apply_time_offsets([5, 6, 7], [0, 1, 4], [1, 1, 1], [0.5, 0.6, 0.7], 161, 1)
    assert list(tok) == [6, 7] and list(frm) == [161, 164]
    tok, frm, dur, conf = oracle.apply_time_offsets([5, 6], [0, 3], [1, 1], [0.5, 0.6], 10, 0)
    assert list(tok) == [5, 6] and list(frm) == [10, 13]


def test_digit_spacing_matches_parakeet_rs():
    # src/decode.rs:151-163
    vocab = ["▁like", "1", "0", "0", "<blk>"]
    r = text_oracle.decode(vocab, [0, 1, 2, 3], [0, 1, 2, 3], [0.9] * 4, 1.0)
    assert r["text"] == "like 100"
    assert r["tokens"][1][1] == " 1"


def test_chunk_spans_the_token_range():
    # src/decode.rs:165-179
    vocab = ["▁hello", "▁world", "<blk>"]
    r = text_oracle.decode(vocab, [0, 1], [0, 4], [0.9] * 2, 1.0)
    start, end, text = r["chunks"][0]
    assert text == "hello world" and start == 0.0 and end > start


def test_blank_defaults_to_last_token():
    # src/vocab.rs:67-74
    toks, blank = text_oracle.parse_vocab("a 0\nb 1\n")
    assert blank == 1
    toks, blank = text_oracle.parse_vocab("<blk> 0\nb 1\n")
    assert blank == 0
