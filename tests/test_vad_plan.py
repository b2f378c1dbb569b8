"""Planning of the VAD long-form mode (speech regions, silence splits, region tasks, region results): the oracle
against the reference's known answers, and the library's host logic through the C ABI against both.  No GPU."""
import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

import oracle
import scriptrs_b200 as sb
from oracle import text_oracle
from oracle import vad_oracle as vo

W = vo.VAD_WINDOW_SAMPLES


def seg_pair(**kw):
    return sb.VadSegmentationConfig(**kw), vo.Segmentation(**kw)


# ---------------------------------------------------------------- the reference's known answers
def test_speech_regions_trim_short_silence():
    p = [0.9, 0.9, 0.1, 0.9, 0.9]                                    # planner.rs:324-335
    assert len(vo.detect_speech_regions(p, len(p) * W, 0.85, vo.Segmentation())) == 1
    r = sb.detect_speech_regions(p, len(p) * W, 0.85)
    assert r == vo.detect_speech_regions(p, len(p) * W, 0.85, vo.Segmentation()) == [(0, 5 * W)]


def test_silence_split_prefers_internal_gap():
    p = [0.9, 0.9, 0.9, 0.2, 0.2, 0.2, 0.2, 0.9, 0.9, 0.9]           # planner.rs:337-355
    region = (0, len(p) * W)
    for segs in (vo.plan_region_subsegments(region, p, vo.Segmentation(), 5 * W),
                 sb.plan_region_subsegments(region, p, max_chunk_samples=5 * W)):
        assert len(segs) == 2 and segs[0][1] <= 5 * W
        assert segs == [(0, 3 * W), (7 * W, 10 * W)]


def test_no_silence_returns_none_for_overlap_fallback():
    p = [0.9] * 10                                                   # planner.rs:357-374
    region = (0, len(p) * W)
    assert vo.plan_region_subsegments(region, p, vo.Segmentation(), 4 * W) is None
    assert sb.plan_region_subsegments(region, p, max_chunk_samples=4 * W) is None


def test_short_region_stays_as_a_single_segment_task():
    tasks = []                                                       # long_form.rs:682-704
    kind, idx = vo.build_region_plan((16_000, 32_000), [], vo.Segmentation(), 240_000, tasks)
    assert kind == vo.SEGMENTS and idx == [0] and tasks == [(16_000, 32_000, 0, 0)]
    t, r = sb.plan_vad([(16_000, 32_000)], [])
    assert t == tasks and r == [(1, 0, 1)]


def test_overlap_plan_keeps_window_order_and_context_offsets():
    kw = dict(max_speech_duration=1.0, min_silence_at_max_speech=10.0, use_max_possible_silence_at_max_speech=False)
    s_lib, s_ora = seg_pair(**kw)                                    # long_form.rs:706-736
    probs = [1.0] * -(-96_000 // 512)
    tasks = []
    kind, idx = vo.build_region_plan((0, 96_000), probs, s_ora, 48_000, tasks, max_model_samples=240_000)
    assert kind == vo.OVERLAP and len(idx) == len(tasks)
    assert all(a[2] <= b[2] for a, b in zip(tasks, tasks[1:]))
    assert all(t[3] <= t[2] for t in tasks)
    cfg = sb.LongFormConfig(segmentation=s_lib)
    cfg.transcription.max_audio_samples = 48_000
    t, r = sb.plan_vad([(0, 96_000)], probs, cfg)
    assert t == tasks and r == [(0, 0, len(tasks))]


def test_defaults_mirror_the_reference():
    c = sb.LongFormConfig().to_c()                                    # planner.rs:19-27,52-68
    assert abs(c.vad.default_threshold - 0.85) < 1e-7
    s = c.segmentation
    assert (s.min_speech_duration, s.min_silence_duration, s.max_speech_duration, s.speech_padding) == (0.15, 0.75, 14.0, 0.1)
    assert abs(s.silence_threshold_for_split - 0.3) < 1e-7 and s.has_negative_threshold == 0
    assert abs(s.negative_threshold_offset - 0.15) < 1e-7 and s.min_silence_at_max_speech == 0.098
    assert s.use_max_possible_silence_at_max_speech == 1
    d = sb._lib.LongFormConfigC()
    sb.lib().sb_default_longform_config(d)
    assert bytes(d) == bytes(c)
    assert sb.vad_num_windows(0) == 0 and sb.vad_num_windows(1) == 1 and sb.vad_num_windows(1024) == 2


# ---------------------------------------------------------------- differential against the oracle
def prob_track(rng, n):
    """Piecewise speech / silence / in-between probabilities with noise, like a detector's output."""
    out = np.empty(n, np.float32)
    i = 0
    while i < n:
        run = int(rng.integers(1, 120))
        level = rng.choice([0.02, 0.2, 0.5, 0.72, 0.9, 0.99])
        out[i:i + run] = np.clip(level + rng.normal(0, 0.08, min(run, n - i)), 0, 1)
        i += run
    return out


@pytest.mark.parametrize("seed", range(40))
def test_detect_and_plan_match_the_oracle(seed):
    rng = np.random.default_rng(seed)
    n = int(rng.integers(1, 4000))
    probs = prob_track(rng, n)
    audio_len = int(n * W - rng.integers(0, W)) if rng.random() < 0.8 else int(rng.integers(1, n * W + 2000))
    kw = {}
    if seed % 3 == 1:
        kw = dict(min_speech_duration=float(rng.uniform(0, 1)), min_silence_duration=float(rng.uniform(0, 2)),
                  speech_padding=float(rng.uniform(0, 1.5)), silence_threshold_for_split=float(rng.uniform(0.05, 0.8)),
                  min_silence_at_max_speech=float(rng.uniform(0, 0.5)))
    if seed % 3 == 2:
        kw = dict(negative_threshold=float(rng.uniform(0.0, 0.9)), speech_padding=-1.0)
    s_lib, s_ora = seg_pair(**kw)
    thr = float(rng.choice([0.5, 0.85, 0.1]))
    regions = sb.detect_speech_regions(probs, audio_len, thr, s_lib)
    assert regions == vo.detect_speech_regions(probs, audio_len, thr, s_ora)
    max_chunk = int(rng.choice([240_000, 48_000, 16_000]))
    for region in regions:
        rp = vo.region_probability_slice(probs, region)
        assert sb.plan_region_subsegments(region, rp, s_lib, max_chunk) == \
            vo.plan_region_subsegments(region, rp, s_ora, max_chunk)
    cfg = sb.LongFormConfig(segmentation=s_lib)
    cfg.transcription.max_audio_samples = max_chunk
    tasks, rts = sb.plan_vad(regions, probs, cfg)
    o_tasks, o_rts = vo.build_execution_plan(regions, probs, s_ora, max_chunk)
    assert tasks == o_tasks
    assert rts == [(k, idx[0] if idx else len(o_tasks), len(idx)) for k, idx in o_rts]
    # every task lies inside its region and, for segments, fits the chunk limit or fails loudly later
    for (k, first, cnt), region in zip(rts, regions):
        for t in tasks[first:first + cnt]:
            assert region[0] - (1280 if k == 0 else 0) <= t[0] <= t[1] <= region[1]


def test_equal_silences_take_the_last_one():
    # two silences of equal length inside the search range: Iterator::max_by_key keeps the later one
    p = [0.9] * 3 + [0.1] * 4 + [0.9] * 3 + [0.1] * 4 + [0.9] * 6
    region = (0, len(p) * W)
    want = vo.plan_region_subsegments(region, p, vo.Segmentation(), 16 * W)
    assert want == [(0, 10 * W), (14 * W, 20 * W)]
    assert sb.plan_region_subsegments(region, p, max_chunk_samples=16 * W) == want


def test_empty_inputs():
    assert sb.detect_speech_regions([], 16000) == []
    assert sb.detect_speech_regions([0.9, 0.9], 0) == []
    assert sb.detect_speech_regions([0.1] * 50, 50 * W) == []
    assert sb.plan_vad([], [0.5] * 4) == ([], [])


# ---------------------------------------------------------------- region results
VOCAB = ["▁the", "▁a", "▁cat", "s", "▁sat", "▁on", "▁mat", "1", "<blk>"]


def raw(tok, frm):
    n = len(tok)
    return sb.RawTranscription(np.array(tok, np.uint32), np.array(frm, np.int64), np.ones(n, np.int64),
                               np.full(n, 0.5, np.float32))


def oracle_region_result(audio_len, tasks, region_tasks, windows):
    """build_parallel_result (long_form.rs:344-419,649-661) from the oracle's text decoder and merge."""
    tokens, chunks = [], []
    for kind, first, cnt in region_tasks:
        if kind == vo.SEGMENTS:
            rt = []
            for i in range(first, first + cnt):
                w = windows[i]
                d = text_oracle.decode(VOCAB, w.token_ids, w.frame_indices, w.confidences,
                                       (tasks[i][1] - tasks[i][0]) / 16000)
                shift = tasks[i][0] / 16000
                rt += [(a, b, s + shift, e + shift, c) for a, b, s, e, c in d["tokens"]]
        else:
            m = oracle.merge_windows([(w.token_ids, w.frame_indices, w.durations, w.confidences)
                                      for w in windows[first:first + cnt]])
            rt = text_oracle.decode(VOCAB, m[0], m[1], m[3], audio_len / 16000)["tokens"]
        if rt:
            chunks.append((rt[0][2], rt[-1][3], "".join(t[1] for t in rt).strip()))
            tokens += rt
    return dict(text=" ".join(c[2] for c in chunks), chunks=chunks, tokens=tokens)


def test_region_results_shift_segments_and_merge_overlaps():
    vocab = sb.Vocabulary.from_tokens(VOCAB)
    audio_len = 16000 * 60
    tasks = [(16_000, 80_000, 0, 0), (100_000, 150_000, 0, 0),          # a Segments region of two tasks
             (200_000, 438_080, 200_000, 0), (404_800, 600_000, 406_080, 1280),  # an Overlap region
             (700_000, 700_100, 0, 0)]                                   # a Segments region without tokens
    region_tasks = [(1, 0, 2), (0, 2, 2), (1, 4, 1)]
    windows = [raw([0, 2, 3], [2, 10, 12]), raw([4], [5]),
               raw([5, 0, 6], [160, 300, 340]), raw([0, 6, 7], [300, 340, 400]), raw([], [])]
    r = sb.longform_finish_regions(vocab, audio_len, tasks, region_tasks, windows)
    o = oracle_region_result(audio_len, tasks, region_tasks, windows)
    assert r.text == o["text"] == "the cats sat on the mat 1"
    assert [(c.start, c.end, c.text) for c in r.chunks] == o["chunks"]
    assert [(t.token_id, t.text, t.start, t.end) for t in r.tokens] == [(a, b, s, e) for a, b, s, e, _ in o["tokens"]]
    assert len(r.chunks) == 2 and r.duration_seconds == 60.0
    # first token of the first segment: frame 2 of a task that starts at second 1
    assert r.tokens[0].start == 2 * 0.08 + 1.0
    # the last token of a segment ends at most at the segment's own duration, then shifted
    assert r.tokens[3].end == min(5 * 0.08 + 0.08, 50_000 / 16000) + 100_000 / 16000


def test_finish_regions_rejects_regions_outside_the_task_list():
    vocab = sb.Vocabulary.from_tokens(VOCAB)
    with pytest.raises(sb.ScriptrsError) as e:
        sb.longform_finish_regions(vocab, 16000, [(0, 100, 0, 0)], [(1, 0, 2)], [raw([], [])])
    assert e.value.status == 11
