"""Host-side logic of the library (planner, offsets, merge, vocabulary, text) through the C ABI,
against the reference's known answers and, differentially, against the CPU oracle.  No GPU needed."""
import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

import oracle
import scriptrs_b200 as sb
from oracle import text_oracle


def raw(tok, frm, dur=None, conf=None):
    n = len(tok)
    return sb.RawTranscription(np.array(tok, np.uint32), np.array(frm, np.int64),
                               np.array(dur if dur is not None else [1] * n, np.int64),
                               np.array(conf if conf is not None else [0.9] * n, np.float32))


# ---------------------------------------------------------------- planner
def test_planner_known_answers():
    oc = sb.OverlapChunkConfig()
    assert (oc.chunk_samples(), oc.overlap_samples(), oc.stride_samples()) == (238_080, 32_000, 206_080)
    chunks = sb.plan_fast(600_000)                       # planner.rs:376-385
    assert len(chunks) > 1 and chunks[1][2] < chunks[0][1]
    assert len(sb.plan_fast(460_800_000)) == 2236
    assert len(sb.plan_fast(96_000)) == 1                # long_form.rs:757-769


@given(st.integers(1, 3_000_000), st.sampled_from([0.0, 0.5, 2.0, 7.5, 100.0]), st.sampled_from([0, 640, 1280, 5000]),
       st.sampled_from([1000, 48_000, 240_000]))
@settings(max_examples=60, deadline=None)
def test_planner_matches_oracle(n, overlap_s, ctx_samples, max_model):
    oc = sb.OverlapChunkConfig(overlap_s, ctx_samples, max_model)
    assert sb.plan_fast(n, oc) == oracle.plan_fast(n, overlap_s, ctx_samples, max_model)
    assert oc.chunk_samples() == oracle.chunk_samples(ctx_samples, max_model)
    assert oc.overlap_samples() == oracle.overlap_samples(overlap_s, ctx_samples, max_model)
    assert oc.stride_samples() == oracle.stride_samples(overlap_s, ctx_samples, max_model)


def test_parallel_worker_count():
    for t, r in ((0, 4), (1, 4), (3, 0), (3, 2), (3, 8)):   # long_form.rs:738-745
        assert sb.parallel_worker_count(t, r) == oracle.parallel_worker_count(t, r)
    assert sb.parallel_worker_count(3, 8) == 3
    assert sb.LongFormConfig().worker_count == 4 and sb.LongFormConfig().mode == sb.LongFormMode.Fast


# ---------------------------------------------------------------- offsets
@given(st.lists(st.tuples(st.integers(0, 2000), st.integers(0, 190)), max_size=40), st.integers(0, 5000),
       st.integers(0, 3))
@settings(max_examples=60, deadline=None)
def test_time_offsets_match_oracle(items, frame_offset, context_frames):
    tok = [t for t, _ in items]
    frm = sorted(f for _, f in items)
    r = sb.apply_time_offsets(raw(tok, frm), frame_offset, context_frames)
    o = oracle.apply_time_offsets(tok, frm, [1] * len(tok), [0.9] * len(tok), frame_offset, context_frames)
    assert np.array_equal(r.token_ids, o[0]) and np.array_equal(r.frame_indices, o[1])


# ---------------------------------------------------------------- merge
def test_merge_known_answers():
    m = sb.merge_overlapping_windows([raw([1, 2, 3], [0, 10, 20]), raw([2, 3, 4], [10, 20, 30])])
    assert list(m.token_ids) == [1, 2, 3, 4]              # merge.rs:208-224
    m = sb.merge_overlapping_windows([raw([1, 2], [0, 10]), raw([9, 10], [8, 18])])
    assert all(a <= b for a, b in zip(m.frame_indices[:-1], m.frame_indices[1:]))  # merge.rs:226-247
    assert len(sb.merge_overlapping_windows([]).token_ids) == 0
    m = sb.merge_overlapping_windows([raw([], []), raw([4], [2]), raw([], [])])
    assert list(m.token_ids) == [4]                       # merge.rs:15-21


def random_windows(rng, n_windows, vocab, monotone=True):
    wins = []
    base = 0
    for _ in range(n_windows):
        n = int(rng.integers(0, 30))
        frames = base + np.sort(rng.integers(0, 188, n)) if monotone else base + rng.integers(0, 188, n)
        toks = rng.integers(0, vocab, n)
        wins.append((toks.astype(np.uint32), frames.astype(np.int64), rng.integers(0, 5, n).astype(np.int64),
                     rng.random(n).astype(np.float32)))
        base += int(rng.integers(100, 200))
    return wins


@pytest.mark.parametrize("vocab,monotone", [(3, True), (8, True), (50, True), (4, False), (1000, True)])
def test_windowed_merge_equals_the_literal_quadratic_merge(vocab, monotone):
    rng = np.random.default_rng(vocab * 2 + monotone)
    for trial in range(60):
        wins = random_windows(rng, int(rng.integers(1, 12)), vocab, monotone)
        got = sb.merge_overlapping_windows([sb.RawTranscription(*w) for w in wins])
        ref = oracle.merge_windows(wins)
        assert np.array_equal(got.token_ids, ref[0]), trial
        assert np.array_equal(got.frame_indices, ref[1])
        assert np.array_equal(got.durations, ref[2])
        assert np.array_equal(got.confidences, ref[3])


def test_merge_with_shared_prefix_of_overlapping_decodes():
    # realistic case: consecutive windows re-decode the same 25-frame overlap
    rng = np.random.default_rng(0)
    wins = []
    stream_tok = rng.integers(0, 1000, 4000).astype(np.uint32)
    stream_frm = np.sort(rng.integers(0, 40 * 161, 4000)).astype(np.int64)
    for k in range(40):
        lo, hi = k * 161, k * 161 + 186
        sel = (stream_frm >= lo) & (stream_frm < hi)
        n = int(sel.sum())
        wins.append((stream_tok[sel], stream_frm[sel], np.ones(n, np.int64), np.full(n, 0.5, np.float32)))
    got = sb.merge_overlapping_windows([sb.RawTranscription(*w) for w in wins])
    ref = oracle.merge_windows(wins)
    assert np.array_equal(got.token_ids, ref[0]) and np.array_equal(got.frame_indices, ref[1])
    assert np.array_equal(got.token_ids, stream_tok[stream_frm < 39 * 161 + 186])


# ---------------------------------------------------------------- vocabulary and text
def test_vocabulary_parsing(tmp_path):
    p = tmp_path / "vocab.txt"
    p.write_text("▁the 0\n▁a 1\ns 2\n<unk> 3\n<blk> 4\n", encoding="utf-8")
    v = sb.Vocabulary.from_file(str(p))
    assert len(v) == 5 and v.blank_id() == 4
    assert sb.Vocabulary.from_text("a 0\nb 1\n").blank_id() == 1    # vocab.rs:49: last id when no <blk>
    assert len(sb.Vocabulary.from_text("a 0\nz 5\n")) == 6          # gaps are filled (vocab.rs:33-35)
    with pytest.raises(sb.ScriptrsError) as e:
        sb.Vocabulary.from_text("a x\n")
    assert e.value.status == 5
    with pytest.raises(sb.ScriptrsError) as e:
        sb.Vocabulary.from_text("\n\n")
    assert e.value.status == 5
    with pytest.raises(sb.ScriptrsError) as e:
        sb.Vocabulary.from_file(str(tmp_path / "missing.txt"))
    assert e.value.status == 4


def test_text_decode_known_answers():
    d = sb.ParakeetTdtDecoder(sb.Vocabulary.from_tokens(["▁like", "1", "0", "0", "<blk>"]))
    r = d.decode(raw([0, 1, 2, 3], [0, 1, 2, 3]), 1.0)           # decode.rs:151-163
    assert r.text == "like 100" and r.tokens[1].text == " 1"
    d = sb.ParakeetTdtDecoder(sb.Vocabulary.from_tokens(["▁hello", "▁world", "<blk>"]))
    r = d.decode(raw([0, 1], [0, 4]), 1.0)                        # decode.rs:165-179
    assert r.chunks[0].text == "hello world" and r.chunks[0].start == 0.0 and r.chunks[0].end > 0.0
    r = d.decode(raw([], []), 2.5)
    assert r.text == "" and r.tokens == [] and r.chunks == [] and r.duration_seconds == 2.5


# letters from well outside Latin: Thai above U+0E30, a Hebrew presentation form, Latin Extended-D, a Roman numeral
# (category Nl), Cherokee, a supplementary-plane letter, a non-letter symbol; and Other_Alphabetic marks, which are
# alphabetic without being letters: a Devanagari vowel sign (Mc), a Hebrew point (Mn), a circled letter (So), and a
# combining accent that is NOT alphabetic (U+0301)
VOCAB = ["▁the", "▁a", "a", "s", "1", "23", "▁", "<unk>", "<pad>", "é", "▁Ünï", "ß", "", "x1", "▁4", "<blk>",
         "ไ", "\ufb2a", "\ua7b5", "\u2167", "\u13a0", "\U00010400", "\u2603", "7", "\u093e", "\u05b0", "\u24b6", "\u0301"]


@given(st.lists(st.tuples(st.integers(0, 29), st.integers(0, 6)), max_size=25), st.floats(0.0, 40.0))
@settings(max_examples=120, deadline=None)
def test_text_decode_matches_oracle(items, duration):
    tok = [t for t, _ in items]
    frm = list(np.cumsum([d for _, d in items])) if items else []
    conf = [0.25 + 0.01 * i for i in range(len(tok))]
    d = sb.ParakeetTdtDecoder(sb.Vocabulary.from_tokens(VOCAB))
    r = d.decode(raw(tok, frm, conf=conf), duration)
    o = text_oracle.decode(VOCAB, tok, frm, conf, duration)
    assert r.text == o["text"]
    assert [(t.token_id, t.text, t.start, t.end) for t in r.tokens] == [(a, b, c, e) for a, b, c, e, _ in o["tokens"]]
    assert [(c.start, c.end, c.text) for c in r.chunks] == o["chunks"]


def test_long_form_finish_builds_the_region_chunk():
    vocab = sb.Vocabulary.from_tokens(["▁hello", "▁world", "▁again", "<blk>"])
    wins = [raw([0, 1], [3, 150]), raw([1, 2], [150, 170])]
    r = sb.longform_finish(vocab, 16000 * 30, wins)
    o_tokens = text_oracle.decode(["▁hello", "▁world", "▁again", "<blk>"], [0, 1, 2], [3, 150, 170], [0.9] * 3, 30.0)
    o = text_oracle.long_form_result(o_tokens["tokens"], 16000 * 30)
    assert r.text == o["text"] == "hello world again"
    assert [(c.start, c.end, c.text) for c in r.chunks] == o["chunks"]
    assert r.duration_seconds == 30.0
    empty = sb.longform_finish(vocab, 16000, [raw([], [])])
    assert empty.text == "" and empty.chunks == [] and empty.tokens == []


def test_alphabetic_table_is_the_unicode_derived_property():
    """needs_digit_spacing (src/decode.rs:114-134) asks char::is_alphabetic: a digit token gets a space in front when
    two or more alphabetic characters end the text so far.  Probed through the text decoder for every kind of
    character the general categories alone would get wrong."""
    import regex

    alpha = regex.compile(r"\p{Alphabetic}")
    probes = ["\u0345", "\u05b0", "\u093e", "\u0903", "\u24b6", "\u2167", "\u0301", "\u20e3", "\u2603", "\u1885",
              "\U0001e947", "\U00016f51", "\u0e31", "\u0e47"]
    for ch in probes:
        vocab = ["x" + ch, "7", "<blk>"]
        r = sb.ParakeetTdtDecoder(sb.Vocabulary.from_tokens(vocab)).decode(raw([0, 1], [0, 2]), 1.0)
        want = "x" + ch + (" 7" if alpha.match(ch) else "7")
        assert r.text == want, (hex(ord(ch)), r.text)
        o = text_oracle.decode(vocab, [0, 1], [0, 2], [0.9, 0.9], 1.0)
        assert o["text"] == want
