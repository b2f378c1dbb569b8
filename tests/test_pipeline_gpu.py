"""The chunk, single-chunk and long-form pipelines (C ABI) against the composition of the stages.

Every stage is parity-checked against the CPU oracle in its own test file; here the pipelines must
equal: GPU stages called one by one + the oracle's host logic (time offsets, overlap merge, text)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

import oracle
from oracle import encoder_oracle as eo
from oracle import text_oracle
from scriptrs_b200 import synth

LAYERS = 2
VOCAB = [f"▁w{i}" if i % 3 == 0 else (str(i % 10) if i % 3 == 1 else chr(97 + i % 26)) for i in range(1024)] + ["<blk>"]


@pytest.fixture(scope="module")
def pipe(ctx):
    import scriptrs_b200 as sb

    w = eo.seeded_weights(eo.EncoderConfig(layers=LAYERS), seed=21, std=0.02, plain_norms=False)
    w.update(oracle.seeded_decoder_weights(22))
    vocab = sb.Vocabulary.from_tokens(VOCAB)
    return sb.TranscriptionPipeline.from_weights(w, vocab, encoder_layers=LAYERS, ctx=ctx)


def stages_by_hand(ctx, audio, tasks):
    """GPU stages one at a time, then the oracle's offsets."""
    import scriptrs_b200 as sb

    fx = sb.ParakeetFeatureExtractor(ctx)
    feats = fx.extract_batch([audio[a:b] for a, b, _, _ in tasks])
    fo = np.zeros(len(feats) + 1, np.int64)
    fo[1:] = np.cumsum([f.shape[0] for f in feats])
    d_feats = torch.from_numpy(np.concatenate(feats)).cuda()
    n_out = sum(sb.encoder_num_frames(f.shape[0]) for f in feats)
    d_enc = torch.empty(n_out, 1024, device="cuda")
    torch.cuda.synchronize()
    eoffs = sb.encode_device(ctx, d_feats.data_ptr(), fo, d_enc.data_ptr())
    ctx.synchronize()
    dec = sb.tdt_decode_device(ctx, d_enc.data_ptr(), eoffs)
    out = []
    for d, (a, b, off, cs) in zip(dec, tasks):
        out.append(oracle.apply_time_offsets(d["tokens"], d["frames"], d["durations"], d["conf"], off // 1280, cs // 1280))
    return out


def test_transcribe_chunks_equals_stages(ctx, pipe):
    import scriptrs_b200 as sb

    audio = synth.long_audio(700_000, 3)
    tasks = oracle.plan_fast(audio.size)
    assert len(tasks) == 4
    got = sb.transcribe_chunks(ctx, audio, tasks)
    ref = stages_by_hand(ctx, audio, tasks)
    for g, r in zip(got, ref):
        assert np.array_equal(g.token_ids, r[0]) and np.array_equal(g.frame_indices, r[1])
        assert np.array_equal(g.durations, r[2]) and np.array_equal(g.confidences, r[3])
    assert sum(len(g.token_ids) for g in got) > 0


def test_long_form_run_equals_stages_plus_oracle_merge_and_text(ctx, pipe):
    import scriptrs_b200 as sb

    audio = synth.long_audio(900_000, 4)
    lf = sb.LongFormTranscriptionPipeline(pipe)
    res = lf.run(audio)
    tasks = oracle.plan_fast(audio.size)
    wins = stages_by_hand(ctx, audio, tasks)
    tok, frm, dur, conf = oracle.merge_windows(wins)
    dec = text_oracle.decode(VOCAB, tok, frm, conf, audio.size / 16000)
    ref = text_oracle.long_form_result(dec["tokens"], audio.size)
    assert res.text == ref["text"]
    assert [(t.token_id, t.text, t.start, t.end) for t in res.tokens] == [(a, b, c, d) for a, b, c, d, _ in ref["tokens"]]
    assert np.allclose([t.confidence for t in res.tokens], [t[4] for t in ref["tokens"]])
    assert [(c.start, c.end, c.text) for c in res.chunks] == ref["chunks"]
    assert res.duration_seconds == audio.size / 16000
    assert len(res.chunks) <= 1  # Fast mode: one Overlap region (long_form.rs:757-769)


def test_single_chunk_run_and_long_form_short_circuit(ctx, pipe):
    import scriptrs_b200 as sb

    audio = synth.clip_audio(200_000, 9)
    res = pipe.run(audio)
    wins = stages_by_hand(ctx, audio, [(0, audio.size, 0, 0)])
    ref = text_oracle.decode(VOCAB, wins[0][0], wins[0][1], wins[0][3], audio.size / 16000)
    assert res.text == ref["text"]
    assert [(t.token_id, t.start, t.end) for t in res.tokens] == [(a, c, d) for a, _, c, d, _ in ref["tokens"]]
    # long_form.rs:161-163: audio that fits one window goes through the inner pipeline unchanged
    lf = sb.LongFormTranscriptionPipeline(pipe)
    res2 = lf.run(audio)
    assert res2.text == res.text and res2.chunks == res.chunks and res2.tokens == res.tokens
    assert lf.run_chunk(audio).text == res.text


def test_error_behaviour(ctx, pipe):
    import scriptrs_b200 as sb

    with pytest.raises(sb.ScriptrsError) as e:
        pipe.run(np.zeros(0, np.float32))                  # pipeline.rs:150
    assert e.value.status == 1
    with pytest.raises(sb.ScriptrsError) as e:
        pipe.run(np.zeros(240_001, np.float32))            # pipeline.rs:153-158
    assert e.value.status == 2 and "15.00s" in e.value.message
    lf = sb.LongFormTranscriptionPipeline(pipe)
    with pytest.raises(sb.ScriptrsError) as e:
        lf.run(np.zeros(0, np.float32))                    # long_form.rs:158
    assert e.value.status == 1
    assert pipe.run(np.zeros(240_000, np.float32)).duration_seconds == 15.0


def test_worker_count_does_not_change_the_result(ctx, pipe):
    import scriptrs_b200 as sb

    audio = synth.long_audio(700_000, 6)
    lf = sb.LongFormTranscriptionPipeline(pipe)
    a = lf.run_with_config(audio, sb.LongFormConfig(worker_count=1))
    b = lf.run_with_config(audio, sb.LongFormConfig(worker_count=8))
    assert a.text == b.text and a.tokens == b.tokens


def test_pieced_host_copy_equals_resident_path(ctx, pipe):
    """Many ordered tasks: the host PCM goes up in three pieces on a copy stream under the kernels; the token
    streams must equal those of the same tasks over a device-resident buffer (single piece).  Short tasks keep
    the 2-block encoder cheap."""
    import scriptrs_b200 as sb

    n_tasks, task_len, stride = 600, 4000, 3000
    audio = synth.long_audio(stride * (n_tasks - 1) + task_len, 17)
    tasks = [(i * stride, i * stride + task_len, i * stride, 0) for i in range(n_tasks)]
    host = sb.transcribe_chunks(ctx, audio, tasks)
    d_audio = torch.from_numpy(audio).cuda()
    torch.cuda.synchronize()
    dev = sb.transcribe_chunks(ctx, None, tasks, audio_ptr=d_audio.data_ptr(), n_samples=audio.size, on_device=True)
    for x, y in zip(host.flat(), dev.flat()):
        assert np.array_equal(x, y)
    # unordered tasks fall back to one copy and must still give each task its own result
    perm = list(reversed(range(n_tasks)))
    shuffled = sb.transcribe_chunks(ctx, audio, [tasks[i] for i in perm])
    for k in (0, 57, n_tasks - 1):
        assert np.array_equal(shuffled[k].token_ids, host[perm[k]].token_ids)
