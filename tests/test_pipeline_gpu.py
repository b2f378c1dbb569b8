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


def model_weights():
    w = eo.seeded_weights(eo.EncoderConfig(layers=LAYERS), seed=21, std=0.02, plain_norms=False)
    w.update(oracle.seeded_decoder_weights(22))
    return w


@pytest.fixture(scope="module")
def pipe(ctx):
    import scriptrs_b200 as sb

    vocab = sb.Vocabulary.from_tokens(VOCAB)
    return sb.TranscriptionPipeline.from_weights(model_weights(), vocab, encoder_layers=LAYERS, ctx=ctx)


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
    # 64 to 511 tasks go up in two pieces (what a GPU sees of an 8 h recording shared by eight)
    some = tasks[100:300]
    host2 = sb.transcribe_chunks(ctx, audio, some)
    for k in range(len(some)):
        assert np.array_equal(host2[k].token_ids, dev[100 + k].token_ids)
        assert np.array_equal(host2[k].frame_indices, dev[100 + k].frame_indices)
    # unordered tasks fall back to one copy and must still give each task its own result
    perm = list(reversed(range(n_tasks)))
    shuffled = sb.transcribe_chunks(ctx, audio, [tasks[i] for i in perm])
    for k in (0, 57, n_tasks - 1):
        assert np.array_equal(shuffled[k].token_ids, host[perm[k]].token_ids)


def test_longform_run_multi_with_two_contexts(ctx, pipe):
    """sb_longform_run_multi with more than one context: the reference's worker pool (src/long_form.rs:266-342) with
    one host thread per context.  Two contexts on the same GPU (own stream and workspaces each) must give the
    single-context result token for token, whatever the worker count says about how the tasks are dealt."""
    import scriptrs_b200 as sb

    second = sb.Context(0)
    try:
        sb.load_model(second, model_weights(), LAYERS, has_encoder=True, has_decoder=True)
        audio = synth.long_audio(1_100_000, 8)
        assert len(sb.plan_fast(audio.size)) == 6
        one = sb.LongFormTranscriptionPipeline(pipe).run(audio)
        both = sb.LongFormTranscriptionPipeline(pipe, extra_contexts=[second])
        for workers in (2, 4):
            two = both.run_with_config(audio, sb.LongFormConfig(worker_count=workers))
            assert two.text == one.text and two.tokens == one.tokens and two.chunks == one.chunks
        assert len(one.tokens) > 0
        # worker_count = 1 leaves the second context idle (long_form.rs:594-600)
        k0 = second.kernel_launches()
        solo = both.run_with_config(audio, sb.LongFormConfig(worker_count=1))
        assert solo.tokens == one.tokens and second.kernel_launches() == k0
    finally:
        second.close()


def test_failing_shard_fails_the_whole_call(ctx, pipe):
    """The first error a worker reports aborts the run (src/long_form.rs:328-332).  The fault is made on the host: the
    second context has no model, so its shard returns SB_MISSING_MODEL_ASSET while the first shard succeeds."""
    import scriptrs_b200 as sb

    empty = sb.Context(0)
    try:
        audio = synth.long_audio(700_000, 6)
        both = sb.LongFormTranscriptionPipeline(pipe, extra_contexts=[empty])
        with pytest.raises(sb.ScriptrsError) as e:
            both.run_with_config(audio, sb.LongFormConfig(worker_count=2))
        assert e.value.status == 3 and "weights" in e.value.message
        # nothing was left half-freed: the healthy context still transcribes, and so does the pair with one worker
        a = sb.LongFormTranscriptionPipeline(pipe).run(audio)
        b = both.run_with_config(audio, sb.LongFormConfig(worker_count=1))
        assert a.tokens == b.tokens
    finally:
        empty.close()


def test_device_side_timeout_flag_fails_the_call(ctx, pipe):
    """A kernel whose bounded wait ran out raises a flag in device memory and returns; every pipeline entry must then
    fail with SB_TIMEOUT instead of handing back tokens computed from unfinished tiles.  The flag is raised from the
    host here (option test_raise_device_error); no kernel waits or faults for this test."""
    import scriptrs_b200 as sb

    audio = synth.long_audio(500_000, 2)
    tasks = sb.plan_fast(audio.size)
    good = sb.transcribe_chunks(ctx, audio, tasks)
    ctx.set_option("test_raise_device_error", 1)
    with pytest.raises(sb.ScriptrsError) as e:
        sb.transcribe_chunks(ctx, audio, tasks)
    assert e.value.status == 10
    # the flag was cleared by the failing call
    again = sb.transcribe_chunks(ctx, audio, tasks)
    for x, y in zip(good.flat(), again.flat()):
        assert np.array_equal(x, y)
    ctx.set_option("test_raise_device_error", 1)
    with pytest.raises(sb.ScriptrsError) as e:
        pipe.run(audio[:100_000])
    assert e.value.status == 10
    ctx.synchronize()


def test_int16_recording_gives_the_f32_token_streams(ctx, pipe):
    """sb_transcribe_chunks_i16: the 16-bit recording crosses to the GPU as it is (half the bytes) and is converted
    inside the frontend kernel; the token streams must equal those of the f32 entry on the recording converted on the
    host as the reference's WAV reader does (value / 32767, examples/transcribe_wav.rs:341-347)."""
    import scriptrs_b200 as sb

    audio = synth.long_audio(700_000, 12)
    pcm16 = np.round(audio * 32767.0).astype(np.int16)
    pcm32 = pcm16.astype(np.float32) / np.float32(32767.0)
    tasks = sb.plan_fast(pcm16.size)
    a = sb.transcribe_chunks(ctx, pcm16, tasks)
    b = sb.transcribe_chunks(ctx, pcm32, tasks)
    assert sum(len(r.token_ids) for r in b) > 0
    for x, y in zip(a.flat(), b.flat()):
        assert np.array_equal(x, y)
    # many ordered tasks: the pieced copy path with 2-byte samples
    n_tasks, task_len, stride = 200, 4000, 3000
    long16 = np.round(synth.long_audio(stride * (n_tasks - 1) + task_len, 18) * 32767.0).astype(np.int16)
    many = [(i * stride, i * stride + task_len, i * stride, 0) for i in range(n_tasks)]
    a = sb.transcribe_chunks(ctx, long16, many)
    b = sb.transcribe_chunks(ctx, long16.astype(np.float32) / np.float32(32767.0), many)
    for x, y in zip(a.flat(), b.flat()):
        assert np.array_equal(x, y)


def test_longform_run_multi_on_two_gpus(ctx, pipe):
    """The same entry with one context per GPU (what a host crate binds for a multi-GPU box); skipped on a
    single-GPU machine."""
    import scriptrs_b200 as sb

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    second = sb.Context(1)
    try:
        sb.load_model(second, model_weights(), LAYERS, has_encoder=True, has_decoder=True)
        audio = synth.long_audio(1_100_000, 8)
        one = sb.LongFormTranscriptionPipeline(pipe).run(audio)
        two = sb.LongFormTranscriptionPipeline(pipe, extra_contexts=[second]).run_with_config(
            audio, sb.LongFormConfig(worker_count=2))
        assert two.text == one.text and two.tokens == one.tokens and two.chunks == one.chunks
        assert second.kernel_launches() > 0
    finally:
        second.close()
