"""The voice-activity network and the VAD long-form mode on the GPU, through the C ABI.

The network is compared with the numpy oracle (float32; tolerance 2e-4 on the probabilities: the kernels sum
in another order and use the fast exponential); the VAD-mode pipeline must equal the composition of its parts:
probabilities -> the oracle's region detection and planning -> chunk transcription -> the region results."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

import oracle
from oracle import encoder_oracle as eo
from oracle import vad_oracle as vo
from scriptrs_b200 import synth

PROB_TOL = 2e-4
LAYERS = 2
VOCAB = [f"▁w{i}" if i % 3 == 0 else (str(i % 10) if i % 3 == 1 else chr(97 + i % 26)) for i in range(1024)] + ["<blk>"]


@pytest.fixture(scope="module")
def pipe(ctx):
    import scriptrs_b200 as sb

    w = eo.seeded_weights(eo.EncoderConfig(layers=LAYERS), seed=21, std=0.02, plain_norms=False)
    w.update(oracle.seeded_decoder_weights(22))
    return sb.TranscriptionPipeline.from_weights(w, sb.Vocabulary.from_tokens(VOCAB), encoder_layers=LAYERS, ctx=ctx)


@pytest.mark.parametrize("cluster", [8, 4])
def test_probabilities_match_the_oracle(ctx, cluster):
    import scriptrs_b200 as sb

    w = synth.seeded_vad_weights(5)
    vad = sb.SileroVad(ctx, w)
    ctx.set_option("vad_cluster", cluster)
    audio = synth.sparse_speech_audio(16000 * 40 + 137, 1)   # the last window holds 137 samples
    got = vad.process(audio)
    want = vo.vad_probabilities(w, audio)
    assert got.shape == want.shape == (1251,)
    assert np.abs(got - want).max() < PROB_TOL
    assert want.std() > 0.02  # the seeded network reacts to its input
    ctx.set_option("vad_cluster", 8)


def test_short_and_ragged_recordings(ctx):
    import scriptrs_b200 as sb

    w = synth.seeded_vad_weights(6)
    vad = sb.SileroVad(ctx, w)
    for n in (1, 63, 512, 513, 8191, 8192 + 64):
        audio = synth.clip_audio(n, 40 + n)
        got = vad.process(audio)
        want = vo.vad_probabilities(w, audio)
        assert got.shape == want.shape == (-(-n // 512),)
        assert np.abs(got - want).max() < PROB_TOL, n
    assert vad.process(np.zeros(0, np.float32)).size == 0     # vad.rs:65-67


def test_state_is_carried_between_passes(ctx):
    import scriptrs_b200 as sb

    w = synth.seeded_vad_weights(7)
    vad = sb.SileroVad(ctx, w)
    audio = synth.sparse_speech_audio(16000 * 25, 2)
    whole = vad.process(audio)
    ctx.set_option("vad_segment_windows", 100)                # 8 passes over 782 windows
    pieces = vad.process(audio)
    ctx.set_option("vad_segment_windows", 131072)
    assert np.array_equal(whole, pieces)
    again = vad.process(audio)                                # the state is reset at the start of every recording
    assert np.array_equal(whole, again)


def test_device_entry_point(ctx):
    import scriptrs_b200 as sb

    w = synth.seeded_vad_weights(5)
    vad = sb.SileroVad(ctx, w)
    audio = synth.sparse_speech_audio(16000 * 10, 3)
    d_audio = torch.from_numpy(audio).cuda()
    d_prob = torch.zeros(sb.vad_num_windows(audio.size), device="cuda")
    torch.cuda.synchronize()
    sb.check(sb.lib().sb_vad_process_device(ctx.handle, d_audio.data_ptr(), audio.size, d_prob.data_ptr()))
    ctx.synchronize()
    assert np.array_equal(d_prob.cpu().numpy(), vad.process(audio))


def test_missing_tensor_and_missing_network(ctx, pipe):
    import scriptrs_b200 as sb

    w = synth.seeded_vad_weights(5)
    del w["decoder.rnn.weight_hh"]
    with pytest.raises(sb.ScriptrsError) as e:
        sb.SileroVad(ctx, w)
    assert e.value.status == 3 and "decoder.rnn.weight_hh" in e.value.message
    fresh = sb.Context(0)
    try:
        with pytest.raises(sb.ScriptrsError) as e:                    # long_form.rs:194-199
            out = np.zeros(4, np.float32)
            n = sb._lib.C.c_int64()
            sb.check(sb.lib().sb_vad_process(fresh.handle, out.ctypes.data, 4, out.ctypes.data, 4, sb._lib.C.byref(n)))
        assert e.value.status == 3
    finally:
        fresh.close()


def test_device_side_timeout_flag_fails_the_network_call(ctx, pipe):
    """Host-side fault injection: the flag that the recurrence kernel raises when its bounded wait for the other
    thread blocks runs out makes sb_vad_process and the VAD mode fail with SB_TIMEOUT; the context stays usable."""
    import scriptrs_b200 as sb

    w = synth.seeded_vad_weights(5)
    vad = sb.SileroVad(ctx, w)
    audio = synth.sparse_speech_audio(16000 * 20, 3)
    good = vad.process(audio)
    ctx.set_option("test_raise_device_error", 1)
    with pytest.raises(sb.ScriptrsError) as e:
        vad.process(audio)
    assert e.value.status == 10
    assert np.array_equal(vad.process(audio), good)      # the flag was cleared by the failing call
    lf = sb.LongFormTranscriptionPipeline(pipe)
    ctx.set_option("test_raise_device_error", 1)
    with pytest.raises(sb.ScriptrsError) as e:
        lf.run_with_config(audio, sb.LongFormConfig(mode=sb.LongFormMode.Vad))
    assert e.value.status == 10
    ctx.synchronize()


def test_energy_detector_weights_find_the_sound(ctx):
    import scriptrs_b200 as sb

    w = synth.energy_vad_weights()
    vad = sb.SileroVad(ctx, w)
    audio = synth.sparse_speech_audio(16000 * 60, 4)
    got = vad.process(audio)
    want = vo.vad_probabilities(w, audio)
    assert np.abs(got - want).max() < PROB_TOL
    assert (got > 0.95).mean() > 0.3 and (got < 0.05).mean() > 0.1
    regions = sb.detect_speech_regions(got, audio.size)
    assert regions == vo.detect_speech_regions(want, audio.size, 0.85, vo.Segmentation()) and len(regions) >= 3


def by_hand(ctx, pipe, audio, probs, cfg):
    """The oracle's plan, the library's chunk transcription, the library's region results."""
    import scriptrs_b200 as sb

    regions = vo.detect_speech_regions(probs, audio.size, cfg.vad.default_threshold, vo.Segmentation())
    tasks, o_rts = vo.build_execution_plan(regions, probs, vo.Segmentation(), cfg.transcription.max_audio_samples)
    rts = [(k, idx[0], len(idx)) for k, idx in o_rts]
    wins = sb.transcribe_chunks(ctx, audio, tasks) if tasks else []
    return regions, tasks, rts, sb.longform_finish_regions(pipe.vocab, audio.size, tasks, rts, wins)


def same_result(a, b):
    assert a.text == b.text and a.duration_seconds == b.duration_seconds
    assert [(c.start, c.end, c.text) for c in a.chunks] == [(c.start, c.end, c.text) for c in b.chunks]
    assert np.array_equal(a.token_ids, b.token_ids) and np.array_equal(a.starts, b.starts)
    assert np.array_equal(a.ends, b.ends) and np.array_equal(a.confidences, b.confidences)


def test_vad_mode_equals_its_parts(ctx, pipe):
    import scriptrs_b200 as sb

    vad = sb.SileroVad(ctx, synth.energy_vad_weights())
    audio = synth.sparse_speech_audio(16000 * 150, 5, speech_seconds=(2.0, 24.0))
    probs = vad.process(audio)
    cfg = sb.LongFormConfig(mode=sb.LongFormMode.Vad)
    regions, tasks, rts, want = by_hand(ctx, pipe, audio, probs, cfg)
    kinds = {k for k, _, _ in rts}
    assert kinds == {0, 1}, "the recording should hold short regions and one longer than a chunk without a silence"
    lf = sb.LongFormTranscriptionPipeline(pipe)
    got = lf.run_with_config(audio, cfg)
    same_result(got, want)
    same_result(lf.run_with_probabilities(audio, probs, cfg), want)
    assert len(got.chunks) <= len(regions) and len(got.token_ids) > 0
    # the run above overlapped the network's passes with the transcription; all of the network first must give the
    # same, and so must short passes (many pieces) with the decoder run in rounds
    ctx.set_option("vad_unstreamed", 1)
    same_result(lf.run_with_config(audio, cfg), want)
    ctx.set_option("vad_unstreamed", 0)
    ctx.set_option("vad_segment_windows", 700)
    ctx.set_option("vad_rows_cap", 1500)
    same_result(lf.run_with_config(audio, cfg), want)
    ctx.set_option("vad_segment_windows", 131072)
    ctx.set_option("vad_rows_cap", 0)
    # chunks are in recording order and inside their regions (with the padding the planner added)
    starts = [c.start for c in got.chunks]
    assert starts == sorted(starts)
    # the Fast mode on the same recording transcribes the silences too: more tasks, another result
    fast = lf.run_with_config(audio, sb.LongFormConfig())
    assert len(fast.chunks) == 1


def test_vad_mode_with_silence_splits(ctx, pipe):
    import scriptrs_b200 as sb

    # probabilities from the caller: one 41 s region with three dips shorter than min_silence_duration, so the
    # region stays whole and is cut at the dips (Segments), not windowed
    n = 16000 * 50
    audio = synth.long_audio(n, 8)
    probs = np.full(sb.vad_num_windows(n), 0.95, np.float32)
    probs[:60] = 0.01
    probs[400:410] = 0.05
    probs[800:812] = 0.05
    probs[1150:1160] = 0.05
    probs[1350:] = 0.01
    cfg = sb.LongFormConfig(mode=sb.LongFormMode.Vad)
    regions, tasks, rts, want = by_hand(ctx, pipe, audio, probs, cfg)
    assert len(regions) == 1 and rts == [(1, 0, 4)]
    got = sb.LongFormTranscriptionPipeline(pipe).run_with_probabilities(audio, probs, cfg)
    same_result(got, want)
    assert len(got.chunks) == 1


def test_vad_mode_without_speech_gives_the_empty_result(ctx, pipe):
    import scriptrs_b200 as sb

    n = 16000 * 20
    audio = synth.long_audio(n, 9)
    lf = sb.LongFormTranscriptionPipeline(pipe)
    r = lf.run_with_probabilities(audio, np.full(sb.vad_num_windows(n), 0.1, np.float32),
                                  sb.LongFormConfig(mode=sb.LongFormMode.Vad))
    assert r.text == "" and r.chunks == [] and len(r.token_ids) == 0 and r.duration_seconds == 20.0
    # audio of at most one chunk takes the single-chunk path whatever the mode (long_form.rs:161-163)
    short = audio[:100_000]
    a = lf.run_with_probabilities(short, np.zeros(sb.vad_num_windows(short.size), np.float32),
                                  sb.LongFormConfig(mode=sb.LongFormMode.Vad))
    same_result(a, pipe.run(short))


def test_vad_mode_needs_the_network(pipe):
    import scriptrs_b200 as sb

    fresh = sb.Context(0)
    try:
        w = eo.seeded_weights(eo.EncoderConfig(layers=1), seed=21, std=0.02, plain_norms=False)
        w.update(oracle.seeded_decoder_weights(22))
        p = sb.TranscriptionPipeline.from_weights(w, sb.Vocabulary.from_tokens(VOCAB), encoder_layers=1, ctx=fresh)
        lf = sb.LongFormTranscriptionPipeline(p)
        with pytest.raises(sb.ScriptrsError) as e:
            lf.run_with_config(synth.long_audio(300_000, 1), sb.LongFormConfig(mode=sb.LongFormMode.Vad))
        assert e.value.status == 3                                     # MissingModelAsset, long_form.rs:194-199
    finally:
        fresh.close()


def test_vad_mode_with_two_contexts(ctx, pipe):
    """Mode 1 of sb_longform_run_multi with two contexts: the first runs the network, the region tasks are dealt to
    both (the first reads the recording it already holds on the GPU, the second its share from the host)."""
    import scriptrs_b200 as sb

    second = sb.Context(0)
    try:
        w = eo.seeded_weights(eo.EncoderConfig(layers=LAYERS), seed=21, std=0.02, plain_norms=False)
        w.update(oracle.seeded_decoder_weights(22))
        sb.load_model(second, w, LAYERS, has_encoder=True, has_decoder=True)
        sb.SileroVad(ctx, synth.energy_vad_weights())
        audio = synth.sparse_speech_audio(16000 * 120, 6, speech_seconds=(2.0, 24.0))
        cfg = sb.LongFormConfig(mode=sb.LongFormMode.Vad)
        one = sb.LongFormTranscriptionPipeline(pipe).run_with_config(audio, cfg)
        both = sb.LongFormTranscriptionPipeline(pipe, extra_contexts=[second])
        k0 = second.kernel_launches()
        two = both.run_with_config(audio, cfg)
        same_result(two, one)
        assert second.kernel_launches() > k0 and len(one.token_ids) > 0
    finally:
        second.close()
