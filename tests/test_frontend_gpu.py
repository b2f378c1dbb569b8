"""Parity of the CUDA frontend (through the C ABI) with the CPU oracle."""
import numpy as np
import pytest

import oracle
from scriptrs_b200 import synth

pytestmark = pytest.mark.gpu

REL_TOL = 1e-4  # per clip: ||gpu - ref||_2 / ||ref||_2 and max|gpu - ref| / max|ref|


def rel_errors(g, r):
    nrm = float(np.linalg.norm(g.astype(np.float64) - r) / max(np.linalg.norm(r.astype(np.float64)), 1e-30))
    peak = float(np.abs(g.astype(np.float64) - r).max() / max(np.abs(r).max(), 1e-30))
    return nrm, peak


@pytest.fixture(scope="module")
def fx(ctx):
    import scriptrs_b200 as sb

    return sb.ParakeetFeatureExtractor(ctx)


def test_tables_match_oracle(fx):
    import scriptrs_b200 as sb

    w, fb = sb.frontend_tables()
    assert np.array_equal(w, oracle.hann_window(400))
    assert np.array_equal(fb, oracle.mel_filterbank())


def test_config0_single_clip(fx):
    a = synth.clip_audio(160000, 0)
    g = fx.extract(a)
    r = oracle.frontend_extract(a)
    assert g.shape == (1001, 128)
    nrm, peak = rel_errors(g, r)
    assert nrm <= REL_TOL and peak <= REL_TOL, (nrm, peak)


def test_raw_logmel_before_normalisation(fx):
    a = synth.clip_audio(48000, 11)
    g = fx.extract(a, normalize=False)
    _, raw = oracle.frontend_extract(a, want_raw=True)
    nrm, peak = rel_errors(g, raw)
    assert nrm <= REL_TOL and peak <= REL_TOL, (nrm, peak)


def test_silent_clips_reproduce_the_sequential_sum_residue(fx):
    for n in (160000, 240000, 480000, 239360):
        z = np.zeros(n, np.float32)
        g = fx.extract(z)
        r = oracle.frontend_extract(z)
        assert np.array_equal(g, r), (n, g[0, 0], r[0, 0])


def test_config1_slice_with_silence(fx):
    clips = synth.clip_batch(12, 480000, base_seed=100)  # clip 3 is all-zero
    g = fx.extract_batch(list(clips))
    for i in range(12):
        r = oracle.frontend_extract(clips[i])
        assert g[i].shape == (3001, 128)
        nrm, peak = rel_errors(g[i], r)
        assert nrm <= REL_TOL and peak <= REL_TOL, (i, nrm, peak)


def test_ragged_batch_and_tiny_clips(fx):
    lens = [1, 100, 159, 160, 161, 399, 400, 511, 512, 513, 5119, 5120, 5121, 16000, 239360, 238080, 212480]
    clips = [synth.clip_audio(n, 1000 + n) for n in lens]
    g = fx.extract_batch(clips)
    for n, gi, c in zip(lens, g, clips):
        r = oracle.frontend_extract(c)
        assert gi.shape == r.shape == (n // 160 + 1, 128)
        if n < 160:
            assert np.isnan(gi).all() and np.isnan(r).all()
            continue
        # few frames: compare un-normalised values too (normalisation is ill-conditioned for T = 2, 3)
        if n >= 5119:
            nrm, peak = rel_errors(gi, r)
            assert nrm <= REL_TOL and peak <= REL_TOL, (n, nrm, peak)
    raw = fx.extract_batch(clips, normalize=False)
    for n, gi, c in zip(lens, raw, clips):
        _, r = oracle.frontend_extract(c, want_raw=True)
        nrm, peak = rel_errors(gi, r)
        assert nrm <= REL_TOL and peak <= REL_TOL, (n, nrm, peak)


def test_speech_with_silent_gaps(fx):
    a = synth.long_audio(239360, 7)
    g = fx.extract(a)
    r = oracle.frontend_extract(a)
    nrm, peak = rel_errors(g, r)
    assert nrm <= REL_TOL and peak <= REL_TOL, (nrm, peak)


def test_reference_property_tests_hold_on_gpu(fx):
    # src/frontend.rs:258-300 re-expressed against the CUDA path
    i = np.arange(16000, dtype=np.float32)
    s = np.sin(np.float32(2 * np.pi) * np.float32(440.0) * i / np.float32(16000)).astype(np.float32)
    f = fx.extract(s)
    assert f.shape == (101, 128)
    assert abs(float(f[:, 0].sum(dtype=np.float32) / np.float32(101))) <= 1e-4


def test_empty_audio_is_rejected(fx):
    import scriptrs_b200 as sb

    with pytest.raises(sb.ScriptrsError) as e:
        fx.extract(np.zeros(0, np.float32))
    assert e.value.status == 1


def _device_features(ctx, fx, pcm_np, offsets, int16=False):
    import torch

    import scriptrs_b200 as sb

    d_pcm = torch.from_numpy(pcm_np).cuda()
    rows = sum(sb.num_frames(int(offsets[i + 1] - offsets[i])) for i in range(len(offsets) - 1))
    d_out = torch.full((rows, 128), float("nan"), device="cuda")
    torch.cuda.synchronize()
    fo = fx.extract_device(d_pcm.data_ptr(), np.asarray(offsets, np.int64), d_out.data_ptr(), int16=int16)
    ctx.synchronize()
    out = d_out.cpu().numpy()
    return [out[fo[i]:fo[i + 1]] for i in range(len(offsets) - 1)]


def test_clip_placement_does_not_change_the_result(ctx, fx):
    """Clips that start at odd sample offsets of the PCM buffer take the 4-byte copy and unaligned load paths of the
    kernel; the features must equal, bit for bit, those of the same clips placed at the start of a buffer."""
    rng = np.random.default_rng(3)
    lens = [16001, 4999, 48002, 1, 161, 23998]
    offs = np.zeros(len(lens) + 1, np.int64)
    offs[1:] = np.cumsum(lens)
    assert {int(o) % 4 for o in offs[:-1]} == {0, 1, 2, 3}
    pcm = np.clip(rng.normal(0, 0.2, int(offs[-1])), -1, 1).astype(np.float32)
    packed = _device_features(ctx, fx, pcm, offs)
    for i, n in enumerate(lens):
        alone = _device_features(ctx, fx, pcm[offs[i]:offs[i + 1]].copy(), [0, n])[0]
        assert np.array_equal(packed[i], alone, equal_nan=True), (i, n)


def test_int16_pcm_equals_the_converted_f32_buffer(ctx, fx):
    """16-bit PCM in: the kernel converts each sample as value / 32767 in f32 (the reference's WAV reader,
    examples/transcribe_wav.rs:341-347); the features must equal those of the f32 path on the buffer converted on the
    host, bit for bit, for every clip placement (offsets 0 .. 7 modulo the 16-byte copy granule)."""
    rng = np.random.default_rng(4)
    lens = [16000, 4001, 48003, 239360, 7, 161, 23998, 5, 1602]
    offs = np.zeros(len(lens) + 1, np.int64)
    offs[1:] = np.cumsum(lens)
    assert len({int(o) % 8 for o in offs[:-1]}) >= 5
    pcm16 = rng.integers(-32768, 32768, int(offs[-1]), dtype=np.int16)
    pcm16[offs[3]:offs[3] + 120000] = 0                        # a long silent stretch
    pcm16[offs[0]], pcm16[offs[0] + 1] = -32768, 32767         # both extremes
    pcm32 = pcm16.astype(np.float32) / np.float32(32767.0)
    a = _device_features(ctx, fx, pcm16, offs, int16=True)
    b = _device_features(ctx, fx, pcm32, offs)
    for i in range(len(lens)):
        assert np.array_equal(a[i], b[i], equal_nan=True), i
    r = oracle.frontend_extract(pcm32[offs[2]:offs[3]])
    nrm, peak = rel_errors(a[2], r)
    assert nrm <= REL_TOL and peak <= REL_TOL, (nrm, peak)
