"""Pins the frontend oracle against the reference's own frontend tests
(src/frontend.rs:243-301) and against the facts its source implies."""
import numpy as np
import pytest

import oracle


def sine(freq, sr, n):
    i = np.arange(n, dtype=np.float32)
    return np.sin(np.float32(2.0) * np.float32(np.pi) * np.float32(freq) * i / np.float32(sr)).astype(np.float32)


def test_stft_concentrates_power_at_the_expected_bin():
    # frontend.rs:258-281
    _, power = oracle.frontend_extract(sine(1000.0, 16000, 16000), want_power=True)
    assert power.shape[0] == 257
    interior = power[:, 2:power.shape[1] - 2]
    assert int((interior.argmax(axis=0) == 32).sum()) > 90


def test_feature_extraction_produces_expected_shape():
    # frontend.rs:283-290
    f = oracle.frontend_extract(sine(440.0, 16000, 16000))
    assert f.shape[1] == 128 and f.shape[0] > 0
    assert f.shape[0] == 16000 // 160 + 1


def test_features_are_column_normalized():
    # frontend.rs:292-300
    f = oracle.frontend_extract(sine(440.0, 16000, 16000))
    col = f[:, 0]
    mean = np.float32(col.sum(dtype=np.float32) / np.float32(col.size))
    assert abs(float(mean)) <= 1e-4


def test_filterbank_structure():
    fb = oracle.mel_filterbank()
    nz = fb != 0
    assert fb.shape == (128, 257)
    assert int(nz.sum()) == 504
    assert nz.sum(axis=1).min() == 1 and nz.sum(axis=1).max() == 12
    assert not nz[:, 0].any() and not nz[:, 256].any()


def test_window_is_symmetric_periodic_minus_one():
    w = oracle.hann_window(400)
    assert w[0] == 0.0 and abs(w[399]) < 1e-6
    assert np.allclose(w, w[::-1], atol=1e-6)


def test_silent_clip_normalises_to_the_rounding_constant():
    # A constant column keeps only the rounding residue of the sequential f32 sum.
    for n, expect in ((160000, 0.9317), (240000, -0.9422), (480000, 0.9536)):
        f = oracle.frontend_extract(np.zeros(n, np.float32))
        assert f.min() == f.max()
        assert abs(float(f[0, 0]) - expect) < 1e-3


def test_single_frame_clip_is_nan_like_the_reference():
    # T = 1 divides by T - 1 = 0 (frontend.rs:235)
    f = oracle.frontend_extract(np.ones(100, np.float32) * 0.1)
    assert f.shape == (1, 128) and np.isnan(f).all()


def test_port_mode_stays_close_to_gold():
    from scriptrs_b200 import synth

    a = synth.clip_audio(32000, 5)
    g = oracle.frontend_extract(a)
    p = oracle.frontend_extract(a, port_f32=True)
    assert np.linalg.norm(g - p) / np.linalg.norm(g) < 1e-4


@pytest.mark.parametrize("n,seed", [(16000 * 2 + 123, 11), (4321, 12), (161, 13)])
def test_oracle_matches_library_stft_and_mel(n, seed):
    """The same features assembled from independent library pieces: torch.stft (with the reference's framing: 256
    zeros on either side, the 400-sample window at the START of each 512-sample frame, src/frontend.rs:121-147), the
    Slaney filterbank of transformers.audio_utils, numpy's log, mean and standard deviation (n - 1, + 1e-5)."""
    torch = pytest.importorskip("torch")
    mel_filter_bank = pytest.importorskip("transformers.audio_utils").mel_filter_bank
    from scriptrs_b200 import synth

    a = synth.clip_audio(n, seed)
    feats, raw, power = oracle.frontend_extract(a, want_raw=True, want_power=True)
    x = torch.from_numpy(a)
    pre = torch.cat([x[:1], x[1:] - 0.97 * x[:-1]]).double()
    padded = torch.cat([torch.zeros(256, dtype=torch.float64), pre, torch.zeros(256, dtype=torch.float64)])
    window = torch.cat([torch.from_numpy(oracle.hann_window(400)).double(), torch.zeros(112, dtype=torch.float64)])
    spec = torch.stft(padded, n_fft=512, hop_length=160, win_length=512, window=window, center=False, return_complex=True)
    p = (spec.real ** 2 + spec.imag ** 2).T.numpy()
    assert p.shape == power.T.shape
    assert np.abs(p - power.T).max() <= 1e-6 * np.abs(p).max()
    lib_fb = mel_filter_bank(257, 128, 0.0, 8000.0, 16000, norm="slaney", mel_scale="slaney")   # [257, 128]
    assert np.abs(lib_fb.T - oracle.mel_filterbank()).max() < 1e-8
    logmel = np.log(p @ lib_fb + 2.0 ** -24)
    assert np.abs(logmel - raw).max() < 2e-4          # f32 sums of 257 terms against f64
    norm = (logmel - logmel.mean(0)) / (logmel.std(0, ddof=1) + 1e-5)
    assert np.linalg.norm(norm - feats) <= 1e-5 * np.linalg.norm(feats)
