"""The C-ABI library loads without a GPU and exports every symbol the public header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "scriptrs_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(sb_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_every_declared_symbol_is_exported():
    import scriptrs_b200 as sb

    lib = ctypes.CDLL(sb.LIB_PATH)
    names = declared_functions()
    assert len(names) >= 10
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_python_signature_table_covers_the_header():
    from scriptrs_b200 import _lib

    assert sorted(_lib.SIGNATURES) == declared_functions()


def test_defaults_match_the_reference():
    # src/config.rs:30-43, src/long_form/planner.rs:94-102, src/long_form.rs:74-87
    from scriptrs_b200 import _lib

    L = _lib.lib()
    c = _lib.LongFormConfigC()
    L.sb_default_longform_config(ctypes.byref(c))
    assert (c.mode, c.worker_count) == (0, 4)
    t = c.transcription
    assert (t.sample_rate, t.feature_size, t.n_fft, t.win_length, t.hop_length) == (16000, 128, 512, 400, 160)
    assert abs(t.preemphasis - 0.97) < 1e-7
    assert (t.max_audio_samples, t.samples_per_encoder_frame) == (240000, 1280)
    assert (c.overlap.overlap_seconds, c.overlap.context_samples, c.overlap.max_model_samples) == (2.0, 1280, 240000)


def test_no_device_means_a_loud_failure_not_a_fallback():
    import scriptrs_b200 as sb

    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        pytest.skip("a GPU is present")
    with pytest.raises(sb.ScriptrsError) as e:
        sb.Context(0)
    assert e.value.status == 8


def test_frame_count_formula():
    import scriptrs_b200 as sb

    for n in (1, 159, 160, 161, 160000, 240000, 480000):
        assert sb.num_frames(n) == n // 160 + 1
