"""Golden vectors (tests/golden/golden.npz, written by tests/golden/make_golden.py from the CPU oracle).

CPU: the oracle still reproduces them.  GPU: the CUDA frontend and both decoders' decision logic match them."""
import os

import numpy as np
import pytest

import oracle
from scriptrs_b200 import synth

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))
CLIPS = {"tone_1s": (16000, 11, False), "tone_ragged_4321": (4321, 12, False), "silent_10s": (160000, 13, True)}


def clip(name):
    n, seed, silent = CLIPS[name]
    assert int(GOLD[name + "_len"]) == n and int(GOLD[name + "_audio_seed"]) == seed
    return synth.clip_audio(n, seed=seed, silent=silent)


@pytest.mark.parametrize("name", list(CLIPS))
def test_oracle_frontend_reproduces_golden(name):
    feats = oracle.frontend_extract(clip(name))
    gold = GOLD[name]
    if name.startswith("silent"):
        assert np.all(feats == gold[0, 0])  # bit-exact constant (sequential f32 column sums)
    else:
        assert feats.shape == gold.shape
        assert np.array_equal(feats, gold)


def test_oracle_replay_reproduces_golden():
    rep = oracle.greedy_replay(GOLD["replay_logits"], time_steps=int(GOLD["replay_time_steps"]))
    assert rep["steps"] == GOLD["replay_logits"].shape[0]
    assert np.array_equal(rep["tokens"], GOLD["replay_tokens"])
    assert np.array_equal(rep["frames"], GOLD["replay_frames"])
    assert np.array_equal(rep["durations"], GOLD["replay_durations"])
    assert np.allclose(rep["conf"], GOLD["replay_conf"], rtol=1e-6)
    assert len(rep["tokens"]) > 5 and (GOLD["replay_durations"] > 0).any()


def test_planner_golden_host_library():
    """The product's C++ planner (host code of the shared library) against the frozen plans."""
    import scriptrs_b200 as sb

    for n, count, s0, e0, sl, el in GOLD["planner_cases"]:
        plan = sb.plan_fast(int(n))
        assert len(plan) == count
        assert (plan[0][0], plan[0][1], plan[-1][0], plan[-1][1]) == (s0, e0, sl, el)


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(CLIPS))
def test_cuda_frontend_matches_golden(ctx, name):
    import scriptrs_b200 as sb

    fx = sb.ParakeetFeatureExtractor(ctx)
    feats = fx.extract(clip(name))
    gold = GOLD[name]
    if name.startswith("silent"):
        assert np.all(feats == gold[0, 0])
    else:
        assert np.linalg.norm(feats - gold) / np.linalg.norm(gold) <= 1e-4
        assert np.abs(feats - gold).max() <= 1e-4 * np.abs(gold).max()


# ---------------------------------------------------------------- VAD mode
def _vad_golden():
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_vad.npz"))


def test_oracle_vad_reproduces_golden():
    from oracle import vad_oracle as vo
    from scriptrs_b200 import synth

    g = _vad_golden()
    audio = synth.sparse_speech_audio(int(g["vad_audio_len"]), int(g["vad_audio_seed"]), speech_seconds=(1.0, 3.0),
                                      silence_seconds=(0.3, 1.0))
    probs = vo.vad_probabilities(synth.seeded_vad_weights(int(g["vad_weights_seed"])), audio)
    assert np.abs(probs - g["vad_probabilities"]).max() < 1e-5   # BLAS summation order may differ between hosts
    regions = vo.detect_speech_regions(g["plan_track"], int(g["plan_audio_len"]), 0.85, vo.Segmentation())
    assert np.array_equal(np.array(regions, np.int64).reshape(-1, 2), g["plan_regions"])


def test_vad_plan_golden_host_library():
    import scriptrs_b200 as sb

    g = _vad_golden()
    regions = sb.detect_speech_regions(g["plan_track"], int(g["plan_audio_len"]))
    assert np.array_equal(np.array(regions, np.int64).reshape(-1, 2), g["plan_regions"])
    tasks, rts = sb.plan_vad(regions, g["plan_track"])
    assert np.array_equal(np.array(tasks, np.int64).reshape(-1, 4), g["plan_tasks"])
    assert np.array_equal(np.array(rts, np.int64).reshape(-1, 3), g["plan_region_tasks"])
    assert {int(k) for k in g["plan_region_tasks"][:, 0]} == {0, 1}


@pytest.mark.gpu
def test_cuda_vad_matches_golden(ctx):
    import scriptrs_b200 as sb
    from scriptrs_b200 import synth

    g = _vad_golden()
    audio = synth.sparse_speech_audio(int(g["vad_audio_len"]), int(g["vad_audio_seed"]), speech_seconds=(1.0, 3.0),
                                      silence_seconds=(0.3, 1.0))
    probs = sb.SileroVad(ctx, synth.seeded_vad_weights(int(g["vad_weights_seed"]))).process(audio)
    assert np.abs(probs - g["vad_probabilities"]).max() < 2e-4
