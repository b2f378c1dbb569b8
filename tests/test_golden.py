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
