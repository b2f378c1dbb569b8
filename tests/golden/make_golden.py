"""Regenerates the golden vectors in this folder from the CPU oracle.

The reference (a Rust / CoreML crate) cannot be built or run where these tests run, and it ships no golden vectors
of its own for this path; what it does ship - the known-answer cases of its planner, merge and text tests - is
restated in tests/test_oracle_*.py.  The files written here freeze the oracle's output on small seeded inputs so
that (a) a change to the oracle shows up as a diff, and (b) the CUDA path can be checked against fixed numbers
without running the oracle.  Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle  # noqa: E402
from scriptrs_b200 import synth  # noqa: E402


def frontend_cases():
    clips = {
        "tone_1s": synth.clip_audio(16000, seed=11),
        "tone_ragged_4321": synth.clip_audio(4321, seed=12),
        "silent_10s": synth.clip_audio(160000, seed=13, silent=True),
    }
    out = {}
    for name, audio in clips.items():
        feats = oracle.frontend_extract(audio)
        if name.startswith("silent"):
            # every element of a silent clip is the same constant per clip length: keep one row
            assert np.all(feats == feats[0, 0])
            feats = feats[:1]
        out[name + "_audio_seed"] = np.array([11, 12, 13][list(clips).index(name)], np.int64)
        out[name + "_len"] = np.array(len(audio), np.int64)
        out[name] = feats.astype(np.float32)
    return out


def decode_case():
    rng = np.random.default_rng(2024)
    t = 40
    logits = rng.standard_normal((11 * t + 2, 1030)).astype(np.float32)
    # make blanks and long durations common enough that the walk ends with a mixed token stream
    logits[:, 1024] += 2.5
    rep = oracle.greedy_replay(logits, time_steps=t)
    n = rep["steps"]
    return {
        "replay_logits": logits[:n],
        "replay_time_steps": np.array(t, np.int64),
        "replay_tokens": np.asarray(rep["tokens"], np.int64),
        "replay_frames": np.asarray(rep["frames"], np.int64),
        "replay_durations": np.asarray(rep["durations"], np.int64),
        "replay_conf": np.asarray(rep["conf"], np.float32),
    }


def planner_cases():
    lens = [1, 238080, 240000, 240001, 444160, 460800000]
    rows = []
    for n in lens:
        plan = oracle.plan_fast(n)
        rows.append((n, len(plan), plan[0][0], plan[0][1], plan[-1][0], plan[-1][1]))
    return {"planner_cases": np.array(rows, np.int64)}


def main():
    blob = {}
    blob.update(frontend_cases())
    blob.update(decode_case())
    blob.update(planner_cases())
    path = os.path.join(HERE, "golden.npz")
    np.savez_compressed(path, **blob)
    print("wrote", path, os.path.getsize(path), "bytes;", ", ".join(sorted(blob)))


if __name__ == "__main__":
    main()
