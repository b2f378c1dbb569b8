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


def vad_cases():
    """The voice-activity network's oracle on a short seeded recording, and the planner on a fixed probability track
    (written to their own file so that the other vectors stay byte for byte what they were)."""
    from oracle import vad_oracle as vo

    w = synth.seeded_vad_weights(5)
    audio = synth.sparse_speech_audio(16000 * 8 + 77, 31, speech_seconds=(1.0, 3.0), silence_seconds=(0.3, 1.0))
    probs = vo.vad_probabilities(w, audio)
    rng = np.random.default_rng(77)
    track = np.clip(np.repeat(rng.choice([0.02, 0.5, 0.95], 60, p=[0.3, 0.1, 0.6]), 25) + rng.normal(0, 0.03, 1500), 0, 1)
    track[200:800] = np.clip(0.95 + rng.normal(0, 0.02, 600), 0, 1)  # 19 s without a silence: overlap windows
    track = track.astype(np.float32)
    n = 1500 * 512 - 100
    regions = vo.detect_speech_regions(track, n, 0.85, vo.Segmentation())
    tasks, rts = vo.build_execution_plan(regions, track, vo.Segmentation(), 240_000)
    return {
        "vad_weights_seed": np.array(5, np.int64), "vad_audio_seed": np.array(31, np.int64),
        "vad_audio_len": np.array(audio.size, np.int64), "vad_probabilities": probs.astype(np.float32),
        "plan_track": track, "plan_audio_len": np.array(n, np.int64),
        "plan_regions": np.array(regions, np.int64).reshape(-1, 2), "plan_tasks": np.array(tasks, np.int64).reshape(-1, 4),
        "plan_region_tasks": np.array([(k, idx[0], len(idx)) for k, idx in rts], np.int64).reshape(-1, 3),
    }


def main():
    vad = vad_cases()
    vpath = os.path.join(HERE, "golden_vad.npz")
    np.savez_compressed(vpath, **vad)
    print("wrote", vpath, os.path.getsize(vpath), "bytes;", ", ".join(sorted(vad)))
    if "--vad-only" in sys.argv:
        return
    blob = {}
    blob.update(frontend_cases())
    blob.update(decode_case())
    blob.update(planner_cases())
    path = os.path.join(HERE, "golden.npz")
    np.savez_compressed(path, **blob)
    print("wrote", path, os.path.getsize(path), "bytes;", ", ".join(sorted(blob)))


if __name__ == "__main__":
    main()
