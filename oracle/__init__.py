"""CPU oracle: ctypes bindings over oracle/_build/liboracle.so.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this module;
it is used by tests/, by ``__graft_entry__.smoke()`` and by the CPU-baseline
leg of ``bench.py``.  Each wrapped function names the reference source it
restates in the C file that defines it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")
_lib = None

N_MELS = 128
N_BINS = 257


def build(force: bool = False) -> str:
    """Compile the C restatement with the Makefile beside it."""
    srcs = [os.path.join(_HERE, f) for f in ("frontend_oracle.c", "decode_oracle.c", "longform_oracle.c")]
    stale = force or not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in srcs
    )
    if stale:
        subprocess.run(["make", "-B", "-C", _HERE], check=True, capture_output=True)
    return _LIB_PATH


class ChunkTask(C.Structure):
    _fields_ = [
        ("audio_start", C.c_int64),
        ("audio_end", C.c_int64),
        ("global_sample_offset", C.c_int64),
        ("context_samples", C.c_int64),
    ]


class TdtWeights(C.Structure):
    _fields_ = [
        ("vocab", C.c_int32), ("n_dur", C.c_int32), ("blank", C.c_int32), ("hidden", C.c_int32),
        ("layers", C.c_int32), ("enc_dim", C.c_int32), ("joint_dim", C.c_int32), ("max_symbols", C.c_int32),
        ("embedding", C.c_void_p), ("w_ih", C.c_void_p), ("w_hh", C.c_void_p), ("b_ih", C.c_void_p),
        ("b_hh", C.c_void_p), ("w_enc", C.c_void_p), ("b_enc", C.c_void_p), ("w_pred", C.c_void_p),
        ("b_pred", C.c_void_p), ("w_out", C.c_void_p), ("b_out", C.c_void_p),
    ]


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.sbo_frontend_extract.restype = C.c_int64
        L.sbo_frontend_extract.argtypes = [C.c_void_p, C.c_int64, C.c_float, C.c_int, C.c_void_p, C.c_int64,
                                           C.c_void_p, C.c_void_p]
        L.sbo_frontend_batch.restype = C.c_int64
        L.sbo_frontend_batch.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_float, C.c_int, C.c_void_p]
        L.sbo_hann_window.argtypes = [C.c_void_p, C.c_int]
        L.sbo_mel_filterbank.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int]
        L.sbo_greedy_replay.restype = C.c_int64
        L.sbo_greedy_replay.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int,
                                        C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p,
                                        C.c_void_p, C.c_void_p]
        L.sbo_tdt_decode.restype = C.c_int64
        L.sbo_tdt_decode.argtypes = [C.POINTER(TdtWeights), C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p,
                                     C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p]
        for name in ("sbo_chunk_samples",):
            getattr(L, name).restype = C.c_int64
            getattr(L, name).argtypes = [C.c_int64, C.c_int64]
        for name in ("sbo_overlap_samples", "sbo_stride_samples"):
            getattr(L, name).restype = C.c_int64
            getattr(L, name).argtypes = [C.c_double, C.c_int64, C.c_int64]
        L.sbo_plan_fast.restype = C.c_int64
        L.sbo_plan_fast.argtypes = [C.c_int64, C.c_double, C.c_int64, C.c_int64, C.c_void_p, C.c_int64]
        L.sbo_parallel_worker_count.restype = C.c_int64
        L.sbo_parallel_worker_count.argtypes = [C.c_int64, C.c_int64]
        L.sbo_apply_time_offsets.restype = C.c_int64
        L.sbo_apply_time_offsets.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                             C.c_int64, C.c_int64]
        L.sbo_merge_windows.restype = C.c_int64
        L.sbo_merge_windows.argtypes = [C.c_void_p] * 5 + [C.c_int64] + [C.c_void_p] * 4 + [C.c_int64]
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


# ----------------------------------------------------------------- frontend
def hann_window(n: int = 400) -> np.ndarray:
    w = np.empty(n, np.float32)
    lib().sbo_hann_window(_p(w), n)
    return w


def mel_filterbank(n_fft: int = 512, n_mels: int = 128, sample_rate: int = 16000) -> np.ndarray:
    fb = np.empty((n_mels, n_fft // 2 + 1), np.float32)
    lib().sbo_mel_filterbank(_p(fb), n_fft, n_mels, sample_rate)
    return fb


def num_frames(n_samples: int) -> int:
    return n_samples // 160 + 1


def frontend_extract(audio: np.ndarray, preemph: float = 0.97, port_f32: bool = False,
                     want_raw: bool = False, want_power: bool = False):
    """Restatement of ParakeetFeatureExtractor::extract.  Returns feats [T,128]
    (and optionally the un-normalised log-mel [T,128] and the power [257,T])."""
    audio = np.ascontiguousarray(audio, np.float32)
    if audio.size == 0:
        raise ValueError("EmptyAudio")
    T = num_frames(audio.size)
    feats = np.empty((T, N_MELS), np.float32)
    raw = np.empty((T, N_MELS), np.float32) if want_raw else None
    power = np.empty((N_BINS, T), np.float32) if want_power else None
    r = lib().sbo_frontend_extract(_p(audio), audio.size, preemph, int(port_f32), _p(feats), T, _p(raw), _p(power))
    assert r == T, r
    out = [feats]
    if want_raw:
        out.append(raw)
    if want_power:
        out.append(power)
    return out[0] if len(out) == 1 else tuple(out)


def frontend_batch(audio: np.ndarray, port_f32: bool = True, preemph: float = 0.97) -> np.ndarray:
    """audio [n_clips, n] -> feats [n_clips, T, 128]."""
    audio = np.ascontiguousarray(audio, np.float32)
    n_clips, n = audio.shape
    T = num_frames(n)
    feats = np.empty((n_clips, T, N_MELS), np.float32)
    r = lib().sbo_frontend_batch(_p(audio), n, n_clips, preemph, int(port_f32), _p(feats))
    assert r == T, r
    return feats


# ------------------------------------------------------------------- decode
def greedy_replay(logits: np.ndarray, time_steps: int, vocab: int = 1025, n_dur: int = 5, blank: int = 1024,
                  max_symbols: int = 10):
    """Drive the reference's greedy state machine with recorded joint logits
    [n_steps, vocab+n_dur].  Returns dict(tokens, frames, durations, conf,
    steps, step_frame, step_ran_predictor)."""
    logits = np.ascontiguousarray(logits, np.float32).reshape(-1, vocab + n_dur)
    n_steps = logits.shape[0]
    cap = max(n_steps, 1)
    tok = np.zeros(cap, np.uint32)
    frm = np.zeros(cap, np.int64)
    dur = np.zeros(cap, np.int64)
    conf = np.zeros(cap, np.float32)
    used = np.zeros(1, np.int64)
    sf = np.zeros(cap, np.int32)
    sp = np.zeros(cap, np.int32)
    n = lib().sbo_greedy_replay(_p(logits), n_steps, time_steps, vocab, n_dur, blank, max_symbols, _p(tok),
                                _p(frm), _p(dur), _p(conf), cap, _p(used), _p(sf), _p(sp))
    if n < 0:
        raise RuntimeError(f"replay failed: {n}")
    s = int(used[0])
    return dict(tokens=tok[:n], frames=frm[:n], durations=dur[:n], conf=conf[:n], steps=s,
                step_frame=sf[:s], step_ran_predictor=sp[:s])


def make_tdt_weights(w: dict, max_symbols: int = 10):
    """w: dict of float32 arrays (embedding, w_ih, w_hh, b_ih, b_hh, w_enc, b_enc,
    w_pred, b_pred, w_out, b_out).  Returns (struct, keepalive)."""
    keep = {k: np.ascontiguousarray(v, np.float32) for k, v in w.items()}
    vocab, hidden = keep["embedding"].shape
    layers = keep["w_ih"].shape[0]
    joint, enc_dim = keep["w_enc"].shape
    width = keep["w_out"].shape[0]
    s = TdtWeights(vocab=vocab, n_dur=width - vocab, blank=vocab - 1, hidden=hidden, layers=layers,
                   enc_dim=enc_dim, joint_dim=joint, max_symbols=max_symbols)
    for k in ("embedding", "w_ih", "w_hh", "b_ih", "b_hh", "w_enc", "b_enc", "w_pred", "b_pred", "w_out", "b_out"):
        setattr(s, k, keep[k].ctypes.data)
    return s, keep


def tdt_decode(weights: dict, enc: np.ndarray, want_trace: bool = False, max_symbols: int = 10):
    """Full fp32 greedy decode of one sequence; enc is time-major [T', enc_dim]."""
    s, keep = make_tdt_weights(weights, max_symbols)
    enc = np.ascontiguousarray(enc, np.float32)
    T = enc.shape[0]
    cap = (max_symbols + 1) * max(T, 1)
    tok = np.zeros(cap, np.uint32)
    frm = np.zeros(cap, np.int64)
    dur = np.zeros(cap, np.int64)
    conf = np.zeros(cap, np.float32)
    used = np.zeros(1, np.int64)
    width = s.vocab + s.n_dur
    trace = np.zeros((cap, width), np.float32) if want_trace else None
    n = lib().sbo_tdt_decode(C.byref(s), _p(enc), T, _p(tok), _p(frm), _p(dur), _p(conf), cap, _p(trace), cap,
                             _p(used))
    if n < 0:
        raise RuntimeError(f"decode failed: {n}")
    out = dict(tokens=tok[:n], frames=frm[:n], durations=dur[:n], conf=conf[:n], steps=int(used[0]))
    if want_trace:
        out["logits"] = trace[: int(used[0])]
    return out


# ---------------------------------------------------------------- long form
def chunk_samples(context_samples=1280, max_model_samples=240000):
    return lib().sbo_chunk_samples(context_samples, max_model_samples)


def overlap_samples(overlap_seconds=2.0, context_samples=1280, max_model_samples=240000):
    return lib().sbo_overlap_samples(overlap_seconds, context_samples, max_model_samples)


def stride_samples(overlap_seconds=2.0, context_samples=1280, max_model_samples=240000):
    return lib().sbo_stride_samples(overlap_seconds, context_samples, max_model_samples)


def plan_fast(audio_len: int, overlap_seconds=2.0, context_samples=1280, max_model_samples=240000):
    """Returns a list of (audio_start, audio_end, global_sample_offset, context_samples)."""
    n = lib().sbo_plan_fast(audio_len, overlap_seconds, context_samples, max_model_samples, None, 0)
    arr = (ChunkTask * max(n, 1))()
    n2 = lib().sbo_plan_fast(audio_len, overlap_seconds, context_samples, max_model_samples, arr, n)
    assert n2 == n
    return [(t.audio_start, t.audio_end, t.global_sample_offset, t.context_samples) for t in arr[:n]]


def parallel_worker_count(task_count: int, requested: int) -> int:
    return lib().sbo_parallel_worker_count(task_count, requested)


def apply_time_offsets(tok, frm, dur, conf, frame_offset: int, context_frames: int):
    tok = np.array(tok, np.uint32)
    frm = np.array(frm, np.int64)
    dur = np.array(dur, np.int64)
    conf = np.array(conf, np.float32)
    n = lib().sbo_apply_time_offsets(_p(tok), _p(frm), _p(dur), _p(conf), tok.size, frame_offset, context_frames)
    return tok[:n], frm[:n], dur[:n], conf[:n]


def merge_windows(windows):
    """windows: list of (tokens, frames, durations, conf).  Literal left fold."""
    offs = np.zeros(len(windows) + 1, np.int64)
    for i, w in enumerate(windows):
        offs[i + 1] = offs[i] + len(w[0])
    total = int(offs[-1])
    cat = lambda k, dt: (np.concatenate([np.asarray(w[k], dt) for w in windows]) if windows and total
                         else np.zeros(0, dt))
    tok, frm, dur, conf = cat(0, np.uint32), cat(1, np.int64), cat(2, np.int64), cat(3, np.float32)
    cap = max(total, 1)
    otok, ofrm, odur, oconf = np.zeros(cap, np.uint32), np.zeros(cap, np.int64), np.zeros(cap, np.int64), np.zeros(cap, np.float32)
    n = lib().sbo_merge_windows(_p(tok), _p(frm), _p(dur), _p(conf), _p(offs), len(windows), _p(otok), _p(ofrm),
                                _p(odur), _p(oconf), cap)
    assert n >= 0, n
    return otok[:n], ofrm[:n], odur[:n], oconf[:n]


# -------------------------------------------------- seeded decoder weights (generated by scriptrs_b200.synth)
def seeded_decoder_weights(seed: int, std: float = 0.05) -> dict:
    """Config-3 predictor / joint weights: N(0, std) per tensor, named as the library's loader expects."""
    from scriptrs_b200 import synth

    return synth.seeded_decoder_weights(seed, std)


def tdt_weights_from_named(w: dict) -> dict:
    return dict(embedding=w["predictor.embedding"], w_ih=w["predictor.lstm.weight_ih"],
                w_hh=w["predictor.lstm.weight_hh"], b_ih=w["predictor.lstm.bias_ih"],
                b_hh=w["predictor.lstm.bias_hh"], w_enc=w["joint.enc.weight"], b_enc=w["joint.enc.bias"],
                w_pred=w["joint.pred.weight"], b_pred=w["joint.pred.bias"], w_out=w["joint.out.weight"],
                b_out=w["joint.out.bias"])
