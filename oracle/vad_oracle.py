"""CPU oracle for the VAD long-form mode.  TEST INFRASTRUCTURE ONLY: never imported by the product package.

Two parts:

* the planner, a literal pure-Python restatement of the reference's logic
    VadSegmentationConfig defaults / effective_negative_threshold   src/long_form/planner.rs:52-80
    detect_speech_regions                                           src/long_form/planner.rs:139-233
    region_probability_slice                                        src/long_form/planner.rs:235-240
    plan_region_subsegments / silence_spans                         src/long_form/planner.rs:242-315
    build_region_plan / push_segment_task / push_overlap_task       src/long_form.rs:508-582
    build_parallel_result / decode_segment_tasks / offset_token     src/long_form.rs:344-419,649-661
  pinned by the reference's known-answer tests (planner.rs:324-374, long_form.rs:682-736), which
  tests/test_oracle_vad.py replays;

* the voice-activity network, numpy float32: the streaming loop of process_coreml_vad
  (src/long_form/vad.rs:61-98: 512-sample windows, 64 samples of context, last window filled with its last
  sample, zero initial state) around the public Silero VAD (16 kHz) network shape.  The reference keeps the
  network in a CoreML file that is not part of its repository, so the network arithmetic is PARITY UNPINNED:
  there is no golden output to check it against, only the I/O contract of src/coreml.rs:188-236 (and an independent
  implementation of the same layers with torch, tests/test_oracle_vad.py).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

SAMPLE_RATE = 16000
VAD_WINDOW_SAMPLES = 512
VAD_CONTEXT_SAMPLES = 64
VAD_STATE_SIZE = 128
MEL_HOP_SAMPLES = 160
SAMPLES_PER_ENCODER_FRAME = 1280
MAX_MODEL_SAMPLES = 240_000

f32 = np.float32


@dataclass
class Segmentation:
    min_speech_duration: float = 0.15
    min_silence_duration: float = 0.75
    max_speech_duration: float = 14.0
    speech_padding: float = 0.1
    silence_threshold_for_split: float = 0.3
    negative_threshold: float | None = None
    negative_threshold_offset: float = 0.15
    min_silence_at_max_speech: float = 0.098
    use_max_possible_silence_at_max_speech: bool = True

    def effective_negative_threshold(self, base: float) -> np.float32:
        if self.negative_threshold is not None:
            return f32(self.negative_threshold)
        return max(f32(base) - f32(self.negative_threshold_offset), f32(0.01))


def _as_usize(x: float) -> int:
    """Rust's `f64 as usize`: truncation towards zero, saturating, NaN -> 0."""
    if math.isnan(x) or x <= 0.0:
        return 0
    return int(min(x, 2.0 ** 63))


def _sat_sub(a: int, b: int) -> int:
    return a - b if a > b else 0


def detect_speech_regions(probabilities, audio_length_samples: int, threshold: float, config: Segmentation):
    probabilities = [f32(p) for p in probabilities]
    if not probabilities or audio_length_samples == 0:
        return []
    hop = VAD_WINDOW_SAMPLES
    min_speech = _as_usize(config.min_speech_duration * float(SAMPLE_RATE))
    min_silence = _as_usize(config.min_silence_duration * float(SAMPLE_RATE))
    pad = _as_usize(config.speech_padding * float(SAMPLE_RATE))
    threshold = f32(threshold)
    negative = config.effective_negative_threshold(threshold)

    triggered = False
    current_start = 0
    temp_end = None
    speeches = []
    for index, p in enumerate(probabilities):
        frame_start = index * hop
        if p >= threshold:
            temp_end = None
            if not triggered:
                triggered = True
                current_start = frame_start
            continue
        if p < negative and triggered:
            if temp_end is None:
                temp_end = frame_start
            if temp_end is not None and _sat_sub(frame_start, temp_end) >= min_silence:
                if _sat_sub(temp_end, current_start) >= min_speech:
                    speeches.append([current_start, temp_end])
                triggered = False
                temp_end = None
    if triggered and _sat_sub(audio_length_samples, current_start) >= min_speech:
        speeches.append([current_start, audio_length_samples])
    if not speeches:
        return []
    adj = speeches
    for i in range(len(adj)):
        if i == 0:
            adj[i][0] = _sat_sub(adj[i][0], pad)
        if i < len(adj) - 1:
            silence = _sat_sub(adj[i + 1][0], adj[i][1])
            if silence < 2 * pad:
                half = silence // 2
                adj[i][1] = min(adj[i][1] + half, audio_length_samples)
                adj[i + 1][0] = _sat_sub(adj[i + 1][0], half)
            else:
                adj[i][1] = min(adj[i][1] + pad, audio_length_samples)
                adj[i + 1][0] = _sat_sub(adj[i + 1][0], pad)
        else:
            adj[i][1] = min(adj[i][1] + pad, audio_length_samples)
    return [(a, b) for a, b in adj if b > a]


def region_probability_slice(probabilities, region):
    a = region[0] // VAD_WINDOW_SAMPLES
    b = -(-region[1] // VAD_WINDOW_SAMPLES)
    n = len(probabilities)
    return probabilities[min(a, n):min(b, n)]


def silence_spans(region, region_probabilities, threshold):
    first = region[0] // VAD_WINDOW_SAMPLES
    spans = []
    start = None
    for index, p in enumerate(region_probabilities):
        sample_start = (first + index) * VAD_WINDOW_SAMPLES
        if f32(p) <= f32(threshold):
            if start is None:
                start = sample_start
            continue
        if start is not None:
            spans.append((max(start, region[0]), min(sample_start, region[1])))
            start = None
    if start is not None:
        spans.append((max(start, region[0]), region[1]))
    return spans


def plan_region_subsegments(region, region_probabilities, config: Segmentation, max_chunk_samples: int):
    if _sat_sub(region[1], region[0]) <= max_chunk_samples:
        return [tuple(region)]
    min_silence = _as_usize(config.min_silence_at_max_speech * float(SAMPLE_RATE))
    spans = [s for s in silence_spans(region, region_probabilities, config.silence_threshold_for_split)
             if _sat_sub(s[1], s[0]) >= min_silence]
    segments = []
    cursor = region[0]
    while _sat_sub(region[1], cursor) > max_chunk_samples:
        search_end = cursor + max_chunk_samples
        best = None
        for s in spans:  # Iterator::max_by_key returns the last maximum
            if s[0] > cursor and s[0] < search_end:
                if best is None or _sat_sub(s[1], s[0]) >= _sat_sub(best[1], best[0]):
                    best = s
        if best is None:
            return None
        segments.append((cursor, best[0]))
        cursor = best[1]
    if cursor < region[1]:
        segments.append((cursor, region[1]))
    return segments


def overlap_chunk_samples(context_samples=SAMPLES_PER_ENCODER_FRAME, max_model_samples=MAX_MODEL_SAMPLES):
    raw = max(_sat_sub(_sat_sub(max_model_samples, context_samples), MEL_HOP_SAMPLES), SAMPLES_PER_ENCODER_FRAME)
    return raw // SAMPLES_PER_ENCODER_FRAME * SAMPLES_PER_ENCODER_FRAME


def overlap_stride_samples(overlap_seconds=2.0, context_samples=SAMPLES_PER_ENCODER_FRAME,
                           max_model_samples=MAX_MODEL_SAMPLES):
    chunk = overlap_chunk_samples(context_samples, max_model_samples)
    requested = _as_usize(overlap_seconds * float(SAMPLE_RATE))
    overlap = min(requested, chunk // 2) // SAMPLES_PER_ENCODER_FRAME * SAMPLES_PER_ENCODER_FRAME
    return max(_sat_sub(chunk, overlap), SAMPLES_PER_ENCODER_FRAME) // SAMPLES_PER_ENCODER_FRAME * SAMPLES_PER_ENCODER_FRAME


def overlap_plan(region, overlap_seconds=2.0, context_samples=SAMPLES_PER_ENCODER_FRAME,
                 max_model_samples=MAX_MODEL_SAMPLES):
    chunk = overlap_chunk_samples(context_samples, max_model_samples)
    stride = overlap_stride_samples(overlap_seconds, context_samples, max_model_samples)
    chunks = []
    start = region[0]
    while start < region[1]:
        end = min(start + chunk, region[1])
        chunks.append((start, end))
        if end == region[1]:
            break
        start += stride
    return chunks


SEGMENTS, OVERLAP = 1, 0


def build_region_plan(region, probabilities, segmentation: Segmentation, max_audio_samples: int, tasks: list,
                      overlap_seconds=2.0, context_samples=SAMPLES_PER_ENCODER_FRAME,
                      max_model_samples=MAX_MODEL_SAMPLES):
    """Appends (audio_start, audio_end, global_sample_offset, context_samples) tuples to `tasks`; returns
    (kind, task_indices)."""
    def push_segment(seg):
        tasks.append((seg[0], seg[1], 0, 0))
        return len(tasks) - 1

    def push_overlap(chunk):
        context_start = _sat_sub(chunk[0], context_samples)
        tasks.append((context_start, chunk[1], chunk[0], chunk[0] - context_start))
        return len(tasks) - 1

    if _sat_sub(region[1], region[0]) <= max_audio_samples:
        return SEGMENTS, [push_segment(region)]
    sub = plan_region_subsegments(region, region_probability_slice(probabilities, region), segmentation,
                                  max_audio_samples)
    if sub is not None:
        return SEGMENTS, [push_segment(s) for s in sub]
    return OVERLAP, [push_overlap(c) for c in overlap_plan(region, overlap_seconds, context_samples, max_model_samples)]


def build_execution_plan(regions, probabilities, segmentation: Segmentation, max_audio_samples: int = MAX_MODEL_SAMPLES,
                         **overlap_kw):
    tasks = []
    region_tasks = [build_region_plan(r, probabilities, segmentation, max_audio_samples, tasks, **overlap_kw)
                    for r in regions]
    return tasks, region_tasks


# ---------------------------------------------------------------------------- network
def _conv1d_relu(x, w, b, stride):
    """x [N, Cin, T], w [Cout, Cin, 3], padding 1."""
    n, cin, t = x.shape
    xp = np.zeros((n, cin, t + 2), f32)
    xp[:, :, 1:-1] = x
    t_out = (t + 2 - 3) // stride + 1
    cols = np.stack([xp[:, :, k:k + stride * (t_out - 1) + 1:stride] for k in range(3)], axis=2)  # [N, Cin, 3, T']
    y = np.einsum("nckt,ock->not", cols, w.astype(f32), dtype=f32, optimize=False) + b.astype(f32)[None, :, None]
    return np.maximum(y, f32(0)).astype(f32)


def _sigmoid(x):
    return (f32(1) / (f32(1) + np.exp(-x.astype(f32)))).astype(f32)


def vad_window_inputs(audio: np.ndarray) -> np.ndarray:
    """[W, 576] model inputs of process_coreml_vad (vad.rs:78-93)."""
    audio = np.asarray(audio, f32)
    n = audio.size
    w = -(-n // VAD_WINDOW_SAMPLES)
    chunks = np.empty((w, VAD_WINDOW_SAMPLES), f32)
    for i in range(w):
        c = audio[i * VAD_WINDOW_SAMPLES:(i + 1) * VAD_WINDOW_SAMPLES]
        chunks[i, :c.size] = c
        if c.size < VAD_WINDOW_SAMPLES:
            chunks[i, c.size:] = c[-1]
    ctx = np.zeros((w, VAD_CONTEXT_SAMPLES), f32)
    ctx[1:] = chunks[:-1, VAD_WINDOW_SAMPLES - VAD_CONTEXT_SAMPLES:]
    return np.concatenate([ctx, chunks], axis=1)


def vad_encode(weights: dict, x: np.ndarray) -> np.ndarray:
    """[W, 576] -> [W, 128]: reflect padding, |STFT| (256-tap basis, stride 128), four ReLU convolutions."""
    xp = np.concatenate([x, x[:, -2:-66:-1]], axis=1)  # 64 reflected samples, edge not repeated
    basis = weights["stft.forward_basis_buffer"].reshape(258, 256).astype(f32)
    frames = np.stack([xp[:, 128 * t:128 * t + 256] for t in range(4)], axis=1)  # [W, 4, 256]
    spec = np.einsum("wtn,cn->wct", frames, basis, dtype=f32)
    mag = np.sqrt(spec[:, :129] ** 2 + spec[:, 129:] ** 2).astype(f32)
    y = mag
    for i, stride in enumerate((1, 2, 2, 1)):
        y = _conv1d_relu(y, weights[f"encoder.{i}.reparam_conv.weight"], weights[f"encoder.{i}.reparam_conv.bias"], stride)
    assert y.shape[1:] == (128, 1)
    return y[:, :, 0]


def vad_probabilities(weights: dict, audio: np.ndarray, return_state: bool = False):
    """One probability per 512-sample window (vad.rs:61-98)."""
    audio = np.asarray(audio, f32)
    if audio.size == 0:
        return np.zeros(0, f32)
    e = vad_encode(weights, vad_window_inputs(audio))
    w_ih = weights["decoder.rnn.weight_ih"].astype(f32)
    w_hh = weights["decoder.rnn.weight_hh"].astype(f32)
    bias = (weights["decoder.rnn.bias_ih"].astype(f32) + weights["decoder.rnn.bias_hh"].astype(f32)).astype(f32)
    w_out = weights["decoder.decoder.2.weight"].reshape(128).astype(f32)
    b_out = f32(weights["decoder.decoder.2.bias"].reshape(1)[0])
    gx = (e @ w_ih.T + bias).astype(f32)
    h = np.zeros(VAD_STATE_SIZE, f32)
    c = np.zeros(VAD_STATE_SIZE, f32)
    probs = np.empty(e.shape[0], f32)
    for s in range(e.shape[0]):
        g = (gx[s] + w_hh @ h).astype(f32)
        i, f, gg, o = _sigmoid(g[:128]), _sigmoid(g[128:256]), np.tanh(g[256:384]).astype(f32), _sigmoid(g[384:])
        c = (f * c + i * gg).astype(f32)
        h = (o * np.tanh(c)).astype(f32)
        probs[s] = _sigmoid(np.array([np.dot(np.maximum(h, f32(0)), w_out) + b_out], f32))[0]
    return (probs, h, c) if return_state else probs
