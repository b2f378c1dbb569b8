"""TranscriptionPipeline / LongFormTranscriptionPipeline: the reference's public API
(src/pipeline.rs:30-99, src/long_form.rs:100-174) over the C ABI.  No CPU fallback: every call
ends in libscriptrs_b200.so."""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field

import numpy as np

from . import _lib
from ._lib import ScriptrsError, check
from .api import Context, TranscriptionConfig, _ptr, load_model


@dataclass
class TimedToken:
    """src/types.rs:1-14"""
    token_id: int
    text: str
    start: float
    end: float
    confidence: float


@dataclass
class TranscriptChunk:
    """src/types.rs:16-26"""
    start: float
    end: float
    text: str


class TranscriptionResult:
    """src/types.rs:28-49.  Token fields are kept as arrays (token_ids, starts, ends, confidences, token
    texts); `.tokens` builds the list of TimedToken on first use."""

    def __init__(self, text, chunks, duration_seconds, token_ids, starts, ends, confidences, token_texts):
        self.text = text
        self.chunks = chunks
        self.duration_seconds = duration_seconds
        self.token_ids, self.starts, self.ends, self.confidences = token_ids, starts, ends, confidences
        self._token_texts = token_texts  # (utf-8 bytes, offsets)
        self._tokens = None

    def __len__(self):
        return len(self.token_ids)

    @property
    def tokens(self):
        if self._tokens is None:
            buf, off = self._token_texts
            self._tokens = [TimedToken(int(self.token_ids[i]), buf[off[i]:off[i + 1]].decode("utf-8"),
                                       float(self.starts[i]), float(self.ends[i]), float(self.confidences[i]))
                            for i in range(len(self.token_ids))]
        return self._tokens


@dataclass
class RawTranscription:
    """src/decode.rs:6-11"""
    token_ids: np.ndarray
    frame_indices: np.ndarray
    durations: np.ndarray
    confidences: np.ndarray


@dataclass
class OverlapChunkConfig:
    """src/long_form/planner.rs:84-102"""
    overlap_seconds: float = 2.0
    context_samples: int = 1280
    max_model_samples: int = 240_000

    def to_c(self):
        return _lib.OverlapConfigC(self.overlap_seconds, self.context_samples, self.max_model_samples)

    def chunk_samples(self) -> int:
        return int(_lib.lib().sb_overlap_chunk_samples(C.byref(self.to_c())))

    def overlap_samples(self) -> int:
        return int(_lib.lib().sb_overlap_overlap_samples(C.byref(self.to_c())))

    def stride_samples(self) -> int:
        return int(_lib.lib().sb_overlap_stride_samples(C.byref(self.to_c())))


class LongFormMode:
    """src/long_form.rs:89-98"""
    Fast = 0
    Vad = 1


@dataclass
class VadConfig:
    """src/long_form/planner.rs:11-27"""
    default_threshold: float = 0.85

    def to_c(self):
        return _lib.VadConfigC(self.default_threshold)


@dataclass
class VadSegmentationConfig:
    """src/long_form/planner.rs:29-81"""
    min_speech_duration: float = 0.15
    min_silence_duration: float = 0.75
    max_speech_duration: float = 14.0
    speech_padding: float = 0.1
    silence_threshold_for_split: float = 0.3
    negative_threshold: float | None = None
    negative_threshold_offset: float = 0.15
    min_silence_at_max_speech: float = 0.098
    use_max_possible_silence_at_max_speech: bool = True

    def threshold(self, default_threshold: float) -> float:
        return default_threshold

    def to_c(self):
        return _lib.VadSegmentationConfigC(
            self.min_speech_duration, self.min_silence_duration, self.max_speech_duration, self.speech_padding,
            self.silence_threshold_for_split, 0 if self.negative_threshold is None else 1,
            0.0 if self.negative_threshold is None else self.negative_threshold, self.negative_threshold_offset,
            self.min_silence_at_max_speech, 1 if self.use_max_possible_silence_at_max_speech else 0)


@dataclass
class LongFormConfig:
    """src/long_form.rs:56-87.  worker_count: parallel chunk workers; a worker is a GPU shard here."""
    mode: int = LongFormMode.Fast
    worker_count: int = 4
    transcription: TranscriptionConfig = field(default_factory=TranscriptionConfig)
    vad: VadConfig = field(default_factory=VadConfig)
    segmentation: VadSegmentationConfig = field(default_factory=VadSegmentationConfig)
    overlap: OverlapChunkConfig = field(default_factory=OverlapChunkConfig)

    def to_c(self):
        return _lib.LongFormConfigC(self.mode, self.worker_count, self.transcription.to_c(), self.vad.to_c(),
                                    self.segmentation.to_c(), self.overlap.to_c())


VAD_WINDOW_SAMPLES = 512  # src/constants.rs:7


def vad_num_windows(n_samples: int) -> int:
    return int(_lib.lib().sb_vad_num_windows(n_samples))


def detect_speech_regions(probabilities, audio_len: int, threshold: float = 0.85,
                          config: VadSegmentationConfig | None = None):
    """src/long_form/planner.rs:139-233: list of (start, end) sample ranges."""
    p = np.ascontiguousarray(probabilities, np.float32)
    sc = (config or VadSegmentationConfig()).to_c()
    n = C.c_int64()
    L = _lib.lib()
    check(L.sb_vad_detect_speech_regions(_ptr(p) if p.size else None, p.size, audio_len, threshold, C.byref(sc), None,
                                         0, C.byref(n)))
    arr = (_lib.SampleRangeC * max(n.value, 1))()
    check(L.sb_vad_detect_speech_regions(_ptr(p) if p.size else None, p.size, audio_len, threshold, C.byref(sc), arr,
                                         n.value, C.byref(n)))
    return [(r.start, r.end) for r in arr[: n.value]]


def plan_region_subsegments(region, region_probabilities, config: VadSegmentationConfig | None = None,
                            max_chunk_samples: int = 240_000):
    """src/long_form/planner.rs:242-284: list of (start, end), or None where no usable silence exists."""
    p = np.ascontiguousarray(region_probabilities, np.float32)
    sc = (config or VadSegmentationConfig()).to_c()
    rg = _lib.SampleRangeC(int(region[0]), int(region[1]))
    cap = p.size + 2
    arr = (_lib.SampleRangeC * cap)()
    n = C.c_int64()
    check(_lib.lib().sb_vad_plan_region_subsegments(C.byref(rg), _ptr(p) if p.size else None, p.size, C.byref(sc),
                                                    max_chunk_samples, arr, cap, C.byref(n)))
    if n.value < 0:
        return None
    return [(r.start, r.end) for r in arr[: n.value]]


def plan_vad(regions, probabilities, config: LongFormConfig | None = None):
    """build_execution_plan (src/long_form.rs:421-437,508-548): (tasks, region_tasks); a task is (audio_start,
    audio_end, global_sample_offset, context_samples), a region task (kind, first_task, n_tasks) with kind 0 =
    Overlap, 1 = Segments."""
    p = np.ascontiguousarray(probabilities, np.float32)
    lc = (config or LongFormConfig()).to_c()
    rg = (_lib.SampleRangeC * max(len(regions), 1))(*[_lib.SampleRangeC(int(a), int(b)) for a, b in regions])
    n = C.c_int64()
    L = _lib.lib()
    check(L.sb_plan_vad(C.byref(lc), rg, len(regions), _ptr(p) if p.size else None, p.size, None, 0, C.byref(n), None, 0))
    tasks = (_lib.ChunkTaskC * max(n.value, 1))()
    rts = (_lib.RegionTaskC * max(len(regions), 1))()
    check(L.sb_plan_vad(C.byref(lc), rg, len(regions), _ptr(p) if p.size else None, p.size, tasks, n.value, C.byref(n),
                        rts, len(regions)))
    return ([(t.audio_start, t.audio_end, t.global_sample_offset, t.context_samples) for t in tasks[: n.value]],
            [(r.kind, r.first_task, r.n_tasks) for r in rts[: len(regions)]])


def plan_fast(audio_len: int, overlap: OverlapChunkConfig | None = None):
    """build_fast_execution_plan: list of (audio_start, audio_end, global_sample_offset, context_samples)."""
    oc = (overlap or OverlapChunkConfig()).to_c()
    n = C.c_int64()
    check(_lib.lib().sb_plan_fast(C.byref(oc), audio_len, None, 0, C.byref(n)))
    arr = (_lib.ChunkTaskC * max(n.value, 1))()
    check(_lib.lib().sb_plan_fast(C.byref(oc), audio_len, arr, n.value, C.byref(n)))
    return [(t.audio_start, t.audio_end, t.global_sample_offset, t.context_samples) for t in arr[: n.value]]


def parallel_worker_count(task_count: int, requested: int) -> int:
    return int(_lib.lib().sb_parallel_worker_count(task_count, requested))


def apply_time_offsets(raw: RawTranscription, frame_offset: int, context_frames: int) -> RawTranscription:
    tok = np.array(raw.token_ids, np.uint32)
    frm = np.array(raw.frame_indices, np.int64)
    dur = np.array(raw.durations, np.int64)
    conf = np.array(raw.confidences, np.float32)
    n = C.c_int64()
    check(_lib.lib().sb_apply_time_offsets(_ptr(tok), _ptr(frm), _ptr(dur), _ptr(conf), tok.size, frame_offset,
                                           context_frames, C.byref(n)))
    k = n.value
    return RawTranscription(tok[:k], frm[:k], dur[:k], conf[:k])


class RawBatch:
    """Per-task token streams of one batch as flat arrays; behaves like a list of RawTranscription."""

    def __init__(self, offsets, token_ids, frame_indices, durations, confidences):
        self.offsets, self.token_ids, self.frame_indices = offsets, token_ids, frame_indices
        self.durations, self.confidences = durations, confidences

    def __len__(self):
        return len(self.offsets) - 1

    def __getitem__(self, i):
        if isinstance(i, slice):
            return [self[k] for k in range(*i.indices(len(self)))]
        if i < 0:
            i += len(self)
        a, b = int(self.offsets[i]), int(self.offsets[i + 1])
        return RawTranscription(self.token_ids[a:b], self.frame_indices[a:b], self.durations[a:b], self.confidences[a:b])

    def __iter__(self):
        return (self[i] for i in range(len(self)))

    def flat(self):
        return self.token_ids, self.frame_indices, self.durations, self.confidences, self.offsets

    @classmethod
    def concat(cls, parts):
        """Batches of consecutive task blocks -> one batch."""
        offs = [np.zeros(1, np.int64)]
        base = 0
        for p in parts:
            offs.append(p.offsets[1:] + base)
            base += int(p.offsets[-1])
        cat = lambda attr: np.concatenate([getattr(p, attr) for p in parts])
        return cls(np.concatenate(offs), cat("token_ids"), cat("frame_indices"), cat("durations"), cat("confidences"))


def _concat(windows):
    if isinstance(windows, RawBatch):
        t, f, d, c, o = windows.flat()
        return t, f, d, c, np.ascontiguousarray(o, np.int64), int(o[-1])
    offs = np.zeros(len(windows) + 1, np.int64)
    for i, w in enumerate(windows):
        offs[i + 1] = offs[i] + len(w.token_ids)
    total = int(offs[-1])

    def cat(attr, dt):
        return (np.concatenate([np.asarray(getattr(w, attr), dt) for w in windows]) if total else np.zeros(0, dt))

    return (cat("token_ids", np.uint32), cat("frame_indices", np.int64), cat("durations", np.int64),
            cat("confidences", np.float32), offs, total)


def merge_overlapping_windows(windows) -> RawTranscription:
    """src/long_form/merge.rs:3-13"""
    tok, frm, dur, conf, offs, total = _concat(windows)
    cap = max(total, 1)
    o = (np.zeros(cap, np.uint32), np.zeros(cap, np.int64), np.zeros(cap, np.int64), np.zeros(cap, np.float32))
    n = C.c_int64()
    check(_lib.lib().sb_merge_windows(_ptr(tok), _ptr(frm), _ptr(dur), _ptr(conf), _ptr(offs), len(windows),
                                      _ptr(o[0]), _ptr(o[1]), _ptr(o[2]), _ptr(o[3]), cap, C.byref(n)))
    k = n.value
    return RawTranscription(o[0][:k], o[1][:k], o[2][:k], o[3][:k])


class Vocabulary:
    """src/vocab.rs:9-61"""

    def __init__(self, handle):
        self._h = handle

    @classmethod
    def from_file(cls, path: str) -> "Vocabulary":
        h = C.c_void_p()
        check(_lib.lib().sb_vocab_load(os.fsencode(path), C.byref(h)))
        return cls(h)

    @classmethod
    def from_text(cls, text: str) -> "Vocabulary":
        b = text.encode("utf-8")
        h = C.c_void_p()
        check(_lib.lib().sb_vocab_from_text(b, len(b), C.byref(h)))
        return cls(h)

    @classmethod
    def from_tokens(cls, tokens) -> "Vocabulary":
        return cls.from_text("".join(f"{t} {i}\n" for i, t in enumerate(tokens)))

    def blank_id(self) -> int:
        return int(_lib.lib().sb_vocab_blank_id(self._h))

    def __len__(self):
        return int(_lib.lib().sb_vocab_size(self._h))

    def __del__(self):
        try:
            if self._h:
                _lib.lib().sb_vocab_free(self._h)
                self._h = None
        except Exception:
            pass


def _take_result(h) -> TranscriptionResult:
    L = _lib.lib()
    try:
        n = int(L.sb_result_num_tokens(h))
        ids, starts, ends = np.zeros(n, np.uint32), np.zeros(n, np.float64), np.zeros(n, np.float64)
        confs, offs = np.zeros(n, np.float32), np.zeros(n + 1, np.int64)
        need = C.c_int64()
        check(L.sb_result_tokens_bulk(h, None, None, None, None, None, None, 0, C.byref(need)))
        buf = C.create_string_buffer(max(need.value, 1))
        check(L.sb_result_tokens_bulk(h, _ptr(ids), _ptr(starts), _ptr(ends), _ptr(confs), _ptr(offs), buf,
                                      need.value, C.byref(need)))
        chunks = []
        for i in range(L.sb_result_num_chunks(h)):
            txt, a, b = C.c_char_p(), C.c_double(), C.c_double()
            check(L.sb_result_chunk(h, i, C.byref(a), C.byref(b), C.byref(txt)))
            chunks.append(TranscriptChunk(a.value, b.value, txt.value.decode("utf-8")))
        return TranscriptionResult(L.sb_result_text(h).decode("utf-8"), chunks, L.sb_result_duration(h), ids, starts,
                                   ends, confs, (buf.raw[: need.value], offs))
    finally:
        L.sb_result_free(h)


class ParakeetTdtDecoder:
    """src/decode.rs:29-104"""

    def __init__(self, vocab: Vocabulary):
        self.vocab = vocab

    def decode(self, raw: RawTranscription, duration_seconds: float) -> TranscriptionResult:
        tok = np.ascontiguousarray(raw.token_ids, np.uint32)
        frm = np.ascontiguousarray(raw.frame_indices, np.int64)
        conf = np.ascontiguousarray(raw.confidences, np.float32)
        h = C.c_void_p()
        check(_lib.lib().sb_text_decode(self.vocab._h, _ptr(tok), _ptr(frm), _ptr(conf), tok.size, conf.size,
                                        float(duration_seconds), C.byref(h)))
        return _take_result(h)


def _audio(a) -> np.ndarray:
    return np.ascontiguousarray(a, np.float32).reshape(-1)


def transcribe_chunks(ctx: Context, audio: np.ndarray, tasks, config: TranscriptionConfig | None = None,
                      audio_ptr: int | None = None, n_samples: int | None = None, on_device: bool = False,
                      sample_format: str = "float32"):
    """Batched transcribe_task for a list of (audio_start, audio_end, global_sample_offset, context_samples).
    Returns a RawBatch (a list-like of RawTranscription).  `audio_ptr`/`n_samples` let a caller pass pinned host memory, or,
    with on_device=True, a device pointer.  An int16 array (or sample_format="int16" with audio_ptr) is 16-bit PCM: it
    crosses to the GPU as it is and is converted (value / 32767) inside the frontend kernel."""
    int16 = False
    if audio_ptr is None:
        if isinstance(audio, np.ndarray) and audio.dtype == np.int16:
            audio = np.ascontiguousarray(audio).reshape(-1)   # 16-bit PCM goes to the GPU as it is
            int16 = True
        else:
            audio = _audio(audio)
        audio_ptr, n_samples = audio.ctypes.data, audio.size
    elif sample_format == "int16":
        int16 = True
    arr = (_lib.ChunkTaskC * max(len(tasks), 1))()
    for i, t in enumerate(tasks):
        arr[i] = _lib.ChunkTaskC(*[int(x) for x in t])
    cfg = (config or TranscriptionConfig()).to_c()
    h = C.c_void_p()
    if int16 and on_device:
        raise ScriptrsError(11, "16-bit PCM is taken from host memory")
    fn = (_lib.lib().sb_transcribe_chunks_device if on_device else
          (_lib.lib().sb_transcribe_chunks_i16 if int16 else _lib.lib().sb_transcribe_chunks))
    check(fn(ctx.handle, C.c_void_p(audio_ptr), n_samples, arr, len(tasks), C.byref(cfg), C.byref(h)))
    L = _lib.lib()
    try:
        n_items, total = int(L.sb_raw_batch_size(h)), int(L.sb_raw_batch_total(h))
        offs = np.zeros(n_items + 1, np.int64)
        tok, frm = np.zeros(total, np.uint32), np.zeros(total, np.int64)
        dur, conf = np.zeros(total, np.int64), np.zeros(total, np.float32)
        check(L.sb_raw_batch_flatten(h, _ptr(offs), _ptr(tok), _ptr(frm), _ptr(dur), _ptr(conf)))
    finally:
        L.sb_raw_batch_free(h)
    return RawBatch(offs, tok, frm, dur, conf)


def longform_finish(vocab: Vocabulary, audio_len: int, windows) -> TranscriptionResult:
    """Merge per-task token streams (task order), decode, build the long-form result."""
    tok, frm, dur, conf, offs, _ = _concat(windows)
    h = C.c_void_p()
    check(_lib.lib().sb_longform_finish(vocab._h, audio_len, _ptr(tok), _ptr(frm), _ptr(dur), _ptr(conf), _ptr(offs),
                                        len(windows), C.byref(h)))
    return _take_result(h)


def longform_finish_regions(vocab: Vocabulary, audio_len: int, tasks, region_tasks, windows) -> TranscriptionResult:
    """build_parallel_result (src/long_form.rs:344-374) from per-task token streams in task order."""
    tok, frm, dur, conf, offs, _ = _concat(windows)
    ts = (_lib.ChunkTaskC * max(len(tasks), 1))(*[_lib.ChunkTaskC(*map(int, t)) for t in tasks])
    rs = (_lib.RegionTaskC * max(len(region_tasks), 1))(*[_lib.RegionTaskC(*map(int, r)) for r in region_tasks])
    h = C.c_void_p()
    check(_lib.lib().sb_longform_finish_regions(vocab._h, audio_len, ts, len(tasks), rs, len(region_tasks), _ptr(tok),
                                                _ptr(frm), _ptr(dur), _ptr(conf), _ptr(offs), C.byref(h)))
    return _take_result(h)


class SileroVad:
    """src/long_form/vad.rs:9-29: per-window speech probabilities of a recording, on the context's GPU."""

    def __init__(self, ctx: Context, weights: dict | None = None, path: str | None = None):
        self.ctx = ctx
        L = _lib.lib()
        if path is not None:
            check(L.sb_vad_load_file(ctx.handle, path.encode()))
        else:
            keep = {k: np.ascontiguousarray(v, np.float32) for k, v in weights.items()}
            arr = (_lib.TensorC * len(keep))()
            for i, (k, v) in enumerate(keep.items()):
                arr[i] = _lib.TensorC(k.encode(), v.ctypes.data, v.size)
            check(L.sb_vad_load(ctx.handle, arr, len(keep)))

    def process(self, audio, config: VadConfig | None = None) -> np.ndarray:
        a = _audio(audio)
        out = np.zeros(vad_num_windows(a.size), np.float32)
        n = C.c_int64()
        check(_lib.lib().sb_vad_process(self.ctx.handle, _ptr(a) if a.size else None, a.size,
                                        _ptr(out) if out.size else None, out.size, C.byref(n)))
        return out[: n.value]


class TranscriptionPipeline:
    """Single-chunk pipeline (src/pipeline.rs:21-99).  Audio: mono 16 kHz float32."""

    def __init__(self, ctx: Context, vocab: Vocabulary):
        self.ctx = ctx
        self.vocab = vocab
        self._config = TranscriptionConfig()

    @classmethod
    def from_weights(cls, weights: dict, vocab: Vocabulary, encoder_layers: int = 24, scale_input: bool = False,
                     device: int = 0, ctx: Context | None = None) -> "TranscriptionPipeline":
        """Stands where the reference has from_dir / from_bundle (src/pipeline.rs:35-54): the caller hands
        over named float32 tensors instead of a CoreML bundle directory."""
        ctx = ctx or Context(device)
        load_model(ctx, weights, encoder_layers, scale_input, has_encoder=True, has_decoder=True)
        return cls(ctx, vocab)

    @classmethod
    def from_dir(cls, models_dir: str, device: int = 0, ctx: Context | None = None,
                 fp8_weights: bool = False) -> "TranscriptionPipeline":
        """src/pipeline.rs:35-46: builds the pipeline from a local bundle directory, here
        `<models_dir>/parakeet-v2/model.safetensors` + `<models_dir>/parakeet-v2/vocab.txt`.  A missing file raises
        MissingModelAsset with its path (src/models.rs:53-66)."""
        from . import weights

        model_path, vocab_path = weights.validate_bundle(models_dir)
        vocab = Vocabulary.from_file(vocab_path)
        ctx = ctx or Context(device)
        weights.load_model_file(ctx, model_path, fp8_weights=fp8_weights)
        return cls(ctx, vocab)

    def config(self) -> TranscriptionConfig:
        return self._config

    def run(self, audio) -> TranscriptionResult:
        return self.run_with_config(audio, self._config)

    def run_with_config(self, audio, config: TranscriptionConfig) -> TranscriptionResult:
        a = _audio(audio)
        cfg = config.to_c()
        h = C.c_void_p()
        check(_lib.lib().sb_pipeline_run(self.ctx.handle, self.vocab._h, _ptr(a) if a.size else None, a.size,
                                         C.byref(cfg), C.byref(h)))
        return _take_result(h)


class LongFormTranscriptionPipeline:
    """Long-form pipeline (src/long_form.rs:44-174): overlap chunking (Fast) or VAD-planned regions (Vad; load the
    network with SileroVad(inner.ctx, ...) first, else MissingModelAsset as in long_form.rs:194-199)."""

    def __init__(self, inner: TranscriptionPipeline, extra_contexts=()):
        self.inner = inner
        self.contexts = [inner.ctx, *extra_contexts]
        self.default_config = LongFormConfig()
        self.vad = None

    @classmethod
    def from_dir(cls, models_dir: str, device: int = 0, fp8_weights: bool = False) -> "LongFormTranscriptionPipeline":
        """src/long_form.rs:100-123: the base bundle must be present; the VAD network file
        (`<models_dir>/vad/silero-vad.safetensors`) is optional here and needed only when the Vad mode is used
        (load_vad, src/long_form.rs:663-670)."""
        from . import weights

        lf = cls(TranscriptionPipeline.from_dir(models_dir, device=device, fp8_weights=fp8_weights))
        path = weights.vad_path(models_dir)
        if os.path.exists(path):
            lf.vad = SileroVad(lf.inner.ctx, path=path)
        return lf

    def run(self, audio) -> TranscriptionResult:
        return self.run_with_config(audio, self.default_config)

    def run_chunk(self, audio) -> TranscriptionResult:
        return self.inner.run(audio)

    def run_with_config(self, audio, config: LongFormConfig) -> TranscriptionResult:
        a = _audio(audio)
        cfg = config.to_c()
        h = C.c_void_p()
        hs = (C.c_void_p * len(self.contexts))(*[c.handle for c in self.contexts])
        check(_lib.lib().sb_longform_run_multi(hs, len(self.contexts), self.inner.vocab._h,
                                               _ptr(a) if a.size else None, a.size, C.byref(cfg), C.byref(h)))
        return _take_result(h)

    def run_with_probabilities(self, audio, probabilities, config: LongFormConfig | None = None) -> TranscriptionResult:
        """run_vad_long_form (src/long_form.rs:188-216) with the caller's per-window speech probabilities."""
        a = _audio(audio)
        p = np.ascontiguousarray(probabilities, np.float32)
        cfg = (config or self.default_config).to_c()
        h = C.c_void_p()
        hs = (C.c_void_p * len(self.contexts))(*[c.handle for c in self.contexts])
        check(_lib.lib().sb_longform_run_with_probabilities(hs, len(self.contexts), self.inner.vocab._h,
                                                            _ptr(a) if a.size else None, a.size, C.byref(cfg),
                                                            _ptr(p) if p.size else None, p.size, C.byref(h)))
        return _take_result(h)
