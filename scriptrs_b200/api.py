"""Host-side mirror of the reference's interface for the transcription hot path.

Names, argument meaning and error behaviour follow the reference crate
(src/frontend.rs, src/pipeline.rs, src/long_form.rs); every call goes through
the C ABI of libscriptrs_b200.so and from there to the sm_100a kernels.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import _lib
from ._lib import ScriptrsError, check

SAMPLE_RATE = 16000
MAX_MODEL_SAMPLES = 240_000
MEL_HOP_SAMPLES = 160
ENCODER_SUBSAMPLING = 8
SAMPLES_PER_ENCODER_FRAME = MEL_HOP_SAMPLES * ENCODER_SUBSAMPLING
SECONDS_PER_ENCODER_FRAME = SAMPLES_PER_ENCODER_FRAME / SAMPLE_RATE
ENCODER_HIDDEN_SIZE = 1024
DECODER_HIDDEN_SIZE = 640
DECODER_LAYERS = 2
MAX_TOKENS_PER_STEP = 10


@dataclass
class TranscriptionConfig:
    """src/config.rs:10-43."""
    sample_rate: int = SAMPLE_RATE
    feature_size: int = 128
    n_fft: int = 512
    win_length: int = 400
    hop_length: int = MEL_HOP_SAMPLES
    preemphasis: float = 0.97
    max_audio_samples: int = MAX_MODEL_SAMPLES
    samples_per_encoder_frame: int = SAMPLES_PER_ENCODER_FRAME

    def max_duration_seconds(self) -> float:
        return self.max_audio_samples / self.sample_rate

    def max_feature_frames(self) -> int:
        return self.max_audio_samples // self.hop_length + 1

    def to_c(self) -> _lib.TranscriptionConfigC:
        return _lib.TranscriptionConfigC(self.sample_rate, self.feature_size, self.n_fft, self.win_length,
                                         self.hop_length, self.preemphasis, self.max_audio_samples,
                                         self.samples_per_encoder_frame)


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


class Context:
    """One GPU's context (sb_ctx).  Not thread-safe, like the reference's pipelines."""

    def __init__(self, device: int = 0):
        self._h = C.c_void_p()
        check(_lib.lib().sb_ctx_create(device, C.byref(self._h)))
        self.device = device

    @property
    def handle(self):
        return self._h

    def set_stream(self, cuda_stream_ptr: int | None):
        check(_lib.lib().sb_ctx_set_stream(self._h, C.c_void_p(cuda_stream_ptr or 0)))

    def synchronize(self):
        check(_lib.lib().sb_ctx_synchronize(self._h))

    def kernel_launches(self) -> int:
        return int(_lib.lib().sb_ctx_kernel_launches(self._h))

    def set_option(self, name: str, value: int):
        check(_lib.lib().sb_ctx_set_option(self._h, name.encode(), int(value)))

    def set_profiling(self, on: bool):
        check(_lib.lib().sb_ctx_set_profiling(self._h, int(on)))

    def profile_report(self) -> dict:
        """{label: (milliseconds, launches)} since the last report (synchronises)."""
        buf = C.create_string_buffer(1 << 16)
        _lib.lib().sb_ctx_profile_report(self._h, buf, len(buf))
        out = {}
        for line in buf.value.decode().splitlines():
            name, ms, n = line.rsplit(" ", 2)
            out[name] = (float(ms), int(n))
        return out

    def close(self):
        if self._h:
            _lib.lib().sb_ctx_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def frontend_tables():
    """(hann window [400], mel filterbank [128, 257]) as the library builds them."""
    w = np.empty(400, np.float32)
    fb = np.empty((128, 257), np.float32)
    check(_lib.lib().sb_frontend_tables(_ptr(w), _ptr(fb)))
    return w, fb


def num_frames(n_samples: int) -> int:
    return int(_lib.lib().sb_frontend_num_frames(n_samples))


class ParakeetFeatureExtractor:
    """Mirror of the reference's feature extractor (src/frontend.rs:11-148) on the GPU."""

    def __init__(self, ctx: Context, config: TranscriptionConfig | None = None):
        self.ctx = ctx
        self.config = config or TranscriptionConfig()
        c = self.config
        if (c.n_fft, c.win_length, c.hop_length, c.feature_size, c.sample_rate) != (512, 400, 160, 128, 16000):
            raise ScriptrsError(11, "the kernels are specialised for n_fft 512 / win 400 / hop 160 / 128 mels / 16 kHz")

    def extract(self, audio: np.ndarray, normalize: bool = True) -> np.ndarray:
        """One clip -> [T, 128] f32.  Empty audio raises EmptyAudio (frontend.rs:105)."""
        audio = np.ascontiguousarray(audio, np.float32).reshape(-1)
        out = self.extract_batch([audio], normalize)
        return out[0]

    def extract_batch(self, clips, normalize: bool = True):
        """List of 1-D clips -> list of [T_i, 128] arrays (one batched launch)."""
        clips = [np.ascontiguousarray(c, np.float32).reshape(-1) for c in clips]
        if len(clips) == 0 or any(c.size == 0 for c in clips):
            raise ScriptrsError(1, "audio input was empty")
        offs = np.zeros(len(clips) + 1, np.int64)
        offs[1:] = np.cumsum([c.size for c in clips])
        pcm = np.concatenate(clips)
        frames = [num_frames(c.size) for c in clips]
        feats = np.empty((int(sum(frames)), 128), np.float32)
        fo = np.zeros(len(clips) + 1, np.int64)
        check(_lib.lib().sb_frontend_host(self.ctx.handle, _ptr(pcm), _ptr(offs), len(clips),
                                          float(self.config.preemphasis), int(normalize), _ptr(feats), _ptr(fo)))
        return [feats[fo[i]:fo[i + 1]] for i in range(len(clips))]

    def extract_device(self, d_pcm: int, clip_offsets: np.ndarray, d_feats: int, normalize: bool = True,
                       int16: bool = False):
        """Device pointers in and out; asynchronous on the context's stream.  Returns frame offsets.
        int16=True: d_pcm holds 16-bit PCM (converted as value / 32767 inside the kernel)."""
        clip_offsets = np.ascontiguousarray(clip_offsets, np.int64)
        n = clip_offsets.size - 1
        fo = np.zeros(n + 1, np.int64)
        fn = _lib.lib().sb_frontend_device_i16 if int16 else _lib.lib().sb_frontend_device
        check(fn(self.ctx.handle, C.c_void_p(d_pcm), _ptr(clip_offsets), n, float(self.config.preemphasis),
                 int(normalize), C.c_void_p(d_feats), _ptr(fo)))
        return fo


def gemm(ctx: Context, d_a: int, d_w: int, d_out: int, M: int, N: int, K: int, d_bias: int = 0, act: int = 0,
         out_mode: int = 0, alpha: float = 1.0, fp8: bool = False, d_row_scale: int = 0, d_col_scale: int = 0):
    """out = epilogue(A[M,K] @ W[N,K]^T) on the tcgen05 GEMM; device pointers; asynchronous."""
    check(_lib.lib().sb_gemm(ctx.handle, C.c_void_p(d_a), C.c_void_p(d_w), C.c_void_p(d_bias or None),
                             C.c_void_p(d_row_scale or None), C.c_void_p(d_col_scale or None), C.c_void_p(d_out),
                             M, N, K, int(fp8), act, out_mode, float(alpha)))


def load_model(ctx: Context, weights: dict, encoder_layers: int, scale_input: bool = False,
               has_encoder: bool = True, has_decoder: bool = False, fp8_weights: bool = False):
    """Uploads a dict of named float32 arrays (see sb_model_load for the names)."""
    keep = {k: np.ascontiguousarray(v, np.float32) for k, v in weights.items()}
    arr = (_lib.TensorC * max(len(keep), 1))()
    for i, (k, v) in enumerate(keep.items()):
        arr[i] = _lib.TensorC(k.encode(), v.ctypes.data, v.size)
    desc = _lib.ModelDescC(encoder_layers, int(scale_input), int(has_encoder), int(has_decoder), int(fp8_weights))
    check(_lib.lib().sb_model_load(ctx.handle, C.byref(desc), arr, len(keep)))


def encoder_num_frames(feature_frames: int) -> int:
    return int(_lib.lib().sb_encoder_num_frames(feature_frames))


def encode_device(ctx: Context, d_feats: int, frame_offsets: np.ndarray, d_out: int) -> np.ndarray:
    """Packed features -> packed encoder output; device pointers; returns the T' prefix sums."""
    frame_offsets = np.ascontiguousarray(frame_offsets, np.int64)
    n = frame_offsets.size - 1
    eo = np.zeros(n + 1, np.int64)
    check(_lib.lib().sb_encode_device(ctx.handle, C.c_void_p(d_feats), _ptr(frame_offsets), n, C.c_void_p(d_out),
                                      _ptr(eo)))
    return eo


def tdt_decode_device(ctx: Context, d_enc: int, enc_offsets: np.ndarray, max_tokens: int | None = None,
                      trace_cap: int = 0):
    """Greedy TDT decode of packed encoder output on the device.  Returns a list of dicts
    (tokens, frames, durations, conf[, logits, steps]) per clip, like the reference's RawTranscription."""
    enc_offsets = np.ascontiguousarray(enc_offsets, np.int64)
    n = enc_offsets.size - 1
    lens = np.diff(enc_offsets)
    if max_tokens is None:
        max_tokens = int(max(1, MAX_TOKENS_PER_STEP * int(lens.max(initial=1))))
    tok = np.zeros((n, max_tokens), np.uint32)
    frm = np.zeros((n, max_tokens), np.int64)
    dur = np.zeros((n, max_tokens), np.int64)
    conf = np.zeros((n, max_tokens), np.float32)
    cnt = np.zeros(n, np.int64)
    steps = np.zeros(n, np.int64)
    trace = np.zeros((n, trace_cap, 1030), np.float32) if trace_cap else None
    check(_lib.lib().sb_tdt_decode_device(ctx.handle, C.c_void_p(d_enc), _ptr(enc_offsets), n, max_tokens, _ptr(tok),
                                          _ptr(frm), _ptr(dur), _ptr(conf), _ptr(cnt), _ptr(trace), trace_cap,
                                          _ptr(steps)))
    out = []
    for i in range(n):
        k = int(cnt[i])
        d = dict(tokens=tok[i, :k].copy(), frames=frm[i, :k].copy(), durations=dur[i, :k].copy(),
                 conf=conf[i, :k].copy(), steps=int(steps[i]))
        if trace is not None:
            d["logits"] = trace[i, : int(steps[i])]
        out.append(d)
    return out


def frontend_device_noalloc(d_pcm: int, clip_offsets: np.ndarray, d_feats: int, normalize: bool = True,
                            preemphasis: float = 0.97, stream: int = 0) -> np.ndarray:
    """Frontend for callers that must not allocate: no context, fixed scratch inside the library, at most
    1024 clips, current device, asynchronous on `stream`.  Returns the frame offsets."""
    clip_offsets = np.ascontiguousarray(clip_offsets, np.int64)
    n = clip_offsets.size - 1
    fo = np.zeros(n + 1, np.int64)
    check(_lib.lib().sb_frontend_device_noalloc(C.c_void_p(d_pcm), _ptr(clip_offsets), n, float(preemphasis),
                                                int(normalize), C.c_void_p(d_feats), _ptr(fo),
                                                C.c_void_p(stream or None)))
    return fo
