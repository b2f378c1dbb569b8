"""ctypes loader for libscriptrs_b200.so (the C ABI declared in include/scriptrs_b200.h).

There is no CPU fallback: if the shared library is missing this module raises,
and creating a context without a B200 fails with SB_UNSUPPORTED_PLATFORM.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libscriptrs_b200.so")

SB_OK = 0
STATUS_NAMES = {
    0: "SB_OK", 1: "SB_EMPTY_AUDIO", 2: "SB_AUDIO_TOO_LONG", 3: "SB_MISSING_MODEL_ASSET", 4: "SB_IO",
    5: "SB_INVALID_VOCABULARY", 6: "SB_INVALID_MODEL_OUTPUT", 7: "SB_BACKEND", 8: "SB_UNSUPPORTED_PLATFORM",
    9: "SB_CUDA_ERROR", 10: "SB_TIMEOUT", 11: "SB_INVALID_ARGUMENT", 12: "SB_BUFFER_TOO_SMALL",
}


class TranscriptionConfigC(C.Structure):
    _fields_ = [("sample_rate", C.c_int64), ("feature_size", C.c_int64), ("n_fft", C.c_int64),
                ("win_length", C.c_int64), ("hop_length", C.c_int64), ("preemphasis", C.c_float),
                ("max_audio_samples", C.c_int64), ("samples_per_encoder_frame", C.c_int64)]


class OverlapConfigC(C.Structure):
    _fields_ = [("overlap_seconds", C.c_double), ("context_samples", C.c_int64), ("max_model_samples", C.c_int64)]


class VadConfigC(C.Structure):
    _fields_ = [("default_threshold", C.c_float)]


class VadSegmentationConfigC(C.Structure):
    _fields_ = [("min_speech_duration", C.c_double), ("min_silence_duration", C.c_double),
                ("max_speech_duration", C.c_double), ("speech_padding", C.c_double),
                ("silence_threshold_for_split", C.c_float), ("has_negative_threshold", C.c_int32),
                ("negative_threshold", C.c_float), ("negative_threshold_offset", C.c_float),
                ("min_silence_at_max_speech", C.c_double), ("use_max_possible_silence_at_max_speech", C.c_int32)]


class LongFormConfigC(C.Structure):
    _fields_ = [("mode", C.c_int32), ("worker_count", C.c_int64), ("transcription", TranscriptionConfigC),
                ("vad", VadConfigC), ("segmentation", VadSegmentationConfigC), ("overlap", OverlapConfigC)]


class SampleRangeC(C.Structure):
    _fields_ = [("start", C.c_int64), ("end", C.c_int64)]


class RegionTaskC(C.Structure):
    _fields_ = [("kind", C.c_int32), ("first_task", C.c_int64), ("n_tasks", C.c_int64)]


class TensorC(C.Structure):
    _fields_ = [("name", C.c_char_p), ("data", C.c_void_p), ("numel", C.c_int64)]


class ModelDescC(C.Structure):
    _fields_ = [("encoder_layers", C.c_int32), ("scale_input", C.c_int32), ("has_encoder", C.c_int32),
                ("has_decoder", C.c_int32), ("fp8_weights", C.c_int32)]


class ChunkTaskC(C.Structure):
    _fields_ = [("audio_start", C.c_int64), ("audio_end", C.c_int64), ("global_sample_offset", C.c_int64),
                ("context_samples", C.c_int64)]


_lib = None

_VP = C.c_void_p
_I64 = C.c_int64
_I32 = C.c_int32

# name -> (restype, argtypes); one entry per symbol declared in include/scriptrs_b200.h
SIGNATURES = {
    "sb_last_error": (C.c_char_p, []),
    "sb_status_string": (C.c_char_p, [_I32]),
    "sb_default_transcription_config": (None, [C.POINTER(TranscriptionConfigC)]),
    "sb_default_overlap_config": (None, [C.POINTER(OverlapConfigC)]),
    "sb_default_longform_config": (None, [C.POINTER(LongFormConfigC)]),
    "sb_default_vad_config": (None, [C.POINTER(VadConfigC)]),
    "sb_default_vad_segmentation_config": (None, [C.POINTER(VadSegmentationConfigC)]),
    "sb_ctx_create": (_I32, [_I32, C.POINTER(_VP)]),
    "sb_ctx_destroy": (None, [_VP]),
    "sb_ctx_set_stream": (_I32, [_VP, _VP]),
    "sb_ctx_synchronize": (_I32, [_VP]),
    "sb_ctx_kernel_launches": (_I64, [_VP]),
    "sb_ctx_set_option": (_I32, [_VP, C.c_char_p, _I64]),
    "sb_ctx_set_profiling": (_I32, [_VP, _I32]),
    "sb_ctx_profile_report": (_I64, [_VP, C.c_char_p, _I64]),
    "sb_frontend_tables": (_I32, [_VP, _VP]),
    "sb_frontend_num_frames": (_I64, [_I64]),
    "sb_frontend_device": (_I32, [_VP, _VP, _VP, _I64, C.c_float, _I32, _VP, _VP]),
    "sb_frontend_device_i16": (_I32, [_VP, _VP, _VP, _I64, C.c_float, _I32, _VP, _VP]),
    "sb_frontend_host": (_I32, [_VP, _VP, _VP, _I64, C.c_float, _I32, _VP, _VP]),
    "sb_frontend_device_noalloc": (_I32, [_VP, _VP, _I64, C.c_float, _I32, _VP, _VP, _VP]),
    "sb_model_load": (_I32, [_VP, C.POINTER(ModelDescC), C.POINTER(TensorC), _I64]),
    "sb_model_load_file": (_I32, [_VP, C.POINTER(ModelDescC), C.c_char_p, C.c_char_p]),
    "sb_weights_file_list": (_I64, [C.c_char_p, C.c_char_p, _I64]),
    "sb_encoder_num_frames": (_I64, [_I64]),
    "sb_encode_device": (_I32, [_VP, _VP, _VP, _I64, _VP, _VP]),
    "sb_tdt_decode_device": (_I32, [_VP, _VP, _VP, _I64, _I64, _VP, _VP, _VP, _VP, _VP, _VP, _I64, _VP]),
    "sb_overlap_chunk_samples": (_I64, [C.POINTER(OverlapConfigC)]),
    "sb_overlap_overlap_samples": (_I64, [C.POINTER(OverlapConfigC)]),
    "sb_overlap_stride_samples": (_I64, [C.POINTER(OverlapConfigC)]),
    "sb_plan_fast": (_I32, [C.POINTER(OverlapConfigC), _I64, _VP, _I64, C.POINTER(_I64)]),
    "sb_parallel_worker_count": (_I64, [_I64, _I64]),
    "sb_apply_time_offsets": (_I32, [_VP, _VP, _VP, _VP, _I64, _I64, _I64, C.POINTER(_I64)]),
    "sb_merge_windows": (_I32, [_VP, _VP, _VP, _VP, _VP, _I64, _VP, _VP, _VP, _VP, _I64, C.POINTER(_I64)]),
    "sb_vad_num_windows": (_I64, [_I64]),
    "sb_vad_detect_speech_regions": (_I32, [_VP, _I64, _I64, C.c_float, C.POINTER(VadSegmentationConfigC), _VP, _I64,
                                            C.POINTER(_I64)]),
    "sb_vad_plan_region_subsegments": (_I32, [C.POINTER(SampleRangeC), _VP, _I64, C.POINTER(VadSegmentationConfigC), _I64,
                                              _VP, _I64, C.POINTER(_I64)]),
    "sb_plan_vad": (_I32, [C.POINTER(LongFormConfigC), _VP, _I64, _VP, _I64, _VP, _I64, C.POINTER(_I64), _VP, _I64]),
    "sb_vocab_load": (_I32, [C.c_char_p, C.POINTER(_VP)]),
    "sb_vocab_from_text": (_I32, [C.c_char_p, _I64, C.POINTER(_VP)]),
    "sb_vocab_free": (None, [_VP]),
    "sb_vocab_size": (_I64, [_VP]),
    "sb_vocab_blank_id": (_I64, [_VP]),
    "sb_text_decode": (_I32, [_VP, _VP, _VP, _VP, _I64, _I64, C.c_double, C.POINTER(_VP)]),
    "sb_result_text": (C.c_char_p, [_VP]),
    "sb_result_duration": (C.c_double, [_VP]),
    "sb_result_num_tokens": (_I64, [_VP]),
    "sb_result_num_chunks": (_I64, [_VP]),
    "sb_result_token": (_I32, [_VP, _I64, C.POINTER(C.c_uint32), C.POINTER(C.c_char_p), C.POINTER(C.c_double),
                               C.POINTER(C.c_double), C.POINTER(C.c_float)]),
    "sb_result_chunk": (_I32, [_VP, _I64, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_char_p)]),
    "sb_result_tokens_bulk": (_I32, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _I64, C.POINTER(_I64)]),
    "sb_result_free": (None, [_VP]),
    "sb_raw_batch_size": (_I64, [_VP]),
    "sb_raw_batch_get": (_I32, [_VP, _I64, C.POINTER(_I64), C.POINTER(_VP), C.POINTER(_VP), C.POINTER(_VP),
                                C.POINTER(_VP)]),
    "sb_raw_batch_total": (_I64, [_VP]),
    "sb_raw_batch_flatten": (_I32, [_VP, _VP, _VP, _VP, _VP, _VP]),
    "sb_raw_batch_free": (None, [_VP]),
    "sb_transcribe_chunks": (_I32, [_VP, _VP, _I64, _VP, _I64, C.POINTER(TranscriptionConfigC), C.POINTER(_VP)]),
    "sb_transcribe_chunks_i16": (_I32, [_VP, _VP, _I64, _VP, _I64, C.POINTER(TranscriptionConfigC), C.POINTER(_VP)]),
    "sb_transcribe_chunks_device": (_I32, [_VP, _VP, _I64, _VP, _I64, C.POINTER(TranscriptionConfigC), C.POINTER(_VP)]),
    "sb_pipeline_run": (_I32, [_VP, _VP, _VP, _I64, C.POINTER(TranscriptionConfigC), C.POINTER(_VP)]),
    "sb_longform_run": (_I32, [_VP, _VP, _VP, _I64, C.POINTER(LongFormConfigC), C.POINTER(_VP)]),
    "sb_longform_run_multi": (_I32, [C.POINTER(_VP), _I64, _VP, _VP, _I64, C.POINTER(LongFormConfigC), C.POINTER(_VP)]),
    "sb_longform_finish": (_I32, [_VP, _I64, _VP, _VP, _VP, _VP, _VP, _I64, C.POINTER(_VP)]),
    "sb_longform_finish_regions": (_I32, [_VP, _I64, _VP, _I64, _VP, _I64, _VP, _VP, _VP, _VP, _VP, C.POINTER(_VP)]),
    "sb_longform_run_with_probabilities": (_I32, [C.POINTER(_VP), _I64, _VP, _VP, _I64, C.POINTER(LongFormConfigC), _VP,
                                                  _I64, C.POINTER(_VP)]),
    "sb_vad_load": (_I32, [_VP, C.POINTER(TensorC), _I64]),
    "sb_vad_load_file": (_I32, [_VP, C.c_char_p]),
    "sb_vad_process": (_I32, [_VP, _VP, _I64, _VP, _I64, C.POINTER(_I64)]),
    "sb_vad_process_device": (_I32, [_VP, _VP, _I64, _VP]),
    "sb_gemm": (_I32, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _I64, _I64, _I64, _I32, _I32, _I32, C.c_float]),
}


class ScriptrsError(RuntimeError):
    """Mirror of the reference's TranscriptionError (src/error.rs): `.status` is the sb_status code."""

    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status
        self.message = message


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m scriptrs_b200.build` "
                "(there is no CPU fallback for the CUDA path)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status: int):
    if status != SB_OK:
        msg = lib().sb_last_error().decode("utf-8", "replace")
        raise ScriptrsError(status, msg)
