"""scriptrs_b200: B200-native (sm_100a) transcription hot path behind a C ABI.

The compute lives in libscriptrs_b200.so (built from csrc/ by `scriptrs_b200.build`);
this package is the host-side mirror of the reference's interface.
"""
from ._lib import ScriptrsError, lib, LIB_PATH  # noqa: F401
from .api import *  # noqa: F401,F403
from .pipeline import *  # noqa: F401,F403
from .pipeline import (LongFormConfig, LongFormMode, LongFormTranscriptionPipeline, OverlapChunkConfig,  # noqa: F401
                       ParakeetTdtDecoder, RawBatch, RawTranscription, TimedToken, TranscriptChunk, TranscriptionPipeline,
                       TranscriptionResult, Vocabulary, apply_time_offsets, longform_finish,
                       merge_overlapping_windows, parallel_worker_count, plan_fast, transcribe_chunks)
