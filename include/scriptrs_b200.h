/*
 * scriptrs_b200 — C ABI of the B200 (sm_100a) transcription hot path.
 *
 * This is the boundary a host crate binds instead of the reference's CoreML
 * backend.  Every entry point takes plain pointers and sizes.  All functions
 * return an sb_status (0 = success); sb_last_error() gives the message of the
 * last failure on the calling thread.  A context (sb_ctx) belongs to one GPU
 * and must be used by one host thread at a time, like the reference's
 * pipelines, which are Clone but not Sync (src/frontend.rs:16, src/model.rs:18).
 *
 * Citations name the reference interface each entry point replaces, by path
 * within the reference project.
 */
#ifndef SCRIPTRS_B200_H
#define SCRIPTRS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes: the variants of TranscriptionError (src/error.rs:5-40) plus
 * device-side conditions.  SB_BACKEND stands where the reference reports
 * CoreMl(String). */
typedef enum sb_status {
    SB_OK = 0,
    SB_EMPTY_AUDIO = 1,          /* EmptyAudio */
    SB_AUDIO_TOO_LONG = 2,       /* AudioTooLong { max_seconds, actual_seconds } */
    SB_MISSING_MODEL_ASSET = 3,  /* MissingModelAsset { path } */
    SB_IO = 4,                   /* Io */
    SB_INVALID_VOCABULARY = 5,   /* InvalidVocabulary */
    SB_INVALID_MODEL_OUTPUT = 6, /* InvalidModelOutput */
    SB_BACKEND = 7,              /* CoreMl(String) in the reference */
    SB_UNSUPPORTED_PLATFORM = 8, /* UnsupportedPlatform */
    SB_CUDA_ERROR = 9,
    SB_TIMEOUT = 10,             /* a bounded device-side wait ran out */
    SB_INVALID_ARGUMENT = 11,
    SB_BUFFER_TOO_SMALL = 12
} sb_status;

typedef struct sb_ctx sb_ctx;

/* TranscriptionConfig (src/config.rs:10-43), field for field. */
typedef struct sb_transcription_config {
    int64_t sample_rate;               /* 16000 */
    int64_t feature_size;              /* 128 */
    int64_t n_fft;                     /* 512 */
    int64_t win_length;                /* 400 */
    int64_t hop_length;                /* 160 */
    float preemphasis;                 /* 0.97 */
    int64_t max_audio_samples;         /* 240000 */
    int64_t samples_per_encoder_frame; /* 1280 */
} sb_transcription_config;

/* OverlapChunkConfig (src/long_form/planner.rs:84-102). */
typedef struct sb_overlap_config {
    double overlap_seconds;    /* 2.0 */
    int64_t context_samples;   /* 1280 */
    int64_t max_model_samples; /* 240000 */
} sb_overlap_config;

/* LongFormConfig (src/long_form.rs:56-87).  mode 0 = Fast (the only mode built).
 * worker_count keeps the reference's meaning of "parallel chunk workers"; here a
 * worker is a GPU shard. */
typedef struct sb_longform_config {
    int32_t mode;
    int64_t worker_count; /* 4 */
    sb_transcription_config transcription;
    sb_overlap_config overlap;
} sb_longform_config;

/* ChunkTask (src/long_form.rs:468-476). */
typedef struct sb_chunk_task {
    int64_t audio_start;
    int64_t audio_end;
    int64_t global_sample_offset;
    int64_t context_samples;
} sb_chunk_task;

/* ---------------------------------------------------------------- library */

/* Message of the last failure on this thread ("" if none). */
const char* sb_last_error(void);
/* Text of a status code. */
const char* sb_status_string(int32_t status);
/* Fills the defaults of src/config.rs:30-43, planner.rs:94-102, long_form.rs:74-87. */
void sb_default_transcription_config(sb_transcription_config* cfg);
void sb_default_overlap_config(sb_overlap_config* cfg);
void sb_default_longform_config(sb_longform_config* cfg);

/* Creates a context on CUDA device `device` (frontend tables, stream, workspaces).
 * Replaces ParakeetFeatureExtractor::new (src/frontend.rs:88-102) and the
 * per-worker pipeline construction of src/long_form.rs:288-295. */
int32_t sb_ctx_create(int32_t device, sb_ctx** out);
void sb_ctx_destroy(sb_ctx* ctx);
/* Launch on `stream` (a cudaStream_t) instead of the context's own stream; NULL restores it. */
int32_t sb_ctx_set_stream(sb_ctx* ctx, void* stream);
/* Blocks until all work submitted through this context has finished. */
int32_t sb_ctx_synchronize(sb_ctx* ctx);
/* Number of kernels this context has launched since creation. */
int64_t sb_ctx_kernel_launches(const sb_ctx* ctx);

/* --------------------------------------------------------------- frontend */

/* Host copies of the frontend's constant tables: hann_window (src/frontend.rs:161-165)
 * and create_mel_filterbank (src/frontend.rs:188-223).  window: win_length floats;
 * filterbank: 128 x 257 floats, row-major. */
int32_t sb_frontend_tables(float* window, float* filterbank);

/* Number of feature frames for n_samples (src/frontend.rs:124-127): n/160 + 1. */
int64_t sb_frontend_num_frames(int64_t n_samples);

/* Batched ParakeetFeatureExtractor::extract (src/frontend.rs:104-118).
 *   d_pcm        device pointer; clip i is d_pcm[clip_offsets[i] .. clip_offsets[i+1])
 *   clip_offsets host array of n_clips + 1 sample offsets (ascending)
 *   d_feats      device pointer, [sum_i T_i x 128] f32, clip after clip, each clip
 *                time-major [T_i x 128] as the reference returns it
 *   frame_offsets host array of n_clips + 1, written by the call (prefix sums of T_i);
 *                may be NULL
 *   normalize    non-zero: per-feature normalisation (src/frontend.rs:225-241);
 *                zero: stop after ln(mel + 2^-24)
 * An empty clip fails with SB_EMPTY_AUDIO (src/frontend.rs:105).  A clip shorter
 * than 160 samples has one frame and normalises to NaN, as in the reference. */
int32_t sb_frontend_device(sb_ctx* ctx, const float* d_pcm, const int64_t* clip_offsets, int64_t n_clips,
                           float preemphasis, int32_t normalize, float* d_feats, int64_t* frame_offsets);

/* Same through host buffers: copies the PCM in, runs, copies the features out. */
int32_t sb_frontend_host(sb_ctx* ctx, const float* pcm, const int64_t* clip_offsets, int64_t n_clips,
                         float preemphasis, int32_t normalize, float* feats, int64_t* frame_offsets);

/* ------------------------------------------------------------------ GEMM */

/* Tensor-core GEMM building block of the encoder: out = epilogue(A[M x K] * W[N x K]^T).
 * No counterpart in the reference, whose encoder arithmetic is inside a CoreML blob
 * (src/coreml.rs:75-135); exported so that the kernel can be tested and profiled alone.
 *   d_a, d_w   device pointers, row-major bf16 (fp8 = 0) or e4m3 (fp8 = 1); W in nn.Linear layout
 *   d_bias     [N] f32 or NULL;  d_row_scale [M] / d_col_scale [N] f32 or NULL (fp8 only)
 *   act        0 none, 1 SiLU, 2 ReLU
 *   out_mode   0: bf16 out = act(.)   1: f32 out = alpha * act(.)   2: f32 out += alpha * act(.)
 * Requires N % 128 == 0 and K % 64 == 0 (bf16) or K % 128 == 0 (fp8).  Asynchronous on the
 * context's stream; a device-side wait that ran out is reported by sb_ctx_synchronize. */
int32_t sb_gemm(sb_ctx* ctx, const void* d_a, const void* d_w, const float* d_bias, const float* d_row_scale,
                const float* d_col_scale, void* d_out, int64_t M, int64_t N, int64_t K, int32_t fp8, int32_t act,
                int32_t out_mode, float alpha);

#ifdef __cplusplus
}
#endif
#endif /* SCRIPTRS_B200_H */
