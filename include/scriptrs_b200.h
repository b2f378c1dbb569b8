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

/* VadConfig (src/long_form/planner.rs:11-27). */
typedef struct sb_vad_config {
    float default_threshold; /* 0.85: positive speech threshold on the per-window probabilities */
} sb_vad_config;

/* VadSegmentationConfig (src/long_form/planner.rs:29-68), field for field; the Option<f32>
 * negative_threshold is the pair (has_negative_threshold, negative_threshold). */
typedef struct sb_vad_segmentation_config {
    double min_speech_duration;        /* 0.15 */
    double min_silence_duration;       /* 0.75 */
    double max_speech_duration;        /* 14.0 (carried; the reference's planner does not read it) */
    double speech_padding;             /* 0.1 */
    float silence_threshold_for_split; /* 0.3 */
    int32_t has_negative_threshold;    /* 0 = None */
    float negative_threshold;
    float negative_threshold_offset;   /* 0.15 */
    double min_silence_at_max_speech;  /* 0.098 */
    int32_t use_max_possible_silence_at_max_speech; /* 1 (carried; the reference's planner does not read it) */
} sb_vad_segmentation_config;

/* LongFormConfig (src/long_form.rs:56-87), field for field.  mode 0 = Fast (overlap chunks over the whole
 * recording, the default), 1 = Vad (speech regions from per-window probabilities first).  worker_count keeps
 * the reference's meaning of "parallel chunk workers"; here a worker is a GPU shard. */
typedef struct sb_longform_config {
    int32_t mode;
    int64_t worker_count; /* 4 */
    sb_transcription_config transcription;
    sb_vad_config vad;
    sb_vad_segmentation_config segmentation;
    sb_overlap_config overlap;
} sb_longform_config;

/* SampleRange (src/long_form/planner.rs:5-9). */
typedef struct sb_sample_range {
    int64_t start;
    int64_t end;
} sb_sample_range;

/* RegionTask (src/long_form.rs:488-499): a run of consecutive tasks and how their token streams are joined.
 * kind 0 = Overlap (windows merged by merge_overlapping_windows), 1 = Segments (each task decoded on its
 * own and shifted to its place in the recording). */
typedef struct sb_region_task {
    int32_t kind;
    int64_t first_task;
    int64_t n_tasks;
} sb_region_task;

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
void sb_default_vad_config(sb_vad_config* cfg);                           /* planner.rs:19-27 */
void sb_default_vad_segmentation_config(sb_vad_segmentation_config* cfg); /* planner.rs:52-68 */

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

/* Tuning and test switches.  "fp8" (0/1): run the feed-forward, QKV and first pointwise GEMMs of every
 * Conformer block in FP8 e4m3 (per-row activation scales, per-output-channel weight scales, fp32
 * accumulation); needs a model loaded with fp8_weights.  "fp8_mask" (bits: 1 feed-forward up, 2 feed-forward
 * down, 4 QKV, 8 first pointwise; default 8, the subset that keeps the encoder output within 5e-2 of an fp32
 * evaluation with seeded random weights; 15 = all four): which of those products take the e4m3 path when "fp8" is on.
 * "fp8_hidden_amax" (0/1): scale the e4m3 hidden row of the feed-forward module by its true maximum (one more
 * pass over the row) instead of a bound known before the product runs.  "test_raise_device_error" (0/1): sets
 * the device flag that a kernel raises when a bounded wait runs out (host-side fault injection for tests).
 * "simt_subsample" (0/1): run the first two sub-sampling stages in fp32 on CUDA cores instead of the fp16
 * tensor-core kernel.  "simt_attention" (0/1): run the relative-position attention on CUDA cores
 * instead of the tensor-core kernel; "simt_decode" (0/1): run the TDT predictor and joint in plain fp32 on
 * CUDA cores (one persistent kernel) instead of the split-bf16 tensor-core steps; "gemm_pair_tiles" (0/1/2,
 * process-wide): two-CTA 256 x 256 GEMM tiles never / where they pay (default) / wherever they fit;
 * "vad_unstreamed" (0/1): in the VAD long-form mode run the whole voice-activity network before the first
 * transcription kernel instead of beside the transcription; "vad_rows_cap" (default 0 = sized from the recording): encoder
 * frames the streamed VAD mode keeps before it runs the decoder over them (more tasks than fit are decoded in rounds);
 * "vad_stream_pass_windows" (default 49152): largest pass of the network in the streamed VAD mode;
 * "vad_cluster" (4 or 8, default 8): thread blocks in the cluster that runs the VAD network's recurrence;
 * "vad_segment_windows" (default 131072): windows the VAD network processes per pass (its work buffers hold 2560 bytes
 * per window; the recurrent state is carried from pass to pass);
 * "workspace_budget_mb":
 * MB of encoder intermediates per group of clips (default 49152: the 2236 chunks of an 8 h recording form one group; a
 * batch allocates only what it needs). */
int32_t sb_ctx_set_option(sb_ctx* ctx, const char* name, int64_t value);

/* In-situ timing (off by default): CUDA events around every kernel launch, summed per kernel label.
 * sb_ctx_profile_report synchronises, writes lines "label milliseconds launches" into buf (NUL
 * terminated, truncated to cap) and resets the counters; it returns the full length. */
int32_t sb_ctx_set_profiling(sb_ctx* ctx, int32_t on);
int64_t sb_ctx_profile_report(sb_ctx* ctx, char* buf, int64_t cap);

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

/* The same for 16-bit PCM (d_pcm holds int16 samples): each sample is converted as value / 32767 in f32, the
 * conversion of the reference's WAV reader for 16-bit files (examples/transcribe_wav.rs:341-347), inside the
 * kernel's sample read, so the features equal those of sb_frontend_device on the converted buffer bit for bit. */
int32_t sb_frontend_device_i16(sb_ctx* ctx, const int16_t* d_pcm, const int64_t* clip_offsets, int64_t n_clips,
                               float preemphasis, int32_t normalize, float* d_feats, int64_t* frame_offsets);

/* Same through host buffers: copies the PCM in, runs, copies the features out. */
int32_t sb_frontend_host(sb_ctx* ctx, const float* pcm, const int64_t* clip_offsets, int64_t n_clips,
                         float preemphasis, int32_t normalize, float* feats, int64_t* frame_offsets);

/* The batched frontend for callers that must not allocate.  It has no counterpart in the reference
 * (whose extractor keeps its scratch in a RefCell workspace on the host, src/frontend.rs:16,40-57).
 * sb_frontend_device grows work buffers inside the context with cudaMalloc when a batch is larger
 * than any before, and cudaMalloc / cudaFree synchronise the whole device.  That is wrong for an
 * ingest thread that extracts features while other streams of the same GPU encode and decode, and
 * impossible for a host that has given all device memory to its own pool.  This variant needs no
 * context and calls no cudaMalloc, cudaFree or allocating library routine: tables and clip metadata
 * live in a device array of fixed size (about 32 KB) that every GPU loading the library holds until the
 * process exits.
 *   - at most 1024 clips per call; more fails with SB_INVALID_ARGUMENT;
 *   - runs on the CURRENT device, on `stream` (a cudaStream_t; NULL = default stream); arguments and
 *     results are those of sb_frontend_device, bit for bit;
 *   - the first call on a device looks up the array's address and fills the tables: make it before
 *     any stream capture (first calls from several host threads take turns on a mutex); a call on a
 *     stream that is capturing is refused with SB_INVALID_ARGUMENT, because the clip metadata is
 *     copied from the host stack of the call;
 *   - all calls on a device share the array, which keeps the last call's contents (nothing in it has
 *     to be zero); calls whose kernels overlap on the GPU race on it, so serialise them. */
int32_t sb_frontend_device_noalloc(const float* d_pcm, const int64_t* clip_offsets, int64_t n_clips,
                                   float preemphasis, int32_t normalize, float* d_feats, int64_t* frame_offsets,
                                   void* stream);

/* ------------------------------------------------------------------ model */

/* One named fp32 tensor in host memory. */
typedef struct sb_tensor {
    const char* name;
    const float* data;
    int64_t numel;
} sb_tensor;

/* What to load.  The network shape is fixed to Parakeet-TDT-0.6B (128 mels, 256 sub-sampling
 * channels, d_model 1024, 8 heads, FF 4096, depthwise k = 9; predictor 2 x LSTM(640), joint 640,
 * 1025 tokens + 5 durations); the number of Conformer blocks is free so that tests can run a
 * shallow stack. */
typedef struct sb_model_desc {
    int32_t encoder_layers; /* 24 */
    int32_t scale_input;    /* multiply the sub-sampling output by sqrt(d_model) */
    int32_t has_encoder;
    int32_t has_decoder;
    int32_t fp8_weights;    /* also keep e4m3 copies (one scale per output channel) of the Conformer
                               blocks' feed-forward, QKV and first pointwise weights, for the "fp8" option */
} sb_model_desc;

/* Uploads the weights to the context's GPU in the layouts the kernels use (bf16 GEMM operands,
 * fused QKV, BatchNorm folded into the depthwise taps, projected relative-position table).
 * Replaces ParakeetModel::from_bundle (src/model.rs:22-35) / ModelBundle (src/models.rs:31-104).
 * Tensor names: "subsampling.layers.{0,2,3,5,6}.{weight,bias}", "subsampling.linear.*",
 * "layers.<i>.{feed_forward1,feed_forward2}.linear{1,2}.*", "layers.<i>.self_attn.{q,k,v,o}_proj.*",
 * "layers.<i>.self_attn.{relative_k_proj.weight,bias_u,bias_v}", "layers.<i>.conv.{pointwise_conv1,
 * depthwise_conv,pointwise_conv2}.*", "layers.<i>.conv.norm.{weight,bias,running_mean,running_var}",
 * "layers.<i>.norm_{feed_forward1,self_att,conv,feed_forward2,out}.*", "predictor.embedding",
 * "predictor.lstm.{weight_ih,weight_hh,bias_ih,bias_hh}" (layers stacked, gate order i,f,g,o),
 * "joint.{enc,pred,out}.{weight,bias}".  A missing tensor fails with SB_MISSING_MODEL_ASSET. */
int32_t sb_model_load(sb_ctx* ctx, const sb_model_desc* desc, const sb_tensor* tensors, int64_t n_tensors);

/* The same from a weight file on disk: ModelBundle::from_dir + validate_base (src/models.rs:31-66) with one file in
 * place of the reference's three compiled CoreML model directories.  The file uses the safetensors layout: 8 bytes
 * little-endian header length N, N bytes of JSON {"<tensor name>": {"dtype": "F32" | "F16" | "BF16", "shape": [...],
 * "data_offsets": [begin, end]}, ..., optional "__metadata__": {...}}, then the tensor bytes (offsets count from the
 * end of the header; row-major, little-endian).  Tensor names are those listed for sb_model_load, optionally behind
 * `name_prefix` (e.g. "encoder."; NULL for none; tensors without the prefix are ignored).  F16 / BF16 tensors are
 * widened to f32 on load.  desc->encoder_layers < 0 takes the number of "layers.<i>." blocks found in the file.
 * A path that does not exist fails with SB_MISSING_MODEL_ASSET (MissingModelAsset { path }), an unreadable or
 * malformed file with SB_IO, a missing or mis-shaped tensor with SB_MISSING_MODEL_ASSET. */
int32_t sb_model_load_file(sb_ctx* ctx, const sb_model_desc* desc, const char* path, const char* name_prefix);

/* Host only (no GPU needed): the tensors of a weight file as text lines "name dtype d0xd1x...", written into buf
 * (NUL terminated, truncated to cap).  Returns the full length, or minus an sb_status on failure. */
int64_t sb_weights_file_list(const char* path, char* buf, int64_t cap);

/* ---------------------------------------------------------------- encoder */

/* Encoder frames for a number of feature frames: three times L <- (L - 1) / 2 + 1
 * (1501 -> 188, the reference's ENCODER_SUBSAMPLING = 8, src/constants.rs:4). */
int64_t sb_encoder_num_frames(int64_t feature_frames);

/* Batched ParakeetModelInner::run_encoder (src/model.rs:327-342; CoreML contract src/coreml.rs:75-135).
 *   d_feats        device, packed [sum_i T_i x 128] f32 (the output of sb_frontend_device)
 *   frame_offsets  host, n_clips + 1 prefix sums of T_i
 *   d_out          device, packed [sum_i T'_i x 1024] f32, time-major per clip
 *   enc_offsets    host, n_clips + 1, written with the prefix sums of T'_i
 * Each clip is encoded with its exact length (no padding frames), which is what the reference's
 * blob does with `mel_length`.  T_i may not exceed 1501 (T' <= 188).  Asynchronous on the stream. */
int32_t sb_encode_device(sb_ctx* ctx, const float* d_feats, const int64_t* frame_offsets, int64_t n_clips,
                         float* d_out, int64_t* enc_offsets);

/* ----------------------------------------------------------------- decode */

/* Batched ParakeetModel::greedy_decode (src/model.rs:64-95) with the state machine of
 * GreedyDecodeState (src/model.rs:98-214); the predictor (run_decoder, src/model.rs:344-364) and the
 * joint decision (run_joint, src/model.rs:366-384: token arg-max over 1025, duration arg-max over 5,
 * confidence = max softmax) run for the whole batch at once: by default every loop iteration is a short
 * sequence of tensor-core products and element-wise kernels replayed from a CUDA graph by the host, which
 * reads an "any sequence alive" word every few iterations; with the option "simt_decode" the whole loop
 * runs inside one persistent fp32 kernel.
 *   d_enc         device, packed [sum_i T'_i x 1024] f32, time-major per clip
 *   enc_offsets   host, n_clips + 1 prefix sums of T'_i
 *   max_tokens    capacity per clip of the four output arrays (host, [n_clips x max_tokens]);
 *                 a clip can emit at most 10 * T' tokens
 *   n_tokens      host [n_clips]: tokens emitted per clip (RawTranscription lengths)
 *   logits_trace  optional host [n_clips x trace_cap x 1030]: the joint logits of every loop
 *                 iteration, for replaying the reference's control flow; n_steps (optional, host
 *                 [n_clips]) receives the iterations per clip
 * frame_indices are encoder-frame indices local to the clip, recorded before the advance
 * (src/model.rs:190-193).  Blocking: results are on the host when the call returns.
 * SB_BUFFER_TOO_SMALL if a clip emitted more than max_tokens. */
int32_t sb_tdt_decode_device(sb_ctx* ctx, const float* d_enc, const int64_t* enc_offsets, int64_t n_clips,
                             int64_t max_tokens, uint32_t* token_ids, int64_t* frame_indices, int64_t* durations,
                             float* confidences, int64_t* n_tokens, float* logits_trace, int64_t trace_cap,
                             int64_t* n_steps);

/* -------------------------------------------------------- long-form host logic */

/* OverlapChunkConfig::{chunk,overlap,stride}_samples (src/long_form/planner.rs:104-122):
 * 238080 / 32000 / 206080 with the defaults. */
int64_t sb_overlap_chunk_samples(const sb_overlap_config* cfg);
int64_t sb_overlap_overlap_samples(const sb_overlap_config* cfg);
int64_t sb_overlap_stride_samples(const sb_overlap_config* cfg);

/* build_fast_execution_plan (src/long_form.rs:439-459): OverlapChunkConfig::plan
 * (src/long_form/planner.rs:124-136) followed by push_overlap_task (src/long_form.rs:566-582), which
 * prepends up to context_samples of left context to every chunk but the first.  *n_tasks receives
 * the task count; tasks may be NULL to size the buffer. */
int32_t sb_plan_fast(const sb_overlap_config* cfg, int64_t audio_len, sb_chunk_task* tasks, int64_t cap,
                     int64_t* n_tasks);

/* parallel_worker_count (src/long_form.rs:594-600). */
int64_t sb_parallel_worker_count(int64_t task_count, int64_t requested_workers);

/* apply_time_offsets (src/pipeline.rs:219-252), in place on the four arrays; *n_out = tokens kept. */
int32_t sb_apply_time_offsets(uint32_t* token_ids, int64_t* frame_indices, int64_t* durations, float* confidences,
                              int64_t n, int64_t frame_offset, int64_t context_frames, int64_t* n_out);

/* merge_overlapping_windows (src/long_form/merge.rs:3-13): left fold over the windows in order.
 * Window w is elements [win_off[w], win_off[w+1]) of the input arrays.  Same result as the
 * reference; cost proportional to the overlaps, not to the transcript length. */
int32_t sb_merge_windows(const uint32_t* token_ids, const int64_t* frame_indices, const int64_t* durations,
                         const float* confidences, const int64_t* win_off, int64_t n_windows, uint32_t* out_token_ids,
                         int64_t* out_frame_indices, int64_t* out_durations, float* out_confidences, int64_t out_cap,
                         int64_t* n_out);

/* ------------------------------------------------ VAD planning (LongFormMode::Vad) host logic */

/* Windows process_coreml_vad walks over n_samples (src/long_form/vad.rs:72,78): ceil(n / 512). */
int64_t sb_vad_num_windows(int64_t n_samples);

/* detect_speech_regions (src/long_form/planner.rs:139-233): hysteresis over the per-window speech
 * probabilities (window w covers samples [512 w, 512 w + 512)), minimum speech and silence spans, then padding
 * shared between neighbouring regions.  *n_regions receives the count; regions may be NULL to size the buffer. */
int32_t sb_vad_detect_speech_regions(const float* probabilities, int64_t n_probabilities, int64_t audio_len,
                                     float threshold, const sb_vad_segmentation_config* cfg, sb_sample_range* regions,
                                     int64_t cap, int64_t* n_regions);

/* plan_region_subsegments (src/long_form/planner.rs:242-284) over the probabilities of the region's windows
 * (region_probability_slice, planner.rs:235-240): cuts a region longer than max_chunk_samples at its longest
 * silences.  *n_segments is -1 where the reference returns None (no usable silence: overlap fallback). */
int32_t sb_vad_plan_region_subsegments(const sb_sample_range* region, const float* region_probabilities,
                                       int64_t n_probabilities, const sb_vad_segmentation_config* cfg,
                                       int64_t max_chunk_samples, sb_sample_range* segments, int64_t cap,
                                       int64_t* n_segments);

/* build_execution_plan + build_region_plan (src/long_form.rs:421-437,508-548): one region task per speech
 * region — a single segment if it fits max_audio_samples, else silence-split segments, else overlap windows
 * over the region.  `probabilities` covers the whole recording.  tasks / region_tasks may be NULL to size. */
int32_t sb_plan_vad(const sb_longform_config* cfg, const sb_sample_range* regions, int64_t n_regions,
                    const float* probabilities, int64_t n_probabilities, sb_chunk_task* tasks, int64_t task_cap,
                    int64_t* n_tasks, sb_region_task* region_tasks, int64_t region_cap);

/* ----------------------------------------------------------- vocabulary and text */

typedef struct sb_vocab sb_vocab;
typedef struct sb_result sb_result;       /* TranscriptionResult (src/types.rs:28-49) */
typedef struct sb_raw_batch sb_raw_batch; /* one RawTranscription (src/decode.rs:6-11) per task */

/* Vocabulary::from_file (src/vocab.rs:15-52): lines "<token> <id>"; the blank is the id of "<blk>" /
 * "<blank>", else the last id.  SB_IO if the file cannot be read, SB_INVALID_VOCABULARY if malformed. */
int32_t sb_vocab_load(const char* path, sb_vocab** out);
int32_t sb_vocab_from_text(const char* text, int64_t len, sb_vocab** out);
void sb_vocab_free(sb_vocab* vocab);
int64_t sb_vocab_size(const sb_vocab* vocab);
int64_t sb_vocab_blank_id(const sb_vocab* vocab); /* Vocabulary::blank_id (src/vocab.rs:58-60) */

/* ParakeetTdtDecoder::decode (src/decode.rs:39-104).  confidences may hold fewer than n entries
 * (missing ones read as 0, src/decode.rs:80). */
int32_t sb_text_decode(const sb_vocab* vocab, const uint32_t* token_ids, const int64_t* frame_indices,
                       const float* confidences, int64_t n, int64_t n_confidences, double duration_seconds,
                       sb_result** out);

/* TranscriptionResult accessors; strings stay valid until sb_result_free. */
const char* sb_result_text(const sb_result* r);
double sb_result_duration(const sb_result* r);
int64_t sb_result_num_tokens(const sb_result* r);
int64_t sb_result_num_chunks(const sb_result* r);
int32_t sb_result_token(const sb_result* r, int64_t i, uint32_t* token_id, const char** text, double* start,
                        double* end, float* confidence); /* TimedToken (src/types.rs:1-14) */
int32_t sb_result_chunk(const sb_result* r, int64_t i, double* start, double* end,
                        const char** text);               /* TranscriptChunk (src/types.rs:16-26) */
/* All tokens at once: arrays of sb_result_num_tokens entries (any may be NULL); the token texts are
 * written back to back (UTF-8, no terminators) into text_buf with text_offsets[i] .. text_offsets[i+1]
 * delimiting token i (text_offsets has n + 1 entries).  *text_len receives the bytes needed. */
int32_t sb_result_tokens_bulk(const sb_result* r, uint32_t* token_ids, double* starts, double* ends,
                              float* confidences, int64_t* text_offsets, char* text_buf, int64_t text_cap,
                              int64_t* text_len);
void sb_result_free(sb_result* r);

int64_t sb_raw_batch_size(const sb_raw_batch* b);
int32_t sb_raw_batch_get(const sb_raw_batch* b, int64_t i, int64_t* n, const uint32_t** token_ids,
                         const int64_t** frame_indices, const int64_t** durations, const float** confidences);
/* The whole batch as flat arrays: sb_raw_batch_total tokens; task i is [offsets[i], offsets[i+1])
 * (offsets has size + 1 entries; the data arrays may be NULL). */
int64_t sb_raw_batch_total(const sb_raw_batch* b);
int32_t sb_raw_batch_flatten(const sb_raw_batch* b, int64_t* offsets, uint32_t* token_ids, int64_t* frame_indices,
                             int64_t* durations, float* confidences);
void sb_raw_batch_free(sb_raw_batch* b);

/* ------------------------------------------------------------------ pipelines */

/* transcribe_task (src/long_form.rs:584-592) for a whole list of tasks at once: ChunkPreparer::prepare
 * (src/pipeline.rs:200-216) + transcribe_prepared_raw (src/pipeline.rs:121-138), i.e. frontend ->
 * encoder -> greedy decode -> apply_time_offsets, batched on this context's GPU.  `audio` is the whole
 * recording in host memory (pinned memory makes the copy faster); task i covers
 * audio[audio_start, audio_end).  An empty task fails with SB_EMPTY_AUDIO, one longer than
 * cfg->max_audio_samples with SB_AUDIO_TOO_LONG.  cfg may be NULL for the defaults. */
int32_t sb_transcribe_chunks(sb_ctx* ctx, const float* audio, int64_t n_samples, const sb_chunk_task* tasks,
                             int64_t n_tasks, const sb_transcription_config* cfg, sb_raw_batch** out);

/* The same for a 16-bit PCM recording in host memory: half the bytes cross to the GPU, and the conversion to
 * f32 (value / 32767, examples/transcribe_wav.rs:341-347, which the reference's caller does per sample on the
 * CPU before run()) happens inside the frontend kernel.  Token streams equal those of sb_transcribe_chunks on
 * the converted recording. */
int32_t sb_transcribe_chunks_i16(sb_ctx* ctx, const int16_t* audio, int64_t n_samples, const sb_chunk_task* tasks,
                                 int64_t n_tasks, const sb_transcription_config* cfg, sb_raw_batch** out);

/* The same with the recording already in device memory (d_audio is a device pointer). */
int32_t sb_transcribe_chunks_device(sb_ctx* ctx, const float* d_audio, int64_t n_samples, const sb_chunk_task* tasks,
                                    int64_t n_tasks, const sb_transcription_config* cfg, sb_raw_batch** out);

/* TranscriptionPipeline::run_with_config (src/pipeline.rs:81-89): one chunk of at most
 * cfg->max_audio_samples samples (SB_AUDIO_TOO_LONG beyond, SB_EMPTY_AUDIO if empty). */
int32_t sb_pipeline_run(sb_ctx* ctx, const sb_vocab* vocab, const float* audio, int64_t n_samples,
                        const sb_transcription_config* cfg, sb_result** out);

/* LongFormTranscriptionPipeline::run_with_config (src/long_form.rs:153-166): audio of at most
 * max_audio_samples goes through the single-chunk path; longer audio is planned into overlap chunks
 * (mode 0, Fast) or into speech regions found by the loaded VAD network (mode 1, Vad: sb_vad_load first, else
 * SB_MISSING_MODEL_ASSET as in long_form.rs:194-199), transcribed on this GPU, merged and decoded
 * (src/long_form.rs:188-245,344-419). */
int32_t sb_longform_run(sb_ctx* ctx, const sb_vocab* vocab, const float* audio, int64_t n_samples,
                        const sb_longform_config* cfg, sb_result** out);

/* The same over several GPUs of one process: run_parallel_regions (src/long_form.rs:266-314) with
 * min(worker_count, n_ctx, tasks) workers, each worker being one context's GPU with its own host
 * thread; tasks are dealt in contiguous blocks and results are reassembled in task order
 * (src/long_form.rs:316-342).  The first failing worker fails the call.  In mode 1 the first context runs the VAD
 * network (one recurrence per recording: it does not shard); with one worker its passes run beside the
 * transcription of the regions already found, with several the whole network runs first, as in the reference
 * (src/long_form.rs:188-216). */
int32_t sb_longform_run_multi(sb_ctx** ctxs, int64_t n_ctx, const sb_vocab* vocab, const float* audio,
                              int64_t n_samples, const sb_longform_config* cfg, sb_result** out);

/* Tail of the long-form path for callers that ran sb_transcribe_chunks themselves (one process per
 * GPU): decode_overlap_tasks + build_chunk + build_result (src/long_form.rs:404-419,622-647) over
 * the per-task token streams, concatenated in task order. */
int32_t sb_longform_finish(const sb_vocab* vocab, int64_t audio_len, const uint32_t* token_ids,
                           const int64_t* frame_indices, const int64_t* durations, const float* confidences,
                           const int64_t* win_off, int64_t n_windows, sb_result** out);

/* build_parallel_result (src/long_form.rs:344-374) for callers that ran sb_transcribe_chunks themselves on a
 * plan of region tasks (sb_plan_vad, or one Overlap region for the Fast mode): Overlap regions are merged and
 * decoded against the recording's duration (decode_overlap_tasks, long_form.rs:404-419); the tasks of a
 * Segments region are decoded one by one against their own duration and shifted by their start
 * (decode_segment_tasks, long_form.rs:376-402,649-661); each region with tokens becomes one chunk.  Task i's
 * tokens are elements [win_off[i], win_off[i+1]) of the arrays. */
int32_t sb_longform_finish_regions(const sb_vocab* vocab, int64_t audio_len, const sb_chunk_task* tasks,
                                   int64_t n_tasks, const sb_region_task* region_tasks, int64_t n_regions,
                                   const uint32_t* token_ids, const int64_t* frame_indices, const int64_t* durations,
                                   const float* confidences, const int64_t* win_off, sb_result** out);

/* run_vad_long_form (src/long_form.rs:188-216) from the probabilities on: for callers that bring their own
 * voice-activity detector.  No speech region gives the empty result (TranscriptionResult::empty) with the
 * recording's duration.  Audio of at most max_audio_samples takes the single-chunk path whatever the mode
 * (long_form.rs:161-163). */
int32_t sb_longform_run_with_probabilities(sb_ctx** ctxs, int64_t n_ctx, const sb_vocab* vocab, const float* audio,
                                           int64_t n_samples, const sb_longform_config* cfg,
                                           const float* probabilities, int64_t n_probabilities, sb_result** out);

/* ------------------------------------------------------------------ VAD network */

/* Loads the streaming voice-activity network that sb_longform_run uses in mode 1 (SileroVad::new,
 * src/long_form/vad.rs:15-19; asset "vad/silero-vad.mlmodelc", src/models.rs:10).  The network has the public
 * Silero VAD (16 kHz) shape behind the reference's I/O contract (src/coreml.rs:188-236: audio [576] = 64
 * context + 512 new samples, h / c [128] in, probability and h / c out):
 *   "stft.forward_basis_buffer" [258, 1, 256]   real rows 0..128, imaginary rows 129..257; stride 128 over the
 *                                               576 samples extended by 64 reflected on the right -> 4 frames
 *   "encoder.{0,1,2,3}.reparam_conv.{weight,bias}"  Conv1d k = 3, padding 1, strides 1, 2, 2, 1:
 *                                               129 -> 128 -> 64 -> 64 -> 128 channels, ReLU after each
 *   "decoder.rnn.{weight_ih,weight_hh,bias_ih,bias_hh}"  LSTMCell(128, 128), gate order i, f, g, o
 *   "decoder.decoder.2.{weight,bias}"           ReLU, Conv1d 128 -> 1 (k = 1), sigmoid
 * A missing tensor fails with SB_MISSING_MODEL_ASSET. */
int32_t sb_vad_load(sb_ctx* ctx, const sb_tensor* tensors, int64_t n_tensors);
/* The same from a weight file in the layout sb_model_load_file reads (names optionally behind "_model."). */
int32_t sb_vad_load_file(sb_ctx* ctx, const char* path);

/* SileroVad::process (src/long_form/vad.rs:61-98) for a whole recording in host memory: one probability per
 * 512-sample window; the last window is filled up with its last sample; every window sees the 64 samples
 * before it (zeros for the first) and the recurrent state left by the window before.  The convolutional part
 * runs for all windows at once, the recurrence as one persistent kernel.  probabilities needs
 * sb_vad_num_windows(n_samples) entries.  SB_MISSING_MODEL_ASSET if no network is loaded; empty audio gives
 * zero probabilities (vad.rs:65-67). */
int32_t sb_vad_process(sb_ctx* ctx, const float* audio, int64_t n_samples, float* probabilities, int64_t cap,
                       int64_t* n_probabilities);
/* The same with the recording and the result in device memory (asynchronous on the context's stream; a device-side
 * wait that ran out is reported by sb_ctx_synchronize, and by sb_vad_process itself as SB_TIMEOUT). */
int32_t sb_vad_process_device(sb_ctx* ctx, const float* d_audio, int64_t n_samples, float* d_probabilities);

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
