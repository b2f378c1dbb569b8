// Stage drivers above the kernels: decode set-up / read-back and the chunk pipeline (pipeline.cu).
#pragma once
#include <stdint.h>

#include <vector>

#include "context.h"

namespace sb {

// Tokens of one clip as the reference's RawTranscription (src/decode.rs:6-11).
struct RawTokens {
    std::vector<uint32_t> token_ids;
    std::vector<int64_t> frame_indices;
    std::vector<int64_t> durations;
    std::vector<float> confidences;
};

void decode_workspace_free(sb_ctx* c);

int32_t frontend_run(sb_ctx* c, const void* d_pcm, SampleFormat fmt, const int64_t* clip_start, const int64_t* clip_len,
                     int64_t n_clips, float preemphasis, bool normalize, float* d_feats, int64_t* frame_offsets);

// Runs the TDT decoder over packed encoder output already on the device.  Blocking.
int32_t tdt_decode(sb_ctx* c, const float* d_enc, const int64_t* enc_offsets, int64_t n_clips, int64_t max_tokens,
                   uint32_t* token_ids, int64_t* frame_indices, int64_t* durations, float* confidences,
                   int64_t* n_tokens, float* logits_trace, int64_t trace_cap, int64_t* n_steps);

}  // namespace sb
