// Internal interface of the batched TDT greedy decoder (decode.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "model.h"

namespace sb {

struct DecodeWeights {
    const float *embedding, *w_ih, *w_hh, *b_gates, *w_pred, *b_pred, *w_out, *b_out;
};

// All pointers are device memory.  Per-sequence arrays have n_seq entries; h/c/h_new/c_new are
// [layers][n_seq][640]; outputs are [n_seq][max_tokens].
struct DecodeState {
    int n_seq;
    int max_tokens;
    int trace_cap;  // rows of logits trace per sequence (0 = no trace)
    const float* enc_proj;  // [sum T' x 640]
    const int* enc_off;     // [n_seq] first row of each sequence in enc_proj
    const int* enc_len;     // [n_seq] T'
    int *frame_idx, *emitted, *last_token, *cache_valid, *n_tokens, *n_steps;
    float *h, *c, *h_new, *c_new, *pred, *logits;
    float* z;  // [n_seq][640] joint input relu(enc_proj[frame] + pred), kept current for every live sequence
    uint32_t* out_tokens;
    int *out_frames, *out_durs;
    float* out_conf;
    float* trace;   // [n_seq][trace_cap][1030] or null
    int* overflow;  // set if a sequence produced more than max_tokens tokens
    long long* timing;  // optional [12]: clock cycles block 0 spent per phase / barrier (null = off)
};

cudaError_t decode_enc_projection(const float* d_enc, const float* w_enc, const float* b_enc, float* d_proj, int rows,
                                  cudaStream_t stream);
cudaError_t decode_launch(const DecodeWeights& w, const DecodeState& s, int max_steps, int sm_count,
                          cudaStream_t stream);


size_t decode_tc_weight_bytes();
cudaError_t decode_tc_prepare(const DecodeWeights& w, const float* w_enc, DecodeTcWeights* t, void* storage,
                              cudaStream_t st);
size_t decode_tc_scratch_bytes(int64_t enc_rows, int n_seq);
cudaError_t decode_tc_enc_projection(const DecodeTcWeights& t, const float* d_enc, const float* b_enc, float* d_proj,
                                     int64_t rows, void* scratch, int sm_count, int* d_error, int64_t* launches,
                                     cudaStream_t st);
cudaError_t decode_tc_run(const DecodeWeights& w, const DecodeTcWeights& t, const DecodeState& s, int max_steps,
                          void* scratch_after_enc, int* d_alive, int sm_count, int* d_error, int64_t* launches,
                          cudaStream_t st);

}  // namespace sb
