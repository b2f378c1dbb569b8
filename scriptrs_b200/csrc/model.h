// Device-resident model: FastConformer encoder, LSTM predictor and joint network.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "context.h"

namespace sb {

constexpr int kDModel = 1024;
constexpr int kHeads = 8;
constexpr int kHeadDim = 128;
constexpr int kFF = 4096;
constexpr int kConvK = 9;
constexpr int kSubC = 256;
constexpr int kMaxEncFrames = 188;                  // 1501 mel frames -> 751 -> 376 -> 188
constexpr int kPosRows = 2 * kMaxEncFrames - 1;     // relative positions 187 .. -187

constexpr int kPredHidden = 640;
constexpr int kPredLayers = 2;
constexpr int kJointDim = 640;
constexpr int kVocab = 1025;
constexpr int kDurations = 5;
constexpr int kJointOut = kVocab + kDurations;
constexpr int kMaxSymbols = 10;

typedef __nv_bfloat16 bf16;

struct LayerWeights {
    float *ln_ff1_g, *ln_ff1_b, *ln_att_g, *ln_att_b, *ln_conv_g, *ln_conv_b, *ln_ff2_g, *ln_ff2_b, *ln_out_g, *ln_out_b;
    bf16 *ff1_w1, *ff1_w2, *ff2_w1, *ff2_w2;  // [4096 x 1024], [1024 x 4096]
    float *ff1_b1, *ff1_b2, *ff2_b1, *ff2_b2;
    bf16* qkv_w;   // [3072 x 1024] rows: q | k | v
    float* qkv_b;  // [3072]
    bf16* o_w;     // [1024 x 1024]
    float* o_b;
    bf16* pos_proj;  // [kPosRows x 1024]: row p = W_r * pos(187 - p), computed once at load
    float *bias_u, *bias_v;  // [1024] (head-major)
    float* pos_vp;           // [kPosRows x 8]: bias_v . pos_proj per table row and head
    bf16* pw1_w;  // [2048 x 1024]
    float* pw1_b;
    float* dw_w;  // [9 x 1024] tap-major, BatchNorm folded in
    float* dw_b;  // [1024], depthwise bias and BatchNorm shift folded
    bf16* pw2_w;  // [1024 x 1024]
    float* pw2_b;
    // e4m3 copies with one scale per output channel (w = q * scale[n]) for the FP8 path
    uint8_t *ff1_w1_q, *ff1_w2_q, *ff2_w1_q, *ff2_w2_q, *qkv_w_q, *pw1_w_q;
    float *ff1_w1_s, *ff1_w2_s, *ff2_w1_s, *ff2_w2_s, *qkv_w_s, *pw1_w_s;
    // bound on |W1 y + b1| per unit of ||y||_2: largest row norm of W1, and max |b1| (scale of the e4m3 hidden row)
    float ff1_wn, ff1_bmax, ff2_wn, ff2_bmax;
};

// Split-bf16 copies of the predictor / joint weights for the tensor-core path (decode_tc.cu): every row is
// [hi | lo | hi] over a tripled K; the joint output matrix and bias are padded to 1152 rows.
struct DecodeTcWeights {
    bf16 *w0 = nullptr, *w1 = nullptr;  // [2560 x 3 * 1280]  ([W_ih | W_hh] of each LSTM layer)
    bf16* wp = nullptr;                 // [640 x 3 * 640]
    bf16* wo = nullptr;                 // [1152 x 3 * 640]
    bf16* wenc = nullptr;               // [640 x 3 * 1024]
    float* b_out = nullptr;             // [1152]
};

struct Model {
    int layers = 0;
    float xscale = 1.0f;
    bool has_encoder = false, has_decoder = false, has_fp8 = false;
    // sub-sampling
    float *sub0_w = nullptr, *sub0_b = nullptr;  // [256 x 9], [256]
    float *dw1_w = nullptr, *dw1_b = nullptr;    // [9 x 256] tap-major, [256]
    void *sub0_frag = nullptr, *dw1_pairs = nullptr;  // fp16 operands of the tensor-core kernel for these two stages (subsample.h)
    float *dw2_w = nullptr, *dw2_b = nullptr;
    bf16 *pw1_w = nullptr, *pw2_w = nullptr;     // [256 x 256]
    float *pw1_b = nullptr, *pw2_b = nullptr;
    bf16* lin_w = nullptr;                       // [1024 x 4096], columns permuted to (f * 256 + c)
    float* lin_b = nullptr;
    std::vector<LayerWeights> L;
    // predictor + joint (fp32)
    float *embedding = nullptr, *w_ih = nullptr, *w_hh = nullptr, *b_gates = nullptr;  // b_gates = b_ih + b_hh
    bf16* enc_proj_w = nullptr;  // [640 x 1024] bf16 copy for the tensor-core projection
    float *w_enc = nullptr, *b_enc = nullptr, *w_pred = nullptr, *b_pred = nullptr, *w_out = nullptr, *b_out = nullptr;
    DecodeTcWeights tc;  // split-bf16 copies for the tensor-core decoder
    std::vector<void*> allocations;
};

}  // namespace sb
