// First two sub-sampling stages on the tensor cores (subsample.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace sb {

constexpr int kMelBins = 128;
constexpr int kSubChannels = 256;

cudaError_t subsample_configure();
// Host-side weight preparation (called once at model load):
//   frags: subsample_frag_count() x uint2, fp16 B fragments of the first convolution (taps + bias)
//   pairs: 10 x 128 fp16 pairs of the depthwise stage (nine taps, then the bias)
size_t subsample_frag_count();
void subsample_build_frags(const float* w0 /*[256 x 9]*/, const float* b0 /*[256]*/, uint2* frags);
void subsample_build_dw(const float* w1_tap_major /*[9 x 256]*/, const float* b1 /*[256]*/, uint32_t* out_pairs);
// feats f32 [sum T x 128] -> out bf16 [sum T2 x 32 x 256]; d_t0 / d_t1 / d_t2: device prefix sums of T, T1, T2.
cudaError_t subsample_conv0_dw1_launch(const float* feats, const int64_t* d_t0, const int* d_t1, const int* d_t2, int n_clips,
                                       int max_t2, const void* w0_frag, const void* w1_pairs, void* out, cudaStream_t st);

}  // namespace sb
