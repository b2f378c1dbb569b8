// Relative-position attention on tensor cores (attention.cu).
#pragma once
#include <cuda_runtime.h>

#include "model.h"

namespace sb {

cudaError_t attention_configure();
// vp[p][h] = v_h . pos_proj[p][h] for the 375 table rows (once per layer at model load)
cudaError_t pos_bias_launch(const bf16* pos_proj, const float* bias_v, float* vp, cudaStream_t st);
// qkv [rows x 3072] bf16 -> out [rows x 1024] bf16; one launch
cudaError_t attention_launch(const bf16* qkv, int rows, const int* d_t3_off, int n_clips, const bf16* pos_proj,
                             const float* bias_u, const float* pos_vp, bf16* out, int sm_count, int* d_error,
                             cudaStream_t st);

}  // namespace sb
