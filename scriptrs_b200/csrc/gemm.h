// Tensor-core GEMM for the encoder / joint projections (see gemm.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace sb {

// kActGlu: the N accumulator columns are groups of 32 = 16 values followed by their 16 gates; the output has N / 2
// columns, out[16 g + i] = v[32 g + i] * sigmoid(v[32 g + 16 + i]) (bf16 output, N % 256 == 0).
enum GemmAct : int { kActNone = 0, kActSilu = 1, kActRelu = 2, kActGlu = 3 };
enum GemmOut : int {
    kOutBf16 = 0,      // out[M x N] bf16 = act(acc * scales + bias)
    kOutF32 = 1,       // out[M x N] f32  = act(acc * scales + bias) * alpha
    kOutResidual = 2,  // out[M x N] f32 += alpha * act(acc * scales + bias)
    kOutFp8 = 3,       // out[M x N] e4m3 = act(acc * scales + bias) / out_row_scale[m]   (N % 256 == 0)
};

struct GemmArgs {
    const void* a;           // [M x K] row-major, bf16 (or e4m3 when fp8)
    const void* w;           // [N x K] row-major (nn.Linear layout), same type
    const float* bias;       // [N] or null
    const float* row_scale;  // fp8 only: per-row activation scale [M], or null
    const float* col_scale;  // fp8 only: per-output-channel weight scale [N], or null
    const float* out_row_scale;  // kOutFp8: per-row scale of the e4m3 output [M]
    void* out;
    int M, N, K;
    int ldo;                 // leading dimension of out in elements
    int act;
    int out_mode;
    float alpha;
    bool fp8;
};

// Process-wide switch for two-CTA 256 x 256 tiles: 0 never, 1 for the products that gain from them (default),
// 2 for every product with at least one such tile per pair of SMs.
void gemm_set_pair_tiles(int mode);
// One-time set-up (driver entry point for tensor maps, shared-memory opt-in).
cudaError_t gemm_configure(const char** why);
// Launches the tcgen05 GEMM on `stream`.  `d_error` is a device int that the kernel
// sets non-zero if a bounded wait ran out.  Returns cudaErrorInvalidValue for shapes
// the kernel does not cover (N % 128 != 0, K % 64 (bf16) / 128 (fp8) != 0).
cudaError_t gemm_launch(const GemmArgs& g, int sm_count, int* d_error, cudaStream_t stream);

}  // namespace sb
