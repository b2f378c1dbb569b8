// FastConformer encoder (Parakeet-TDT-0.6B shape) on sm_100a.
//
// The reference runs this network as an opaque CoreML blob behind
// ParakeetModelInner::run_encoder (src/model.rs:327-342, I/O contract src/coreml.rs:75-135):
// normalised log-mel [T x 128] in, [T' x 1024] out with T' = ceil-halved three times.
// Here a batch of clips is packed row-wise (variable length, no padding): all position-wise
// projections run as tcgen05 GEMMs over the packed rows (gemm.cu); the kernels in this file
// cover what is not a GEMM and respect clip boundaries.
//
//   sub_conv0_dw1_kernel conv2d(1 -> 256, k3, s2, p1) + ReLU fused with the first depthwise conv2d(k3, s2, p1), in fp32 on
//                        CUDA cores: the in-library cross-check (option "simt_subsample") of the tensor-core kernel
//                        in subsample.cu, which is the one the encoder runs
//   sub_dw_kernel        second depthwise conv2d(k3, s2, p1) + bias (feeds the pointwise GEMM)
//   layernorm_kernel     one warp per 1024-wide row, fp32 statistics, bf16 or f32 output
//   relpos_attention_kernel  per (clip, head): scores = ((q + u) k^T + (q + v) p^T[i - j]) / sqrt(128),
//                        softmax, PV; the relative shift is index arithmetic, never materialised
//   dwconv_kernel        depthwise conv k = 9 ('same' within the clip) + folded BatchNorm + SiLU (GLU: GEMM epilogue)
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <vector>

#include "attention.h"
#include "encoder.h"
#include "gemm.h"
#include "subsample.h"
#include "tc_ptx.cuh"

namespace sb {

namespace {

// ---------------------------------------------------------------- sub-sampling
// First two stages in one kernel: 3x3 stride-2 convolution of the mel image (1 -> 256 channels, ReLU) followed by
// the 3x3 stride-2 depthwise convolution, without the [T/2 x 64 x 256] intermediate ever reaching memory.
//   feats f32 [sum T x 128]  ->  out bf16 [sum T2 x 32 x 256]
// grid (ceil(max T2 / TO), clips), 256 threads = 256 channels.  A CTA produces TO output time rows: it stages the
// 4 TO + 3 mel rows they depend on in shared memory, and every thread walks the 32 output frequencies keeping a
// sliding window: per step it reads four new mel columns of each staged row (one 16-byte broadcast read), forms
// the two new columns of the 2 TO + 1 first-stage rows, and combines them with the column carried over from the
// previous step.  First-stage values outside [0, T1) x [0, 64) are the second stage's zero padding.
template <int TO>
__global__ void __launch_bounds__(256)
sub_conv0_dw1_kernel(const float* __restrict__ feats, const int64_t* __restrict__ t0_off,
                     const int* __restrict__ t1_off, const int* __restrict__ t2_off, const float* __restrict__ w0,
                     const float* __restrict__ b0, const float* __restrict__ w1, const float* __restrict__ b1,
                     bf16* __restrict__ out) {
    constexpr int NY = 2 * TO + 1, NX = 4 * TO + 3, XS = kMels + 8;  // mel column f sits at index f + 4
    __shared__ __align__(16) float xs[NX][XS];
    const int clip = blockIdx.y, to0 = blockIdx.x * TO;
    const int out_base = t2_off[clip];
    const int T2 = t2_off[clip + 1] - out_base;
    if (to0 >= T2) return;
    const int64_t base = t0_off[clip];
    const int T = (int)(t0_off[clip + 1] - base);
    const int T1 = t1_off[clip + 1] - t1_off[clip];
    for (int i = threadIdx.x; i < NX * XS; i += 256) {
        const int row = i / XS, col = i % XS - 4;
        const int r = 4 * to0 - 3 + row;
        float v = 0.0f;
        if (r >= 0 && r < T && col >= 0 && col < kMels) v = feats[(base + r) * kMels + col];
        xs[row][i % XS] = v;
    }
    __syncthreads();
    const int c = threadIdx.x;
    float wa[9], wb[9];
#pragma unroll
    for (int i = 0; i < 9; ++i) {
        wa[i] = w0[c * 9 + i];
        wb[i] = w1[i * kSubC + c];
    }
    const float ba = b0[c], bb = b1[c];
    float ymask[NY], prev[NY], carry[NX];
#pragma unroll
    for (int k = 0; k < NY; ++k) {
        const int r = 2 * to0 - 1 + k;
        ymask[k] = (r >= 0 && r < T1) ? 1.0f : 0.0f;
        prev[k] = 0.0f;  // first-stage column -1
    }
#pragma unroll
    for (int x = 0; x < NX; ++x) carry[x] = 0.0f;  // mel column -1
    bf16* o = out + (size_t)(out_base + to0) * 32 * kSubC + c;
#pragma unroll 1
    for (int fo = 0; fo < 32; ++fo) {
        float ya[NY], yb[NY];  // first-stage columns 2 fo and 2 fo + 1
#pragma unroll
        for (int k = 0; k < NY; ++k) ya[k] = yb[k] = ba;
#pragma unroll
        for (int x = 0; x < NX; ++x) {
            const float4 nw = *reinterpret_cast<const float4*>(&xs[x][4 * fo + 4]);  // mel columns 4 fo .. 4 fo + 3
            const float x0 = carry[x];
            carry[x] = nw.w;
#pragma unroll
            for (int et = 0; et < 3; ++et) {
                if ((x - et) % 2 != 0 || x - et < 0 || (x - et) / 2 >= NY) continue;
                const int k = (x - et) / 2;
                ya[k] = fmaf(wa[et * 3 + 0], x0, ya[k]);
                ya[k] = fmaf(wa[et * 3 + 1], nw.x, ya[k]);
                ya[k] = fmaf(wa[et * 3 + 2], nw.y, ya[k]);
                yb[k] = fmaf(wa[et * 3 + 0], nw.y, yb[k]);
                yb[k] = fmaf(wa[et * 3 + 1], nw.z, yb[k]);
                yb[k] = fmaf(wa[et * 3 + 2], nw.w, yb[k]);
            }
        }
#pragma unroll
        for (int k = 0; k < NY; ++k) {
            ya[k] = fmaxf(ya[k], 0.0f) * ymask[k];
            yb[k] = fmaxf(yb[k], 0.0f) * ymask[k];
        }
#pragma unroll
        for (int j = 0; j < TO; ++j) {
            float acc = bb;
#pragma unroll
            for (int dt = 0; dt < 3; ++dt) {
                acc = fmaf(wb[dt * 3 + 0], prev[2 * j + dt], acc);
                acc = fmaf(wb[dt * 3 + 1], ya[2 * j + dt], acc);
                acc = fmaf(wb[dt * 3 + 2], yb[2 * j + dt], acc);
            }
            if (to0 + j < T2) o[((size_t)j * 32 + fo) * kSubC] = __float2bfloat16(acc);
        }
#pragma unroll
        for (int k = 0; k < NY; ++k) prev[k] = yb[k];
    }
}

// Depthwise 3x3 stride-2 stage: in bf16 [sum Tin x Fin x 256] -> out bf16 [sum Tout x Fin/2 x 256], channels last.
// grid (ceil(max Tout / (2 TO)), clips), 256 threads: each half of the CTA produces TO output time rows, a thread
// owns two channels (4-byte loads, a warp reads 128 contiguous bytes) and walks the output frequencies with a
// sliding window: per step it loads the two new input columns of the 2 TO + 1 rows it needs and reuses the column
// carried over from the previous step.  w is tap-major [9 x 256].
template <int TO>
__global__ void __launch_bounds__(256)
sub_dw_kernel(const bf16* __restrict__ in, const int* __restrict__ tin_off, const int* __restrict__ tout_off, int fin,
              const float* __restrict__ w, const float* __restrict__ b, bf16* __restrict__ out) {
    constexpr int NR = 2 * TO + 1;
    const int clip = blockIdx.y;
    const int out_base = tout_off[clip];
    const int Tout = tout_off[clip + 1] - out_base;
    const int to0 = (blockIdx.x * 2 + (threadIdx.x >> 7)) * TO;
    if (to0 >= Tout) return;
    const int in_base = tin_off[clip];
    const int Tin = tin_off[clip + 1] - in_base;
    const int fout = fin >> 1;
    const int cp = (threadIdx.x & 127) * 2;
    float2 wt[9];
#pragma unroll
    for (int i = 0; i < 9; ++i) wt[i] = *reinterpret_cast<const float2*>(w + i * kSubC + cp);
    const float2 bias = *reinterpret_cast<const float2*>(b + cp);
    const __nv_bfloat162* rowp[NR];
    bool rok[NR];
    float2 carry[NR];
#pragma unroll
    for (int k = 0; k < NR; ++k) {
        const int r = 2 * to0 - 1 + k;
        rok[k] = r >= 0 && r < Tin;
        rowp[k] = reinterpret_cast<const __nv_bfloat162*>(in + (size_t)(in_base + (rok[k] ? r : 0)) * fin * kSubC + cp);
        carry[k] = make_float2(0.0f, 0.0f);  // input column -1
    }
    const __nv_bfloat162 zero2 = __floats2bfloat162_rn(0.0f, 0.0f);
#pragma unroll 2
    for (int fo = 0; fo < fout; ++fo) {
        float2 ca[NR], cb[NR];  // input columns 2 fo and 2 fo + 1
#pragma unroll
        for (int k = 0; k < NR; ++k) {
            const __nv_bfloat162 va = rok[k] ? __ldg(rowp[k] + (size_t)(2 * fo) * (kSubC / 2)) : zero2;
            const __nv_bfloat162 vb = rok[k] ? __ldg(rowp[k] + (size_t)(2 * fo + 1) * (kSubC / 2)) : zero2;
            ca[k] = __bfloat1622float2(va);
            cb[k] = __bfloat1622float2(vb);
        }
#pragma unroll
        for (int j = 0; j < TO; ++j) {
            float2 acc = bias;
#pragma unroll
            for (int dt = 0; dt < 3; ++dt) {
                const int k = 2 * j + dt;
                acc.x = fmaf(wt[dt * 3 + 0].x, carry[k].x, acc.x);
                acc.y = fmaf(wt[dt * 3 + 0].y, carry[k].y, acc.y);
                acc.x = fmaf(wt[dt * 3 + 1].x, ca[k].x, acc.x);
                acc.y = fmaf(wt[dt * 3 + 1].y, ca[k].y, acc.y);
                acc.x = fmaf(wt[dt * 3 + 2].x, cb[k].x, acc.x);
                acc.y = fmaf(wt[dt * 3 + 2].y, cb[k].y, acc.y);
            }
            if (to0 + j < Tout)
                *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)(out_base + to0 + j) * fout + fo) * kSubC + cp) =
                    __floats2bfloat162_rn(acc.x, acc.y);
        }
#pragma unroll
        for (int k = 0; k < NR; ++k) carry[k] = cb[k];
    }
}

// ---------------------------------------------------------------- LayerNorm
// One warp per row of 1024; the row stays in registers (8 float4 per lane).
__device__ __forceinline__ void ln_row(float4 (&v)[8], const float* __restrict__ gamma, const float* __restrict__ beta,
                                       int lane) {
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float mean = s * (1.0f / kDModel);
    float q = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float a = v[k].x - mean, b = v[k].y - mean, c = v[k].z - mean, d = v[k].w - mean;
        q += (a * a + b * b) + (c * c + d * d);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
    const float rstd = rsqrtf(q * (1.0f / kDModel) + 1e-5f);
    const float4* g4 = reinterpret_cast<const float4*>(gamma);
    const float4* b4 = reinterpret_cast<const float4*>(beta);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float4 g = g4[lane + 32 * k], b = b4[lane + 32 * k];
        v[k].x = (v[k].x - mean) * rstd * g.x + b.x;
        v[k].y = (v[k].y - mean) * rstd * g.y + b.y;
        v[k].z = (v[k].z - mean) * rstd * g.z + b.z;
        v[k].w = (v[k].w - mean) * rstd * g.w + b.w;
    }
}

// OUT_F32: write f32 (in place allowed), else bf16.  With pre_gamma the row is first normalised with
// (pre_gamma, pre_beta) and that result written back to x as f32: the closing LayerNorm of one Conformer block
// and the opening one of the next in a single pass over the row.
template <bool OUT_F32>
__global__ void __launch_bounds__(256)
layernorm_kernel(float* x, const float* __restrict__ pre_gamma, const float* __restrict__ pre_beta,
                 const float* __restrict__ gamma, const float* __restrict__ beta, void* out, int rows) {
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    float4* xr = reinterpret_cast<float4*>(x + (size_t)row * kDModel);
    float4 v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = xr[lane + 32 * k];
    if (pre_gamma) {
        ln_row(v, pre_gamma, pre_beta, lane);
#pragma unroll
        for (int k = 0; k < 8; ++k) xr[lane + 32 * k] = v[k];
    }
    ln_row(v, gamma, beta, lane);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        if (OUT_F32) {
            reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + (size_t)row * kDModel)[lane + 32 * k] = v[k];
        } else {
            __nv_bfloat162 p0 = __floats2bfloat162_rn(v[k].x, v[k].y), p1 = __floats2bfloat162_rn(v[k].z, v[k].w);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&p0);
            pk.y = *reinterpret_cast<uint32_t*>(&p1);
            reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(out) + (size_t)row * kDModel)[lane + 32 * k] = pk;
        }
    }
}

__device__ __forceinline__ uint32_t cvt4_e4m3(float a, float b, float c, float d) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);  // cvt2_e4m3 pairs: byte 0 = a, 1 = b, 2 = c, 3 = d
}

// LayerNorm with an e4m3 output row and its scale: q = y / scale, scale = max|y| / 448.  pre_gamma as above.
__global__ void __launch_bounds__(256)
layernorm_fp8_kernel(float* x, const float* __restrict__ pre_gamma, const float* __restrict__ pre_beta,
                     const float* __restrict__ gamma, const float* __restrict__ beta, uint8_t* __restrict__ out,
                     float* __restrict__ row_scale, int rows, float* __restrict__ next_scale, float wn, float bmax) {
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    float4* xr = reinterpret_cast<float4*>(x + (size_t)row * kDModel);
    float4 v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = xr[lane + 32 * k];
    if (pre_gamma) {
        ln_row(v, pre_gamma, pre_beta, lane);
#pragma unroll
        for (int k = 0; k < 8; ++k) xr[lane + 32 * k] = v[k];
    }
    ln_row(v, gamma, beta, lane);
    float amax = 0.0f, ss = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[k].x), fabsf(v[k].y)), fmaxf(fabsf(v[k].z), fabsf(v[k].w))));
        ss += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
    }
    // Scale of the NEXT GEMM's e4m3 output row: |silu(w . y + b)| <= ||y|| max_n ||w_n|| + max |b| (Cauchy-Schwarz;
    // 7 % head-room for the rounding of y and w to e4m3).  Loose by a few binades, which e4m3 absorbs.
    if (next_scale && lane == 0)
        next_scale[row] = fmaxf(1.07f * sqrtf(ss) * wn + bmax, 0.28f) * (1.0f / 448.0f);
    const float scale = amax > 0.0f ? amax * (1.0f / 448.0f) : 1.0f;
    const float inv = 1.0f / scale;
    if (lane == 0) row_scale[row] = scale;
    uint32_t* o32 = reinterpret_cast<uint32_t*>(out + (size_t)row * kDModel);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        o32[lane + 32 * k] = cvt4_e4m3(v[k].x * inv, v[k].y * inv, v[k].z * inv, v[k].w * inv);
    }
}

// bf16 [rows x 4096] -> e4m3 [rows x 4096] + per-row scale (one warp per row, the row stays in registers).
__global__ void __launch_bounds__(256)
quantize_rows4096_kernel(const bf16* __restrict__ in, uint8_t* __restrict__ out, float* __restrict__ row_scale,
                         int rows) {
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const uint4* src = reinterpret_cast<const uint4*>(in + (size_t)row * kFF);
    uint4 raw[16];
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        raw[k] = src[lane + 32 * k];
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[k]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h2[e]);
            amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = amax > 0.0f ? amax * (1.0f / 448.0f) : 1.0f;
    const float inv = 1.0f / scale;
    if (lane == 0) row_scale[row] = scale;
    uint2* dst = reinterpret_cast<uint2*>(out + (size_t)row * kFF);
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[k]);
        const float2 f0 = __bfloat1622float2(h2[0]), f1 = __bfloat1622float2(h2[1]);
        const float2 f2 = __bfloat1622float2(h2[2]), f3 = __bfloat1622float2(h2[3]);
        uint32_t w[2];
        w[0] = cvt4_e4m3(f0.x * inv, f0.y * inv, f1.x * inv, f1.y * inv);
        w[1] = cvt4_e4m3(f2.x * inv, f2.y * inv, f3.x * inv, f3.y * inv);
        dst[lane + 32 * k] = make_uint2(w[0], w[1]);
    }
}

// ---------------------------------------------------------------- relative-position attention
constexpr int kAttThreads = 256;
constexpr int kRowStride = kHeadDim + 2;  // bf16 elements; 65 words -> conflict-free column walks

__device__ __forceinline__ float dot128(const float* __restrict__ q, const bf16* __restrict__ row) {
    float acc = 0.0f;
    const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(row);
#pragma unroll 16
    for (int d = 0; d < kHeadDim / 2; ++d) {
        const float2 f = __bfloat1622float2(r2[d]);
        acc = fmaf(q[2 * d], f.x, acc);
        acc = fmaf(q[2 * d + 1], f.y, acc);
    }
    return acc;
}

// qkv bf16 [rows x 3072]; pos bf16 [kPosRows x 1024] (row p <-> relative position 187 - p);
// out bf16 [rows x 1024].  grid (heads, clips).
__global__ void __launch_bounds__(kAttThreads)
relpos_attention_kernel(const bf16* __restrict__ qkv, const int* __restrict__ t3_off, const bf16* __restrict__ pos,
                        const float* __restrict__ bias_u, const float* __restrict__ bias_v, bf16* __restrict__ out) {
    extern __shared__ __align__(16) unsigned char att_smem[];
    const int head = blockIdx.x, clip = blockIdx.y;
    const int r0 = t3_off[clip];
    const int t = t3_off[clip + 1] - r0;
    if (t <= 0) return;
    bf16* Ks = reinterpret_cast<bf16*>(att_smem);
    bf16* Vs = Ks + (size_t)kMaxEncFrames * kRowStride;
    bf16* Ps = Vs + (size_t)kMaxEncFrames * kRowStride;                 // 2t - 1 rows
    float* wbuf = reinterpret_cast<float*>(Ps + (size_t)kPosRows * kRowStride);  // per warp: qu[128], qv[128], p[192]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // stage K, V (this head) and the 2t - 1 position rows for relative positions t-1 .. -(t-1)
    for (int i = tid; i < t * (kHeadDim / 2); i += kAttThreads) {
        const int j = i / (kHeadDim / 2), d2 = i % (kHeadDim / 2);
        const bf16* src = qkv + (size_t)(r0 + j) * (3 * kDModel) + head * kHeadDim + 2 * d2;
        *reinterpret_cast<__nv_bfloat162*>(Ks + j * kRowStride + 2 * d2) =
            *reinterpret_cast<const __nv_bfloat162*>(src + kDModel);
        *reinterpret_cast<__nv_bfloat162*>(Vs + j * kRowStride + 2 * d2) =
            *reinterpret_cast<const __nv_bfloat162*>(src + 2 * kDModel);
    }
    const int p0 = (kMaxEncFrames - 1) - (t - 1);  // table row of relative position t - 1
    for (int i = tid; i < (2 * t - 1) * (kHeadDim / 2); i += kAttThreads) {
        const int pl = i / (kHeadDim / 2), d2 = i % (kHeadDim / 2);
        *reinterpret_cast<__nv_bfloat162*>(Ps + pl * kRowStride + 2 * d2) =
            *reinterpret_cast<const __nv_bfloat162*>(pos + (size_t)(p0 + pl) * kDModel + head * kHeadDim + 2 * d2);
    }
    __syncthreads();

    float* qu = wbuf + warp * (2 * kHeadDim + 192);
    float* qv = qu + kHeadDim;
    float* pr = qv + kHeadDim;
    const float scale = 0.08838834764831845f;  // 1 / sqrt(128)
    for (int i = warp; i < t; i += kAttThreads / 32) {
        const bf16* qrow = qkv + (size_t)(r0 + i) * (3 * kDModel) + head * kHeadDim;
        for (int d = lane; d < kHeadDim; d += 32) {
            const float q = __bfloat162float(qrow[d]);
            qu[d] = q + bias_u[head * kHeadDim + d];
            qv[d] = q + bias_v[head * kHeadDim + d];
        }
        __syncwarp();
        float mx = -INFINITY;
        for (int j = lane; j < t; j += 32) {
            const float ac = dot128(qu, Ks + j * kRowStride);
            // relative position i - j lives in local row (t - 1) - (i - j)
            const float bd = dot128(qv, Ps + ((t - 1) - i + j) * kRowStride);
            const float s = (ac + bd) * scale;
            pr[j] = s;
            mx = fmaxf(mx, s);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float sum = 0.0f;
        for (int j = lane; j < t; j += 32) {
            const float e = __expf(pr[j] - mx);
            pr[j] = e;
            sum += e;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float inv = 1.0f / sum;
        __syncwarp();
        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
        for (int j = 0; j < t; ++j) {
            const float p = pr[j];
            const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(Vs + j * kRowStride + 4 * lane);
            const float2 f0 = __bfloat1622float2(v2[0]), f1 = __bfloat1622float2(v2[1]);
            a0 = fmaf(p, f0.x, a0); a1 = fmaf(p, f0.y, a1); a2 = fmaf(p, f1.x, a2); a3 = fmaf(p, f1.y, a3);
        }
        __nv_bfloat162 o0 = __floats2bfloat162_rn(a0 * inv, a1 * inv), o1 = __floats2bfloat162_rn(a2 * inv, a3 * inv);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&o0);
        pk.y = *reinterpret_cast<uint32_t*>(&o1);
        *reinterpret_cast<uint2*>(out + (size_t)(r0 + i) * kDModel + head * kHeadDim + 4 * lane) = pk;
        __syncwarp();
    }
}

constexpr size_t kAttSmemBytes = ((size_t)(2 * kMaxEncFrames + kPosRows) * kRowStride) * sizeof(bf16) +
                                 (size_t)(kAttThreads / 32) * (2 * kHeadDim + 192) * sizeof(float);

// ---------------------------------------------------------------- depthwise conv + BN + SiLU
// in bf16 [rows x 1024] (the GLU is applied by the epilogue of the first pointwise GEMM) -> out bf16 [rows x 1024].
// grid (time blocks of 32, clips); a CTA walks the four 256-channel blocks of its rows: the bf16 tile
// [40 rows x 256 channels] of the next block arrives by cp.async (zero outside the clip) while the current one is
// convolved; each thread convolves two channels over 16 rows, reading its window straight from the bf16 tile.
constexpr int kDwRows = 32;
constexpr int kDwHalo = (kConvK - 1) / 2;
constexpr int kDwTileRows = kDwRows + kConvK - 1;
__global__ void __launch_bounds__(256)
dwconv_kernel(const bf16* __restrict__ in, const int* __restrict__ t3_off, const float* __restrict__ w,
              const float* __restrict__ b, bf16* __restrict__ out) {
    __shared__ __align__(16) bf16 tile[2][kDwTileRows][256];
    const int clip = blockIdx.y;
    const int r0 = t3_off[clip];
    const int t = t3_off[clip + 1] - r0;
    const int tb = blockIdx.x * kDwRows;
    if (tb >= t) return;
    auto fetch = [&](int zb, int buf) {
        for (int idx = threadIdx.x; idx < kDwTileRows * 32; idx += 256) {
            const int r = idx >> 5, v8 = (idx & 31) * 8;
            const int tt = tb - kDwHalo + r;
            const bool ok = tt >= 0 && tt < t;
            const bf16* src = in + (size_t)(r0 + (ok ? tt : 0)) * kDModel + zb * 256 + v8;
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(&tile[buf][r][v8]);
            const int bytes = ok ? 16 : 0;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch(0, 0);
    const int cp = (threadIdx.x & 127) * 2, rh = (threadIdx.x >> 7) * (kDwRows / 2);
    for (int zb = 0; zb < kDModel / 256; ++zb) {
        const int buf = zb & 1;
        if (zb + 1 < kDModel / 256) fetch(zb + 1, buf ^ 1);
        else asm volatile("cp.async.commit_group;" ::: "memory");
        const int c0 = zb * 256;
        float w0[kConvK], w1[kConvK];
#pragma unroll
        for (int k = 0; k < kConvK; ++k) {
            const float2 wk = *reinterpret_cast<const float2*>(w + k * kDModel + c0 + cp);
            w0[k] = wk.x;
            w1[k] = wk.y;
        }
        const float2 bb = *reinterpret_cast<const float2*>(b + c0 + cp);
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();  // this block's tile is complete
        float2 win[kDwRows / 2 + kConvK - 1];
#pragma unroll
        for (int r = 0; r < kDwRows / 2 + kConvK - 1; ++r)
            win[r] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&tile[buf][rh + r][cp]));
#pragma unroll
        for (int r = 0; r < kDwRows / 2; ++r) {
            if (tb + rh + r >= t) break;
            float a0 = bb.x, a1 = bb.y;
#pragma unroll
            for (int k = 0; k < kConvK; ++k) {
                a0 = fmaf(w0[k], win[r + k].x, a0);
                a1 = fmaf(w1[k], win[r + k].y, a1);
            }
            a0 = ptx::silu_fast(a0);
            a1 = ptx::silu_fast(a1);
            *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(r0 + tb + rh + r) * kDModel + c0 + cp) =
                __floats2bfloat162_rn(a0, a1);
        }
        __syncthreads();  // the buffer is refilled two iterations from now
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
}

cudaError_t run_gemm(sb_ctx* c, const char* label, const void* a, const bf16* w, const float* bias, void* out, int M, int N,
                     int K, int act, int mode, float alpha) {
    GemmArgs g{};
    g.a = a; g.w = w; g.bias = bias; g.out = out; g.M = M; g.N = N; g.K = K; g.ldo = act == kActGlu ? N / 2 : N; g.act = act;
    g.out_mode = mode; g.alpha = alpha; g.fp8 = false;
    c->launches += 1;
    c->prof.begin(label, c->stream);
    cudaError_t e = gemm_launch(g, c->sm_count, c->d_error, c->stream);
    c->prof.end(c->stream);
    return e;
}

cudaError_t run_gemm_fp8(sb_ctx* c, const char* label, const uint8_t* a, const float* a_scale, const uint8_t* w,
                         const float* w_scale, const float* bias, void* out, int M, int N, int K, int act, int mode,
                         float alpha, const float* out_row_scale = nullptr) {
    GemmArgs g{};
    g.a = a; g.w = w; g.bias = bias; g.row_scale = a_scale; g.col_scale = w_scale; g.out = out; g.M = M; g.N = N; g.K = K;
    g.ldo = act == kActGlu ? N / 2 : N; g.act = act; g.out_mode = mode; g.alpha = alpha; g.fp8 = true; g.out_row_scale = out_row_scale;
    c->launches += 1;
    c->prof.begin(label, c->stream);
    cudaError_t e = gemm_launch(g, c->sm_count, c->d_error, c->stream);
    c->prof.end(c->stream);
    return e;
}

#define PROF(label, launch)              \
    do {                                 \
        c->prof.begin(label, st);        \
        launch;                          \
        c->prof.end(st);                 \
    } while (0)

#define ENC_CUDA(expr)                       \
    do {                                     \
        cudaError_t _e = (expr);             \
        if (_e != cudaSuccess) return _e;    \
    } while (0)

}  // namespace

cudaError_t encoder_configure() {
    cudaError_t e = attention_configure();
    if (e != cudaSuccess) return e;
    e = subsample_configure();
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(relpos_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)kAttSmemBytes);
}

int encoder_out_frames(int mel_frames) {
    int t = mel_frames;
    for (int i = 0; i < 3; ++i) t = (t - 1) / 2 + 1;
    return t;
}

// Runs the encoder on clips [c0, c1) of a packed feature batch.  frame_off: host prefix sums of mel
// frames per clip (size n + 1, relative to d_feats).  d_out receives [sum T' x 1024] f32 for the group,
// written at row enc_off[c0].
static cudaError_t encode_group(sb_ctx* c, const Model& m, const float* d_feats, const int64_t* frame_off, int c0, int c1,
                                const int* enc_off_all, float* d_out, EncoderWorkspace& ws) {
    const int n = c1 - c0;
    std::vector<int64_t> t0(n + 1);
    std::vector<int> t1(n + 1), t2(n + 1), t3(n + 1);
    t0[0] = frame_off[c0];
    t1[0] = t2[0] = t3[0] = 0;
    for (int i = 0; i < n; ++i) {
        const int T = (int)(frame_off[c0 + i + 1] - frame_off[c0 + i]);
        const int a = (T - 1) / 2 + 1, b = (a - 1) / 2 + 1, d = (b - 1) / 2 + 1;
        t0[i + 1] = t0[i] + T;
        t1[i + 1] = t1[i] + a;
        t2[i + 1] = t2[i] + b;
        t3[i + 1] = t3[i] + d;
    }
    const int R2 = t2[n], R3 = t3[n];
    const int max_t3 = [&] { int mx = 0; for (int i = 0; i < n; ++i) mx = std::max(mx, t3[i + 1] - t3[i]); return mx; }();
    if (max_t3 > kMaxEncFrames) return cudaErrorInvalidValue;
    cudaStream_t st = c->stream;
    // offsets -> device (one buffer: t0 as int64, then three int arrays)
    const size_t off_bytes = sizeof(int64_t) * (n + 1) + 3 * sizeof(int) * (n + 1) + 64;
    ENC_CUDA(ws.offsets.ensure(off_bytes));
    int64_t* d_t0 = ws.offsets.as<int64_t>();
    int* d_t1 = reinterpret_cast<int*>(d_t0 + (n + 1));
    int* d_t2 = d_t1 + (n + 1);
    int* d_t3 = d_t2 + (n + 1);
    ENC_CUDA(cudaMemcpyAsync(d_t0, t0.data(), sizeof(int64_t) * (n + 1), cudaMemcpyHostToDevice, st));
    ENC_CUDA(cudaMemcpyAsync(d_t1, t1.data(), sizeof(int) * (n + 1), cudaMemcpyHostToDevice, st));
    ENC_CUDA(cudaMemcpyAsync(d_t2, t2.data(), sizeof(int) * (n + 1), cudaMemcpyHostToDevice, st));
    ENC_CUDA(cudaMemcpyAsync(d_t3, t3.data(), sizeof(int) * (n + 1), cudaMemcpyHostToDevice, st));

    ENC_CUDA(ws.y1.ensure((size_t)R2 * 32 * kSubC * sizeof(bf16)));
    ENC_CUDA(ws.y2.ensure((size_t)R2 * 32 * kSubC * sizeof(bf16)));
    ENC_CUDA(ws.y3.ensure((size_t)R3 * 16 * kSubC * sizeof(bf16)));
    ENC_CUDA(ws.y4.ensure((size_t)R3 * 16 * kSubC * sizeof(bf16)));
    ENC_CUDA(ws.x.ensure((size_t)R3 * kDModel * sizeof(float)));
    ENC_CUDA(ws.a.ensure((size_t)R3 * kDModel * sizeof(bf16)));
    ENC_CUDA(ws.h.ensure((size_t)R3 * kFF * sizeof(bf16)));
    ENC_CUDA(ws.att.ensure((size_t)R3 * kDModel * sizeof(bf16)));
    if (c->fp8 && m.has_fp8) {
        ENC_CUDA(ws.h8.ensure((size_t)R3 * kFF));
        ENC_CUDA(ws.rs.ensure((size_t)R3 * 2 * sizeof(float)));
    }

    // sub-sampling
    {
        constexpr int kTO = 2;
        int max_t2 = 0;
        for (int i = 0; i < n; ++i) max_t2 = std::max(max_t2, t2[i + 1] - t2[i]);
        const dim3 grid((max_t2 + kTO - 1) / kTO, n);
        if (c->simt_subsample) {
            PROF("sub_conv0_dw1_simt", (sub_conv0_dw1_kernel<kTO><<<grid, 256, 0, st>>>(d_feats, d_t0, d_t1, d_t2, m.sub0_w, m.sub0_b,
                                                                                       m.dw1_w, m.dw1_b, ws.y1.as<bf16>())));
        } else {
            c->prof.begin("sub_conv0_dw1", st);
            ENC_CUDA(subsample_conv0_dw1_launch(d_feats, d_t0, d_t1, d_t2, n, max_t2, m.sub0_frag, m.dw1_pairs, ws.y1.p, st));
            c->prof.end(st);
        }
        c->launches += 1;
    }
    ENC_CUDA(run_gemm(c, "gemm_sub_pw", ws.y1.p, m.pw1_w, m.pw1_b, ws.y2.p, R2 * 32, kSubC, kSubC, kActRelu, kOutBf16, 1.0f));
    PROF("sub_dw2", (sub_dw_kernel<2><<<dim3((max_t3 + 3) / 4, n), 256, 0, st>>>(ws.y2.as<bf16>(), d_t2, d_t3, 32, m.dw2_w, m.dw2_b,
                                                                                ws.y3.as<bf16>())));
    c->launches += 1;
    ENC_CUDA(run_gemm(c, "gemm_sub_pw", ws.y3.p, m.pw2_w, m.pw2_b, ws.y4.p, R3 * 16, kSubC, kSubC, kActRelu, kOutBf16, 1.0f));
    float* x = ws.x.as<float>();
    ENC_CUDA(run_gemm(c, "gemm_sub_linear", ws.y4.p, m.lin_w, m.lin_b, x, R3, kDModel, 16 * kSubC, kActNone, kOutF32, m.xscale));

    const int ln_grid = (R3 + 7) / 8;
    bf16* a = ws.a.as<bf16>();
    bf16* h = ws.h.as<bf16>();
    bf16* att = ws.att.as<bf16>();
    const bool fp8 = c->fp8 && m.has_fp8;
    uint8_t* a8 = reinterpret_cast<uint8_t*>(a);        // e4m3 LayerNorm output shares the bf16 buffer
    uint8_t* h8 = ws.h8.as<uint8_t>();
    float* rs_a = ws.rs.as<float>();
    float* rs_h = rs_a + R3;
    // feed-forward module: x += 0.5 * W2 silu(W1 LN(x) + b1) + b2
    auto feed_forward = [&](const float* pg, const float* pb, const float* g, const float* b, const bf16* w1, const uint8_t* w1q, const float* w1s,
                            const float* b1, const bf16* w2, const uint8_t* w2q, const float* w2s,
                            const float* b2, float wn, float bmax) -> cudaError_t {
        if (fp8 && (c->fp8_mask & 3) == 3 && !c->fp8_hidden_amax) {
            // LayerNorm -> e4m3; up-projection writes the e4m3 hidden row with a scale bounded in advance
            PROF("layernorm_fp8", (layernorm_fp8_kernel<<<ln_grid, 256, 0, st>>>(x, pg, pb, g, b, a8, rs_a, R3, rs_h, wn, bmax)));
            ENC_CUDA(run_gemm_fp8(c, "gemm_ff_up_fp8", a8, rs_a, w1q, w1s, b1, h8, R3, kFF, kDModel, kActSilu, kOutFp8, 1.0f, rs_h));
            ENC_CUDA(run_gemm_fp8(c, "gemm_ff_down_fp8", h8, rs_h, w2q, w2s, b2, x, R3, kDModel, kFF, kActNone, kOutResidual, 0.5f));
            c->launches += 1;
        } else if (fp8 && (c->fp8_mask & 3)) {
            if (c->fp8_mask & 1) {
                PROF("layernorm_fp8", (layernorm_fp8_kernel<<<ln_grid, 256, 0, st>>>(x, pg, pb, g, b, a8, rs_a, R3, nullptr, 0.0f, 0.0f)));
                ENC_CUDA(run_gemm_fp8(c, "gemm_ff_up_fp8", a8, rs_a, w1q, w1s, b1, h, R3, kFF, kDModel, kActSilu, kOutBf16, 1.0f));
            } else {
                PROF("layernorm", (layernorm_kernel<false><<<ln_grid, 256, 0, st>>>(x, pg, pb, g, b, a, R3)));
                ENC_CUDA(run_gemm(c, "gemm_ff_up", a, w1, b1, h, R3, kFF, kDModel, kActSilu, kOutBf16, 1.0f));
            }
            if (c->fp8_mask & 2) {
                PROF("quantize_rows", (quantize_rows4096_kernel<<<ln_grid, 256, 0, st>>>(h, h8, rs_h, R3)));
                ENC_CUDA(run_gemm_fp8(c, "gemm_ff_down_fp8", h8, rs_h, w2q, w2s, b2, x, R3, kDModel, kFF, kActNone, kOutResidual, 0.5f));
                c->launches += 1;
            } else {
                ENC_CUDA(run_gemm(c, "gemm_ff_down", h, w2, b2, x, R3, kDModel, kFF, kActNone, kOutResidual, 0.5f));
            }
            c->launches += 1;
        } else {
            PROF("layernorm", (layernorm_kernel<false><<<ln_grid, 256, 0, st>>>(x, pg, pb, g, b, a, R3)));
            ENC_CUDA(run_gemm(c, "gemm_ff_up", a, w1, b1, h, R3, kFF, kDModel, kActSilu, kOutBf16, 1.0f));
            ENC_CUDA(run_gemm(c, "gemm_ff_down", h, w2, b2, x, R3, kDModel, kFF, kActNone, kOutResidual, 0.5f));
            c->launches += 1;
        }
        return cudaSuccess;
    };
    // LayerNorm followed by a projection to bf16 (QKV, first pointwise conv)
    auto norm_project = [&](const char* label, const char* label8, const float* g, const float* b, const bf16* w,
                            const uint8_t* wq, const float* wsc, const float* bias, int N, int act) -> cudaError_t {
        if (fp8 && (c->fp8_mask & (N == 3 * kDModel ? 4 : 8))) {
            PROF("layernorm_fp8", (layernorm_fp8_kernel<<<ln_grid, 256, 0, st>>>(x, nullptr, nullptr, g, b, a8, rs_a, R3, nullptr, 0.0f, 0.0f)));
            ENC_CUDA(run_gemm_fp8(c, label8, a8, rs_a, wq, wsc, bias, h, R3, N, kDModel, act, kOutBf16, 1.0f));
        } else {
            PROF("layernorm", (layernorm_kernel<false><<<ln_grid, 256, 0, st>>>(x, nullptr, nullptr, g, b, a, R3)));
            ENC_CUDA(run_gemm(c, label, a, w, bias, h, R3, N, kDModel, act, kOutBf16, 1.0f));
        }
        c->launches += 1;
        return cudaSuccess;
    };
    for (int l = 0; l < m.layers; ++l) {
        const LayerWeights& L = m.L[l];
        // x += 0.5 * FF1(LN x)
        // (for blocks after the first, the previous block's closing LayerNorm runs inside this one's first)
        const float* pre_g = l > 0 ? m.L[l - 1].ln_out_g : nullptr;
        const float* pre_b = l > 0 ? m.L[l - 1].ln_out_b : nullptr;
        ENC_CUDA(feed_forward(pre_g, pre_b, L.ln_ff1_g, L.ln_ff1_b, L.ff1_w1, L.ff1_w1_q, L.ff1_w1_s, L.ff1_b1, L.ff1_w2, L.ff1_w2_q,
                              L.ff1_w2_s, L.ff1_b2, L.ff1_wn, L.ff1_bmax));
        // x += MHA(LN x)
        ENC_CUDA(norm_project("gemm_qkv", "gemm_qkv_fp8", L.ln_att_g, L.ln_att_b, L.qkv_w, L.qkv_w_q, L.qkv_w_s, L.qkv_b,
                              3 * kDModel, kActNone));
        if (c->simt_attention) {
            PROF("relpos_attention_simt", (relpos_attention_kernel<<<dim3(kHeads, n), kAttThreads, kAttSmemBytes, st>>>(
                                              h, d_t3, L.pos_proj, L.bias_u, L.bias_v, att)));
        } else {
            c->prof.begin("relpos_attention_tc", st);
            ENC_CUDA(attention_launch(h, R3, d_t3, n, L.pos_proj, L.bias_u, L.pos_vp, att, c->sm_count, c->d_error, st));
            c->prof.end(st);
            c->launches += 1;
        }
        ENC_CUDA(run_gemm(c, "gemm_attn_out", att, L.o_w, L.o_b, x, R3, kDModel, kDModel, kActNone, kOutResidual, 1.0f));
        // x += Conv(LN x)
        ENC_CUDA(norm_project("gemm_conv_pw1", "gemm_conv_pw1_fp8", L.ln_conv_g, L.ln_conv_b, L.pw1_w, L.pw1_w_q,
                              L.pw1_w_s, L.pw1_b, 2 * kDModel, kActGlu));  // h = GLU(W1 LN(x) + b1), [rows x 1024]
        PROF("dwconv", (dwconv_kernel<<<dim3((max_t3 + kDwRows - 1) / kDwRows, n), 256, 0, st>>>(
                               h, d_t3, L.dw_w, L.dw_b, att)));
        ENC_CUDA(run_gemm(c, "gemm_conv_pw2", att, L.pw2_w, L.pw2_b, x, R3, kDModel, kDModel, kActNone, kOutResidual, 1.0f));
        // x += 0.5 * FF2(LN x)
        ENC_CUDA(feed_forward(nullptr, nullptr, L.ln_ff2_g, L.ln_ff2_b, L.ff2_w1, L.ff2_w1_q, L.ff2_w1_s, L.ff2_b1, L.ff2_w2, L.ff2_w2_q,
                              L.ff2_w2_s, L.ff2_b2, L.ff2_wn, L.ff2_bmax));
        // x = LN_out(x): the last block writes straight into the caller's buffer; the others leave it to the
        // next block's first LayerNorm
        if (l == m.layers - 1) {
            float* dst = d_out + (size_t)enc_off_all[c0] * kDModel;
            PROF("layernorm", (layernorm_kernel<true><<<ln_grid, 256, 0, st>>>(x, nullptr, nullptr, L.ln_out_g, L.ln_out_b, dst, R3)));
            c->launches += 1;
        }
        c->launches += 1;  // depthwise convolution
    }
    if (m.layers == 0)
        ENC_CUDA(cudaMemcpyAsync(d_out + (size_t)enc_off_all[c0] * kDModel, x, (size_t)R3 * kDModel * sizeof(float),
                                 cudaMemcpyDeviceToDevice, st));
    return cudaGetLastError();
}

cudaError_t encoder_forward(sb_ctx* c, const Model& m, const float* d_feats, const int64_t* frame_off, int n_clips,
                            float* d_out, int* enc_off, EncoderWorkspace& ws, size_t workspace_budget_bytes) {
    enc_off[0] = 0;
    for (int i = 0; i < n_clips; ++i)
        enc_off[i + 1] = enc_off[i] + encoder_out_frames((int)(frame_off[i + 1] - frame_off[i]));
    // group clips so that the intermediates of a group fit the budget
    int c0 = 0;
    while (c0 < n_clips) {
        size_t bytes = 0;
        int c1 = c0;
        while (c1 < n_clips) {
            const size_t T = (size_t)(frame_off[c1 + 1] - frame_off[c1]);
            const size_t T2 = ((T - 1) / 2 + 1 - 1) / 2 + 1, T3 = (T2 - 1) / 2 + 1;
            // two [T2 x 32 x 256] and two [T3 x 16 x 256] bf16 sub-sampling stages, then per encoder frame the f32
            // stream, bf16 LayerNorm / attention outputs, the 4096-wide hidden row (bf16 and e4m3)
            const size_t need = T2 * 32 * kSubC * 2 * 2 + T3 * 16 * kSubC * 2 * 2 +
                                T3 * (kDModel * (4 + 2 + 2) + kFF * (2 + 1) + 16);
            if (c1 > c0 && (bytes + need > workspace_budget_bytes || c1 - c0 >= 32768)) break;
            bytes += need;
            ++c1;
        }
        ENC_CUDA(encode_group(c, m, d_feats, frame_off, c0, c1, enc_off, d_out, ws));
        c0 = c1;
    }
    return cudaSuccess;
}

}  // namespace sb
