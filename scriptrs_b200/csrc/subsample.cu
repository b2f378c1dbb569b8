// First two stages of the dw-striding sub-sampling on sm_100a, in one kernel:
//   conv2d(1 -> 256, k3, s2, p1) + ReLU          as a product [positions x 16] x [16 x 256] on the tensor cores
//   depthwise conv2d(256, k3, s2, p1) + bias     on packed fp16 pairs
// Part of the encoder that the reference runs as a CoreML blob (src/model.rs:327-342, contract src/coreml.rs:75-135).
//   feats f32 [sum T x 128]  ->  out bf16 [sum T2 x 32 x 256]   (channels last; T1 = (T-1)/2+1, T2 = (T1-1)/2+1)
// The [T1 x 64 x 256] map between the two stages never reaches memory.
//
// grid (ceil(max T2 / 2), clips), 256 threads.  A CTA produces 2 output time rows: it stages the 11 mel rows they
// depend on, gathers the 3 x 3 input patches of the 5 x 64 first-stage positions into an im2col tile of fp16
// (9 taps, a constant 1 that carries the bias, 6 zeros: K = 16), and then walks the channels in four blocks of 64:
//   product   mma.m16n8k16 (fp16 in, fp32 accumulate): each warp takes first-stage position tiles of 16 and all
//             8 channel tiles of the block; ReLU, rows outside the clip forced to zero (they are the second stage's
//             padding), fp16 pairs into a [5 rows x 65 columns x 64 channels] tile (column slot 0 = padding)
//   depthwise each thread owns a channel pair and four output frequencies per row and slides a 3 x 9 window over
//             the tile; fp16 multiply-adds (the result is rounded to bf16 anyway), bf16 pairs out, 128 bytes per warp
// fp16 keeps 11 significant bits of the normalised features and of the weights; the accumulation of the first stage
// is fp32.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "subsample.h"

namespace sb {

namespace {

constexpr int kTO = 2;                // output time rows per CTA
constexpr int kNY = 2 * kTO + 1;      // first-stage rows per CTA
constexpr int kNX = 4 * kTO + 3;      // mel rows per CTA
constexpr int kXS = kMelBins + 8;     // floats per staged mel row; mel column f sits at index f + 4
constexpr int kPos = kNY * 64;        // first-stage positions per CTA
constexpr int kY0Stride = 72;         // halfs per (row, column slot) of the first-stage tile: 64 channels + 8 (36 words:
                                      // the eight positions x four channel pairs one store instruction writes fall
                                      // into 32 different banks)

struct __align__(16) SmemLayout {
    float xs[kNX][kXS];
    __half im2col[kPos][16];
    __half y0[kNY][65][kY0Stride];
};

__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint2 b) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b.x), "r"(b.y));
}

__device__ __forceinline__ uint32_t relu_pack(float a, float b) {
    const __half2 h = __hmax2(__floats2half2_rn(a, b), __float2half2_rn(0.0f));
    return *reinterpret_cast<const uint32_t*>(&h);
}

__global__ void __launch_bounds__(256, 3)
sub_conv0_dw1_tc_kernel(const float* __restrict__ feats, const int64_t* __restrict__ t0_off, const int* __restrict__ t1_off,
                        const int* __restrict__ t2_off, const uint2* __restrict__ w0_frag, const __half2* __restrict__ w1h,
                        __nv_bfloat16* __restrict__ out) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    SmemLayout& sm = *reinterpret_cast<SmemLayout*>(smem_raw);
    const int clip = blockIdx.y, to0 = blockIdx.x * kTO;
    const int out_base = t2_off[clip];
    const int T2 = t2_off[clip + 1] - out_base;
    if (to0 >= T2) return;
    const int64_t base = t0_off[clip];
    const int T = (int)(t0_off[clip + 1] - base);
    const int T1 = t1_off[clip + 1] - t1_off[clip];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // mel rows 4 to0 - 3 .. 4 to0 + 4 TO - 1, zero outside the clip and outside the 128 columns
    for (int i = tid; i < kNX * kXS; i += 256) {
        const int row = i / kXS, col = i % kXS - 4;
        const int r = 4 * to0 - 3 + row;
        float v = 0.0f;
        if (r >= 0 && r < T && col >= 0 && col < kMelBins) v = feats[(base + r) * kMelBins + col];
        sm.xs[row][i % kXS] = v;
    }
    // column slot 0 of the first-stage tile is the zero padding left of frequency 0
    for (int i = tid; i < kNY * kY0Stride; i += 256) sm.y0[i / kY0Stride][0][i % kY0Stride] = __float2half(0.0f);
    __syncthreads();
    // im2col: position (first-stage row ry, frequency f) <- its 3 x 3 patch, then 1 (bias), then zeros
    for (int pos = tid; pos < kPos; pos += 256) {
        const int ry = pos >> 6, f = pos & 63;
        __half h[16];
#pragma unroll
        for (int dt = 0; dt < 3; ++dt)
#pragma unroll
            for (int df = 0; df < 3; ++df) h[3 * dt + df] = __float2half_rn(sm.xs[2 * ry + dt][2 * f + df + 3]);
        h[9] = __float2half(1.0f);
#pragma unroll
        for (int k = 10; k < 16; ++k) h[k] = __float2half(0.0f);
        uint4* dst = reinterpret_cast<uint4*>(sm.im2col[pos]);
        dst[0] = *reinterpret_cast<const uint4*>(&h[0]);
        dst[1] = *reinterpret_cast<const uint4*>(&h[8]);
    }
    __syncthreads();

    const int g = lane >> 2, t = lane & 3;
    const uint32_t* im = reinterpret_cast<const uint32_t*>(&sm.im2col[0][0]);  // 8 words per position
    uint32_t* y0w = reinterpret_cast<uint32_t*>(&sm.y0[0][0][0]);              // kY0Stride / 2 words per (row, slot)
    const __half2* y0h = reinterpret_cast<const __half2*>(&sm.y0[0][0][0]);
    const int cp = lane, pg = warp;  // depthwise stage: channel pair within the block, group of four output frequencies

    for (int zb = 0; zb < 4; ++zb) {
        // ---- first stage for channels 64 zb .. 64 zb + 63
        uint2 bfrag[8];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) bfrag[nt] = __ldg(w0_frag + (zb * 8 + nt) * 32 + lane);
        for (int mt = warp; mt < kNY * 4; mt += 8) {
            const int ry = mt >> 2, f0 = (mt & 3) * 16;
            const int p0 = ry * 64 + f0 + g;
            uint32_t a[4];
            a[0] = im[p0 * 8 + t];
            a[1] = im[(p0 + 8) * 8 + t];
            a[2] = im[p0 * 8 + 4 + t];
            a[3] = im[(p0 + 8) * 8 + 4 + t];
            const int r = 2 * to0 - 1 + ry;
            const bool valid = r >= 0 && r < T1;  // rows outside the first-stage map are the second stage's padding
            uint32_t* dst0 = y0w + (ry * 65 + f0 + g + 1) * (kY0Stride / 2) + t;
            uint32_t* dst1 = dst0 + 8 * (kY0Stride / 2);
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                mma_f16(c, a, bfrag[nt]);
                dst0[nt * 4] = valid ? relu_pack(c[0], c[1]) : 0u;
                dst1[nt * 4] = valid ? relu_pack(c[2], c[3]) : 0u;
            }
        }
        __syncthreads();
        // ---- depthwise stage for the same channels
        {
            __half2 w[9];
#pragma unroll
            for (int k = 0; k < 9; ++k) w[k] = __ldg(w1h + k * (kSubChannels / 2) + zb * 32 + cp);
            const __half2 bias = __ldg(w1h + 9 * (kSubChannels / 2) + zb * 32 + cp);
#pragma unroll
            for (int j = 0; j < kTO; ++j) {
                if (to0 + j >= T2) break;
                __half2 acc[4] = {bias, bias, bias, bias};
#pragma unroll
                for (int dt = 0; dt < 3; ++dt) {
                    __half2 v[9];
                    const __half2* rowp = y0h + ((2 * j + dt) * 65 + 8 * pg) * (kY0Stride / 2) + cp;
#pragma unroll
                    for (int s = 0; s < 9; ++s) v[s] = rowp[s * (kY0Stride / 2)];
#pragma unroll
                    for (int o = 0; o < 4; ++o)
#pragma unroll
                        for (int df = 0; df < 3; ++df) acc[o] = __hfma2(w[3 * dt + df], v[2 * o + df], acc[o]);
                }
                __nv_bfloat16* orow = out + ((size_t)(out_base + to0 + j) * 32 + 4 * pg) * kSubChannels + zb * 64 + 2 * cp;
#pragma unroll
                for (int o = 0; o < 4; ++o) {
                    const float2 f = __half22float2(acc[o]);
                    *reinterpret_cast<__nv_bfloat162*>(orow + (size_t)o * kSubChannels) = __floats2bfloat162_rn(f.x, f.y);
                }
            }
        }
        __syncthreads();  // the tile is overwritten by the next channel block
    }
}

}  // namespace

size_t subsample_frag_count() { return (size_t)4 * 8 * 32; }

// w0 [256 x 9] (channel-major, taps 3 dt + df), b0 [256] -> B fragments of mma.m16n8k16 for every channel tile:
// lane (g = lane >> 2, t = lane & 3) of tile (zb, nt) holds {k = 2t, 2t+1} and {k = 2t+8, 2t+9} of channel
// 64 zb + 8 nt + g, with k < 9 the taps, k = 9 the bias (the im2col tile holds a 1 there) and zeros above.
void subsample_build_frags(const float* w0, const float* b0, uint2* frags) {
    for (int zb = 0; zb < 4; ++zb)
        for (int nt = 0; nt < 8; ++nt)
            for (int lane = 0; lane < 32; ++lane) {
                const int g = lane >> 2, t = lane & 3, ch = 64 * zb + 8 * nt + g;
                auto tap = [&](int k) { return k < 9 ? w0[ch * 9 + k] : (k == 9 ? b0[ch] : 0.0f); };
                const __half2 lo = __floats2half2_rn(tap(2 * t), tap(2 * t + 1));
                const __half2 hi = __floats2half2_rn(tap(2 * t + 8), tap(2 * t + 9));
                uint2 v;
                v.x = *reinterpret_cast<const uint32_t*>(&lo);
                v.y = *reinterpret_cast<const uint32_t*>(&hi);
                frags[(zb * 8 + nt) * 32 + lane] = v;
            }
}

// w1 tap-major [9 x 256] f32 and b1 [256] -> [10 x 128] fp16 pairs (row 9 = bias)
void subsample_build_dw(const float* w1_tap_major, const float* b1, uint32_t* out_pairs) {
    for (int k = 0; k < 10; ++k)
        for (int c2 = 0; c2 < kSubChannels / 2; ++c2) {
            const float a = k < 9 ? w1_tap_major[k * kSubChannels + 2 * c2] : b1[2 * c2];
            const float b = k < 9 ? w1_tap_major[k * kSubChannels + 2 * c2 + 1] : b1[2 * c2 + 1];
            const __half2 h = __floats2half2_rn(a, b);
            out_pairs[k * (kSubChannels / 2) + c2] = *reinterpret_cast<const uint32_t*>(&h);
        }
}

cudaError_t subsample_configure() {
    return cudaFuncSetAttribute(sub_conv0_dw1_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SmemLayout));
}

cudaError_t subsample_conv0_dw1_launch(const float* feats, const int64_t* d_t0, const int* d_t1, const int* d_t2, int n_clips,
                                       int max_t2, const void* w0_frag, const void* w1_pairs, void* out, cudaStream_t st) {
    if (n_clips <= 0 || max_t2 <= 0) return cudaSuccess;
    const dim3 grid((max_t2 + kTO - 1) / kTO, n_clips);
    sub_conv0_dw1_tc_kernel<<<grid, 256, sizeof(SmemLayout), st>>>(feats, d_t0, d_t1, d_t2, static_cast<const uint2*>(w0_frag),
                                                                  static_cast<const __half2*>(w1_pairs),
                                                                  static_cast<__nv_bfloat16*>(out));
    return cudaGetLastError();
}

}  // namespace sb
