// Log-mel frontend for sm_100a: PCM f32 -> normalised log-mel [T x 128] per clip.
//
// Replaces the reference's CPU feature extractor (src/frontend.rs:104-241):
// pre-emphasis 0.97, 256-sample zero padding on both sides, Hann window of 400
// left-aligned in a 512-point real FFT, power spectrum, 128-bin Slaney mel
// filterbank, ln(x + 2^-24), per-feature mean / variance normalisation over
// all frames of the clip.
//
// Three kernels:
//   logmel_kernel     a CTA walks four consecutive 32-frame tiles of a clip (tables and twiddles set up once, the
//                     next tile's raw samples arriving by cp.async while the current one is transformed);
//                     one warp per frame: pre-emphasised samples staged in shared
//                     memory, 256-point complex FFT of the even/odd-packed frame
//                     (8 x 8 x 4 decomposition: two register radix-8 passes with
//                     one shared-memory transpose, then a radix-4 across four
//                     adjacent lanes with shuffles), real-FFT untangling + power,
//                     sparse mel filterbank (504 non-zero taps), ln.
//   colstats_kernel   one thread per (clip, feature) walks the clip's frames in
//                     order and accumulates the mean and the variance exactly as
//                     the reference does (strictly sequential f32 sums, left to
//                     right): for a constant column (an all-zero clip) the result
//                     is made of the rounding residue of that sum alone, so any
//                     other summation order gives a different answer.
//   normalize_kernel  (v - mean) / std, elementwise, float4.
#include <cuda_runtime.h>
#include <stdint.h>

#include "frontend.h"

namespace sb {

namespace {

constexpr int kWarpsPerCta = 8;
constexpr int kThreads = kWarpsPerCta * 32;
constexpr int kFramesPerTile = 32;
constexpr int kTilesPerCta = 4;                                    // consecutive tiles of one clip per CTA
constexpr int kTileSamples = (kFramesPerTile - 1) * kHop + kWin;  // 5360
constexpr int kRawSamples = kTileSamples + 8 + 1;                  // the tile plus the sample before it
constexpr int kS1Stride = 36;                                      // float2 per k1 row, conflict-free
constexpr int kWarpScratchF2 = 8 * kS1Stride;                      // 288 float2 (>= 272 for the Z layout)
constexpr int kPowerPad = 272;                                     // 257 bins + slack for padded mel taps

struct __align__(16) SmemLayout {
    float xs[2][kRawSamples + 3];          // raw samples of the current and the next tile (cp.async ring)
    float ys[kTileSamples + 8];            // pre-emphasised, zero-padded samples of the tile
    float window[kWin];                    // Hann window
    float2 tw_post[132];                   // 0.5 * exp(-2*pi*i*k/512), k = 0..128
    float melw[kMaxTaps * kMels];          // tap-major: melw[j * 128 + m]
    int16_t mel_start[kMels];
    int16_t mel_cnt[kMels];
    float2 scratch[kWarpsPerCta][kWarpScratchF2];
    float power[kWarpsPerCta][kPowerPad];
};

__device__ __forceinline__ float2 cadd(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
__device__ __forceinline__ float2 csub(float2 a, float2 b) { return make_float2(a.x - b.x, a.y - b.y); }
__device__ __forceinline__ float2 cmul(float2 a, float2 b) {
    return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x);
}
// multiply by -i
__device__ __forceinline__ float2 mul_mi(float2 a) { return make_float2(a.y, -a.x); }

// Forward 8-point DFT, natural order in and out.
__device__ __forceinline__ void fft8(float2 (&a)[8]) {
    const float h = 0.70710678118654752440f;
    float2 b0 = cadd(a[0], a[4]), b1 = csub(a[0], a[4]);
    float2 b2 = cadd(a[2], a[6]), b3 = mul_mi(csub(a[2], a[6]));
    float2 b4 = cadd(a[1], a[5]), b5 = csub(a[1], a[5]);
    float2 b6 = cadd(a[3], a[7]), b7 = mul_mi(csub(a[3], a[7]));
    float2 e0 = cadd(b0, b2), e2 = csub(b0, b2), e1 = cadd(b1, b3), e3 = csub(b1, b3);
    float2 o0 = cadd(b4, b6), o2 = csub(b4, b6), o1 = cadd(b5, b7), o3 = csub(b5, b7);
    // W8^1 = (1 - i)/sqrt2, W8^2 = -i, W8^3 = (-1 - i)/sqrt2
    float2 t1 = make_float2((o1.x + o1.y) * h, (o1.y - o1.x) * h);
    float2 t2 = mul_mi(o2);
    float2 t3 = make_float2((o3.y - o3.x) * h, -(o3.x + o3.y) * h);
    a[0] = cadd(e0, o0); a[4] = csub(e0, o0);
    a[1] = cadd(e1, t1); a[5] = csub(e1, t1);
    a[2] = cadd(e2, t2); a[6] = csub(e2, t2);
    a[3] = cadd(e3, t3); a[7] = csub(e3, t3);
}

__device__ __forceinline__ float2 twiddle(int num, int den) {
    // exp(-2*pi*i*num/den)
    float s, c;
    sincospif(-2.0f * (float)num / (float)den, &s, &c);
    return make_float2(c, s);
}

__global__ void __launch_bounds__(kThreads, 2)
logmel_kernel(const float* __restrict__ pcm, const int64_t* __restrict__ clip_start,
              const int64_t* __restrict__ clip_len, const int64_t* __restrict__ frame_off, float* __restrict__ out, float preemph,
              const FrontendTables* __restrict__ tables) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    SmemLayout& sm = *reinterpret_cast<SmemLayout*>(smem_raw);

    const int clip = blockIdx.y;
    const int64_t c0 = clip_start[clip];
    const int64_t n = clip_len[clip];
    const int64_t fo = frame_off[clip];
    const int T = (int)(frame_off[clip + 1] - fo);
    const int tile0 = blockIdx.x * kTilesPerCta;
    if (tile0 * kFramesPerTile >= T) return;

    const int tid = threadIdx.x;
    const float* x = pcm + c0;
    // Raw samples of a tile -> shared memory, asynchronously; sample g of the clip sits at index g - s0 + 1, so
    // that the sample before the tile is there too; zero outside the clip (frontend.rs:59-65).
    auto fetch = [&](int tile, int buf) {
        const int64_t s0 = (int64_t)tile * kFramesPerTile * kHop - kPad;
        for (int i = tid; i < kRawSamples; i += kThreads) {
            const int64_t g = s0 - 1 + i;
            const bool in = g >= 0 && g < n && tile * kFramesPerTile < T;
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(&sm.xs[buf][i]);
            const int bytes = in ? 4 : 0;
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(x + (in ? g : 0)), "r"(bytes) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch(tile0, 0);
    // Tables -> shared memory.
    for (int i = tid; i < kWin; i += kThreads) sm.window[i] = tables->window[i];
    for (int i = tid; i < kMaxTaps * kMels; i += kThreads) sm.melw[i] = tables->melw[i];
    for (int i = tid; i < kMels; i += kThreads) {
        sm.mel_start[i] = tables->mel_start[i];
        sm.mel_cnt[i] = tables->mel_cnt[i];
    }
    for (int i = tid; i <= 128; i += kThreads) sm.tw_post[i] = tables->tw_post[i];

    const int warp = tid >> 5, lane = tid & 31;
    float2* sc = sm.scratch[warp];
    float* pw = sm.power[warp];
    if (lane < kPowerPad - 257) pw[257 + lane] = 0.0f;

    // Lane-constant twiddles.
    float2 tw1[8], tw2[8];
    const int k1s = lane >> 2, r2 = lane & 3;
#pragma unroll
    for (int k = 1; k < 8; ++k) {
        tw1[k] = twiddle(lane * k, 256);
        tw2[k] = twiddle(r2 * k, 32);
    }

    for (int tt = 0; tt < kTilesPerCta; ++tt) {
        const int f0 = (tile0 + tt) * kFramesPerTile;
        if (f0 >= T) break;
        const int buf = tt & 1;
        if (tt + 1 < kTilesPerCta) fetch(tile0 + tt + 1, buf ^ 1);  // lands while this tile is transformed
        else asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();  // this tile's raw samples are visible; the previous tile's frames are done with ys
        // Pre-emphasis (frontend.rs:150-159): y[0] = x[0]; y[i] = x[i] - c * x[i-1], product rounded first.
        {
            const int64_t s0 = (int64_t)f0 * kHop - kPad;
            const float* xr = sm.xs[buf];
            for (int i = tid; i < kTileSamples + 8; i += kThreads) {
                const int64_t g = s0 + i;
                sm.ys[i] = (g >= 0 && g < n) ? __fsub_rn(xr[i + 1], __fmul_rn(preemph, xr[i])) : 0.0f;
            }
        }
        __syncthreads();
        for (int fl = warp; fl < kFramesPerTile; fl += kWarpsPerCta) {
            const int f = f0 + fl;
            if (f >= T) break;
            const float* ys = sm.ys + fl * kHop;

            // ---- stage 1: z[n] = (x[2n], x[2n+1]) windowed; DFT-8 over n1 with n = 32*n1 + lane
            float2 a[8];
#pragma unroll
            for (int n1 = 0; n1 < 8; ++n1) {
                const int nn = 32 * n1 + lane;
                if (nn < kWin / 2) {
                    const float2 v = *reinterpret_cast<const float2*>(ys + 2 * nn);
                    const float2 w = *reinterpret_cast<const float2*>(sm.window + 2 * nn);
                    a[n1] = make_float2(__fmul_rn(v.x, w.x), __fmul_rn(v.y, w.y));
                } else {
                    a[n1] = make_float2(0.0f, 0.0f);
                }
            }
            fft8(a);
            sc[lane] = a[0];
#pragma unroll
            for (int k = 1; k < 8; ++k) sc[k * kS1Stride + lane] = cmul(a[k], tw1[k]);
            __syncwarp();

            // ---- stage 2: for (k1, r2): DFT-8 over r1 of B[4*r1 + r2]
#pragma unroll
            for (int r1 = 0; r1 < 8; ++r1) a[r1] = sc[k1s * kS1Stride + 4 * r1 + r2];
            __syncwarp();
            fft8(a);
#pragma unroll
            for (int k = 1; k < 8; ++k) a[k] = cmul(a[k], tw2[k]);

            // ---- stage 3: DFT-4 over r2 across the four adjacent lanes, by shuffles.
            // After it lane r2 holds k3 = bitrev2(r2).
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                float2 v = a[k];
                float2 p = make_float2(__shfl_xor_sync(0xffffffffu, v.x, 2), __shfl_xor_sync(0xffffffffu, v.y, 2));
                v = (r2 & 2) ? csub(p, v) : cadd(v, p);
                if (r2 == 3) v = mul_mi(v);
                p = make_float2(__shfl_xor_sync(0xffffffffu, v.x, 1), __shfl_xor_sync(0xffffffffu, v.y, 1));
                v = (r2 & 1) ? csub(p, v) : cadd(v, p);
                a[k] = v;
            }
            const int k3 = ((r2 & 1) << 1) | (r2 >> 1);
            // Z[k], k = k1 + 8*k2 + 64*k3, stored at k + 4*(k >> 6) (bank-conflict-free).
#pragma unroll
            for (int k2 = 0; k2 < 8; ++k2) sc[k1s + 8 * k2 + 68 * k3] = a[k2];
            __syncwarp();

            // ---- real-FFT untangling and power for bins k and 256 - k, k = 1..128.
            //   E = (Z[k] + conj(Z[256-k])) / 2,  O = -i (Z[k] - conj(Z[256-k])) / 2
            //   X[k] = E + W512^k O,  X[256-k] = conj(E - W512^k O)
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                const int k = 1 + lane + 32 * m;
                const int kc = 256 - k;
                const float2 zk = sc[k + 4 * (k >> 6)];
                const float2 zc = sc[kc + 4 * (kc >> 6)];
                const float2 e = make_float2(0.5f * (zk.x + zc.x), 0.5f * (zk.y - zc.y));
                const float2 d = make_float2(zk.x - zc.x, zk.y + zc.y);       // Z[k] - conj(Z[256-k])
                const float2 o = make_float2(d.y, -d.x);                       // -i * d
                const float2 t = cmul(o, sm.tw_post[k]);                       // includes the 1/2
                const float2 xp = cadd(e, t), xm = csub(e, t);
                pw[k] = __fadd_rn(__fmul_rn(xp.x, xp.x), __fmul_rn(xp.y, xp.y));
                pw[kc] = __fadd_rn(__fmul_rn(xm.x, xm.x), __fmul_rn(xm.y, xm.y));
            }
            if (lane == 0) {
                const float2 z0 = sc[0];
                const float dc = z0.x + z0.y, ny = z0.x - z0.y;
                pw[0] = dc * dc;
                pw[256] = ny * ny;
            }
            __syncwarp();

            // ---- sparse mel filterbank + ln(mel + 2^-24), frontend.rs:110-115
            float* orow = out + (fo + f) * (int64_t)kMels;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int m = lane + 32 * i;
                const int st = sm.mel_start[m], cnt = sm.mel_cnt[m];
                float acc = 0.0f;
                for (int j = 0; j < cnt; ++j) acc = fmaf(sm.melw[j * kMels + m], pw[st + j], acc);
                orow[m] = logf(__fadd_rn(acc, 5.9604644775390625e-08f));
            }
            __syncwarp();
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
}

// frontend.rs:225-236: strictly sequential f32 accumulation per (clip, feature).
__global__ void __launch_bounds__(kMels)
colstats_kernel(const float* __restrict__ feat, const int64_t* __restrict__ frame_off,
                float* __restrict__ mean_out, float* __restrict__ std_out) {
    const int clip = blockIdx.x, f = threadIdx.x;
    const int64_t fo = frame_off[clip];
    const int T = (int)(frame_off[clip + 1] - fo);
    const float* col = feat + fo * kMels + f;
    float sum = 0.0f;
    int t = 0;
    for (; t + 8 <= T; t += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = col[(int64_t)(t + u) * kMels];
#pragma unroll
        for (int u = 0; u < 8; ++u) sum = __fadd_rn(sum, v[u]);
    }
    for (; t < T; ++t) sum = __fadd_rn(sum, col[(int64_t)t * kMels]);
    const float mean = __fdiv_rn(sum, (float)T);
    float acc = 0.0f;
    t = 0;
    for (; t + 8 <= T; t += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = col[(int64_t)(t + u) * kMels];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const float d = __fsub_rn(v[u], mean);
            acc = __fadd_rn(acc, __fmul_rn(d, d));
        }
    }
    for (; t < T; ++t) {
        const float d = __fsub_rn(col[(int64_t)t * kMels], mean);
        acc = __fadd_rn(acc, __fmul_rn(d, d));
    }
    // variance / (T - 1); T == 1 divides 0 by 0 and yields NaN exactly as the reference does.
    const float variance = __fdiv_rn(acc, __fsub_rn((float)T, 1.0f));
    mean_out[clip * kMels + f] = mean;
    std_out[clip * kMels + f] = __fadd_rn(__fsqrt_rn(variance), 1e-5f);
}

// frontend.rs:237-239
__global__ void __launch_bounds__(256)
normalize_kernel(float* __restrict__ feat, const int64_t* __restrict__ frame_off,
                 const float* __restrict__ mean, const float* __restrict__ stdv, int rows_per_cta) {
    const int clip = blockIdx.y;
    const int64_t fo = frame_off[clip];
    const int T = (int)(frame_off[clip + 1] - fo);
    const int r0 = blockIdx.x * rows_per_cta;
    if (r0 >= T) return;
    const int r1 = min(T, r0 + rows_per_cta);
    const int c4 = (threadIdx.x & 31) * 4;
    const float4 mu = *reinterpret_cast<const float4*>(mean + clip * kMels + c4);
    const float4 sd = *reinterpret_cast<const float4*>(stdv + clip * kMels + c4);
    for (int r = r0 + (threadIdx.x >> 5); r < r1; r += 8) {
        float4* p = reinterpret_cast<float4*>(feat + (fo + r) * kMels + c4);
        float4 v = *p;
        v.x = __fdiv_rn(__fsub_rn(v.x, mu.x), sd.x);
        v.y = __fdiv_rn(__fsub_rn(v.y, mu.y), sd.y);
        v.z = __fdiv_rn(__fsub_rn(v.z, mu.z), sd.z);
        v.w = __fdiv_rn(__fsub_rn(v.w, mu.w), sd.w);
        *p = v;
    }
}

}  // namespace

size_t frontend_smem_bytes() { return sizeof(SmemLayout); }

cudaError_t frontend_configure() {
    return cudaFuncSetAttribute(logmel_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)sizeof(SmemLayout));
}

cudaError_t frontend_launch(const float* pcm, const int64_t* d_clip_start, const int64_t* d_clip_len,
                            const int64_t* d_frame_off, int n_clips,
                            int max_frames, float preemph, const FrontendTables* d_tables, float* feats,
                            float* d_mean, float* d_std, bool normalize, cudaStream_t stream) {
    if (n_clips <= 0) return cudaSuccess;
    const int tiles = (max_frames + kFramesPerTile - 1) / kFramesPerTile;
    dim3 grid((tiles + kTilesPerCta - 1) / kTilesPerCta, n_clips);
    logmel_kernel<<<grid, kThreads, sizeof(SmemLayout), stream>>>(pcm, d_clip_start, d_clip_len, d_frame_off, feats,
                                                                 preemph, d_tables);
    if (normalize) {
        colstats_kernel<<<n_clips, kMels, 0, stream>>>(feats, d_frame_off, d_mean, d_std);
        const int rows_per_cta = 64;
        dim3 g2((max_frames + rows_per_cta - 1) / rows_per_cta, n_clips);
        normalize_kernel<<<g2, 256, 0, stream>>>(feats, d_frame_off, d_mean, d_std, rows_per_cta);
    }
    return cudaGetLastError();
}

}  // namespace sb
