// Log-mel frontend for sm_100a: PCM (f32 or 16-bit) -> normalised log-mel [T x 128] per clip, one kernel.
//
// Replaces the reference's CPU feature extractor (src/frontend.rs:104-241):
// pre-emphasis 0.97, 256-sample zero padding on both sides, Hann window of 400
// left-aligned in a 512-point real FFT, power spectrum, 128-bin Slaney mel
// filterbank, ln(x + 2^-24), per-feature mean / variance normalisation over
// all frames of the clip.
//
// frontend_clip_kernel: one CTA (8 warps) per clip, two CTAs per SM.
//   rows      The clip is walked 16 frames at a time.  The raw samples of the next 16 frames arrive by cp.async
//             (16-byte pieces where the clip's placement allows it) while the current ones are transformed; one
//             pass turns them into pre-emphasised, zero-padded samples (16-bit input is converted here).  Each
//             warp then transforms two frames, sixteen lanes per frame (frontend_core.cuh: two register radix-16
//             passes around one shared-memory transpose, untangling + power, sparse mel filterbank, ln), and leaves
//             the two log-mel rows in a 16-row stage in shared memory.  At the top of the next step the stage is
//             written out with 16-byte stores, and threads 0..127 add its rows to their column sums.
//   statistics The reference sums every column strictly left to right in f32 (frontend.rs:225-236); for a constant
//             column (an all-zero clip) the result consists of the rounding residue of exactly that order, so the
//             order is kept: thread c owns column c.  The first sum comes from the stage (no re-read); the second
//             pass (squared deviations) streams the clip's rows back through a cp.async ring per warp.
//   normalise (v - mean) / std over the clip's rows, 16-byte loads and stores, all threads.
// While one CTA of an SM is in its two bandwidth-bound tail passes the other one keeps the SM's issue slots busy
// with transforms, so the passes cost little wall time although they re-read the clip's rows.  The kernel is bound by
// shared-memory wavefronts and issue slots, not by DRAM: the filterbank taps and as much state as fits live in
// registers (128 per thread, two CTAs per SM), and buffers are laid out so that the two frames of a warp use
// different banks.
#include <cuda_runtime.h>
#include <stdint.h>

#include "frontend.h"
#include "frontend_core.cuh"

namespace sb {

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kStepFrames = 2 * kWarps;                           // 16 frames per step
constexpr int kRawElems = 2816;  // the step's samples + the one before them + up to 7 of alignment shift, in 16-byte pieces
constexpr int kRingRows = 16;    // rows per ring slot of the second statistics pass
constexpr int kRingSlots = 4;

constexpr int kStageStride = kMels + 16;  // floats per stage row: the two frames of a warp write different banks

struct __align__(16) SmemLayout {
    float2 scratch[kWarps][2][fe::kFrameScratch];  // per frame: transpose buffer, then Z, then the power bins; the
                                                   // statistics ring after the last step
    float raw[kRawElems];                          // raw samples of the next step (16-bit input: first half)
    float ys[kRawElems + 8];                       // pre-emphasised samples of this step, indexed like raw (+ ys_off)
    float stage[kStepFrames][kStageStride];        // log-mel rows of one step
    float window[kWin];
    float2 tw_post[132];
    float2 twid[256];
    float mean[kMels];
    float stdv[kMels];
    int16_t mel_start[kMels];
};
static_assert(sizeof(float2) * kWarps * 2 * fe::kFrameScratch >= sizeof(float) * 4 * kRingSlots * kRingRows * 32,
              "the statistics ring must fit in the transform scratch");

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <typename TIn>
struct Sample;
template <>
struct Sample<float> {
    static constexpr int kPerPiece = 4;  // samples per 16 bytes
    static __device__ __forceinline__ float get(const void* raw, int j) { return static_cast<const float*>(raw)[j]; }
};
template <>
struct Sample<int16_t> {
    static constexpr int kPerPiece = 8;
    static __device__ __forceinline__ float get(const void* raw, int j) {
        return fe::pcm16_to_f32(static_cast<const int16_t*>(raw)[j]);
    }
};

template <typename TIn>
__global__ void __launch_bounds__(kThreads, 2)
frontend_clip_kernel(const TIn* __restrict__ pcm, const int64_t* __restrict__ clip_start,
                     const int64_t* __restrict__ clip_len, const int64_t* __restrict__ frame_off,
                     float* __restrict__ out, float preemph, const FrontendTables* __restrict__ tables, int normalize) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    SmemLayout& sm = *reinterpret_cast<SmemLayout*>(smem_raw);
    constexpr int PP = Sample<TIn>::kPerPiece;

    const int clip = blockIdx.x;
    const int64_t c0 = clip_start[clip];
    const int64_t n = clip_len[clip];
    const int64_t fo = frame_off[clip];
    const int T = (int)(frame_off[clip + 1] - fo);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const TIn* x = pcm + c0;
    // Placement of the clip in memory: shared-memory index j of a step's buffers holds clip sample gbase + j, with
    // gbase chosen so that index 0 sits on a 16-byte boundary of the PCM buffer.  `shift` (0 .. PP-1) is how far the
    // sample before the step lies above that boundary; it is the same for every step (a step is 2560 samples).
    const int64_t elem0 = (int64_t)(reinterpret_cast<uintptr_t>(pcm) / sizeof(TIn)) + c0;   // absolute element index
    const int shift = (int)(((elem0 - kPad - 1) % PP + PP) % PP);
    // A frame's first sample sits at index shift + 1 + 160 fl of the pre-emphasised buffer; the transform reads sample
    // pairs with 8-byte loads, so an odd shift + 1 (a clip that starts on an odd sample of the PCM buffer) moves the
    // whole buffer up by one element.
    const int ys_off = (shift + 1) & 1;
    const int n_steps = (T + kStepFrames - 1) / kStepFrames;

    // Raw samples of a step -> shared memory, asynchronously; zero outside the clip (frontend.rs:59-65).
    auto fetch = [&](int step) {
        const int64_t gbase = (int64_t)step * kStepFrames * kHop - kPad - 1 - shift;
        TIn* dst = reinterpret_cast<TIn*>(sm.raw);
        if (gbase >= 0 && gbase + kRawElems <= n) {  // the whole step lies inside the clip
            const TIn* src = x + gbase;
            for (int q = tid; q < kRawElems / PP; q += kThreads) cp_async16(smem_addr(dst + q * PP), src + q * PP, 16);
        } else {
            for (int q = tid; q < kRawElems / PP; q += kThreads) {
                const int64_t g = gbase + (int64_t)q * PP;
                const uint32_t d = smem_addr(dst + q * PP);
                if (g >= 0 && g + PP <= n) {
                    cp_async16(d, x + g, 16);
                } else if (g + PP <= 0 || g >= n) {
                    *reinterpret_cast<uint4*>(dst + q * PP) = make_uint4(0u, 0u, 0u, 0u);
                } else if constexpr (sizeof(TIn) == 4) {
#pragma unroll
                    for (int e = 0; e < PP; ++e) {
                        const bool in = g + e >= 0 && g + e < n;
                        cp_async4(d + 4 * e, x + (in ? g + e : 0), in ? 4 : 0);
                    }
                } else {
                    // 16-bit samples at a clip edge: plain loads (cp.async moves at least four bytes)
#pragma unroll
                    for (int e = 0; e < PP; ++e) {
                        const bool in = g + e >= 0 && g + e < n;
                        dst[q * PP + e] = in ? x[g + e] : TIn(0);
                    }
                }
            }
        }
        cp_async_commit();
    };
    fetch(0);

    // Tables -> shared memory.
    for (int i = tid; i < kWin; i += kThreads) sm.window[i] = tables->window[i];
    for (int i = tid; i < 132; i += kThreads) sm.tw_post[i] = tables->tw_post[i];
    for (int i = tid; i < 256; i += kThreads) sm.twid[i] = tables->twid[i];
    for (int i = tid; i < kMels; i += kThreads) sm.mel_start[i] = tables->mel_start[i];
    const float log_floor = tables->log_floor;

    float sum = 0.0f;  // threads 0..127: running sum of column tid, frontend.rs:230
    // Rows of a finished step: out to memory (16-byte stores), and into the column sums in frame order.
    auto flush = [&](int step) {
        const int f0 = step * kStepFrames;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int idx = tid + kThreads * k, row = idx >> 5, c4 = idx & 31;
            if (f0 + row < T)
                reinterpret_cast<float4*>(out + (fo + f0 + row) * kMels)[c4] = reinterpret_cast<const float4*>(sm.stage[row])[c4];
        }
        if (tid < kMels) {
            const int rows = min(kStepFrames, T - f0);
            if (rows == kStepFrames) {
#pragma unroll
                for (int r = 0; r < kStepFrames; ++r) sum = __fadd_rn(sum, sm.stage[r][tid]);
            } else {
                for (int r = 0; r < rows; ++r) sum = __fadd_rn(sum, sm.stage[r][tid]);
            }
        }
    };

    const int half = lane >> 4, p = lane & 15;
    float taps[kMelTapRows];  // this lane's filterbank taps (rows 16 g + p)
    fe::load_mel_taps(p, tables->melw, taps);
    for (int step = 0; step < n_steps; ++step) {
        cp_async_wait<0>();
        __syncthreads();  // this step's raw samples are in; the previous step's rows are all in the stage
        if (step > 0) flush(step - 1);
        // Pre-emphasis (frontend.rs:150-159): y[0] = x[0]; y[i] = x[i] - c * x[i-1], product rounded first; zero outside
        // the clip (the padding is added after the pre-emphasis, frontend.rs:59-65).
        {
            const int64_t gbase = (int64_t)step * kStepFrames * kHop - kPad - 1 - shift;
            const void* raw = sm.raw;
            const bool inside = gbase >= 0 && gbase + kRawElems <= n;
            for (int q = tid; q < kRawElems / 4; q += kThreads) {
                const int j = 4 * q;
                float xs[5];
                xs[0] = j > 0 ? Sample<TIn>::get(raw, j - 1) : 0.0f;
#pragma unroll
                for (int e = 0; e < 4; ++e) xs[e + 1] = Sample<TIn>::get(raw, j + e);
                float4 y;
                float* yv = reinterpret_cast<float*>(&y);
                const int64_t g = gbase + j;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float v = __fsub_rn(xs[e + 1], __fmul_rn(preemph, xs[e]));
                    yv[e] = (inside || (g + e >= 0 && g + e < n)) ? v : 0.0f;
                }
                if (ys_off == 0) {
                    *reinterpret_cast<float4*>(sm.ys + j) = y;
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e) sm.ys[j + 1 + e] = yv[e];
                }
            }
        }
        __syncthreads();  // samples ready; the stage and the raw buffer are free again
        if (step + 1 < n_steps) fetch(step + 1);  // lands while this step is transformed
        {
            const int fl = 2 * warp + half;                                // frame of the step this half-warp transforms
            const float* ysf = sm.ys + shift + 1 + ys_off + fl * kHop;     // its 400 samples
            float2* B = sm.scratch[warp][half];
            fe::pass1(p, ysf, sm.window, sm.twid, B);
            __syncwarp();
            {
                float2 z[16];
                fe::pass2(p, B, z);
                __syncwarp();
                fe::store_z(p, z, B);
            }
            __syncwarp();
            float* pwf = reinterpret_cast<float*>(B);  // the power bins take Z's place once every lane holds its Z values
            {
                float2 zk[8], zc[8], z0;
                fe::untangle_load(p, B, zk, zc, z0);
                __syncwarp();
                fe::untangle_store(p, zk, zc, z0, sm.tw_post, pwf);
            }
            __syncwarp();
            fe::mel_rows(p, pwf, taps, sm.mel_start, log_floor, sm.stage[fl]);
        }
    }
    __syncthreads();
    flush(n_steps - 1);
    if (!normalize) return;

    // ---- statistics, frontend.rs:225-236.  Thread c (< 128) owns column c; warp w streams rows of columns
    // 32 w .. 32 w + 31 through its own ring of kRingSlots x kRingRows rows.
    __syncthreads();  // every row of the clip has been stored by this CTA
    const float* rows = out + fo * kMels;
    if (warp < kMels / 32) {
        const float mean = __fdiv_rn(sum, (float)T);
        float* ring = reinterpret_cast<float*>(&sm.scratch[0][0][0]) + warp * (kRingSlots * kRingRows * 32);
        const int n_blk = (T + kRingRows - 1) / kRingRows;
        auto issue = [&](int blk) {
            if (blk < n_blk) {
                float* slot = ring + (blk % kRingSlots) * (kRingRows * 32);
#pragma unroll
                for (int k = 0; k < kRingRows * 8 / 32; ++k) {
                    const int q = lane + 32 * k, r = q >> 3, ch = q & 7;
                    const int row = blk * kRingRows + r;
                    const bool in = row < T;
                    cp_async16(smem_addr(slot + r * 32 + 4 * ch), rows + (int64_t)(in ? row : 0) * kMels + 32 * warp + 4 * ch,
                               in ? 16 : 0);
                }
            }
            cp_async_commit();
        };
#pragma unroll
        for (int s = 0; s < kRingSlots - 1; ++s) issue(s);
        float acc = 0.0f;
        for (int blk = 0; blk < n_blk; ++blk) {
            issue(blk + kRingSlots - 1);  // refills the slot that was read one iteration ago
            cp_async_wait<kRingSlots - 1>();
            __syncwarp();
            const float* slot = ring + (blk % kRingSlots) * (kRingRows * 32);
            const int nr = min(kRingRows, T - blk * kRingRows);
            if (nr == kRingRows) {
#pragma unroll
                for (int r = 0; r < kRingRows; ++r) {
                    const float d = __fsub_rn(slot[r * 32 + lane], mean);
                    acc = __fadd_rn(acc, __fmul_rn(d, d));
                }
            } else {
                for (int r = 0; r < nr; ++r) {
                    const float d = __fsub_rn(slot[r * 32 + lane], mean);
                    acc = __fadd_rn(acc, __fmul_rn(d, d));
                }
            }
            __syncwarp();  // all lanes are done with the slot before the next issue overwrites it
        }
        cp_async_wait<0>();
        // variance / (T - 1); T == 1 divides 0 by 0 and yields NaN exactly as the reference does.
        const float variance = __fdiv_rn(acc, __fsub_rn((float)T, 1.0f));
        sm.mean[tid] = mean;
        sm.stdv[tid] = __fadd_rn(__fsqrt_rn(variance), 1e-5f);
    }
    __syncthreads();
    // ---- normalise, frontend.rs:237-239: (v - mean) / std with the IEEE quotient.  For a divisor in the range below
    // the quotient is formed from the correctly rounded reciprocal and one exact-remainder correction, three
    // instructions, which gives the correctly rounded result (Markstein's correction step; checked against the
    // hardware division on 4e8 operand pairs, all-ones significands included); any other divisor takes __fdiv_rn.
    {
        const int c4 = tid & 31;
        const float4 mu = reinterpret_cast<const float4*>(sm.mean)[c4];
        const float4 sd = reinterpret_cast<const float4*>(sm.stdv)[c4];
        auto plain = [](float d) {
            const uint32_t b = __float_as_uint(d);
            return d >= 7.62939453125e-06f && d < 128.0f && (b & 0x7FFFFFu) != 0x7FFFFFu;  // 2^-17 <= d < 2^7
        };
        const bool fast = plain(sd.x) && plain(sd.y) && plain(sd.z) && plain(sd.w);
        const float4 rc = make_float4(__frcp_rn(sd.x), __frcp_rn(sd.y), __frcp_rn(sd.z), __frcp_rn(sd.w));
        auto quot = [](float x, float d, float r) {
            const float q = __fmul_rn(x, r);
            return fmaf(fmaf(-q, d, x), r, q);
        };
        float4* rows4 = reinterpret_cast<float4*>(out + fo * kMels);
        constexpr int U = 8;
        for (int r0 = tid >> 5; r0 < T; r0 += 8 * U) {
            float4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int r = r0 + 8 * u;
                if (r < T) v[u] = __ldcg(rows4 + (int64_t)r * 32 + c4);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int r = r0 + 8 * u;
                if (r < T) {
                    float4 o;
                    const float a = __fsub_rn(v[u].x, mu.x), b = __fsub_rn(v[u].y, mu.y);
                    const float c = __fsub_rn(v[u].z, mu.z), d = __fsub_rn(v[u].w, mu.w);
                    if (fast) {
                        o.x = quot(a, sd.x, rc.x);
                        o.y = quot(b, sd.y, rc.y);
                        o.z = quot(c, sd.z, rc.z);
                        o.w = quot(d, sd.w, rc.w);
                    } else {
                        o.x = __fdiv_rn(a, sd.x);
                        o.y = __fdiv_rn(b, sd.y);
                        o.z = __fdiv_rn(c, sd.z);
                        o.w = __fdiv_rn(d, sd.w);
                    }
                    rows4[(int64_t)r * 32 + c4] = o;
                }
            }
        }
    }
}

}  // namespace

size_t frontend_smem_bytes() { return sizeof(SmemLayout); }

cudaError_t frontend_configure() {
    cudaError_t e = cudaFuncSetAttribute(frontend_clip_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)sizeof(SmemLayout));
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(frontend_clip_kernel<int16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)sizeof(SmemLayout));
}

cudaError_t frontend_launch(const void* pcm, SampleFormat fmt, const int64_t* d_clip_start, const int64_t* d_clip_len,
                            const int64_t* d_frame_off, int n_clips, float preemph, const FrontendTables* d_tables,
                            float* feats, bool normalize, cudaStream_t stream) {
    if (n_clips <= 0) return cudaSuccess;
    // 16-byte row accesses of the feature matrix and 4- / 2-byte aligned samples
    if ((reinterpret_cast<uintptr_t>(feats) & 15) || (reinterpret_cast<uintptr_t>(pcm) & (fmt == kSampleI16 ? 1 : 3)))
        return cudaErrorMisalignedAddress;
    if (fmt == kSampleI16)
        frontend_clip_kernel<int16_t><<<n_clips, kThreads, sizeof(SmemLayout), stream>>>(
            static_cast<const int16_t*>(pcm), d_clip_start, d_clip_len, d_frame_off, feats, preemph, d_tables, normalize ? 1 : 0);
    else
        frontend_clip_kernel<float><<<n_clips, kThreads, sizeof(SmemLayout), stream>>>(
            static_cast<const float*>(pcm), d_clip_start, d_clip_len, d_frame_off, feats, preemph, d_tables, normalize ? 1 : 0);
    return cudaGetLastError();
}

}  // namespace sb
