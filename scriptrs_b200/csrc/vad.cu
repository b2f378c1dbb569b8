// Streaming voice-activity network of the VAD long-form mode (SileroVad::process, src/long_form/vad.rs:61-98,
// behind the I/O contract of src/coreml.rs:188-236), for a whole recording at once.
//
// The reference feeds one 576-sample input (64 samples of context + 512 new ones) and the recurrent state to a
// CoreML model per window, 31.25 times per second of audio.  Only the LSTM cell depends on the window before;
// everything in front of it depends on the window's own samples.  So the work splits in two:
//
//   vad_encode_kernel   all windows in parallel, 16 windows per CTA: reflect padding, the short-time Fourier
//                       magnitudes (4 frames x 129 bins), the four ReLU convolutions and the input half of the
//                       LSTM gates (W_ih e + b_ih + b_hh), written as 512 floats per window;
//   vad_lstm_kernel     the recurrence, one thread-block cluster for the whole recording: the 512 x 128
//                       recurrent matrix stays in the registers of the cluster's CTAs (it is as large as one SM's
//                       register file, hence several SMs), the hidden vector goes from SM to SM through
//                       distributed shared memory, its arrival counted by an mbarrier at the destination;
//   vad_prob_kernel     ReLU, the 128 -> 1 output layer and the sigmoid, a warp per window.
//
// All arithmetic is fp32.
#include "vad.h"

#include <cooperative_groups.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <string>
#include <vector>

namespace cg = cooperative_groups;

namespace sb {

namespace {

constexpr int kTileWindows = 16;            // windows per CTA of the encode kernel
constexpr int kEncThreads = 256;
constexpr int kXsStride = kVadPadded + 4;   // 644: rows 16 bytes apart modulo 128, conflict-free float4 reads
constexpr int kT1 = kVadFrames + 2;         // 6: four steps with a zero on either side
constexpr int kT2 = 4;                      // two steps with a zero on either side
constexpr int kRegionFloats = 12416;        // >= 129 * 16 * 6 and >= 16 * 644, a multiple of 4

struct EncodeParams {
    const float* audio;
    int64_t n_samples;
    int64_t first_window;  // of this pass, in the recording
    int n_windows;         // in this pass
    const float *basis, *w1, *b1, *w2, *b2, *w3, *b3, *w4, *b4, *wih, *bsum;
    float* gx;             // [n_windows x 512]
};

__device__ __forceinline__ float4 ldg4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }

__global__ void __launch_bounds__(kEncThreads, 2) vad_encode_kernel(const EncodeParams p) {
    extern __shared__ __align__(16) float smem[];
    float* r0 = smem;                  // samples, then layer-1 output, then layer-3 output
    float* r1 = smem + kRegionFloats;  // magnitudes, then layer-2 output, then layer-4 output
    const int tid = threadIdx.x;
    const int64_t w_base = (int64_t)blockIdx.x * kTileWindows;  // within the pass

    // ---- samples: 64 of context (zeros before the recording), 512 new (the last sample repeated past the end),
    //      64 reflected
    for (int i = tid; i < kTileWindows * kVadPadded; i += kEncThreads) {
        const int w = i / kVadPadded, j = i - w * kVadPadded;
        const int jj = j < kVadInput ? j : 2 * kVadInput - 2 - j;  // reflect without repeating the edge sample
        int64_t s = (p.first_window + w_base + w) * kVadWindow - kVadContext + jj;
        float v = 0.0f;
        if (s >= 0) {
            if (s >= p.n_samples) s = p.n_samples - 1;
            v = __ldg(p.audio + s);
        }
        r0[w * kXsStride + j] = v;
    }
    __syncthreads();

    // ---- magnitudes: a task is one window (its four frames) times three bins
    for (int task = tid; task < kTileWindows * 43; task += kEncThreads) {
        const int w = task % kTileWindows, b0 = (task / kTileWindows) * 3;
        float re[3][4], im[3][4];
#pragma unroll
        for (int j = 0; j < 3; ++j)
#pragma unroll
            for (int t = 0; t < 4; ++t) re[j][t] = im[j][t] = 0.0f;
        const float* xs = r0 + w * kXsStride;
#pragma unroll 4
        for (int n = 0; n < kVadFilter; n += 4) {
            float4 a[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) a[t] = *reinterpret_cast<const float4*>(xs + 128 * t + n);
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                const float4 br = ldg4(p.basis + (b0 + j) * kVadFilter + n);
                const float4 bi = ldg4(p.basis + (kVadBins + b0 + j) * kVadFilter + n);
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    re[j][t] = fmaf(a[t].x, br.x, re[j][t]);
                    re[j][t] = fmaf(a[t].y, br.y, re[j][t]);
                    re[j][t] = fmaf(a[t].z, br.z, re[j][t]);
                    re[j][t] = fmaf(a[t].w, br.w, re[j][t]);
                    im[j][t] = fmaf(a[t].x, bi.x, im[j][t]);
                    im[j][t] = fmaf(a[t].y, bi.y, im[j][t]);
                    im[j][t] = fmaf(a[t].z, bi.z, im[j][t]);
                    im[j][t] = fmaf(a[t].w, bi.w, im[j][t]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            float* m = r1 + (b0 + j) * (kTileWindows * kT1) + w * kT1;
            m[0] = 0.0f;
            m[5] = 0.0f;
#pragma unroll
            for (int t = 0; t < 4; ++t) m[1 + t] = sqrtf(fmaf(re[j][t], re[j][t], im[j][t] * im[j][t]));
        }
    }
    __syncthreads();

    // ---- layer 1: 129 -> 128 channels, k = 3, stride 1, four steps.  Thread: one window, eight channels.
    {
        const int w = tid % kTileWindows, co = (tid / kTileWindows) * 8;
        float acc[8][4];
        {
            const float4 ba = ldg4(p.b1 + co), bb = ldg4(p.b1 + co + 4);
            const float b[8] = {ba.x, ba.y, ba.z, ba.w, bb.x, bb.y, bb.z, bb.w};
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int t = 0; t < 4; ++t) acc[j][t] = b[j];
        }
#pragma unroll 3
        for (int ci = 0; ci < kVadBins; ++ci) {
            const float2* mp = reinterpret_cast<const float2*>(r1 + ci * (kTileWindows * kT1) + w * kT1);
            const float2 m01 = mp[0], m23 = mp[1], m45 = mp[2];
            const float m[6] = {m01.x, m01.y, m23.x, m23.y, m45.x, m45.y};
#pragma unroll
            for (int tap = 0; tap < 3; ++tap) {
                const float4 wa = ldg4(p.w1 + (ci * 3 + tap) * 128 + co), wb = ldg4(p.w1 + (ci * 3 + tap) * 128 + co + 4);
                const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int t = 0; t < 4; ++t) acc[j][t] = fmaf(wv[j], m[t + tap], acc[j][t]);
            }
        }
        // the samples in r0 were last read by the magnitude stage, which ended at the barrier above
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float* o = r0 + (co + j) * (kTileWindows * kT1) + w * kT1;
            o[0] = 0.0f;
            o[5] = 0.0f;
#pragma unroll
            for (int t = 0; t < 4; ++t) o[1 + t] = fmaxf(acc[j][t], 0.0f);
        }
    }
    __syncthreads();

    // ---- layer 2: 128 -> 64 channels, k = 3, stride 2, two steps.  Thread: one window, four channels.
    {
        const int w = tid % kTileWindows, co = (tid / kTileWindows) * 4;
        float acc[4][2];
        {
            const float4 b = ldg4(p.b2 + co);
            acc[0][0] = acc[0][1] = b.x;
            acc[1][0] = acc[1][1] = b.y;
            acc[2][0] = acc[2][1] = b.z;
            acc[3][0] = acc[3][1] = b.w;
        }
        for (int ci = 0; ci < 128; ++ci) {
            const float2* mp = reinterpret_cast<const float2*>(r0 + ci * (kTileWindows * kT1) + w * kT1);
            const float2 m01 = mp[0], m23 = mp[1], m45 = mp[2];
            const float m[5] = {m01.x, m01.y, m23.x, m23.y, m45.x};
#pragma unroll
            for (int tap = 0; tap < 3; ++tap) {
                const float4 wa = ldg4(p.w2 + (ci * 3 + tap) * 64 + co);
                const float wv[4] = {wa.x, wa.y, wa.z, wa.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[j][0] = fmaf(wv[j], m[tap], acc[j][0]);
                    acc[j][1] = fmaf(wv[j], m[2 + tap], acc[j][1]);
                }
            }
        }
        // r1 still holds the magnitudes, which layer 1 finished reading before the barrier above
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float4 o;
            o.x = 0.0f;
            o.y = fmaxf(acc[j][0], 0.0f);
            o.z = fmaxf(acc[j][1], 0.0f);
            o.w = 0.0f;
            *reinterpret_cast<float4*>(r1 + (co + j) * (kTileWindows * kT2) + w * kT2) = o;
        }
    }
    __syncthreads();

    // ---- layer 3: 64 -> 64 channels, k = 3, stride 2, one step.  Thread: one window, four channels.
    {
        const int w = tid % kTileWindows, co = (tid / kTileWindows) * 4;
        float acc[4];
        {
            const float4 b = ldg4(p.b3 + co);
            acc[0] = b.x; acc[1] = b.y; acc[2] = b.z; acc[3] = b.w;
        }
        for (int ci = 0; ci < 64; ++ci) {
            const float4 mv = *reinterpret_cast<const float4*>(r1 + ci * (kTileWindows * kT2) + w * kT2);
            const float m[3] = {mv.x, mv.y, mv.z};
#pragma unroll
            for (int tap = 0; tap < 3; ++tap) {
                const float4 wa = ldg4(p.w3 + (ci * 3 + tap) * 64 + co);
                acc[0] = fmaf(wa.x, m[tap], acc[0]);
                acc[1] = fmaf(wa.y, m[tap], acc[1]);
                acc[2] = fmaf(wa.z, m[tap], acc[2]);
                acc[3] = fmaf(wa.w, m[tap], acc[3]);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) r0[(co + j) * kTileWindows + w] = fmaxf(acc[j], 0.0f);  // layer 2 finished with r0
    }
    __syncthreads();

    // ---- layer 4: 64 -> 128 channels, one step in, one step out: only the centre tap meets data
    {
        const int w = tid % kTileWindows, co = (tid / kTileWindows) * 8;
        float acc[8];
        {
            const float4 ba = ldg4(p.b4 + co), bb = ldg4(p.b4 + co + 4);
            acc[0] = ba.x; acc[1] = ba.y; acc[2] = ba.z; acc[3] = ba.w;
            acc[4] = bb.x; acc[5] = bb.y; acc[6] = bb.z; acc[7] = bb.w;
        }
        for (int ci = 0; ci < 64; ++ci) {
            const float a = r0[ci * kTileWindows + w];
            const float4 wa = ldg4(p.w4 + ci * 128 + co), wb = ldg4(p.w4 + ci * 128 + co + 4);
            acc[0] = fmaf(wa.x, a, acc[0]); acc[1] = fmaf(wa.y, a, acc[1]);
            acc[2] = fmaf(wa.z, a, acc[2]); acc[3] = fmaf(wa.w, a, acc[3]);
            acc[4] = fmaf(wb.x, a, acc[4]); acc[5] = fmaf(wb.y, a, acc[5]);
            acc[6] = fmaf(wb.z, a, acc[6]); acc[7] = fmaf(wb.w, a, acc[7]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) r1[(co + j) * kTileWindows + w] = fmaxf(acc[j], 0.0f);  // layer 3 finished with r1
    }
    __syncthreads();

    // ---- input half of the LSTM gates.  Thread: four windows, eight gate rows.
    {
        const int wq = (tid % 4) * 4, g = (tid / 4) * 8;
        float acc[8][4];
        {
            const float4 ba = ldg4(p.bsum + g), bb = ldg4(p.bsum + g + 4);
            const float b[8] = {ba.x, ba.y, ba.z, ba.w, bb.x, bb.y, bb.z, bb.w};
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[j][i] = b[j];
        }
        for (int k = 0; k < kVadState; ++k) {
            const float4 e = *reinterpret_cast<const float4*>(r1 + k * kTileWindows + wq);
            const float ev[4] = {e.x, e.y, e.z, e.w};
            const float4 wa = ldg4(p.wih + k * kVadGates + g), wb = ldg4(p.wih + k * kVadGates + g + 4);
            const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[j][i] = fmaf(wv[j], ev[i], acc[j][i]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int64_t w = w_base + wq + i;
            if (w >= p.n_windows) continue;
            float* o = p.gx + w * kVadGates + g;
            *reinterpret_cast<float4*>(o) = make_float4(acc[0][i], acc[1][i], acc[2][i], acc[3][i]);
            *reinterpret_cast<float4*>(o + 4) = make_float4(acc[4][i], acc[5][i], acc[6][i], acc[7][i]);
        }
    }
}

// 1 / (1 + 2^(k x)) with the hardware's exponential and reciprocal (relative error about 2^-22 each): k = -log2(e)
// gives the logistic function, k = -2 log2(e) gives (tanh(x) + 1) / 2.  2^(k x) overflows to +inf for very negative
// x, and the reciprocal of +inf is 0.
__device__ __forceinline__ float logistic_pow2(float x, float k) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * k));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return r;
}
constexpr float kNegLog2e = -1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t cluster_addr(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}

// 4-byte store into another CTA's shared memory that, once it has landed, counts 4 bytes on that CTA's mbarrier
__device__ __forceinline__ void store_remote_tx(uint32_t remote_data, float v, uint32_t remote_mbar) {
    asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.u32 [%0], %1, [%2];" ::"r"(remote_data),
                 "r"(__float_as_uint(v)), "r"(remote_mbar)
                 : "memory");
}

__device__ __forceinline__ void mbar_init(uint32_t mbar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"(bytes) : "memory");
}

// Waits for the phase of the given parity to complete; gives up (false) after about a second.  Each try_wait
// suspends the warp for at most a microsecond (the hint), so the clock is read once in 1024 polls.
__device__ __forceinline__ bool mbar_wait(uint32_t mbar, uint32_t parity) {
    unsigned long long t0 = 0;
    for (uint32_t i = 1;; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(mbar), "r"(parity), "r"(1000u)
            : "memory");
        if (done) return true;
        if ((i & 1023u) == 0) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > 1000000000ull) return false;
        }
    }
}

// The recurrence over the n windows of a pass.  A cluster of C CTAs; CTA r owns hidden units [r U, r U + U),
// U = 128 / C, i.e. gate rows' [4 r U, 4 (r + 1) U) of the permuted matrices.  Two threads per row, each with half
// of the row's columns in registers; the 8 lanes of a unit (4 gates x 2 halves) sit next to each other in a warp
// and all of them end a step holding the unit's new h, so a warp holds 4 units.
//
// Exchange of the hidden vector: two buffers of 128 floats per CTA, used in turn, each with an mbarrier.  After
// step s lane j < C of a unit stores the unit's h (4 bytes) into buffer (s + 1) & 1 of CTA j with st.async, which
// adds 4 bytes to that CTA's transaction count: one instruction per warp, 128 small packets per CTA and step
// (gathering a warp's four units into one 16-byte store, or a CTA's units into one store per destination behind
// a CTA barrier, costs more in shuffles and barriers than the fewer packets save: 43.5 and 46.7 ms per hour of
// audio against 41.8).  A warp starts step s + 1 when its CTA's barrier has counted all 512 bytes.  There is no
// barrier among the warps of a CTA inside the loop.  A warp can be at most one step ahead of any other warp of
// the cluster (a step needs everybody's output of the step before), so two buffers are enough, nothing is
// overwritten while it is still read, and no warp can miss a phase.  Every wait is bounded: a warp whose wait gave
// up raises *error and leaves the loop, which stops the others' input, so they give up too, and all meet at the
// closing cluster barrier.
template <int C>
__global__ void __launch_bounds__(2 * kVadGates / C, 1)
vad_lstm_kernel(const float* __restrict__ gx, const float* __restrict__ whh, float* __restrict__ state,
                float* __restrict__ hout, int n, int* __restrict__ error) {
    constexpr int kRows = kVadGates / C;  // gate rows of this CTA
    constexpr int kUnits = kVadState / C;
    constexpr int kThreads = 2 * kRows;
    constexpr int kDepth = 16;            // gate inputs are fetched this many windows ahead
    static_assert(C <= 8, "lane j < C sends to CTA j: one lane per unit lane");
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int tid = threadIdx.x, lane = tid & 31;
    const int part = tid & 1, row_local = tid >> 1, q = row_local & 3, unit_local = row_local >> 2;
    const int row = rank * kRows + row_local;
    const int unit = rank * kUnits + unit_local;

    __shared__ __align__(16) float hs[2][kVadState];
    // Gate inputs on their way from global memory: slot s % kDepth holds step s's value for every thread.  They come
    // by cp.async, one group per step, because loads into registers this far ahead end up waiting for one another
    // (a warp has few scoreboards), which puts a DRAM round trip into every step.
    __shared__ float gring[kDepth][kThreads];
    __shared__ __align__(8) uint64_t mbar[2];

    float2 w[32];  // pairs, for the two-wide fp32 multiply-add
    {
        // thread `part` of a row holds the 16-byte column chunks part, part + 2, ...: the two lanes of a row read
        // neighbouring chunks of h, which lie in different banks
        const float4* src = reinterpret_cast<const float4*>(whh + (size_t)row * kVadState) + part;
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const float4 v = __ldg(src + 2 * k);
            w[2 * k] = make_float2(v.x, v.y);
            w[2 * k + 1] = make_float2(v.z, v.w);
        }
    }
    if (tid < kVadState) hs[0][tid] = state[tid];
    float c = state[kVadState + unit];
    float h = state[unit];
    const uint32_t mbar0 = smem_u32(&mbar[0]), mbar1 = smem_u32(&mbar[1]);
    if (tid == 0) {
        mbar_init(mbar0, 1);
        mbar_init(mbar1, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // phase for the input of step 1 (buffer 1) and of step 2 (buffer 0)
        if (n >= 1) mbar_expect_tx(mbar1, kVadState * 4);
        if (n >= 2) mbar_expect_tx(mbar0, kVadState * 4);
    }
    // lane j < C of a unit's eight lanes sends the unit's h to CTA j
    const int unit_lane = lane & 7;
    const uint32_t dst_rank = unit_lane < C ? unit_lane : 0;
    const uint32_t dst_h = cluster_addr(smem_u32(&hs[0][unit]), dst_rank);
    const uint32_t dst_mbar0 = cluster_addr(mbar0, dst_rank), dst_mbar1 = cluster_addr(mbar1, dst_rank);

    const float* gx_row = gx + row;
    const uint32_t gring_mine = smem_u32(&gring[0][tid]);
    auto fetch = [&](int step) {
        if (step < n)
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(gring_mine + (uint32_t)(step % kDepth) * kThreads * 4),
                         "l"(gx_row + (size_t)step * kVadGates)
                         : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int j = 0; j < kDepth; ++j) fetch(j);
    cluster.sync();  // barriers initialised and hs[0] filled everywhere before the first remote store

    // the cell candidate (gate 2) is a tanh: 2 / (1 + e^(-2 x)) - 1; the other gates are logistic
    const float gate_k = q == 2 ? 2.0f * kNegLog2e : kNegLog2e;
    const float gate_mul = q == 2 ? 2.0f : 1.0f, gate_add = q == 2 ? -1.0f : 0.0f;
    const int base = lane & ~7;
    bool alive = true;
    for (int s = 0; s < n; ++s) {
        const int cur = s & 1;
        // this step's gate input has long arrived; read it and reuse its slot before waiting for the others' h
        asm volatile("cp.async.wait_group %0;" ::"n"(kDepth - 1) : "memory");
        const float gxv = gring[s % kDepth][tid];
        fetch(s + kDepth);
        const bool ok = s == 0 || mbar_wait(cur ? mbar1 : mbar0, (uint32_t)((s - 1) >> 1) & 1u);
        const float4* hv = reinterpret_cast<const float4*>(&hs[cur][0]) + part;
        float2 a0 = make_float2(0.0f, 0.0f), a1 = a0, a2 = a0, a3 = a0;
#pragma unroll
        for (int k = 0; k < 16; k += 2) {
            const float4 u = hv[2 * k], v = hv[2 * k + 2];
            a0 = __ffma2_rn(w[2 * k], make_float2(u.x, u.y), a0);
            a1 = __ffma2_rn(w[2 * k + 1], make_float2(u.z, u.w), a1);
            a2 = __ffma2_rn(w[2 * k + 2], make_float2(v.x, v.y), a2);
            a3 = __ffma2_rn(w[2 * k + 3], make_float2(v.z, v.w), a3);
        }
        float pre = ((a0.x + a0.y) + (a1.x + a1.y)) + ((a2.x + a2.y) + (a3.x + a3.y));
        pre += __shfl_xor_sync(0xffffffffu, pre, 1);
        pre += gxv;
        const float act = fmaf(gate_mul, logistic_pow2(pre, gate_k), gate_add);
        const float gi = __shfl_sync(0xffffffffu, act, base);
        const float gf = __shfl_sync(0xffffffffu, act, base + 2);
        const float gg = __shfl_sync(0xffffffffu, act, base + 4);
        const float go = __shfl_sync(0xffffffffu, act, base + 6);
        c = fmaf(gf, c, gi * gg);
        h = go * fmaf(2.0f, logistic_pow2(c, 2.0f * kNegLog2e), -1.0f);
        if (unit_lane < C) store_remote_tx(dst_h + (uint32_t)((cur ^ 1) * kVadState * 4), h, cur ? dst_mbar0 : dst_mbar1);
        if (unit_lane == 0) hout[(size_t)s * kVadState + unit] = h;
        // Everything that is not on the path from the others' h to this warp's h comes after the send.  The buffer
        // just read is armed for its next phase, the input of step s + 2 (its bytes cannot be complete before this
        // CTA has sent step s + 1, and bytes that arrive before the arming are counted all the same).  And a wait
        // that gave up ends the warp's loop only here: the arithmetic ran on stale input and the result is void.
        if (tid == 0 && ok && s > 0 && s + 2 <= n) mbar_expect_tx(cur ? mbar1 : mbar0, kVadState * 4);
        alive = __all_sync(0xffffffffu, ok);
        if (!alive) {
            *error = 1;
            break;
        }
    }
    // the output of the last step is in flight to every CTA's shared memory: wait for it before anyone exits
    if (alive && n > 0 && !mbar_wait((n & 1) ? mbar1 : mbar0, (uint32_t)((n - 1) >> 1) & 1u)) *error = 1;
    if (unit_lane == 0) {
        state[unit] = h;
        state[kVadState + unit] = c;
    }
    cluster.sync();
}

__global__ void vad_prob_kernel(const float* __restrict__ hout, const float* __restrict__ wout, float bout,
                                float* __restrict__ prob, int n) {
    const int w = (int)((blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
    if (w >= n) return;
    const float4 h = __ldcs(reinterpret_cast<const float4*>(hout + (size_t)w * kVadState) + lane);
    const float4 k = ldg4(wout + 4 * lane);
    float a = fmaxf(h.x, 0.0f) * k.x;
    a = fmaf(fmaxf(h.y, 0.0f), k.y, a);
    a = fmaf(fmaxf(h.z, 0.0f), k.z, a);
    a = fmaf(fmaxf(h.w, 0.0f), k.w, a);
#pragma unroll
    for (int o = 16; o; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
    if (lane == 0) prob[w] = 1.0f / (1.0f + expf(-(a + bout)));
}

constexpr size_t kEncSmem = 2 * kRegionFloats * sizeof(float);

template <int C>
cudaError_t launch_lstm(const float* gx, const float* whh, float* state, float* hout, int n, int* error, cudaStream_t st) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(C);
    cfg.blockDim = dim3(2 * kVadGates / C);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = C;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, vad_lstm_kernel<C>, gx, whh, state, hout, n, error);
}

const sb_tensor* find(const sb_tensor* t, int64_t n, const std::string& name) {
    for (int64_t i = 0; i < n; ++i) {
        if (!t[i].name) continue;
        std::string have = t[i].name;
        if (have.compare(0, 7, "_model.") == 0) have = have.substr(7);
        if (have == name) return &t[i];
    }
    return nullptr;
}

cudaError_t upload(const std::vector<float>& v, float** out) {
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(out), v.size() * sizeof(float));
    if (e != cudaSuccess) return e;
    return cudaMemcpy(*out, v.data(), v.size() * sizeof(float), cudaMemcpyHostToDevice);
}

}  // namespace

void VadModel::release() {
    for (float* p : {basis, w1, b1, w2, b2, w3, b3, w4, b4, wih, bsum, whh, wout})
        if (p) cudaFree(p);
    gx[0].release();
    gx[1].release();
    hout.release();
    state.release();
    audio.release();
    prob.release();
    host_prob.release();
}

cudaError_t vad_configure() {
    return cudaFuncSetAttribute(vad_encode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kEncSmem);
}

int32_t vad_load(sb_ctx* c, const sb_tensor* tensors, int64_t n_tensors) {
    struct Want { const char* name; int64_t numel; };
    static const Want wants[] = {
        {"stft.forward_basis_buffer", 258 * 256},
        {"encoder.0.reparam_conv.weight", 128 * 129 * 3}, {"encoder.0.reparam_conv.bias", 128},
        {"encoder.1.reparam_conv.weight", 64 * 128 * 3},  {"encoder.1.reparam_conv.bias", 64},
        {"encoder.2.reparam_conv.weight", 64 * 64 * 3},   {"encoder.2.reparam_conv.bias", 64},
        {"encoder.3.reparam_conv.weight", 128 * 64 * 3},  {"encoder.3.reparam_conv.bias", 128},
        {"decoder.rnn.weight_ih", 512 * 128}, {"decoder.rnn.weight_hh", 512 * 128},
        {"decoder.rnn.bias_ih", 512},         {"decoder.rnn.bias_hh", 512},
        {"decoder.decoder.2.weight", 128},    {"decoder.decoder.2.bias", 1},
    };
    const float* src[sizeof(wants) / sizeof(wants[0])];
    for (size_t i = 0; i < sizeof(wants) / sizeof(wants[0]); ++i) {
        const sb_tensor* t = find(tensors, n_tensors, wants[i].name);
        if (!t || !t->data) return fail(SB_MISSING_MODEL_ASSET, std::string("missing model asset: vad tensor ") + wants[i].name);
        if (t->numel != wants[i].numel)
            return fail(SB_INVALID_ARGUMENT, std::string("vad tensor ") + wants[i].name + " has " + std::to_string(t->numel) +
                                                 " elements, expected " + std::to_string(wants[i].numel));
        src[i] = t->data;
    }
    SB_CUDA(cudaSetDevice(c->device));
    SB_CUDA(vad_configure());
    VadModel* m = new VadModel();
    auto bail = [&](cudaError_t e) {
        m->release();
        delete m;
        return cuda_fail(e, "vad weight upload");
    };
    cudaError_t e;
    // [out][in][tap] -> [in][tap][out]
    auto conv_layout = [](const float* w, int co, int ci) {
        std::vector<float> r((size_t)co * ci * 3);
        for (int o = 0; o < co; ++o)
            for (int i = 0; i < ci; ++i)
                for (int t = 0; t < 3; ++t) r[((size_t)i * 3 + t) * co + o] = w[((size_t)o * ci + i) * 3 + t];
        return r;
    };
    if ((e = upload(std::vector<float>(src[0], src[0] + 258 * 256), &m->basis)) != cudaSuccess) return bail(e);
    if ((e = upload(conv_layout(src[1], 128, 129), &m->w1)) != cudaSuccess) return bail(e);
    if ((e = upload(std::vector<float>(src[2], src[2] + 128), &m->b1)) != cudaSuccess) return bail(e);
    if ((e = upload(conv_layout(src[3], 64, 128), &m->w2)) != cudaSuccess) return bail(e);
    if ((e = upload(std::vector<float>(src[4], src[4] + 64), &m->b2)) != cudaSuccess) return bail(e);
    if ((e = upload(conv_layout(src[5], 64, 64), &m->w3)) != cudaSuccess) return bail(e);
    if ((e = upload(std::vector<float>(src[6], src[6] + 64), &m->b3)) != cudaSuccess) return bail(e);
    {
        std::vector<float> r((size_t)64 * 128);
        for (int o = 0; o < 128; ++o)
            for (int i = 0; i < 64; ++i) r[(size_t)i * 128 + o] = src[7][((size_t)o * 64 + i) * 3 + 1];
        if ((e = upload(r, &m->w4)) != cudaSuccess) return bail(e);
    }
    if ((e = upload(std::vector<float>(src[8], src[8] + 128), &m->b4)) != cudaSuccess) return bail(e);
    {
        // gate rows in PyTorch order (i, f, g, o blocks of 128) -> row' = 4 * unit + gate
        std::vector<float> wih((size_t)128 * 512), whh((size_t)512 * 128), bs(512);
        for (int g = 0; g < 4; ++g)
            for (int u = 0; u < 128; ++u) {
                const int from = g * 128 + u, to = 4 * u + g;
                for (int k = 0; k < 128; ++k) {
                    wih[(size_t)k * 512 + to] = src[9][(size_t)from * 128 + k];
                    whh[(size_t)to * 128 + k] = src[10][(size_t)from * 128 + k];
                }
                bs[to] = src[11][from] + src[12][from];
            }
        if ((e = upload(wih, &m->wih)) != cudaSuccess) return bail(e);
        if ((e = upload(whh, &m->whh)) != cudaSuccess) return bail(e);
        if ((e = upload(bs, &m->bsum)) != cudaSuccess) return bail(e);
    }
    if ((e = upload(std::vector<float>(src[13], src[13] + 128), &m->wout)) != cudaSuccess) return bail(e);
    m->bout = src[14][0];
    if ((e = m->state.ensure(2 * kVadState * sizeof(float))) != cudaSuccess) return bail(e);
    if (c->vad) {
        cudaStreamSynchronize(c->stream);
        c->vad->release();
        delete c->vad;
    }
    c->vad = m;
    return SB_OK;
}

const float* vad_resident_audio(const sb_ctx* c) { return c->vad ? c->vad->audio.as<float>() : nullptr; }

int32_t vad_begin(sb_ctx* c, int64_t max_pass_windows, cudaStream_t st, bool two_buffers) {
    if (!c->vad) return fail(SB_MISSING_MODEL_ASSET, "missing model asset: vad network (sb_vad_load)");
    VadModel& m = *c->vad;
    SB_CUDA(cudaSetDevice(c->device));
    SB_CUDA(m.gx[0].ensure((size_t)max_pass_windows * kVadGates * sizeof(float)));
    if (two_buffers) SB_CUDA(m.gx[1].ensure((size_t)max_pass_windows * kVadGates * sizeof(float)));
    SB_CUDA(m.hout.ensure((size_t)max_pass_windows * kVadState * sizeof(float)));
    SB_CUDA(cudaMemsetAsync(m.state.p, 0, 2 * kVadState * sizeof(float), st));  // vad.rs:73-74
    return SB_OK;
}

int32_t vad_encode_pass(sb_ctx* c, cudaStream_t st, const float* d_audio, int64_t n_samples, int64_t first, int n, int buf) {
    VadModel& m = *c->vad;
    EncodeParams p{d_audio, n_samples, first, n,       m.basis, m.w1, m.b1, m.w2,
                   m.b2,    m.w3,      m.b3,  m.w4,    m.b4,    m.wih, m.bsum, m.gx[buf].as<float>()};
    c->prof.begin("vad_encode", st);
    vad_encode_kernel<<<(n + kTileWindows - 1) / kTileWindows, kEncThreads, kEncSmem, st>>>(p);
    c->prof.end(st);
    SB_CUDA(cudaGetLastError());
    c->launches += 1;
    return SB_OK;
}

int32_t vad_recur_pass(sb_ctx* c, cudaStream_t st, int64_t first, int n, int buf, float* d_prob) {
    VadModel& m = *c->vad;
    c->prof.begin("vad_lstm", st);
    float *gxp = m.gx[buf].as<float>(), *stp = m.state.as<float>(), *hop = m.hout.as<float>();
    cudaError_t e = c->vad_cluster == 4 ? launch_lstm<4>(gxp, m.whh, stp, hop, n, c->d_error, st)
                                        : launch_lstm<8>(gxp, m.whh, stp, hop, n, c->d_error, st);
    c->prof.end(st);
    SB_CUDA(e);
    c->prof.begin("vad_prob", st);
    vad_prob_kernel<<<(n + 7) / 8, 256, 0, st>>>(m.hout.as<float>(), m.wout, m.bout, d_prob + first, n);
    c->prof.end(st);
    SB_CUDA(cudaGetLastError());
    c->launches += 2;
    return SB_OK;
}

int32_t vad_process_device(sb_ctx* c, const float* d_audio, int64_t n_samples, float* d_prob) {
    if (!c->vad) return fail(SB_MISSING_MODEL_ASSET, "missing model asset: vad network (sb_vad_load)");
    if (n_samples <= 0) return SB_OK;
    const int64_t total = (n_samples + kVadWindow - 1) / kVadWindow;
    const int64_t seg = std::min<int64_t>(total, c->vad_segment_windows);
    int32_t s = vad_begin(c, seg, c->stream, false);
    if (s != SB_OK) return s;
    for (int64_t first = 0; first < total; first += seg) {
        const int n = (int)std::min<int64_t>(seg, total - first);
        if ((s = vad_encode_pass(c, c->stream, d_audio, n_samples, first, n, 0)) != SB_OK) return s;
        if ((s = vad_recur_pass(c, c->stream, first, n, 0, d_prob)) != SB_OK) return s;
    }
    return SB_OK;
}

}  // namespace sb
