// Relative-position multi-head attention on tcgen05 tensor cores (sm_100a): persistent CTAs, one (clip, head)
// item at a time, the next item's Q, K and V fetched while the current one is in its softmax / P V phases.
//
//   scores(i, j) = ((q_i + u) . k_j + (q_i + v) . p_{i-j}) / sqrt(128),  softmax over j,  out_i = sum_j P(i, j) v_j
// with p_r the projected sinusoidal embedding of relative position r (model.h: row (187 - r) of the
// per-layer table).  Part of the encoder that the reference runs as a CoreML blob
// (src/model.rs:327-342); T' <= 188 frames per clip, 8 heads of 128.
//
// For each block of 128 query rows:
//   TMA      Q [128 x 128], K [192 x 128] and the 320 table rows this block can reach, 128-byte swizzled
//   MMA 1    S_ac = Q K^T            (128 x 192, fp32, tensor memory columns 0..191)
//   MMA 2    S_bd = Q Pseg^T         (128 x 320, columns 192..511): column q of row i is relative
//            position i - j for j = q - ((T'-1) - i - first_row); the "relative shift" is therefore a
//            per-row offset, applied when each thread copies its own row out of tensor memory
//   softmax  four threads per query row (each a quarter of the columns): the shifted S_bd row goes through a private
//            fp32 row of shared memory, the scores S_ac + S_bd stay in registers; max, exp2, sum; probabilities
//            written as the bf16 A operand
//   MMA 3    O = P V                  (128 x 128; V is read as it lies in memory, as an MN-major B operand)
//   store    O / sum -> bf16, staged through shared memory, coalesced rows
// The u and v biases enter as per-key (u.k_j, computed here) and per-position (v.p, computed at model
// load) scalars written into the accumulators before the products are issued, so Q goes to the tensor
// cores untouched.  All mbarrier waits are bounded, and every
// wait is followed by a block-wide vote so that all threads leave the loop together.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

#include "attention.h"
#include "tc_ptx.cuh"

namespace sb {

namespace {

using namespace ptx;

constexpr int kAT = 128;             // query rows per block
constexpr int kATh = 512;            // threads per CTA: four per query row, each owning a quarter of the columns
constexpr int kNK = 192;             // key columns of S_ac (T' padded)
constexpr int kNP = 320;             // table rows per query block (256 + 64)
constexpr int kSStride = 189;        // floats per shifted S_bd row (odd: conflict-free reads)
constexpr int kR1 = 97280;           // table rows (2 x 40 KB) / shifted S_bd rows (128 x 189 x 4) / probabilities + output staging
constexpr int kR2 = 49152;           // K (2 x 24 KB), resident for both query blocks
constexpr int kR3 = 32768;           // Q (2 x 16 KB)
constexpr int kR4 = 49152;           // V (2 blocks of 64 d x 192 key rows)
constexpr int kPOff = 0;             // probabilities inside region 1 (3 x 16 KB)
constexpr int kOOff = 49152;         // output staging inside region 1
constexpr int kTailOff = 128 * kSStride * 4;  // 512 spare bytes of region 1 that no other use touches
constexpr int kSmall = (kNK + kNP) * 4 + 3 * kAT * 4 + 64;
constexpr int kAttSmem = kR1 + kR2 + kR3 + kR4 + kSmall;
constexpr int kOStride = 272;        // bytes per staged output row (256 + 16)
constexpr uint32_t kBoxBytes = 64 * 128;  // one TMA box: 64 rows x 128 bytes
static_assert(kAttSmem <= 232448, "shared memory budget");
static_assert(kOOff + kAT * kOStride <= kTailOff && 2 * 40960 <= kTailOff && kTailOff + kAT * 4 <= kR1, "region 1 layout");

__device__ __forceinline__ uint32_t idesc_bf16(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

__global__ void __launch_bounds__(kATh, 1)
relpos_attention_tc_kernel(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_pos,
                           const int* __restrict__ t3_off, int n_items,
                           const float* __restrict__ bias_u, const float* __restrict__ pos_vp,
                           bf16* __restrict__ out, int* __restrict__ error) {
    extern __shared__ __align__(1024) unsigned char att_dyn[];
    const uint32_t base = smem_u32(att_dyn);
    if (base & 1023u) {  // the swizzled operand tiles need 1024-byte alignment
        if (threadIdx.x == 0) atomicExch(error, 2);
        return;
    }
    unsigned char* bp = att_dyn;
    const uint32_t r1 = base, r2 = r1 + kR1, r3 = r2 + kR2, r4 = r3 + kR3;
    unsigned char* p1 = bp;
    unsigned char* p2 = bp + kR1;
    float* pre = reinterpret_cast<float*>(bp + kR1 + kR2 + kR3 + kR4);  // [uk (192) | vp (320)]: accumulator preload
    float* uk = pre;
    float* vp = pre + kNK;
    float* part = vp + kNP;  // [3][128] row partials of quarters 0..2 (maxima, later sums); also u while u.k is formed
    float* part3 = reinterpret_cast<float*>(p1 + kTailOff);  // [128] partials of quarter 3
    const uint32_t bar0 = r4 + kR4 + (kNK + kNP + 3 * kAT) * 4;  // seven barriers, then tmem slot, abort flag
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(part + 3 * kAT) + 14;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t bar_qk = bar0, bar_q2 = bar0 + 8, bar_tab = bar0 + 16, bar_v = bar0 + 24;
    const uint32_t bar_sbd = bar0 + 32, bar_sac = bar0 + 40, bar_o = bar0 + 48;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int lg = warp & 3;   // tensor-memory lane group of this warp: rows 32 lg .. 32 lg + 31 of the block
    const int qd = warp >> 2;  // column quarter
    const int rl = 32 * lg + lane;
    auto part_of = [&](int q) -> float* { return q < 3 ? part + q * kAT : part3; };
    // work items: (clip, head) pairs, strided over the persistent CTAs; empty clips are skipped
    auto next_item = [&](int it) {
        while (it < n_items && t3_off[(it >> 3) + 1] - t3_off[it >> 3] <= 0) it += gridDim.x;
        return it;
    };
    // Q rows of query block qb and (qb == 0) the K rows of an item -> regions 3 and 2
    auto load_q = [&](int it, int qb, uint32_t bar) {
        const int head = it & 7, row0 = t3_off[it >> 3];
        mbar_expect_tx(bar, (qb == 0 ? 10 : 4) * kBoxBytes);
        for (int kb = 0; kb < 2; ++kb) {
            const int col = head * kHeadDim + kb * 64;
            for (int h = 0; h < 2; ++h)
                tma_load_2d(r3 + kb * 16384 + h * kBoxBytes, &map_qkv, bar, col, row0 + qb * kAT + h * 64);
            if (qb == 0)
                for (int h = 0; h < 3; ++h)   // K rows 0 .. 191, kept for the second block
                    tma_load_2d(r2 + kb * 24576 + h * kBoxBytes, &map_qkv, bar, kDModel + col, row0 + h * 64);
        }
    };
    // V as it lies in memory, [192 j x 128 d]: an MN-major B operand, two blocks of 64 d, each 192 key rows of
    // 128 bytes.  Rows beyond T' belong to the next clip (or are zero fill) and meet probabilities that are zero.
    auto load_v = [&](int it) {
        const int head = it & 7, row0 = t3_off[it >> 3];
        mbar_expect_tx(bar_v, 6 * kBoxBytes);
        for (int h = 0; h < 2; ++h)
            for (int kb = 0; kb < 3; ++kb)
                tma_load_2d(r4 + h * 24576 + kb * kBoxBytes, &map_qkv, bar_v, 2 * kDModel + head * kHeadDim + h * 64,
                            row0 + kb * 64);
    };

    if (tid == 0) {
        for (int i = 0; i < 7; ++i) mbar_init(bar0 + 8 * i, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tq = tmem + ((uint32_t)(lg * 32) << 16);

    const float sc2 = 0.08838834764831845f * 1.4426950408889634f;  // log2(e) / sqrt(128)
    uint32_t ph_qk = 0, ph_q2 = 0, ph_tab = 0, ph_v = 0, ph_sbd = 0, ph_sac = 0, ph_o = 0;
    bool ok = true;

    int item = next_item(blockIdx.x);
    if (item < n_items && tid == 0) {
        load_q(item, 0, bar_qk);
        load_v(item);
    }
    while (item < n_items && ok) {
        const int head = item & 7, clip = item >> 3;
        const int row0 = t3_off[clip];
        const int t = t3_off[clip + 1] - row0;
        const int next = next_item(item + gridDim.x);
        const int p_first = (kMaxEncFrames - 1) - (t - 1);  // table row of relative position t - 1
        const int n_blocks = (t + kAT - 1) / kAT;
        if (tid < kHeadDim) part[tid] = bias_u[head * kHeadDim + tid];  // u, until the first partials are written

        for (int qb = 0; qb < n_blocks && ok; ++qb) {
            const int i0 = qb * kAT;
            const bool last = qb == n_blocks - 1;
            const int plo = max(0, (t - 1) - (i0 + kAT - 1));  // first local table row this block can reach
            if (tid == 0) {
                mbar_expect_tx(bar_tab, 10 * kBoxBytes);
                for (int kb = 0; kb < 2; ++kb)
                    for (int h = 0; h < 5; ++h)   // table rows plo .. plo + 319
                        tma_load_2d(r1 + kb * 40960 + h * kBoxBytes, &map_pos, bar_tab, head * kHeadDim + kb * 64,
                                    p_first + plo + h * 64);
            }
            // v . p for the table rows of this block, written into the S_bd accumulators while the loads fly
            if (tid < kNP) {
                const int p = p_first + plo + tid;
                vp[tid] = p < kPosRows ? pos_vp[p * kHeads + head] : 0.0f;
            }
            __syncthreads();
#pragma unroll 1
            for (int c = kNK / 16 + qd; c < (kNK + kNP) / 16; c += 4) {
                uint32_t v[16];
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const uint4 x = *reinterpret_cast<const uint4*>(pre + 16 * c + 4 * g);
                    v[4 * g] = x.x; v[4 * g + 1] = x.y; v[4 * g + 2] = x.z; v[4 * g + 3] = x.w;
                }
                tmem_st16(tq + 16 * c, v);
            }
            if (qb == 0) {
                if (!__syncthreads_and(mbar_wait(bar_qk, ph_qk, abort_flag))) { ok = false; break; }
                ph_qk ^= 1;
                // u . k_j from the swizzled K tile
                if (tid < kNK) {
                    const int j = tid;
                    float acc = 0.0f;
                    if (j < t) {
#pragma unroll
                        for (int ch = 0; ch < 16; ++ch) {
                            const int kb = ch >> 3, c8 = ch & 7;
                            const uint4 raw = *reinterpret_cast<const uint4*>(p2 + kb * 24576 + j * 128 + ((c8 ^ (j & 7)) << 4));
                            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float2 f = __bfloat1622float2(h2[e]);
                                acc = fmaf(part[ch * 8 + 2 * e], f.x, acc);
                                acc = fmaf(part[ch * 8 + 2 * e + 1], f.y, acc);
                            }
                        }
                    }
                    uk[j] = acc;
                }
                __syncthreads();
            } else {
                if (!__syncthreads_and(mbar_wait(bar_q2, ph_q2, abort_flag))) { ok = false; break; }
                ph_q2 ^= 1;
            }
            // columns [0, 192) of the accumulators start from u . k_j, the same in every row
#pragma unroll 1
            for (int c = qd; c < kNK / 16; c += 4) {
                uint32_t v[16];
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const uint4 x = *reinterpret_cast<const uint4*>(pre + 16 * c + 4 * g);
                    v[4 * g] = x.x; v[4 * g + 1] = x.y; v[4 * g + 2] = x.z; v[4 * g + 3] = x.w;
                }
                tmem_st16(tq + 16 * c, v);
            }
            tmem_wait_st();
            tc_fence_before();
            if (!__syncthreads_and(mbar_wait(bar_tab, ph_tab, abort_flag))) { ok = false; break; }
            ph_tab ^= 1;
            if (tid == 0) {
                tc_fence_after();
                // S_bd first: its read-out (the shift pass) can start while S_ac is still being formed
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int kb = k >> 2, ko = (k & 3) * 2;
                    const uint64_t a = make_smem_desc(r3 + kb * 16384) + ko;
                    tc_mma<false>(tmem + kNK, a, make_smem_desc(r1 + kb * 40960) + ko, idesc_bf16(256), 1u);
                    tc_mma<false>(tmem + kNK + 256, a, make_smem_desc(r1 + kb * 40960 + 256 * 128) + ko, idesc_bf16(64), 1u);
                }
                tc_commit(bar_sbd);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int kb = k >> 2, ko = (k & 3) * 2;
                    const uint64_t a = make_smem_desc(r3 + kb * 16384) + ko;
                    tc_mma<false>(tmem, a, make_smem_desc(r2 + kb * 24576) + ko, idesc_bf16(kNK), 1u);
                }
                tc_commit(bar_sac);
            }
            if (!__syncthreads_and(mbar_wait(bar_sbd, ph_sbd, abort_flag))) { ok = false; break; }
            ph_sbd ^= 1;
            tc_fence_after();

            const int i = i0 + rl;
            const bool warp_live = i0 + 32 * lg < t;  // some row of this warp exists
            float* srow = reinterpret_cast<float*>(p1) + rl * kSStride;
            float s[48];
            float mx = -INFINITY;
            if (warp_live) {
                // S_bd: the relative shift is a per-row offset, applied while each thread copies its quarter of its
                // row out of tensor memory: column q of S_bd is key j = q - shift
                const int shift = (t - 1) - i - plo;
                const int shift_hi = __shfl_sync(0xffffffffu, shift, 0), shift_lo = shift_hi - 31;
                float* srow_sh = srow - shift;
#pragma unroll 1
                for (int c = 0; c < 5; ++c) {
                    const int q0 = 80 * qd + 16 * c;
                    if (q0 + 15 < shift_lo || q0 >= shift_hi + t) continue;  // no lane has a key in this chunk
                    uint32_t v[16];
                    tmem_ld16(tq + kNK + q0, v);
                    tmem_wait_ld();
                    if (q0 >= shift_hi && q0 + 15 < shift_lo + t) {
#pragma unroll
                        for (int jj = 0; jj < 16; ++jj) srow_sh[q0 + jj] = __uint_as_float(v[jj]);
                    } else {
#pragma unroll
                        for (int jj = 0; jj < 16; ++jj)
                            if ((unsigned)(q0 + jj - shift) < (unsigned)t) srow_sh[q0 + jj] = __uint_as_float(v[jj]);
                    }
                }
            }
            // (the vote also orders the four threads' shares of a shifted row before they are read)
            if (!__syncthreads_and(mbar_wait(bar_sac, ph_sac, abort_flag))) { ok = false; break; }
            ph_sac ^= 1;
            tc_fence_after();
            // Q (and, after the last block, K) are no longer needed: fetch what comes next into their place
            if (tid == 0) {
                if (!last) {
                    fence_proxy_async();
                    load_q(item, qb + 1, bar_q2);
                } else if (next < n_items) {
                    fence_proxy_async();
                    load_q(next, 0, bar_qk);
                }
            }
            if (warp_live) {
                // scores (kept in registers, unscaled) and the row maximum over this thread's 48 keys
#pragma unroll
                for (int m = 0; m < 3; ++m) {
                    const int j0 = 48 * qd + 16 * m;
                    if (j0 + 15 < t) {
                        uint32_t v[16];
                        tmem_ld16(tq + j0, v);
                        tmem_wait_ld();
#pragma unroll
                        for (int jj = 0; jj < 16; ++jj) {
                            s[16 * m + jj] = __uint_as_float(v[jj]) + srow[j0 + jj];
                            mx = fmaxf(mx, s[16 * m + jj]);
                        }
                    } else if (j0 < t) {
                        uint32_t v[16];
                        tmem_ld16(tq + j0, v);
                        tmem_wait_ld();
#pragma unroll
                        for (int jj = 0; jj < 16; ++jj) {
                            s[16 * m + jj] = j0 + jj < t ? __uint_as_float(v[jj]) + srow[j0 + jj] : -INFINITY;
                            mx = fmaxf(mx, s[16 * m + jj]);
                        }
                    } else {
#pragma unroll
                        for (int jj = 0; jj < 16; ++jj) s[16 * m + jj] = -INFINITY;
                    }
                }
                part_of(qd)[rl] = mx;
            }
            __syncthreads();
            float sum = 0.0f;
            if (warp_live) {
                mx = fmaxf(fmaxf(part[rl], part[kAT + rl]), fmaxf(part[2 * kAT + rl], part3[rl]));
                const float mc = mx * sc2;
                // probabilities -> bf16 A operand (K-major, 128-byte swizzle, three blocks of 64 keys)
#pragma unroll
                for (int m8 = 0; m8 < 6; ++m8) {
                    float e[8];
#pragma unroll
                    for (int u8 = 0; u8 < 8; ++u8) {
                        e[u8] = ex2_approx(fmaf(s[8 * m8 + u8], sc2, -mc));
                        sum += e[u8];
                    }
                    uint4 pk;
                    __nv_bfloat162 q0 = __floats2bfloat162_rn(e[0], e[1]), q1 = __floats2bfloat162_rn(e[2], e[3]);
                    __nv_bfloat162 q2 = __floats2bfloat162_rn(e[4], e[5]), q3 = __floats2bfloat162_rn(e[6], e[7]);
                    pk.x = *reinterpret_cast<uint32_t*>(&q0);
                    pk.y = *reinterpret_cast<uint32_t*>(&q1);
                    pk.z = *reinterpret_cast<uint32_t*>(&q2);
                    pk.w = *reinterpret_cast<uint32_t*>(&q3);
                    const int j8 = 48 * qd + 8 * m8;
                    const int kb = j8 >> 6, ch = (j8 & 63) >> 3;
                    *reinterpret_cast<uint4*>(p1 + kPOff + kb * 16384 + rl * 128 + ((ch ^ (rl & 7)) << 4)) = pk;
                }
            }
            fence_proxy_async();
            tc_fence_before();
            __syncthreads();  // probabilities complete; every thread has read the row maxima
            if (qb == 0) {
                if (!__syncthreads_and(mbar_wait(bar_v, ph_v, abort_flag))) { ok = false; break; }
                ph_v ^= 1;
            }
            if (tid == 0) {
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < kNK / 16; ++k) {
                    const int kb = k >> 2, ko = (k & 3) * 2;
                    tc_mma<false>(tmem, make_smem_desc(r1 + kPOff + kb * 16384) + ko, make_smem_desc_mn(r4 + k * 2048, 24576),
                                  idesc_bf16(kHeadDim) | (1u << 16), k ? 1u : 0u);
                }
                tc_commit(bar_o);
            }
            if (warp_live) part_of(qd)[rl] = sum;  // the partial maxima are dead: the slots now carry the partial sums
            if (!__syncthreads_and(mbar_wait(bar_o, ph_o, abort_flag))) { ok = false; break; }
            ph_o ^= 1;
            tc_fence_after();
            if (last && next < n_items && tid == 0) load_v(next);  // V was read by the tensor cores only
            // O / sum -> bf16 -> staging rows -> coalesced global rows
            if (warp_live) {
                const float inv = i < t ? 1.0f / ((part[rl] + part[kAT + rl]) + (part[2 * kAT + rl] + part3[rl])) : 0.0f;
                uint32_t v[32];
                tmem_ld32(tq + 32 * qd, v);
                tmem_wait_ld();
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint4 pk;
                    __nv_bfloat162 o0 = __floats2bfloat162_rn(__uint_as_float(v[8 * q]) * inv, __uint_as_float(v[8 * q + 1]) * inv);
                    __nv_bfloat162 o1 = __floats2bfloat162_rn(__uint_as_float(v[8 * q + 2]) * inv, __uint_as_float(v[8 * q + 3]) * inv);
                    __nv_bfloat162 o2 = __floats2bfloat162_rn(__uint_as_float(v[8 * q + 4]) * inv, __uint_as_float(v[8 * q + 5]) * inv);
                    __nv_bfloat162 o3 = __floats2bfloat162_rn(__uint_as_float(v[8 * q + 6]) * inv, __uint_as_float(v[8 * q + 7]) * inv);
                    pk.x = *reinterpret_cast<uint32_t*>(&o0);
                    pk.y = *reinterpret_cast<uint32_t*>(&o1);
                    pk.z = *reinterpret_cast<uint32_t*>(&o2);
                    pk.w = *reinterpret_cast<uint32_t*>(&o3);
                    *reinterpret_cast<uint4*>(p1 + kOOff + rl * kOStride + qd * 64 + q * 16) = pk;
                }
            }
            tc_fence_before();
            __syncthreads();
            const int valid = min(kAT, t - i0);
            for (int r = warp; r < valid; r += kATh / 32) {
                const uint2 val = *reinterpret_cast<const uint2*>(p1 + kOOff + r * kOStride + lane * 8);
                *reinterpret_cast<uint2*>(out + (size_t)(row0 + i0 + r) * kDModel + head * kHeadDim + lane * 4) = val;
            }
            fence_proxy_async();  // generic accesses to region 1 are ordered before the next table load lands there
            __syncthreads();      // staging, partials and the u vector are reused by the next block / item
        }
        item = next;
    }

    tc_fence_before();
    __syncthreads();
    if (!ok || *abort_flag) {
        // give copies that may still be in flight time to land before the shared memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) {}
    }
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
    if (tid == 0 && *abort_flag) atomicExch(error, 1);
}

// vp[p][h] = sum_d v[h][d] * pos[p][h * 128 + d].  grid kPosRows, 256 threads (8 warps = 8 heads).
__global__ void __launch_bounds__(256)
pos_bias_kernel(const bf16* __restrict__ pos, const float* __restrict__ bias_v, float* __restrict__ vp) {
    const int p = blockIdx.x, head = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float acc = 0.0f;
    for (int d = lane; d < kHeadDim; d += 32)
        acc = fmaf(bias_v[head * kHeadDim + d], __bfloat162float(pos[(size_t)p * kDModel + head * kHeadDim + d]), acc);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) vp[p * kHeads + head] = acc;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_enc = nullptr;

bool map_bf16(CUtensorMap* m, const void* ptr, int64_t rows, int64_t cols) {
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {64, 64};
    const cuuint32_t estr[2] = {1, 1};
    return g_enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

cudaError_t attention_configure() {
    if (!g_enc) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) return e != cudaSuccess ? e : cudaErrorNotSupported;
        g_enc = reinterpret_cast<EncodeTiledFn>(fn);
    }
    return cudaFuncSetAttribute(relpos_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttSmem);
}

cudaError_t pos_bias_launch(const bf16* pos_proj, const float* bias_v, float* vp, cudaStream_t st) {
    pos_bias_kernel<<<kPosRows, 256, 0, st>>>(pos_proj, bias_v, vp);
    return cudaGetLastError();
}

cudaError_t attention_launch(const bf16* qkv, int rows, const int* d_t3_off, int n_clips, const bf16* pos_proj,
                             const float* bias_u, const float* pos_vp, bf16* out, int sm_count, int* d_error,
                             cudaStream_t st) {
    if (n_clips <= 0 || rows <= 0) return cudaSuccess;
    alignas(64) CUtensorMap mq, mp;
    if (!map_bf16(&mq, qkv, rows, 3 * kDModel) || !map_bf16(&mp, pos_proj, kPosRows, kDModel))
        return cudaErrorInvalidValue;
    const int n_items = n_clips * kHeads;
    relpos_attention_tc_kernel<<<std::min(n_items, sm_count), kATh, kAttSmem, st>>>(mq, mp, d_t3_off, n_items, bias_u, pos_vp,
                                                                                   out, d_error);
    return cudaGetLastError();
}

}  // namespace sb
