// Persistent tcgen05 GEMM for sm_100a:  out = epilogue(A[M x K] * W[N x K]^T).
//
// Used for every position-wise projection of the FastConformer encoder (feed-forward,
// QKV / output, convolution-module pointwise, sub-sampling pointwise and linear) and the
// joint network's encoder projection.  Operands are K-major bf16 (or e4m3), accumulation
// is fp32 in tensor memory.
//
// One CTA per SM, 320 threads, warp-specialised:
//   warp 0      TMA producer: 128-byte-swizzled [128 x 64] A tiles and [BN x 64] W tiles
//               through a multi-stage shared-memory ring (full / empty mbarriers)
//   warp 1      allocates tensor memory, issues tcgen05.mma (M = 128, N = BN, K = 16 per
//               instruction, four per stage) from one lane; tcgen05.commit releases ring
//               slots and publishes finished accumulators
//   warps 2..9  epilogue: each warp owns one 32-lane quadrant of tensor memory and one half of
//               the tile's columns; tcgen05.ld (one row per thread), scales / bias / activation,
//               128-byte-swizzled staging slab in shared memory, TMA store of [32 rows x 128 B]
//               boxes (TMA reduce-add for the residual mode, so the residual stream is never read;
//               rows beyond M are clipped by the tensor map).  Two accumulator buffers (2 x BN
//               columns of tensor memory) let the epilogue of tile i overlap the main loop of i + 1.
// Every wait on an mbarrier is bounded by a cycle budget; when it runs out the kernel sets
// *error, drains, frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

#include "gemm.h"
#include "tc_ptx.cuh"

namespace sb {

namespace {

using namespace ptx;

constexpr int kBM = 128;
constexpr int kBKBytes = 128;  // one 128-byte swizzle row per operand row and stage
constexpr int kGemmThreads = 320;
constexpr int kEpiWarps = 8;
constexpr int kSlabBytes = 32 * 128;  // per epilogue warp: 32 rows x 128 bytes

// CTAS = 2: two CTAs of a cluster share one 256 x BN tile (tcgen05 cta_group::2); each stages its own 128 rows of A
// and its own half of the W rows, so a W tile crosses L2 -> SM once per 256 output rows instead of once per 128.
template <int BN, int CTAS = 1>
struct Cfg {
    static constexpr int kStages = CTAS == 2 ? 6 : (BN == 256 ? 4 : 6);
    static constexpr int kABytes = kBM * kBKBytes;
    static constexpr int kBBytes = (BN / CTAS) * kBKBytes;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarBytes = 256;
    static constexpr int kSmemBytes = kStages * kStageBytes + kEpiWarps * kSlabBytes + kBarBytes + 1024;  // + alignment slack
};

// Instruction descriptor: fp32 accumulate, A and B K-major, M = 128, N = BN.
template <int BN, bool FP8, int CTAS = 1>
__device__ __forceinline__ uint32_t make_idesc() {
    const uint32_t fmt = FP8 ? 0u : 1u;  // kind::f8f6f4: 0 = e4m3; kind::f16: 1 = bf16
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((kBM * CTAS) >> 4) << 24);
}

__device__ __forceinline__ uint32_t cvt4_e4m3(float a, float b, float c, float d) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);  // cvt2_e4m3 pairs: byte 0 = a, 1 = b, 2 = c, 3 = d
}

struct EpiParams {
    const float* bias;
    const float* row_scale;
    const float* col_scale;
    const float* out_row_scale;
    void* out;
    int M, N, K, ldo, act, out_mode;
    float alpha;
};

template <int BN, bool FP8, int CTAS>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
            const __grid_constant__ CUtensorMap tma_out, EpiParams ep, int* __restrict__ error) {
    using C = Cfg<BN, CTAS>;
    // rank of this CTA in its pair (the pair's leader, rank 0, owns the barriers the MMAs wait on)
    const uint32_t rank = CTAS == 2 ? cluster_ctarank() : 0u;
    constexpr int S = C::kStages;
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_dyn + (base - smem_u32(smem_dyn));
    const uint32_t a_base = base;
    const uint32_t b_base = base + S * C::kABytes;
    const uint32_t slab_base = base + S * C::kStageBytes;
    const uint32_t bar_base = slab_base + kEpiWarps * kSlabBytes;
    // barriers: full[S], empty[S], tmem_full[2], tmem_empty[2], then tmem pointer and abort flag
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * S + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * S + 2 + a); };
    uint32_t* tmem_slot =
        reinterpret_cast<uint32_t*>(base_ptr + S * C::kStageBytes + kEpiWarps * kSlabBytes + 8 * (2 * S + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int kTileM = kBM * CTAS;
    const int m_tiles = (ep.M + kTileM - 1) / kTileM;
    const int n_tiles = ep.N / BN;
    const int num_tiles = m_tiles * n_tiles;
    const int k_tiles = ep.K / (FP8 ? 128 : 64);
    const int tile0 = blockIdx.x / CTAS, tile_step = gridDim.x / CTAS;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), kEpiWarps * CTAS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if constexpr (CTAS == 2) {
            tmem_alloc_pair(smem_u32(tmem_slot), 2 * BN);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(smem_u32(tmem_slot), 2 * BN);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (CTAS == 2) cluster_sync();  // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int t = tile0; t < num_tiles && ok; t += tile_step) {
                const int m0 = (t / n_tiles) * kTileM + (int)rank * kBM;
                const int n0 = (t % n_tiles) * BN + (int)rank * (BN / CTAS);
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const int s = it % S;
                    const uint32_t ph = (it / S) & 1;
                    if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag)) { ok = false; break; }
                    const int kc = kt * (FP8 ? 128 : 64);
                    if constexpr (CTAS == 2) {
                        // both CTAs' bytes are counted on the leader's barrier
                        if (rank == 0) mbar_expect_tx(full_bar(s), 2 * C::kStageBytes);
                        const uint32_t lead = mapa(full_bar(s), 0);
                        tma_load_2d_pair(a_base + s * C::kABytes, &tma_a, lead, kc, m0);
                        tma_load_2d_pair(b_base + s * C::kBBytes, &tma_b, lead, kc, n0);
                    } else {
                        mbar_expect_tx(full_bar(s), C::kStageBytes);
                        tma_load_2d(a_base + s * C::kABytes, &tma_a, full_bar(s), kc, m0);
                        tma_load_2d(b_base + s * C::kBBytes, &tma_b, full_bar(s), kc, n0);
                    }
                }
            }
            if (!ok) {
                // give copies already in flight time to land before the CTA exits
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000) {}
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = make_idesc<BN, FP8, CTAS>();
            uint32_t it = 0, lt = 0;
            bool ok = true;
            for (int t = tile0; t < num_tiles && ok; t += tile_step, ++lt) {
                const int acc = lt & 1;
                const uint32_t acc_ph = (lt >> 1) & 1;
                if (!mbar_wait(tempty_bar(acc), acc_ph ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const int s = it % S;
                    const uint32_t ph = (it / S) & 1;
                    if (!mbar_wait(full_bar(s), ph, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t adesc = make_smem_desc(a_base + s * C::kABytes);
                    const uint64_t bdesc = make_smem_desc(b_base + s * C::kBBytes);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        // 32 bytes of K per instruction: +2 in the 16-byte start-address field
                        if constexpr (CTAS == 2) tc_mma_pair<FP8>(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kt | k) ? 1u : 0u);
                        else tc_mma<FP8>(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kt | k) ? 1u : 0u);
                    }
                    if constexpr (CTAS == 2) {
                        // the ring slot is free in both CTAs once these MMAs have read it
                        tc_commit_pair(mapa(empty_bar(s), 0));
                        tc_commit_pair(mapa(empty_bar(s), 1));
                    } else {
                        tc_commit(empty_bar(s));
                    }
                }
                if (ok) {
                    if constexpr (CTAS == 2) {
                        tc_commit_pair(mapa(tfull_bar(acc), 0));
                        tc_commit_pair(mapa(tfull_bar(acc), 1));
                    } else {
                        tc_commit(tfull_bar(acc));
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const int ew = warp - 2;
        const int quad = warp & 3;   // tensor-memory lane quadrant this warp may read
        const int half = ew >> 2;    // which half of the tile's columns
        const uint32_t slab = slab_base + ew * kSlabBytes;
        unsigned char* slab_ptr = base_ptr + S * C::kStageBytes + ew * kSlabBytes;
        const bool out_bf16 = ep.out_mode == kOutBf16;
        const bool out_fp8 = ep.out_mode == kOutFp8;
        const bool glu = ep.act == kActGlu;
        // accumulator columns per slab: 128 bytes per output row in every mode
        const int slab_cols = (out_fp8 || glu) ? 128 : (out_bf16 ? 64 : 32);
        const int sw = lane & 7;
        uint32_t lt = 0;
        bool ok = true;
        for (int t = tile0; t < num_tiles && ok; t += tile_step, ++lt) {
            const int acc = lt & 1;
            const uint32_t acc_ph = (lt >> 1) & 1;
            const int m0 = (t / n_tiles) * kTileM + (int)rank * kBM, n0 = (t % n_tiles) * BN;
            if (!mbar_wait(tfull_bar(acc), acc_ph, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const int row = m0 + quad * 32 + lane;
            const float rs = (FP8 && ep.row_scale && row < ep.M) ? ep.row_scale[row] : 1.0f;
            const float out_inv = (out_fp8 && row < ep.M) ? 1.0f / ep.out_row_scale[row] : 1.0f;
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN;
            const int cbeg = half * (BN / 2), cend = cbeg + BN / 2;
#pragma unroll 1
            for (int c = cbeg; c < cend; c += slab_cols) {
                // the slab is free again once the previous TMA store has read it
                if (lane == 0) bulk_wait_read0();
                __syncwarp();
#pragma unroll 1
                for (int sub = 0; sub * 32 < slab_cols; ++sub) {
                    uint32_t v[32];
                    tmem_ld32(taddr + c + 32 * sub, v);
                    tmem_wait_ld();
                    if (c + 32 * (sub + 1) >= cend) {
                        // this warp has read its part of the accumulator: hand it back to the MMA warp
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            if constexpr (CTAS == 2) mbar_arrive_cluster(mapa(tempty_bar(acc), 0));
                            else mbar_arrive(tempty_bar(acc));
                        }
                    }
                    const int col0 = n0 + c + 32 * sub;
                    float x[32];
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        float4 bb = make_float4(0.f, 0.f, 0.f, 0.f), cs = make_float4(1.f, 1.f, 1.f, 1.f);
                        if (ep.bias) bb = __ldg(reinterpret_cast<const float4*>(ep.bias + col0 + j));
                        if (FP8 && ep.col_scale) cs = __ldg(reinterpret_cast<const float4*>(ep.col_scale + col0 + j));
                        float f0 = __uint_as_float(v[j]), f1 = __uint_as_float(v[j + 1]);
                        float f2 = __uint_as_float(v[j + 2]), f3 = __uint_as_float(v[j + 3]);
                        if (FP8) { f0 *= rs * cs.x; f1 *= rs * cs.y; f2 *= rs * cs.z; f3 *= rs * cs.w; }
                        x[j] = f0 + bb.x; x[j + 1] = f1 + bb.y; x[j + 2] = f2 + bb.z; x[j + 3] = f3 + bb.w;
                    }
                    if (ep.act == kActSilu) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) x[j] = silu_fast(x[j]);
                    } else if (ep.act == kActRelu) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) x[j] = fmaxf(x[j], 0.0f);
                    }
                    if (glu) {
                        // 32 accumulator columns = 16 values and their 16 gates -> 16 outputs = 32 bytes
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            float y[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e)
                                y[e] = gate_fast(x[8 * q + e], x[16 + 8 * q + e]);
                            uint4 pk;
                            __nv_bfloat162 p0 = __floats2bfloat162_rn(y[0], y[1]), p1 = __floats2bfloat162_rn(y[2], y[3]);
                            __nv_bfloat162 p2 = __floats2bfloat162_rn(y[4], y[5]), p3 = __floats2bfloat162_rn(y[6], y[7]);
                            pk.x = *reinterpret_cast<uint32_t*>(&p0);
                            pk.y = *reinterpret_cast<uint32_t*>(&p1);
                            pk.z = *reinterpret_cast<uint32_t*>(&p2);
                            pk.w = *reinterpret_cast<uint32_t*>(&p3);
                            const int ch = 2 * sub + q;
                            *reinterpret_cast<uint4*>(slab_ptr + lane * 128 + ((ch ^ sw) << 4)) = pk;
                        }
                    } else if (out_fp8) {
                        // 32 columns = 32 bytes = chunks 2*sub, 2*sub + 1 of this row
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            uint32_t wd[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float* xv = x + 16 * q + 4 * e;
                                wd[e] = cvt4_e4m3(xv[0] * out_inv, xv[1] * out_inv, xv[2] * out_inv, xv[3] * out_inv);
                            }
                            const int ch = 2 * sub + q;
                            *reinterpret_cast<uint4*>(slab_ptr + lane * 128 + ((ch ^ sw) << 4)) =
                                make_uint4(wd[0], wd[1], wd[2], wd[3]);
                        }
                    } else if (out_bf16) {
                        // 32 columns = 64 bytes = chunks 4*sub .. 4*sub + 3 of this row
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint4 pk;
                            __nv_bfloat162 p0 = __floats2bfloat162_rn(x[8 * q], x[8 * q + 1]);
                            __nv_bfloat162 p1 = __floats2bfloat162_rn(x[8 * q + 2], x[8 * q + 3]);
                            __nv_bfloat162 p2 = __floats2bfloat162_rn(x[8 * q + 4], x[8 * q + 5]);
                            __nv_bfloat162 p3 = __floats2bfloat162_rn(x[8 * q + 6], x[8 * q + 7]);
                            pk.x = *reinterpret_cast<uint32_t*>(&p0);
                            pk.y = *reinterpret_cast<uint32_t*>(&p1);
                            pk.z = *reinterpret_cast<uint32_t*>(&p2);
                            pk.w = *reinterpret_cast<uint32_t*>(&p3);
                            const int ch = 4 * sub + q;
                            *reinterpret_cast<uint4*>(slab_ptr + lane * 128 + ((ch ^ sw) << 4)) = pk;
                        }
                    } else {
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const float4 r = make_float4(ep.alpha * x[4 * q], ep.alpha * x[4 * q + 1],
                                                         ep.alpha * x[4 * q + 2], ep.alpha * x[4 * q + 3]);
                            *reinterpret_cast<float4*>(slab_ptr + lane * 128 + ((q ^ sw) << 4)) = r;
                        }
                    }
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    if (ep.out_mode == kOutResidual) tma_reduce_add_2d(&tma_out, slab, n0 + c, m0 + quad * 32);
                    else tma_store_2d(&tma_out, slab, glu ? (n0 + c) >> 1 : n0 + c, m0 + quad * 32);
                    bulk_commit();
                }
            }
        }
        if (lane == 0) bulk_wait_all();
        __syncwarp();
    }

    tc_fence_before();
    __syncthreads();
    if constexpr (CTAS == 2) cluster_sync();  // neither CTA leaves while the other may still touch its memory
    if (warp == 1) {
        tc_fence_after();
        if constexpr (CTAS == 2) tmem_dealloc_pair(tmem_base, 2 * BN);
        else tmem_dealloc(tmem_base, 2 * BN);
    }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(error, 1);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
int g_pair_tiles = 1;  // process-wide: 0 never, 1 where it pays (see gemm_launch), 2 every product large enough

// 2-D row-major tensor [rows x cols] with a row pitch of `pitch_elems`; boxes of 128 bytes x box_rows, 128-byte swizzle.
bool make_map(CUtensorMap* map, const void* ptr, int rows, int cols, int pitch_elems, CUtensorMapDataType dt,
              int elem_bytes, int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)pitch_elems * elem_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)(kBKBytes / elem_bytes), (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

template <int BN, bool FP8, int CTAS>
cudaError_t launch_t(const GemmArgs& g, int sm_count, int* d_error, cudaStream_t stream) {
    alignas(64) CUtensorMap ma, mb, mo;
    const int eb = FP8 ? 1 : 2;
    const CUtensorMapDataType in_dt = FP8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const bool ob = g.out_mode == kOutBf16, o8 = g.out_mode == kOutFp8;
    const CUtensorMapDataType out_dt = o8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                          : (ob ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32);
    if (!make_map(&ma, g.a, g.M, g.K, g.K, in_dt, eb, kBM) || !make_map(&mb, g.w, g.N, g.K, g.K, in_dt, eb, BN / CTAS) ||
        !make_map(&mo, g.out, g.M, g.act == kActGlu ? g.N / 2 : g.N, g.ldo, out_dt, o8 ? 1 : (ob ? 2 : 4), 32))
        return cudaErrorInvalidValue;
    EpiParams ep{g.bias, g.row_scale, g.col_scale, g.out_row_scale, g.out, g.M, g.N, g.K, g.ldo, g.act, g.out_mode, g.alpha};
    const int tiles = ((g.M + kBM * CTAS - 1) / (kBM * CTAS)) * (g.N / BN);
    if constexpr (CTAS == 2) {
        const int pairs = std::min(tiles, sm_count / 2);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * pairs);
        cfg.blockDim = dim3(kGemmThreads);
        cfg.dynamicSmemBytes = Cfg<BN, CTAS>::kSmemBytes;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        return cudaLaunchKernelEx(&cfg, gemm_kernel<BN, FP8, CTAS>, ma, mb, mo, ep, d_error);
    } else {
        const int grid = tiles < sm_count ? tiles : sm_count;
        gemm_kernel<BN, FP8, CTAS><<<grid, kGemmThreads, Cfg<BN, CTAS>::kSmemBytes, stream>>>(ma, mb, mo, ep, d_error);
        return cudaGetLastError();
    }
}

}  // namespace

void gemm_set_pair_tiles(int mode) { g_pair_tiles = mode; }

cudaError_t gemm_configure(const char** why) {
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
            if (why) *why = "cuTensorMapEncodeTiled is not available from the driver";
            return e != cudaSuccess ? e : cudaErrorNotSupported;
        }
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    cudaError_t e;
#define SB_SET(BN, F8, CT)                                                                                  \
    e = cudaFuncSetAttribute(gemm_kernel<BN, F8, CT>, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                             Cfg<BN, CT>::kSmemBytes);                                                      \
    if (e != cudaSuccess) {                                                                                 \
        if (why) *why = "shared-memory opt-in for the GEMM kernel failed";                                  \
        return e;                                                                                           \
    }
    SB_SET(256, false, 1) SB_SET(128, false, 1) SB_SET(256, true, 1) SB_SET(128, true, 1)
    SB_SET(256, false, 2) SB_SET(256, true, 2)
#undef SB_SET
    return cudaSuccess;
}

cudaError_t gemm_launch(const GemmArgs& g, int sm_count, int* d_error, cudaStream_t stream) {
    if (!g_encode) return cudaErrorNotReady;
    if (g.M <= 0) return cudaSuccess;
    const int kq = g.fp8 ? 128 : 64;
    if (g.N % 128 != 0 || g.K % kq != 0 || g.K <= 0) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(g.a) & 15) || (reinterpret_cast<uintptr_t>(g.w) & 15) ||
        (reinterpret_cast<uintptr_t>(g.out) & 15) || (g.ldo & 7) || (reinterpret_cast<uintptr_t>(g.bias) & 15) ||
        (reinterpret_cast<uintptr_t>(g.col_scale) & 15))
        return cudaErrorInvalidValue;
    // BN = 256 when it divides N and still leaves at least one tile per SM; else 128.
    const int m_tiles = (g.M + kBM - 1) / kBM;
    if (g.out_mode == kOutFp8 && (g.N % 256 != 0 || !g.out_row_scale || (g.ldo & 15))) return cudaErrorInvalidValue;
    if (g.act == kActGlu && (g.N % 256 != 0 || g.out_mode != kOutBf16)) return cudaErrorInvalidValue;
    const bool wide = (g.N % 256 == 0) && (g.out_mode == kOutFp8 || g.act == kActGlu || m_tiles * (g.N / 256) >= sm_count);
    // Two CTAs per 256 x 256 tile when there is at least one such tile per pair of SMs.  Measured in the 8 h encoder
    // step against single-CTA tiles: residual-add products -15 % time (their fp32 epilogue leaves L2 little room
    // for operand traffic), K = 4096 products -9 %, QKV -6 %, the other K = 1024 products unchanged; the K = 256
    // sub-sampling products are 25 % slower (nothing to amortise), so short K stays on single-CTA tiles.
    const bool pair = g_pair_tiles && wide && ((g.M + 2 * kBM - 1) / (2 * kBM)) * (g.N / 256) >= sm_count / 2 &&
                      (g_pair_tiles == 2 || g.K >= 512);
    if (g.fp8) {
        if (pair) return launch_t<256, true, 2>(g, sm_count, d_error, stream);
        return wide ? launch_t<256, true, 1>(g, sm_count, d_error, stream) : launch_t<128, true, 1>(g, sm_count, d_error, stream);
    }
    if (pair) return launch_t<256, false, 2>(g, sm_count, d_error, stream);
    return wide ? launch_t<256, false, 1>(g, sm_count, d_error, stream) : launch_t<128, false, 1>(g, sm_count, d_error, stream);
}

}  // namespace sb
