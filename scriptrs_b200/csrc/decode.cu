// Batched TDT greedy decoding on sm_100a: one persistent cooperative kernel for a whole batch.
//
// Replaces the reference's per-chunk loop (ParakeetModel::greedy_decode and GreedyDecodeState,
// src/model.rs:64-214), which calls two CoreML blobs per iteration (predictor: src/coreml.rs:239-308,
// joint decision: src/coreml.rs:312-359).  The state machine is the reference's, per sequence:
//   h = c = 0, last_token = blank, frame = 0, emitted = 0, predictor cache empty
//   while frame < T':  run the predictor only if its cache is empty; joint(enc[frame], cache);
//                      token = argmax over [0, 1025), duration = argmax over the 5 duration logits;
//                      non-blank: record (token, frame, duration, max-softmax), commit the cached
//                      LSTM state, empty the cache, emitted += 1;
//                      duration > 0: frame += duration, emitted = 0;
//                      else blank or emitted >= 10: frame += 1, emitted = 0.
// Sequences advance at different rates, so every iteration first builds (redundantly in every CTA,
// hence in a deterministic order) the list of live sequences and of those whose predictor must run,
// then runs four skinny fp32 GEMM phases over those lists (LSTM layer 0, layer 1 with the cell update
// fused into the epilogue, predictor projection, joint output) and a per-sequence arg-max / update
// phase, with a grid-wide barrier between phases.  Weights (35 MB fp32) stay L2-resident; the
// encoder projection is hoisted out of the loop.  Sums run in a fixed order, so results are
// reproducible; arg-max ties go to the lowest index.
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "decode.h"

namespace cg = cooperative_groups;

namespace sb {

namespace {

constexpr int kThreads = 256;
constexpr int kTileSeq = 32;   // sequences per tile
constexpr int kTileRow = 64;   // weight rows per tile (LSTM: 16 units x 4 gates)
constexpr int kTileK = 32;
constexpr int kWStride = kTileRow + 1;
constexpr int kXStride = kTileSeq + 1;

enum Phase { kLstm0 = 0, kLstm1 = 1, kPred = 2, kOut = 3 };

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

struct Lists {
    int* act;  // live sequences, ascending
    int* upd;  // live sequences whose predictor cache is empty
    int n_act, n_upd;
};

// Every CTA builds the same lists from the per-sequence state (block-wide ordered compaction).
__device__ void build_lists(const DecodeState& s, int n_seq, int* act, int* upd, int* counts, int* scan) {
    const int tid = threadIdx.x;
    if (tid == 0) { counts[0] = 0; counts[1] = 0; }
    __syncthreads();
    for (int base = 0; base < n_seq; base += kThreads) {
        const int b = base + tid;
        int live = 0, need = 0;
        if (b < n_seq) {
            live = s.frame_idx[b] < s.enc_len[b];
            need = live && !s.cache_valid[b];
        }
        // ordered compaction via ballot within warps, then a serial pass over the 8 warp totals
        const unsigned ml = __ballot_sync(0xffffffffu, live), mn = __ballot_sync(0xffffffffu, need);
        const int warp = tid >> 5, lane = tid & 31;
        if (lane == 0) { scan[warp] = __popc(ml); scan[8 + warp] = __popc(mn); }
        __syncthreads();
        int offl = counts[0], offn = counts[1];
        for (int w = 0; w < warp; ++w) { offl += scan[w]; offn += scan[8 + w]; }
        const unsigned below = (1u << lane) - 1u;
        if (live) act[offl + __popc(ml & below)] = b;
        if (need) upd[offn + __popc(mn & below)] = b;
        __syncthreads();
        if (tid == 0) {
            int tl = 0, tn = 0;
            for (int w = 0; w < 8; ++w) { tl += scan[w]; tn += scan[8 + w]; }
            counts[0] += tl;
            counts[1] += tn;
        }
        __syncthreads();
    }
}

// One phase: C[list x rows] = X[list x K] * W[rows x K]^T, tiled 32 sequences x 64 rows, fp32, K in
// ascending order.  Thread (sg = tid / 16, ul = tid % 16) owns sequences {2 sg, 2 sg + 1} and local rows
// {ul, ul + 16, ul + 32, ul + 48}; for the LSTM phases those four rows are the i, f, g, o gates of one unit.
template <int PHASE>
__device__ void run_phase(const DecodeWeights& w, const DecodeState& s, const int* list, int n_list, float* Ws,
                          float* Xs) {
    constexpr bool lstm = PHASE == kLstm0 || PHASE == kLstm1;
    constexpr int K = lstm ? 2 * kPredHidden : kPredHidden;
    constexpr int rows_total = lstm ? 4 * kPredHidden : (PHASE == kPred ? kJointDim : kJointOut);
    constexpr int row_tiles = lstm ? kPredHidden / 16 : (rows_total + kTileRow - 1) / kTileRow;
    constexpr int layer = PHASE == kLstm1 ? 1 : 0;
    const float* W_a = nullptr;  // first K-half
    const float* W_b = nullptr;  // second K-half (LSTM: hidden-to-hidden)
    if (PHASE == kLstm0 || PHASE == kLstm1) {
        W_a = w.w_ih + (size_t)layer * 4 * kPredHidden * kPredHidden;
        W_b = w.w_hh + (size_t)layer * 4 * kPredHidden * kPredHidden;
    } else if (PHASE == kPred) {
        W_a = w.w_pred;
    } else {
        W_a = w.w_out;
    }
    const int tid = threadIdx.x;
    const int sg = tid >> 4, ul = tid & 15;
    const int seq_tiles = (n_list + kTileSeq - 1) / kTileSeq;
    const int n_tiles = seq_tiles * row_tiles;
    const size_t BH = (size_t)s.n_seq * kPredHidden;

    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int st = tile / row_tiles, rt = tile % row_tiles;
        const int s0 = st * kTileSeq;
        float acc[2][4];
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[a][r] = 0.0f;

        for (int k0 = 0; k0 < K; k0 += kTileK) {
            __syncthreads();
            // weights chunk: 64 rows x 32 k, stored k-major
            for (int i = tid; i < kTileRow * kTileK; i += kThreads) {
                const int r = i >> 5, k = i & 31;
                int grow;
                if (lstm) grow = (r >> 4) * kPredHidden + rt * 16 + (r & 15);
                else grow = rt * kTileRow + r;
                float v = 0.0f;
                if (grow < rows_total) {
                    if (lstm) {
                        const int kk = k0 + k;
                        v = kk < kPredHidden ? W_a[(size_t)grow * kPredHidden + kk]
                                             : W_b[(size_t)grow * kPredHidden + kk - kPredHidden];
                    } else {
                        v = W_a[(size_t)grow * K + k0 + k];
                    }
                }
                Ws[k * kWStride + r] = v;
            }
            // activations chunk: 32 sequences x 32 k, stored k-major
            for (int i = tid; i < kTileSeq * kTileK; i += kThreads) {
                const int sl = i >> 5, k = i & 31;
                const int li = s0 + sl;
                float v = 0.0f;
                if (li < n_list) {
                    const int b = list[li];
                    const int kk = k0 + k;
                    if (PHASE == kLstm0) {
                        v = kk < kPredHidden ? w.embedding[(size_t)s.last_token[b] * kPredHidden + kk]
                                             : s.h[(size_t)b * kPredHidden + kk - kPredHidden];
                    } else if (PHASE == kLstm1) {
                        v = kk < kPredHidden ? s.h_new[(size_t)b * kPredHidden + kk]
                                             : s.h[BH + (size_t)b * kPredHidden + kk - kPredHidden];
                    } else if (PHASE == kPred) {
                        v = s.h_new[BH + (size_t)b * kPredHidden + kk];
                    } else {
                        const size_t row = (size_t)(s.enc_off[b] + s.frame_idx[b]);
                        v = fmaxf(s.enc_proj[row * kJointDim + kk] + s.pred[(size_t)b * kJointDim + kk], 0.0f);
                    }
                }
                Xs[k * kXStride + sl] = v;
            }
            __syncthreads();
#pragma unroll 8
            for (int k = 0; k < kTileK; ++k) {
                const float x0 = Xs[k * kXStride + 2 * sg], x1 = Xs[k * kXStride + 2 * sg + 1];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float wv = Ws[k * kWStride + ul + 16 * r];
                    acc[0][r] = fmaf(x0, wv, acc[0][r]);
                    acc[1][r] = fmaf(x1, wv, acc[1][r]);
                }
            }
        }
        // epilogue
#pragma unroll
        for (int a = 0; a < 2; ++a) {
            const int li = s0 + 2 * sg + a;
            if (li >= n_list) continue;
            const int b = list[li];
            if (lstm) {
                const int u = rt * 16 + ul;
                const float* bg = w.b_gates + (size_t)layer * 4 * kPredHidden;
                const float gi = acc[a][0] + bg[u], gf = acc[a][1] + bg[kPredHidden + u];
                const float gg = acc[a][2] + bg[2 * kPredHidden + u], go = acc[a][3] + bg[3 * kPredHidden + u];
                const size_t idx = (size_t)layer * BH + (size_t)b * kPredHidden + u;
                const float cn = sigmoid_f(gf) * s.c[idx] + sigmoid_f(gi) * tanhf(gg);
                s.c_new[idx] = cn;
                s.h_new[idx] = sigmoid_f(go) * tanhf(cn);
            } else {
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int row = rt * kTileRow + ul + 16 * r;
                    if (row >= rows_total) continue;
                    if (PHASE == kPred) s.pred[(size_t)b * kJointDim + row] = acc[a][r] + w.b_pred[row];
                    else s.logits[(size_t)b * kJointOut + row] = acc[a][r] + w.b_out[row];
                }
            }
        }
    }
}

// One warp per live sequence: arg-max, confidence, record, commit, advance (model.rs:79-90,180-209).
__device__ void decide_phase(const DecodeState& s, const int* act, int n_act, int step) {
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = kThreads / 32;
    const size_t BH = (size_t)s.n_seq * kPredHidden;
    for (int li = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); li < n_act; li += gridDim.x * warps_per_cta) {
        const int b = act[li];
        const float* lg = s.logits + (size_t)b * kJointOut;
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = lane; i < kVocab; i += 32) {
            const float v = lg[i];
            if (v > best) { best = v; bi = i; }  // ascending i per lane: first maximum kept
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        float sum = 0.0f;
        for (int i = lane; i < kVocab; i += 32) sum += expf(lg[i] - best);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        int dur = 0;
        {
            float dv = lg[kVocab];
            for (int i = 1; i < kDurations; ++i)
                if (lg[kVocab + i] > dv) { dv = lg[kVocab + i]; dur = i; }
        }
        const int token = bi;
        if (s.trace && step < s.trace_cap) {
            float* tr = s.trace + ((size_t)b * s.trace_cap + s.n_steps[b]) * kJointOut;
            if (s.n_steps[b] < s.trace_cap)
                for (int i = lane; i < kJointOut; i += 32) tr[i] = lg[i];
        }
        const int frame = s.frame_idx[b];
        const bool emit = token != kVocab - 1;
        if (emit) {
            // commit the cached predictor state (model.rs:188-189)
            for (int l = 0; l < kPredLayers; ++l)
                for (int i = lane; i < kPredHidden; i += 32) {
                    const size_t idx = (size_t)l * BH + (size_t)b * kPredHidden + i;
                    s.h[idx] = s.h_new[idx];
                    s.c[idx] = s.c_new[idx];
                }
        }
        __syncwarp();
        if (lane == 0) {
            int emitted = s.emitted[b];
            if (emit) {
                const int n = s.n_tokens[b];
                if (n < s.max_tokens) {
                    const size_t o = (size_t)b * s.max_tokens + n;
                    s.out_tokens[o] = (uint32_t)token;
                    s.out_frames[o] = frame;
                    s.out_durs[o] = dur;
                    s.out_conf[o] = 1.0f / sum;
                } else {
                    atomicExch(s.overflow, 1);
                }
                s.n_tokens[b] = n + 1;
                s.last_token[b] = token;
                s.cache_valid[b] = 0;
                emitted += 1;
            } else {
                s.cache_valid[b] = 1;
            }
            int nf = frame;
            if (dur > 0) { nf += dur; emitted = 0; }
            else if (!emit || emitted >= kMaxSymbols) { nf += 1; emitted = 0; }
            s.frame_idx[b] = nf;
            s.emitted[b] = emitted;
            s.n_steps[b] += 1;
        }
    }
}

__global__ void __launch_bounds__(kThreads, 2)
tdt_decode_kernel(DecodeWeights w, DecodeState s, int max_steps) {
    cg::grid_group grid = cg::this_grid();
    extern __shared__ __align__(16) unsigned char dsm[];
    float* Ws = reinterpret_cast<float*>(dsm);
    float* Xs = Ws + kTileK * kWStride;
    int* act = reinterpret_cast<int*>(Xs + kTileK * kXStride);
    int* upd = act + s.n_seq;
    int* counts = upd + s.n_seq;
    int* scan = counts + 2;

    for (int step = 0; step < max_steps; ++step) {
        build_lists(s, s.n_seq, act, upd, counts, scan);
        const int n_act = counts[0], n_upd = counts[1];
        if (n_act == 0) break;
        if (n_upd > 0) {
            run_phase<kLstm0>(w, s, upd, n_upd, Ws, Xs);
            grid.sync();
            run_phase<kLstm1>(w, s, upd, n_upd, Ws, Xs);
            grid.sync();
            run_phase<kPred>(w, s, upd, n_upd, Ws, Xs);
            grid.sync();
        }
        run_phase<kOut>(w, s, act, n_act, Ws, Xs);
        grid.sync();
        decide_phase(s, act, n_act, step);
        grid.sync();
    }
}

// Plain fp32 C[M x N] = A[M x K] * W[N x K]^T + bias (hoisted encoder projection), 64 x 64 tiles.
__global__ void __launch_bounds__(256)
sgemm_nt_bias_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                     float* __restrict__ C, int M, int N, int K) {
    __shared__ float As[16][65];
    __shared__ float Bs[16][65];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            const int r = i >> 4, k = i & 15;
            As[k][r] = (m0 + r < M) ? A[(size_t)(m0 + r) * K + k0 + k] : 0.0f;
            Bs[k][r] = (n0 + r < N) ? W[(size_t)(n0 + r) * K + k0 + k] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = As[k][ty + 16 * i]; b[i] = Bs[k][tx + 16 * i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty + 16 * i, n = n0 + tx + 16 * j;
            if (m < M && n < N) C[(size_t)m * N + n] = acc[i][j] + bias[n];
        }
}

size_t decode_smem_bytes(int n_seq) {
    return sizeof(float) * (kTileK * kWStride + kTileK * kXStride) + sizeof(int) * (2 * (size_t)n_seq + 2 + 16);
}

}  // namespace

cudaError_t decode_enc_projection(const float* d_enc, const float* w_enc, const float* b_enc, float* d_proj, int rows,
                                  cudaStream_t stream) {
    if (rows <= 0) return cudaSuccess;
    dim3 grid((kJointDim + 63) / 64, (rows + 63) / 64);
    sgemm_nt_bias_kernel<<<grid, 256, 0, stream>>>(d_enc, w_enc, b_enc, d_proj, rows, kJointDim, kDModel);
    return cudaGetLastError();
}

cudaError_t decode_launch(const DecodeWeights& w, const DecodeState& s, int max_steps, int sm_count,
                          cudaStream_t stream) {
    const size_t smem = decode_smem_bytes(s.n_seq);
    cudaError_t e = cudaFuncSetAttribute(tdt_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, tdt_decode_kernel, kThreads, smem);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) return cudaErrorInvalidConfiguration;
    if (per_sm > 2) per_sm = 2;
    const int grid = sm_count * per_sm;
    DecodeWeights wl = w;
    DecodeState sl = s;
    int ms = max_steps;
    void* args[] = {&wl, &sl, &ms};
    return cudaLaunchCooperativeKernel((const void*)tdt_decode_kernel, dim3(grid), dim3(kThreads), args, smem, stream);
}

}  // namespace sb
