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
// fused into the epilogue, predictor projection which also forms the joint input relu(enc + pred), joint
// output) and a per-sequence arg-max / update phase, with a grid-wide barrier between phases.  Weights (35 MB fp32) stay L2-resident; the
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
constexpr int kTileRow = 64;   // weight rows per tile (LSTM: 16 units x 4 gates, gates adjacent)
constexpr int kTileK = 32;
constexpr int kKPad = kTileK + 4;        // floats per operand row of a chunk in shared memory
constexpr int kRingFloats = 4 * (kTileRow + 64) * kKPad;  // cp.async ring: 4 stages of 64 + 64 rows, or 6 of 64 + 16

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

__device__ __forceinline__ void cp_async16(float* dst_smem, const float* src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst_smem);
    const int bytes = valid ? 16 : 0;  // 0: nothing is read, the destination is zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One phase: C[list x rows] = X[list x K] * W[rows x K]^T in fp32.  Tiles of (16 SPT) sequences x 64 weight rows;
// thread (sg = tid / 16, ul = tid % 16) owns sequences sg * SPT .. + SPT - 1 and local rows ul, ul + 16, ul + 32,
// ul + 48, which for the LSTM phases are the i, f, g, o gates of unit 16 rt + ul, so the cell update stays in the
// thread.  K is walked in chunks of 32 through a cp.async ring (both operands are plain 16-byte row copies; rows are
// padded to 36 floats, which keeps the float4 reads of 8 neighbouring threads on distinct banks).  Every output is
// one fp32 fused-multiply-add chain over ascending k, whatever SPT is, so a sequence's result does not depend on
// how many other sequences are alive.
template <int PHASE, int SPT>
__device__ void run_phase(const DecodeWeights& w, const DecodeState& s, const int* list, int n_list, float* ring) {
    constexpr bool lstm = PHASE == kLstm0 || PHASE == kLstm1;
    constexpr int K = lstm ? 2 * kPredHidden : kPredHidden;
    constexpr int ldw = lstm ? kPredHidden : K;  // row pitch of each weight matrix
    constexpr int rows_total = lstm ? 4 * kPredHidden : (PHASE == kPred ? kJointDim : kJointOut);
    constexpr int row_tiles = lstm ? kPredHidden / 16 : (rows_total + kTileRow - 1) / kTileRow;
    constexpr int layer = PHASE == kLstm1 ? 1 : 0;
    constexpr int seq_t = 16 * SPT;
    constexpr int n_chunks = K / kTileK;
    constexpr int stage_floats = (kTileRow + seq_t) * kKPad;
    constexpr int stages = kRingFloats / stage_floats;
    constexpr int n_xl = (seq_t * 8 + kThreads - 1) / kThreads;  // activation float4 slots per thread
    static_assert(stages >= 3, "ring too small");
    const float* W_a = lstm ? w.w_ih + (size_t)layer * 4 * kPredHidden * kPredHidden : (PHASE == kPred ? w.w_pred : w.w_out);
    const float* W_b = lstm ? w.w_hh + (size_t)layer * 4 * kPredHidden * kPredHidden : W_a;
    const int tid = threadIdx.x;
    const int sg = tid >> 4, ul = tid & 15;
    const int seq_tiles = (n_list + seq_t - 1) / seq_t;
    const int n_tiles = seq_tiles * row_tiles;
    const size_t BH = (size_t)s.n_seq * kPredHidden;
    const int lj = tid & 7, lrow = tid >> 3;  // load slots: float4 lj of rows lrow (+ 32)

    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int st = tile / row_tiles, rt = tile % row_tiles;
        const int s0 = st * seq_t;
        size_t woff[2];
        bool wok[2];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int r = lrow + 32 * q;  // local weight row
            const int grow = lstm ? (r >> 4) * kPredHidden + rt * 16 + (r & 15) : rt * kTileRow + r;
            wok[q] = grow < rows_total;
            woff[q] = (size_t)(wok[q] ? grow : 0) * ldw + 4 * lj;
        }
        const float* xsrc_a[n_xl];
        const float* xsrc_b[n_xl];
        bool xok[n_xl];
#pragma unroll
        for (int q = 0; q < n_xl; ++q) {
            const int lsq = lrow + 32 * q;  // local sequence
            const int li = s0 + lsq;
            xok[q] = lsq < seq_t && li < n_list;
            const int b = xok[q] ? list[li] : 0;
            if (PHASE == kLstm0) {
                xsrc_a[q] = w.embedding + (size_t)s.last_token[b] * kPredHidden;
                xsrc_b[q] = s.h + (size_t)b * kPredHidden;
            } else if (PHASE == kLstm1) {
                xsrc_a[q] = s.h_new + (size_t)b * kPredHidden;
                xsrc_b[q] = s.h + BH + (size_t)b * kPredHidden;
            } else if (PHASE == kPred) {
                xsrc_a[q] = s.h_new + BH + (size_t)b * kPredHidden;
                xsrc_b[q] = xsrc_a[q];
            } else {
                xsrc_a[q] = s.z + (size_t)b * kJointDim;
                xsrc_b[q] = xsrc_a[q];
            }
        }
        auto issue = [&](int chunk) {
            float* Ws = ring + (chunk % stages) * stage_floats;
            float* Xs = Ws + kTileRow * kKPad;
            const bool second = lstm && chunk >= n_chunks / 2;  // LSTM: k >= 640 comes from the recurrent operands
            const int k0 = (second ? chunk - n_chunks / 2 : chunk) * kTileK;
            const float* Wm = second ? W_b : W_a;
#pragma unroll
            for (int q = 0; q < 2; ++q)
                cp_async16(Ws + (lrow + 32 * q) * kKPad + 4 * lj, Wm + woff[q] + k0, wok[q]);
#pragma unroll
            for (int q = 0; q < n_xl; ++q) {
                const int lsq = lrow + 32 * q;
                if (lsq < seq_t)
                    cp_async16(Xs + lsq * kKPad + 4 * lj, (second ? xsrc_b[q] : xsrc_a[q]) + k0 + 4 * lj, xok[q]);
            }
        };
        float acc[SPT][4];
#pragma unroll
        for (int a = 0; a < SPT; ++a)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[a][r] = 0.0f;

        __syncthreads();  // the previous tile's readers are done with the ring
#pragma unroll
        for (int c = 0; c < stages - 1; ++c) {
            if (c < n_chunks) issue(c);
            cp_async_commit();
        }
        for (int c = 0; c < n_chunks; ++c) {
            cp_async_wait<stages - 2>();
            __syncthreads();
            if (c + stages - 1 < n_chunks) issue(c + stages - 1);
            cp_async_commit();
            const float* Ws = ring + (c % stages) * stage_floats;
            const float* Xs = Ws + kTileRow * kKPad;
#pragma unroll
            for (int k = 0; k < kTileK; k += 4) {
                float4 wv[4], xv[SPT];
#pragma unroll
                for (int r = 0; r < 4; ++r) wv[r] = *reinterpret_cast<const float4*>(Ws + (ul + 16 * r) * kKPad + k);
#pragma unroll
                for (int a = 0; a < SPT; ++a) xv[a] = *reinterpret_cast<const float4*>(Xs + (sg * SPT + a) * kKPad + k);
#pragma unroll
                for (int a = 0; a < SPT; ++a)
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        float t = acc[a][r];
                        t = fmaf(xv[a].x, wv[r].x, t);
                        t = fmaf(xv[a].y, wv[r].y, t);
                        t = fmaf(xv[a].z, wv[r].z, t);
                        t = fmaf(xv[a].w, wv[r].w, t);
                        acc[a][r] = t;
                    }
            }
        }
        cp_async_wait<0>();
        // epilogue
#pragma unroll
        for (int a = 0; a < SPT; ++a) {
            const int li = s0 + sg * SPT + a;
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
                const size_t erow = (size_t)(s.enc_off[b] + s.frame_idx[b]) * kJointDim;
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int row = rt * kTileRow + ul + 16 * r;
                    if (row >= rows_total) continue;
                    if (PHASE == kPred) {
                        const float pv = acc[a][r] + w.b_pred[row];
                        s.pred[(size_t)b * kJointDim + row] = pv;
                        s.z[(size_t)b * kJointDim + row] = fmaxf(s.enc_proj[erow + row] + pv, 0.0f);
                    } else {
                        s.logits[(size_t)b * kJointOut + row] = acc[a][r] + w.b_out[row];
                    }
                }
            }
        }
    }
}

// One CTA per live sequence: arg-max, confidence, record, commit, advance (model.rs:79-90,180-209).
// redf / redi: shared scratch of 16 floats and 8 ints.
__device__ void decide_phase(const DecodeState& s, const int* act, int n_act, float* redf, int* redi) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t BH = (size_t)s.n_seq * kPredHidden;
    for (int li = blockIdx.x; li < n_act; li += gridDim.x) {
        const int b = act[li];
        const float* lg = s.logits + (size_t)b * kJointOut;
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = tid; i < kVocab; i += kThreads) {
            const float v = lg[i];
            if (v > best) { best = v; bi = i; }  // ascending i per thread: first maximum kept
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        __syncthreads();  // the scratch is free again
        if (lane == 0) { redf[warp] = best; redi[warp] = bi; }
        __syncthreads();
        best = redf[0];
        bi = redi[0];
#pragma unroll
        for (int wv = 1; wv < kThreads / 32; ++wv) {
            const float ov = redf[wv];
            const int oi = redi[wv];
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        float sum = 0.0f;
        for (int i = tid; i < kVocab; i += kThreads) sum += expf(lg[i] - best);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) redf[8 + warp] = sum;
        __syncthreads();
        sum = 0.0f;
#pragma unroll
        for (int wv = 0; wv < kThreads / 32; ++wv) sum += redf[8 + wv];
        int dur = 0;
        {
            float dv = lg[kVocab];
            for (int i = 1; i < kDurations; ++i)
                if (lg[kVocab + i] > dv) { dv = lg[kVocab + i]; dur = i; }
        }
        const int token = bi;
        const int nsteps = s.n_steps[b];
        if (s.trace && nsteps < s.trace_cap) {
            float* tr = s.trace + ((size_t)b * s.trace_cap + nsteps) * kJointOut;
            for (int i = tid; i < kJointOut; i += kThreads) tr[i] = lg[i];
        }
        const int frame = s.frame_idx[b];
        const bool emit = token != kVocab - 1;
        int emitted = s.emitted[b] + (emit ? 1 : 0);
        int nf = frame;
        if (dur > 0) { nf += dur; emitted = 0; }
        else if (!emit || emitted >= kMaxSymbols) { nf += 1; emitted = 0; }
        if (emit) {
            // commit the cached predictor state (model.rs:188-189); the predictor runs again next iteration
            for (int i = tid; i < kPredLayers * kPredHidden; i += kThreads) {
                const size_t idx = (size_t)(i / kPredHidden) * BH + (size_t)b * kPredHidden + (i % kPredHidden);
                s.h[idx] = s.h_new[idx];
                s.c[idx] = s.c_new[idx];
            }
        } else if (nf < s.enc_len[b]) {
            // the cached predictor output stays valid: refresh the joint input for the new frame
            const size_t erow = (size_t)(s.enc_off[b] + nf) * kJointDim;
            for (int i = tid; i < kJointDim; i += kThreads)
                s.z[(size_t)b * kJointDim + i] = fmaxf(s.enc_proj[erow + i] + s.pred[(size_t)b * kJointDim + i], 0.0f);
        }
        __syncthreads();  // every thread has read the state it needs before thread 0 updates it
        if (tid == 0) {
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
            } else {
                s.cache_valid[b] = 1;
            }
            s.frame_idx[b] = nf;
            s.emitted[b] = emitted;
            s.n_steps[b] = nsteps + 1;
        }
    }
}

__global__ void __launch_bounds__(kThreads, 2)
tdt_decode_kernel(DecodeWeights w, DecodeState s, int max_steps) {
    cg::grid_group grid = cg::this_grid();
    extern __shared__ __align__(16) unsigned char dsm[];
    float* ring = reinterpret_cast<float*>(dsm);
    float* redf = ring + kRingFloats;
    int* redi = reinterpret_cast<int*>(redf + 16);
    int* act = redi + 16;
    int* upd = act + s.n_seq;
    int* counts = upd + s.n_seq;
    int* scan = counts + 2;

    long long tacc[12] = {};
    const bool timed = s.timing != nullptr && blockIdx.x == 0 && threadIdx.x == 0;
    long long tprev = clock64();
    auto lap = [&](int slot) {
        if (timed) {
            const long long now = clock64();
            tacc[slot] += now - tprev;
            tprev = now;
        }
    };
    int steps_done = 0;
    for (int step = 0; step < max_steps; ++step) {
        build_lists(s, s.n_seq, act, upd, counts, scan);
        const int n_act = counts[0], n_upd = counts[1];
        lap(0);
        if (n_act == 0) break;
        ++steps_done;
        // few sequences: 16 per tile (one per thread) so that a phase is short; many: 64 per tile (four per thread)
        const bool small_upd = ((n_upd + 15) / 16) * (kPredHidden / 16) <= (int)gridDim.x;
        const bool small_act = ((n_act + 15) / 16) * ((kJointOut + kTileRow - 1) / kTileRow) <= (int)gridDim.x;
        if (n_upd > 0) {
            if (small_upd) run_phase<kLstm0, 1>(w, s, upd, n_upd, ring); else run_phase<kLstm0, 4>(w, s, upd, n_upd, ring);
            lap(1);
            grid.sync();
            lap(2);
            if (small_upd) run_phase<kLstm1, 1>(w, s, upd, n_upd, ring); else run_phase<kLstm1, 4>(w, s, upd, n_upd, ring);
            lap(3);
            grid.sync();
            lap(4);
            if (small_upd) run_phase<kPred, 1>(w, s, upd, n_upd, ring); else run_phase<kPred, 4>(w, s, upd, n_upd, ring);
            lap(5);
            grid.sync();
            lap(6);
        }
        if (small_act) run_phase<kOut, 1>(w, s, act, n_act, ring); else run_phase<kOut, 4>(w, s, act, n_act, ring);
        lap(7);
        grid.sync();
        lap(8);
        decide_phase(s, act, n_act, redf, redi);
        lap(9);
        grid.sync();
        lap(10);
    }
    if (timed) {
        for (int i = 0; i < 11; ++i) s.timing[i] = tacc[i];
        s.timing[11] = steps_done;
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
    return sizeof(float) * (kRingFloats + 16) + sizeof(int) * (16 + 2 * (size_t)n_seq + 2 + 16);
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
    // A grid-wide barrier over two CTAs per SM costs several times one over a single CTA per SM (measured: about
    // 17 us against 2 us), which only a batch large enough to keep both CTAs in arithmetic repays.
    if (per_sm > 2) per_sm = 2;
    if (s.n_seq < 1024) per_sm = 1;
    const int grid = sm_count * per_sm;
    DecodeWeights wl = w;
    DecodeState sl = s;
    int ms = max_steps;
    void* args[] = {&wl, &sl, &ms};
    return cudaLaunchCooperativeKernel((const void*)tdt_decode_kernel, dim3(grid), dim3(kThreads), args, smem, stream);
}

}  // namespace sb
