// TDT greedy decoding with the predictor and joint products on the tensor cores (sm_100a).
//
// The same state machine as the persistent SIMT kernel in decode.cu (ParakeetModel::greedy_decode and
// GreedyDecodeState, src/model.rs:64-214), stepped from the host: every iteration runs, for ALL sequences of the
// batch at once,
//   GEMM  gates0 = [emb(last_token) | h0] W0^T      cell 0   (c0', h0')
//   GEMM  gates1 = [h0' | h1] W1^T                  cell 1   (c1', h1')
//   GEMM  pred   = h1' Wp^T + bp                    joint input  z = relu(enc_proj[frame] + pred)
//   GEMM  logits = z Wo^T + bo                      decide   (arg-max, confidence, record, commit, advance)
// The reference runs the predictor only after a token was emitted and otherwise reuses its cached output
// (src/model.rs:136-160).  Re-running it from the same committed (last_token, h, c) gives the same numbers, so the
// cache is an optimisation this path does not need: the products are dense over the batch, finished sequences
// are simply masked in the decide step, and no per-step index lists are built.
//
// fp32 operands go to the bf16 tensor cores as three-term splits: x = hi + lo with hi = bf16(x), lo = bf16(x - hi),
// and x . w ~= hi.hi + hi.lo + lo.hi (the dropped terms are below 2^-16 of |x||w|), accumulated in fp32 in tensor
// memory.  The activation row is stored as [hi | hi | lo] and the weight row as [hi | lo | hi] over a tripled K,
// so one ordinary bf16 GEMM forms the sum.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "context.h"
#include "decode.h"
#include "gemm.h"

namespace sb {

namespace {

constexpr int kH = kPredHidden;        // 640
constexpr int kOutPad = 1152;          // joint output rows padded to a multiple of 128

__device__ __forceinline__ void split2(float x, bf16& hi, bf16& lo) {
    hi = __float2bfloat16(x);
    lo = __float2bfloat16(x - __bfloat162float(hi));
}

// dst [rows x 3 cols] = [hi | hi | lo] of src [rows x cols] (activations).
__global__ void __launch_bounds__(256)
split_act_kernel(const float* __restrict__ src, bf16* __restrict__ dst, int64_t rows, int cols) {
    const int64_t n = rows * cols;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
        const int64_t r = i / cols;
        const int c = (int)(i - r * cols);
        bf16 hi, lo;
        split2(src[i], hi, lo);
        bf16* d = dst + r * 3 * cols;
        d[c] = hi;
        d[cols + c] = hi;
        d[2 * cols + c] = lo;
    }
}

// dst [rows_pad x 3 (ca + cb)] = [hi | lo | hi] of the rows of [a | b] (weights; b may be null; rows beyond `rows` zero).
__global__ void __launch_bounds__(256)
split_weight_kernel(const float* __restrict__ a, int ca, const float* __restrict__ b, int cb, bf16* __restrict__ dst,
                    int rows, int rows_pad) {
    const int k = ca + cb;
    const int64_t n = (int64_t)rows_pad * k;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
        const int r = (int)(i / k), c = (int)(i % k);
        float x = 0.0f;
        if (r < rows) x = c < ca ? a[(size_t)r * ca + c] : b[(size_t)r * cb + (c - ca)];
        bf16 hi, lo;
        split2(x, hi, lo);
        bf16* d = dst + (size_t)r * 3 * k;
        d[c] = hi;
        d[k + c] = lo;
        d[2 * k + c] = hi;
    }
}

__global__ void pad_bias_kernel(const float* __restrict__ b, float* __restrict__ out, int n, int n_pad) {
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i < n_pad) out[i] = i < n ? b[i] : 0.0f;
}

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// Writes the split row [hi | hi | lo] element c of a K-wide activation row.
__device__ __forceinline__ void put_split(bf16* row, int k, int c, float x) {
    bf16 hi, lo;
    split2(x, hi, lo);
    row[c] = hi;
    row[k + c] = hi;
    row[2 * k + c] = lo;
}

// First predictor input of every sequence: [emb(blank) | 0].
__global__ void __launch_bounds__(256)
dec_init_kernel(const float* __restrict__ embedding, bf16* __restrict__ a0, int n_seq) {
    const int b = blockIdx.x;
    bf16* row = a0 + (size_t)b * 3 * 2 * kH;
    for (int c = threadIdx.x; c < 2 * kH; c += 256)
        put_split(row, 2 * kH, c, c < kH ? embedding[(size_t)(kVocab - 1) * kH + c] : 0.0f);
}

// LSTM cell of one layer from the gate pre-activations (bias already added): c' = s(f) c + s(i) tanh(g),
// h' = s(o) tanh(c').  Layer 0 also writes the next product's input [h0' | h1], layer 1 writes [h1'].
template <int LAYER>
__global__ void __launch_bounds__(256)
dec_cell_kernel(const float* __restrict__ gates, DecodeState s, bf16* __restrict__ a_next, int* __restrict__ step_counter) {
    const int b = blockIdx.x;
    if (LAYER == 0 && b == 0 && threadIdx.x == 0) *step_counter += 1;  // one iteration = one pass through these kernels
    const size_t BH = (size_t)s.n_seq * kH;
    const float* g = gates + (size_t)b * 4 * kH;
    for (int u = threadIdx.x; u < kH; u += 256) {
        const size_t idx = (size_t)LAYER * BH + (size_t)b * kH + u;
        const float cn = sigmoid_f(g[kH + u]) * s.c[idx] + sigmoid_f(g[u]) * tanhf(g[2 * kH + u]);
        const float hn = sigmoid_f(g[3 * kH + u]) * tanhf(cn);
        s.c_new[idx] = cn;
        s.h_new[idx] = hn;
        if (LAYER == 0) {
            bf16* row = a_next + (size_t)b * 3 * 2 * kH;
            put_split(row, 2 * kH, u, hn);
            put_split(row, 2 * kH, kH + u, s.h[BH + (size_t)b * kH + u]);
        } else {
            put_split(a_next + (size_t)b * 3 * kH, kH, u, hn);
        }
    }
}

// z = relu(enc_proj[frame] + pred) -> split row (live sequences only; the others keep a stale, finite row).
__global__ void __launch_bounds__(256)
dec_joint_in_kernel(DecodeState s, bf16* __restrict__ a3) {
    const int b = blockIdx.x;
    const int frame = s.frame_idx[b];
    if (frame >= s.enc_len[b]) return;
    const size_t erow = (size_t)(s.enc_off[b] + frame) * kJointDim;
    bf16* row = a3 + (size_t)b * 3 * kJointDim;
    for (int c = threadIdx.x; c < kJointDim; c += 256)
        put_split(row, kJointDim, c, fmaxf(s.enc_proj[erow + c] + s.pred[(size_t)b * kJointDim + c], 0.0f));
}

// One CTA per sequence: arg-max, confidence, record, commit, advance (src/model.rs:79-90,180-209), then the next
// iteration's first predictor input [emb(last_token) | h0].  `alive` receives the number of iterations run so far
// (step_counter, advanced by the first cell kernel of the iteration) if any sequence still has frames left.
__global__ void __launch_bounds__(256)
dec_decide_kernel(DecodeState s, const float* __restrict__ embedding, const float* __restrict__ logits, int ld_logits,
                  bf16* __restrict__ a0, const int* __restrict__ step_counter, int* __restrict__ alive) {
    __shared__ float redf[16];
    __shared__ int redi[8];
    const int b = blockIdx.x;
    const int frame = s.frame_idx[b];
    if (frame >= s.enc_len[b]) return;  // finished (block-uniform)
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t BH = (size_t)s.n_seq * kH;
    const float* lg = logits + (size_t)b * ld_logits;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < kVocab; i += 256) {
        const float v = lg[i];
        if (v > best) { best = v; bi = i; }  // ascending i per thread: first maximum kept
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { redf[warp] = best; redi[warp] = bi; }
    __syncthreads();
    best = redf[0];
    bi = redi[0];
#pragma unroll
    for (int wv = 1; wv < 8; ++wv) {
        const float ov = redf[wv];
        const int oi = redi[wv];
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    float sum = 0.0f;
    for (int i = tid; i < kVocab; i += 256) sum += expf(lg[i] - best);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) redf[8 + warp] = sum;
    __syncthreads();
    sum = 0.0f;
#pragma unroll
    for (int wv = 0; wv < 8; ++wv) sum += redf[8 + wv];
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
        for (int i = tid; i < kJointOut; i += 256) tr[i] = lg[i];
    }
    const bool emit = token != kVocab - 1;
    int emitted = s.emitted[b] + (emit ? 1 : 0);
    int nf = frame;
    if (dur > 0) { nf += dur; emitted = 0; }
    else if (!emit || emitted >= kMaxSymbols) { nf += 1; emitted = 0; }
    bf16* row = a0 + (size_t)b * 3 * 2 * kH;
    if (emit) {
        // commit the predictor state that produced this token (src/model.rs:188-189) and form the next input
        for (int i = tid; i < kPredLayers * kH; i += 256) {
            const int l = i / kH, u = i % kH;
            const size_t idx = (size_t)l * BH + (size_t)b * kH + u;
            const float hn = s.h_new[idx];
            s.h[idx] = hn;
            s.c[idx] = s.c_new[idx];
            if (l == 0) put_split(row, 2 * kH, kH + u, hn);
        }
        for (int u = tid; u < kH; u += 256) put_split(row, 2 * kH, u, embedding[(size_t)token * kH + u]);
    }
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
        }
        s.frame_idx[b] = nf;
        s.emitted[b] = emitted;
        s.n_steps[b] = nsteps + 1;
        if (nf < s.enc_len[b]) *alive = *step_counter;  // every writer of a step stores the same value
    }
}

cudaError_t gemm_f32(const bf16* a, const bf16* w, const float* bias, float* out, int M, int N, int K, int sm_count,
                     int* d_error, cudaStream_t st) {
    GemmArgs g{};
    g.a = a;
    g.w = w;
    g.bias = bias;
    g.out = out;
    g.M = M;
    g.N = N;
    g.K = K;
    g.ldo = N;
    g.act = kActNone;
    g.out_mode = kOutF32;
    g.alpha = 1.0f;
    g.fp8 = false;
    return gemm_launch(g, sm_count, d_error, st);
}

}  // namespace

size_t decode_tc_weight_bytes() {
    return sizeof(bf16) * 3 * ((size_t)2 * 4 * kH * 2 * kH + (size_t)kJointDim * kH + (size_t)kOutPad * kJointDim +
                               (size_t)kJointDim * kDModel) + sizeof(float) * kOutPad;
}

cudaError_t decode_tc_prepare(const DecodeWeights& w, const float* w_enc, DecodeTcWeights* t, void* storage,
                              cudaStream_t st) {
    bf16* p = reinterpret_cast<bf16*>(storage);
    const size_t G = (size_t)4 * kH * kH;
    t->w0 = p; p += (size_t)4 * kH * 3 * 2 * kH;
    t->w1 = p; p += (size_t)4 * kH * 3 * 2 * kH;
    t->wp = p; p += (size_t)kJointDim * 3 * kH;
    t->wo = p; p += (size_t)kOutPad * 3 * kJointDim;
    t->wenc = p; p += (size_t)kJointDim * 3 * kDModel;
    t->b_out = reinterpret_cast<float*>(p);
    split_weight_kernel<<<1024, 256, 0, st>>>(w.w_ih, kH, w.w_hh, kH, t->w0, 4 * kH, 4 * kH);
    split_weight_kernel<<<1024, 256, 0, st>>>(w.w_ih + G, kH, w.w_hh + G, kH, t->w1, 4 * kH, 4 * kH);
    split_weight_kernel<<<256, 256, 0, st>>>(w.w_pred, kH, nullptr, 0, t->wp, kJointDim, kJointDim);
    split_weight_kernel<<<512, 256, 0, st>>>(w.w_out, kJointDim, nullptr, 0, t->wo, kJointOut, kOutPad);
    split_weight_kernel<<<512, 256, 0, st>>>(w_enc, kDModel, nullptr, 0, t->wenc, kJointDim, kJointDim);
    pad_bias_kernel<<<(kOutPad + 255) / 256, 256, 0, st>>>(w.b_out, t->b_out, kJointOut, kOutPad);
    return cudaGetLastError();
}

size_t decode_tc_scratch_bytes(int64_t enc_rows, int n_seq) {
    const size_t B = (size_t)n_seq;
    return sizeof(bf16) * ((size_t)enc_rows * 3 * kDModel) +
           sizeof(bf16) * B * (3 * 2 * kH * 2 + 3 * kH + 3 * kJointDim) +
           sizeof(float) * B * (4 * kH + kOutPad) + 256;
}

// enc_proj [rows x 640] = enc [rows x 1024] W_enc^T + b_enc through the split product.
cudaError_t decode_tc_enc_projection(const DecodeTcWeights& t, const float* d_enc, const float* b_enc, float* d_proj,
                                     int64_t rows, void* scratch, int sm_count, int* d_error, int64_t* launches,
                                     cudaStream_t st) {
    if (rows <= 0) return cudaSuccess;
    bf16* a = reinterpret_cast<bf16*>(scratch);
    split_act_kernel<<<2048, 256, 0, st>>>(d_enc, a, rows, kDModel);
    cudaError_t e = gemm_f32(a, t.wenc, b_enc, d_proj, (int)rows, kJointDim, 3 * kDModel, sm_count, d_error, st);
    *launches += 2;
    return e != cudaSuccess ? e : cudaGetLastError();
}

// Runs the greedy loop for s.n_seq sequences.  One iteration (four products, four element-wise kernels) is
// captured into a CUDA graph once per call and replayed; the host launches `check_every` iterations at a time and
// then reads the `alive` word (d_alive[0]; d_alive[1] is the device-side iteration counter).  Iterations launched
// after the last sequence finished find nothing to do.
cudaError_t decode_tc_run(const DecodeWeights& w, const DecodeTcWeights& t, const DecodeState& s, int max_steps,
                          void* scratch_after_enc, int* d_alive, int sm_count, int* d_error, int64_t* launches,
                          cudaStream_t st) {
    const int B = s.n_seq;
    bf16* a0 = reinterpret_cast<bf16*>(scratch_after_enc);
    bf16* a1 = a0 + (size_t)B * 3 * 2 * kH;
    bf16* a2 = a1 + (size_t)B * 3 * 2 * kH;
    bf16* a3 = a2 + (size_t)B * 3 * kH;
    float* gates = reinterpret_cast<float*>(a3 + (size_t)B * 3 * kJointDim);
    float* logits = gates + (size_t)B * 4 * kH;
    int* d_step = d_alive + 1;
    cudaError_t e = cudaMemsetAsync(d_alive, 0, 2 * sizeof(int), st);
    if (e != cudaSuccess) return e;
    dec_init_kernel<<<B, 256, 0, st>>>(w.embedding, a0, B);
    *launches += 1;

    auto iteration = [&]() -> cudaError_t {
        cudaError_t r = gemm_f32(a0, t.w0, w.b_gates, gates, B, 4 * kH, 3 * 2 * kH, sm_count, d_error, st);
        if (r != cudaSuccess) return r;
        dec_cell_kernel<0><<<B, 256, 0, st>>>(gates, s, a1, d_step);
        r = gemm_f32(a1, t.w1, w.b_gates + 4 * kH, gates, B, 4 * kH, 3 * 2 * kH, sm_count, d_error, st);
        if (r != cudaSuccess) return r;
        dec_cell_kernel<1><<<B, 256, 0, st>>>(gates, s, a2, d_step);
        r = gemm_f32(a2, t.wp, w.b_pred, s.pred, B, kJointDim, 3 * kH, sm_count, d_error, st);
        if (r != cudaSuccess) return r;
        dec_joint_in_kernel<<<B, 256, 0, st>>>(s, a3);
        r = gemm_f32(a3, t.wo, t.b_out, logits, B, kOutPad, 3 * kJointDim, sm_count, d_error, st);
        if (r != cudaSuccess) return r;
        dec_decide_kernel<<<B, 256, 0, st>>>(s, w.embedding, logits, kOutPad, a0, d_step, d_alive);
        return cudaGetLastError();
    };

    // capture one iteration; on any capture problem fall back to plain launches
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
        const cudaError_t ce = iteration();
        const cudaError_t ee = cudaStreamEndCapture(st, &graph);
        if (ce != cudaSuccess || ee != cudaSuccess || !graph ||
            cudaGraphInstantiate(&exec, graph, nullptr, nullptr, 0) != cudaSuccess)
            exec = nullptr;
    }
    (void)cudaGetLastError();  // a failed capture leaves a sticky-free error code behind

    constexpr int check_every = 8;
    int h_alive = 0;
    for (int step = 0; step < max_steps; ++step) {
        e = exec ? cudaGraphLaunch(exec, st) : iteration();
        if (e != cudaSuccess) break;
        *launches += 8;
        if ((step + 1) % check_every == 0 || step + 1 == max_steps) {
            e = cudaMemcpyAsync(&h_alive, d_alive, sizeof(int), cudaMemcpyDeviceToHost, st);
            if (e == cudaSuccess) e = cudaStreamSynchronize(st);
            if (e != cudaSuccess) break;
            if (h_alive < step + 1) break;  // no sequence had frames left after the last launched iteration
        }
    }
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace sb
