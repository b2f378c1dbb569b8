// Stage drivers: decoder state set-up and read-back.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "decode.h"
#include "encoder.h"
#include "model.h"
#include "pipeline.h"

namespace sb {

struct DecodeWorkspace {
    Buffer ints, floats, enc_proj, out_tok, out_frm, out_dur, out_conf, trace, timing, tc;
    Buffer h_tok, h_frm, h_dur, h_conf;  // pinned host staging
    DecodeWorkspace() { h_tok.pinned_host = h_frm.pinned_host = h_dur.pinned_host = h_conf.pinned_host = true; }
    void release() {
        ints.release(); floats.release(); enc_proj.release(); out_tok.release(); out_frm.release(); out_dur.release();
        out_conf.release(); trace.release(); timing.release(); tc.release(); h_tok.release(); h_frm.release(); h_dur.release(); h_conf.release();
    }
};

void decode_workspace_free(sb_ctx* c) {
    if (c && c->dec_ws) {
        c->dec_ws->release();
        delete c->dec_ws;
        c->dec_ws = nullptr;
    }
}

constexpr int kMaxSeqPerLaunch = 8192;  // the kernel keeps two index lists of this many ints in shared memory

int32_t tdt_decode(sb_ctx* c, const float* d_enc, const int64_t* enc_offsets, int64_t n_clips, int64_t max_tokens,
                   uint32_t* token_ids, int64_t* frame_indices, int64_t* durations, float* confidences,
                   int64_t* n_tokens, float* logits_trace, int64_t trace_cap, int64_t* n_steps) {
    if (!c || !d_enc || !enc_offsets || !token_ids || !frame_indices || !durations || !confidences || !n_tokens)
        return fail(SB_INVALID_ARGUMENT, "null argument");
    if (!c->model || !c->model->has_decoder) return fail(SB_MISSING_MODEL_ASSET, "no predictor / joint weights loaded");
    if (n_clips <= 0) return fail(SB_EMPTY_AUDIO, "audio input was empty");
    if (max_tokens <= 0 || max_tokens > (1 << 20)) return fail(SB_INVALID_ARGUMENT, "bad max_tokens");
    if (logits_trace && trace_cap <= 0) return fail(SB_INVALID_ARGUMENT, "trace_cap must be positive with a trace");
    SB_CUDA(cudaSetDevice(c->device));
    if (!c->dec_ws) c->dec_ws = new DecodeWorkspace();
    DecodeWorkspace& ws = *c->dec_ws;
    const Model& m = *c->model;
    cudaStream_t st = c->stream;

    for (int64_t g0 = 0; g0 < n_clips; g0 += kMaxSeqPerLaunch) {
        const int n = (int)std::min<int64_t>(kMaxSeqPerLaunch, n_clips - g0);
        const int64_t row0 = enc_offsets[g0];
        const int64_t rows = enc_offsets[g0 + n] - row0;
        std::vector<int> off(n), len(n);
        int max_len = 0;
        for (int i = 0; i < n; ++i) {
            off[i] = (int)(enc_offsets[g0 + i] - row0);
            len[i] = (int)(enc_offsets[g0 + i + 1] - enc_offsets[g0 + i]);
            if (len[i] < 0) return fail(SB_INVALID_ARGUMENT, "encoder offsets must ascend");
            max_len = std::max(max_len, len[i]);
        }
        // int state: enc_off, enc_len, frame_idx, emitted, last_token, cache_valid, n_tokens, n_steps, overflow
        const size_t n_int = (size_t)8 * n + 16;
        SB_CUDA(ws.ints.ensure(n_int * sizeof(int)));
        int* di = ws.ints.as<int>();
        std::vector<int> hi(n_int, 0);
        std::memcpy(hi.data(), off.data(), sizeof(int) * n);
        std::memcpy(hi.data() + n, len.data(), sizeof(int) * n);
        for (int i = 0; i < n; ++i) hi[(size_t)4 * n + i] = kVocab - 1;  // last_token = blank (model.rs:123)
        SB_CUDA(cudaMemcpyAsync(di, hi.data(), n_int * sizeof(int), cudaMemcpyHostToDevice, st));
        // float state: h, c, h_new, c_new [2][n][640], pred [n][640], logits [n][1030]
        const size_t BH = (size_t)n * kPredHidden;
        const size_t n_f = 8 * BH + 2 * (size_t)n * kJointDim + (size_t)n * kJointOut;
        SB_CUDA(ws.floats.ensure(n_f * sizeof(float)));
        float* df = ws.floats.as<float>();
        SB_CUDA(cudaMemsetAsync(df, 0, 4 * BH * sizeof(float), st));  // h = c = 0 (model.rs:114-115)
        SB_CUDA(ws.enc_proj.ensure((size_t)std::max<int64_t>(rows, 1) * kJointDim * sizeof(float)));
        SB_CUDA(ws.out_tok.ensure((size_t)n * max_tokens * sizeof(uint32_t)));
        SB_CUDA(ws.out_frm.ensure((size_t)n * max_tokens * sizeof(int)));
        SB_CUDA(ws.out_dur.ensure((size_t)n * max_tokens * sizeof(int)));
        SB_CUDA(ws.out_conf.ensure((size_t)n * max_tokens * sizeof(float)));
        if (logits_trace) SB_CUDA(ws.trace.ensure((size_t)n * trace_cap * kJointOut * sizeof(float)));

        const bool tc = !c->simt_decode;
        if (tc) {
            SB_CUDA(ws.tc.ensure(decode_tc_scratch_bytes(rows, n)));
            c->prof.begin("decode_enc_projection_tc", st);
            SB_CUDA(decode_tc_enc_projection(m.tc, d_enc + row0 * kDModel, m.b_enc, ws.enc_proj.as<float>(), rows, ws.tc.p,
                                             c->sm_count, c->d_error, &c->launches, st));
            c->prof.end(st);
        } else {
            c->prof.begin("decode_enc_projection", st);
            SB_CUDA(decode_enc_projection(d_enc + row0 * kDModel, m.w_enc, m.b_enc, ws.enc_proj.as<float>(), (int)rows, st));
            c->prof.end(st);
            c->launches += rows > 0 ? 1 : 0;
        }

        DecodeWeights w{m.embedding, m.w_ih, m.w_hh, m.b_gates, m.w_pred, m.b_pred, m.w_out, m.b_out};
        DecodeState s{};
        s.n_seq = n;
        s.max_tokens = (int)max_tokens;
        s.trace_cap = logits_trace ? (int)trace_cap : 0;
        s.enc_proj = ws.enc_proj.as<float>();
        s.enc_off = di;
        s.enc_len = di + n;
        s.frame_idx = di + 2 * n;
        s.emitted = di + 3 * n;
        s.last_token = di + 4 * n;
        s.cache_valid = di + 5 * n;
        s.n_tokens = di + 6 * n;
        s.n_steps = di + 7 * n;
        s.overflow = di + 8 * n;
        s.h = df;
        s.c = df + 2 * BH;
        s.h_new = df + 4 * BH;
        s.c_new = df + 6 * BH;
        s.pred = df + 8 * BH;
        s.z = s.pred + (size_t)n * kJointDim;
        s.logits = s.z + (size_t)n * kJointDim;
        s.out_tokens = ws.out_tok.as<uint32_t>();
        s.out_frames = ws.out_frm.as<int>();
        s.out_durs = ws.out_dur.as<int>();
        s.out_conf = ws.out_conf.as<float>();
        s.trace = logits_trace ? ws.trace.as<float>() : nullptr;
        // SB_DECODE_TIMING=1: block 0's cycle counts per phase / barrier, printed after the kernel
        static const bool want_timing = std::getenv("SB_DECODE_TIMING") != nullptr;
        long long* d_timing = nullptr;
        if (want_timing) {
            SB_CUDA(ws.timing.ensure(12 * sizeof(long long)));
            d_timing = ws.timing.as<long long>();
            SB_CUDA(cudaMemsetAsync(d_timing, 0, 12 * sizeof(long long), st));
        }
        s.timing = d_timing;
        const int max_steps = (kMaxSymbols + 1) * max_len + 2;
        if (max_len > 0 && tc) {
            // the per-sequence buffers follow the split encoder rows in the scratch area
            char* after_enc = static_cast<char*>(ws.tc.p) + sizeof(bf16) * (size_t)rows * 3 * kDModel;
            c->prof.begin("tdt_decode_tc", st);
            SB_CUDA(decode_tc_run(w, m.tc, s, max_steps, after_enc, di + 8 * n + 1, c->sm_count, c->d_error, &c->launches, st));
            c->prof.end(st);
        } else if (max_len > 0) {
            c->prof.begin("tdt_decode", st);
            SB_CUDA(decode_launch(w, s, max_steps, c->sm_count, st));
            c->prof.end(st);
            c->launches += 1;
        }
        // read back: counts first, then only the used columns of the output tables
        std::vector<int> cnt((size_t)2 * n + 1);
        SB_CUDA(cudaMemcpyAsync(cnt.data(), s.n_tokens, sizeof(int) * (2 * n + 1), cudaMemcpyDeviceToHost, st));
        // the flag that a kernel of this stream (GEMM, attention, decoder) raises when one of its bounded waits ran
        // out: everything computed after that is garbage, so the call must not return tokens
        int dev_err = 0;
        SB_CUDA(cudaMemcpyAsync(&dev_err, c->d_error, sizeof(int), cudaMemcpyDeviceToHost, st));
        SB_CUDA(cudaStreamSynchronize(st));
        if (dev_err) {
            SB_CUDA(cudaMemsetAsync(c->d_error, 0, sizeof(int), st));
            return fail(SB_TIMEOUT, "a bounded device-side wait ran out (kernel aborted cleanly); no tokens returned");
        }
        if (d_timing) {
            long long t[12];
            SB_CUDA(cudaMemcpy(t, d_timing, sizeof(t), cudaMemcpyDeviceToHost));
            static const char* names[11] = {"lists", "lstm0", "sync", "lstm1", "sync", "pred", "sync", "out", "sync", "decide", "sync"};
            std::fprintf(stderr, "[decode timing] n_seq=%d steps=%lld kcycles:", n, t[11]);
            for (int i = 0; i < 11; ++i) std::fprintf(stderr, " %s=%lld", names[i], t[i] / 1000);
            std::fprintf(stderr, "\n");
        }
        if (cnt[2 * n]) return fail(SB_BUFFER_TOO_SMALL, "a clip emitted more tokens than max_tokens");
        int max_n = 0;
        for (int i = 0; i < n; ++i) max_n = std::max(max_n, cnt[i]);
        if (max_n > 0) {
            const size_t hb = (size_t)n * max_n * 4;
            SB_CUDA(ws.h_tok.ensure(hb)); SB_CUDA(ws.h_frm.ensure(hb)); SB_CUDA(ws.h_dur.ensure(hb)); SB_CUDA(ws.h_conf.ensure(hb));
            const size_t wbytes = (size_t)max_n * 4, pitch = (size_t)max_tokens * 4;
            SB_CUDA(cudaMemcpy2DAsync(ws.h_tok.p, wbytes, s.out_tokens, pitch, wbytes, n, cudaMemcpyDeviceToHost, st));
            SB_CUDA(cudaMemcpy2DAsync(ws.h_frm.p, wbytes, s.out_frames, pitch, wbytes, n, cudaMemcpyDeviceToHost, st));
            SB_CUDA(cudaMemcpy2DAsync(ws.h_dur.p, wbytes, s.out_durs, pitch, wbytes, n, cudaMemcpyDeviceToHost, st));
            SB_CUDA(cudaMemcpy2DAsync(ws.h_conf.p, wbytes, s.out_conf, pitch, wbytes, n, cudaMemcpyDeviceToHost, st));
        }
        if (logits_trace)
            SB_CUDA(cudaMemcpyAsync(logits_trace + (size_t)g0 * trace_cap * kJointOut, ws.trace.p,
                                    (size_t)n * trace_cap * kJointOut * sizeof(float), cudaMemcpyDeviceToHost, st));
        SB_CUDA(cudaStreamSynchronize(st));
        for (int i = 0; i < n; ++i) {
            const int k = cnt[i];
            n_tokens[g0 + i] = k;
            if (n_steps) n_steps[g0 + i] = cnt[n + i];
            const size_t o = (size_t)(g0 + i) * max_tokens;
            const uint32_t* ht = ws.h_tok.as<uint32_t>() + (size_t)i * max_n;
            const int* hf = ws.h_frm.as<int>() + (size_t)i * max_n;
            const int* hd = ws.h_dur.as<int>() + (size_t)i * max_n;
            const float* hc = ws.h_conf.as<float>() + (size_t)i * max_n;
            for (int j = 0; j < k; ++j) {
                token_ids[o + j] = ht[j];
                frame_indices[o + j] = hf[j];
                durations[o + j] = hd[j];
                confidences[o + j] = hc[j];
            }
        }
    }
    return SB_OK;
}

}  // namespace sb

extern "C" int32_t sb_tdt_decode_device(sb_ctx* ctx, const float* d_enc, const int64_t* enc_offsets, int64_t n_clips,
                                        int64_t max_tokens, uint32_t* token_ids, int64_t* frame_indices,
                                        int64_t* durations, float* confidences, int64_t* n_tokens,
                                        float* logits_trace, int64_t trace_cap, int64_t* n_steps) {
    return sb::tdt_decode(ctx, d_enc, enc_offsets, n_clips, max_tokens, token_ids, frame_indices, durations,
                          confidences, n_tokens, logits_trace, trace_cap, n_steps);
}
