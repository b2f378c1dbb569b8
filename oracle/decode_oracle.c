/*
 * CPU oracle for TDT greedy decoding.  TEST INFRASTRUCTURE ONLY: never linked
 * into or called from the product library.
 *
 * Control flow restates the reference's src/model.rs:
 *   ParakeetModel::greedy_decode            model.rs:64-95
 *   GreedyDecodeState::new                  model.rs:111-125  (h = c = 0, last_token = blank)
 *   ensure_decoder_step (cache)             model.rs:146-162
 *   record_emission                         model.rs:180-196
 *   advance                                 model.rs:198-209
 * and its Python twin dev-tools/python/compare_coreml.py:216-338
 * (argmax over [0, vocab) and [vocab, vocab + n_dur); duration value = index;
 * confidence = max softmax over the token logits, compare_coreml.py:141-145,350-354).
 *
 * The predictor and joint networks are opaque CoreML blobs in the reference
 * (src/coreml.rs:239-359), so their arithmetic is defined here, not restated:
 *   x0      = embedding[last_token]                       (row of [vocab x H]; the blank row is an ordinary row)
 *   layer l : g = W_ih[l] x + b_ih[l] + W_hh[l] h[l] + b_hh[l], gate order i,f,g,o
 *             c' = sigmoid(f) c + sigmoid(i) tanh(g);  h' = sigmoid(o) tanh(c');  x <- h'
 *   dec     = h'[L-1]
 *   z       = relu(W_enc enc_t + b_enc + W_pred dec + b_pred)
 *   logits  = W_out z + b_out                             [vocab + n_dur]
 * Numerics of those two networks are therefore "parity unpinned" against the
 * reference; the control flow is pinned by the source and its Python twin (the
 * reference has no unit test for the loop).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    int32_t vocab;      /* 1025 incl. blank */
    int32_t n_dur;      /* 5 */
    int32_t blank;      /* 1024 */
    int32_t hidden;     /* 640 */
    int32_t layers;     /* 2 */
    int32_t enc_dim;    /* 1024 */
    int32_t joint_dim;  /* 640 */
    int32_t max_symbols;/* 10, constants.rs:17 */
    const float *embedding; /* [vocab x hidden] */
    const float *w_ih;      /* [layers x 4H x H] */
    const float *w_hh;      /* [layers x 4H x H] */
    const float *b_ih;      /* [layers x 4H] */
    const float *b_hh;      /* [layers x 4H] */
    const float *w_enc;     /* [joint x enc_dim] */
    const float *b_enc;     /* [joint] */
    const float *w_pred;    /* [joint x hidden] */
    const float *b_pred;    /* [joint] */
    const float *w_out;     /* [(vocab+n_dur) x joint] */
    const float *b_out;     /* [vocab+n_dur] */
} sbo_tdt_weights;

static int argmax_first(const float *v, int n) {
    int best = 0;
    for (int i = 1; i < n; ++i)
        if (v[i] > v[best]) best = i; /* strict: lowest index wins ties */
    return best;
}

static float max_softmax(const float *v, int n) {
    float mx = v[argmax_first(v, n)];
    float sum = 0.0f;
    for (int i = 0; i < n; ++i) sum += expf(v[i] - mx);
    return 1.0f / sum;
}

/* model.rs:198-209 */
static void advance(int64_t *frame_idx, int *emitted, int token, int duration, int blank, int max_symbols) {
    if (duration > 0) { *frame_idx += duration; *emitted = 0; return; }
    if (token == blank || *emitted >= max_symbols) { *frame_idx += 1; *emitted = 0; }
}

/*
 * Logit replay: drives the state machine of model.rs:64-214 with a recorded
 * sequence of joint outputs, one row of [vocab + n_dur] logits per loop
 * iteration.  Writes the emitted tokens and, per step, the encoder frame the
 * step must have looked at and whether the predictor had to run (cache empty).
 * Returns the number of tokens, or -1 if the trace is too short / -2 if the
 * capacity is too small.  *steps_used receives the number of iterations.
 */
int64_t sbo_greedy_replay(const float *logits, int64_t n_steps, int64_t time_steps, int vocab, int n_dur,
                          int blank, int max_symbols, uint32_t *tokens, int64_t *frames, int64_t *durs,
                          float *conf, int64_t cap, int64_t *steps_used, int32_t *step_frame,
                          int32_t *step_ran_predictor) {
    int64_t frame_idx = 0, n_tok = 0, step = 0;
    int emitted = 0, cache_valid = 0;
    const int width = vocab + n_dur;
    while (frame_idx < time_steps) {
        if (step >= n_steps) return -1;
        if (step_ran_predictor) step_ran_predictor[step] = cache_valid ? 0 : 1;
        cache_valid = 1;
        if (step_frame) step_frame[step] = (int32_t)frame_idx;
        const float *row = logits + step * width;
        int token = argmax_first(row, vocab);
        int duration = argmax_first(row + vocab, n_dur);
        if (token != blank) {
            if (n_tok >= cap) return -2;
            cache_valid = 0; /* take_cached_decoder, model.rs:80 */
            tokens[n_tok] = (uint32_t)token;
            frames[n_tok] = frame_idx; /* before the advance, model.rs:191 */
            durs[n_tok] = duration;
            conf[n_tok] = max_softmax(row, vocab);
            ++n_tok;
            ++emitted;
        }
        advance(&frame_idx, &emitted, token, duration, blank, max_symbols);
        ++step;
    }
    if (steps_used) *steps_used = step;
    return n_tok;
}

static float sigmoidf(float x) { return 1.0f / (1.0f + expf(-x)); }

static void matvec_acc(const float *w, const float *x, int rows, int cols, float *y) {
    for (int r = 0; r < rows; ++r) {
        const float *wr = w + (size_t)r * cols;
        float acc = 0.0f;
        for (int c = 0; c < cols; ++c) acc += wr[c] * x[c];
        y[r] += acc;
    }
}

/*
 * Full fp32 decode of one sequence.  enc is time-major [time_steps x enc_dim].
 * logits_trace (optional) receives one row per loop iteration, capacity
 * trace_cap rows.  Returns the number of tokens or a negative code as above.
 */
int64_t sbo_tdt_decode(const sbo_tdt_weights *w, const float *enc, int64_t time_steps, uint32_t *tokens,
                       int64_t *frames, int64_t *durs, float *conf, int64_t cap, float *logits_trace,
                       int64_t trace_cap, int64_t *steps_used) {
    const int H = w->hidden, L = w->layers, J = w->joint_dim, V = w->vocab, D = w->n_dur, W = V + D;
    float *h = (float *)calloc((size_t)L * H, sizeof(float));
    float *c = (float *)calloc((size_t)L * H, sizeof(float));
    float *h_new = (float *)calloc((size_t)L * H, sizeof(float));
    float *c_new = (float *)calloc((size_t)L * H, sizeof(float));
    float *gates = (float *)malloc(sizeof(float) * 4 * (size_t)H);
    float *pred = (float *)malloc(sizeof(float) * (size_t)J);
    float *z = (float *)malloc(sizeof(float) * (size_t)J);
    float *logits = (float *)malloc(sizeof(float) * (size_t)W);
    /* enc projection hoisted out of the loop: one row per frame. */
    float *encp = (float *)malloc(sizeof(float) * (size_t)(time_steps > 0 ? time_steps : 1) * J);
    for (int64_t t = 0; t < time_steps; ++t) {
        float *row = encp + t * J;
        memcpy(row, w->b_enc, sizeof(float) * (size_t)J);
        matvec_acc(w->w_enc, enc + t * w->enc_dim, J, w->enc_dim, row);
    }
    int64_t frame_idx = 0, n_tok = 0, step = 0, rc = 0;
    int emitted = 0, cache_valid = 0, last_token = w->blank;
    while (frame_idx < time_steps) {
        if (!cache_valid) {
            const float *x = w->embedding + (size_t)last_token * H;
            for (int l = 0; l < L; ++l) {
                for (int g = 0; g < 4 * H; ++g) gates[g] = w->b_ih[l * 4 * H + g] + w->b_hh[l * 4 * H + g];
                matvec_acc(w->w_ih + (size_t)l * 4 * H * H, x, 4 * H, H, gates);
                matvec_acc(w->w_hh + (size_t)l * 4 * H * H, h + l * H, 4 * H, H, gates);
                for (int u = 0; u < H; ++u) {
                    float ig = sigmoidf(gates[u]), fg = sigmoidf(gates[H + u]);
                    float gg = tanhf(gates[2 * H + u]), og = sigmoidf(gates[3 * H + u]);
                    float cn = fg * c[l * H + u] + ig * gg;
                    c_new[l * H + u] = cn;
                    h_new[l * H + u] = og * tanhf(cn);
                }
                x = h_new + l * H;
            }
            memcpy(pred, w->b_pred, sizeof(float) * (size_t)J);
            matvec_acc(w->w_pred, h_new + (L - 1) * H, J, H, pred);
            cache_valid = 1;
        }
        const float *er = encp + frame_idx * J;
        for (int j = 0; j < J; ++j) {
            float v = er[j] + pred[j];
            z[j] = v > 0.0f ? v : 0.0f;
        }
        memcpy(logits, w->b_out, sizeof(float) * (size_t)W);
        matvec_acc(w->w_out, z, W, J, logits);
        if (logits_trace) {
            if (step >= trace_cap) { rc = -1; break; }
            memcpy(logits_trace + step * W, logits, sizeof(float) * (size_t)W);
        }
        int token = argmax_first(logits, V);
        int duration = argmax_first(logits + V, D);
        if (token != w->blank) {
            if (n_tok >= cap) { rc = -2; break; }
            cache_valid = 0;
            memcpy(h, h_new, sizeof(float) * (size_t)L * H);
            memcpy(c, c_new, sizeof(float) * (size_t)L * H);
            tokens[n_tok] = (uint32_t)token;
            frames[n_tok] = frame_idx;
            durs[n_tok] = duration;
            conf[n_tok] = max_softmax(logits, V);
            ++n_tok;
            last_token = token;
            ++emitted;
        }
        advance(&frame_idx, &emitted, token, duration, w->blank, w->max_symbols);
        ++step;
    }
    if (steps_used) *steps_used = step;
    free(h); free(c); free(h_new); free(c_new); free(gates); free(pred); free(z); free(logits); free(encp);
    return rc < 0 ? rc : n_tok;
}
