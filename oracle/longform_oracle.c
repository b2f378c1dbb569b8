/*
 * CPU oracle for the long-form host logic.  TEST INFRASTRUCTURE ONLY: never
 * linked into or called from the product library.
 *
 * Literal restatements of the reference's integer logic:
 *   OverlapChunkConfig::{chunk,overlap,stride}_samples, plan   src/long_form/planner.rs:104-137
 *   push_overlap_task / build_fast_execution_plan              src/long_form.rs:439-459,566-582
 *   parallel_worker_count                                      src/long_form.rs:594-600
 *   apply_time_offsets                                         src/pipeline.rs:219-252
 *   merge_overlapping_windows and helpers                      src/long_form/merge.rs:3-200
 * The merge here is deliberately the reference's quadratic algorithm (whole
 * left transcript scanned against the right window, full LCS table); the
 * product's windowed merge is differential-tested against it.
 *
 * Pinned by the reference's own known-answer tests: planner.rs:376-385,
 * merge.rs:208-247, long_form.rs:738-769 (see tests/test_oracle_longform.py).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define SAMPLE_RATE 16000
#define MEL_HOP 160
#define SAMPLES_PER_ENC_FRAME 1280

typedef struct {
    int64_t audio_start, audio_end, global_sample_offset, context_samples;
} sbo_chunk_task;

static int64_t sat_sub(int64_t a, int64_t b) { return a > b ? a - b : 0; }
static int64_t imax(int64_t a, int64_t b) { return a > b ? a : b; }
static int64_t imin(int64_t a, int64_t b) { return a < b ? a : b; }

/* planner.rs:104-111 */
int64_t sbo_chunk_samples(int64_t context_samples, int64_t max_model_samples) {
    int64_t max_actual = sat_sub(max_model_samples, context_samples);
    int64_t raw = imax(sat_sub(max_actual, MEL_HOP), SAMPLES_PER_ENC_FRAME);
    return raw / SAMPLES_PER_ENC_FRAME * SAMPLES_PER_ENC_FRAME;
}
/* planner.rs:113-117 */
int64_t sbo_overlap_samples(double overlap_seconds, int64_t context_samples, int64_t max_model_samples) {
    double want = overlap_seconds * (double)SAMPLE_RATE;
    int64_t requested = want <= 0.0 ? 0 : (int64_t)want; /* `as usize` saturates at 0 */
    int64_t capped = imin(requested, sbo_chunk_samples(context_samples, max_model_samples) / 2);
    return capped / SAMPLES_PER_ENC_FRAME * SAMPLES_PER_ENC_FRAME;
}
/* planner.rs:119-122 */
int64_t sbo_stride_samples(double overlap_seconds, int64_t context_samples, int64_t max_model_samples) {
    int64_t raw = sat_sub(sbo_chunk_samples(context_samples, max_model_samples),
                          sbo_overlap_samples(overlap_seconds, context_samples, max_model_samples));
    return imax(raw, SAMPLES_PER_ENC_FRAME) / SAMPLES_PER_ENC_FRAME * SAMPLES_PER_ENC_FRAME;
}

/* planner.rs:124-136 + long_form.rs:566-582.  Returns the task count (the
 * tasks array may be NULL to size it), -2 if cap is too small. */
int64_t sbo_plan_fast(int64_t audio_len, double overlap_seconds, int64_t context_samples,
                      int64_t max_model_samples, sbo_chunk_task *tasks, int64_t cap) {
    int64_t chunk = sbo_chunk_samples(context_samples, max_model_samples);
    int64_t stride = sbo_stride_samples(overlap_seconds, context_samples, max_model_samples);
    int64_t n = 0, start = 0;
    while (start < audio_len) {
        int64_t end = imin(start + chunk, audio_len);
        if (tasks) {
            if (n >= cap) return -2;
            int64_t ctx_start = sat_sub(start, context_samples);
            tasks[n].audio_start = ctx_start;
            tasks[n].audio_end = end;
            tasks[n].global_sample_offset = start;
            tasks[n].context_samples = start - ctx_start;
        }
        ++n;
        if (end == audio_len) break;
        start += stride;
    }
    return n;
}

/* long_form.rs:594-600 */
int64_t sbo_parallel_worker_count(int64_t task_count, int64_t requested) {
    if (task_count <= 1) return 1;
    return imin(imax(requested, 1), task_count);
}

/* pipeline.rs:219-252, in place; returns the new token count. */
int64_t sbo_apply_time_offsets(uint32_t *tok, int64_t *frm, int64_t *dur, float *conf, int64_t n,
                               int64_t frame_offset, int64_t context_frames) {
    if (context_frames == 0) {
        for (int64_t i = 0; i < n; ++i) frm[i] += frame_offset;
        return n;
    }
    int64_t k = 0;
    for (int64_t i = 0; i < n; ++i) {
        if (frm[i] < context_frames) continue;
        tok[k] = tok[i]; frm[k] = frm[i] - context_frames + frame_offset; dur[k] = dur[i]; conf[k] = conf[i];
        ++k;
    }
    return k;
}

typedef struct {
    uint32_t *tok; int64_t *frm; int64_t *dur; float *conf; int64_t n, cap;
} raw_t;

static void raw_init(raw_t *r) { memset(r, 0, sizeof(*r)); }
static void raw_free(raw_t *r) { free(r->tok); free(r->frm); free(r->dur); free(r->conf); raw_init(r); }
static void raw_push(raw_t *r, const raw_t *s, int64_t i) {
    if (r->n == r->cap) {
        r->cap = r->cap ? r->cap * 2 : 64;
        r->tok = (uint32_t *)realloc(r->tok, sizeof(uint32_t) * (size_t)r->cap);
        r->frm = (int64_t *)realloc(r->frm, sizeof(int64_t) * (size_t)r->cap);
        r->dur = (int64_t *)realloc(r->dur, sizeof(int64_t) * (size_t)r->cap);
        r->conf = (float *)realloc(r->conf, sizeof(float) * (size_t)r->cap);
    }
    r->tok[r->n] = s->tok[i]; r->frm[r->n] = s->frm[i]; r->dur[r->n] = s->dur[i]; r->conf[r->n] = s->conf[i];
    r->n++;
}
static void raw_extend(raw_t *r, const raw_t *s, int64_t a, int64_t b) {
    for (int64_t i = a; i < b; ++i) raw_push(r, s, i);
}

/* merge.rs:95-103 */
static int tokens_match(const raw_t *l, int64_t li, const raw_t *r, int64_t ri) {
    int64_t d = l->frm[li] - r->frm[ri];
    if (d < 0) d = -d;
    return l->tok[li] == r->tok[ri] && d <= 25;
}

/* merge.rs:36-60: first strictly-longest diagonal run in (left, right) scan order. */
static int64_t contiguous_matches(const raw_t *l, const raw_t *r, int64_t *ml, int64_t *mr) {
    int64_t best = 0, bl = 0, br = 0;
    for (int64_t li = 0; li < l->n; ++li)
        for (int64_t ri = 0; ri < r->n; ++ri) {
            if (!tokens_match(l, li, r, ri)) continue;
            int64_t a = li, b = ri, len = 0;
            while (a < l->n && b < r->n && tokens_match(l, a, r, b)) { ++a; ++b; ++len; }
            if (len > best) { best = len; bl = li; br = ri; }
        }
    for (int64_t i = 0; i < best; ++i) { ml[i] = bl + i; mr[i] = br + i; }
    return best;
}

/* merge.rs:62-93 */
static int64_t lcs_matches(const raw_t *l, const raw_t *r, int64_t *ml, int64_t *mr) {
    int64_t nl = l->n, nr = r->n, w = nr + 1;
    int64_t *dp = (int64_t *)calloc((size_t)(nl + 1) * (size_t)w, sizeof(int64_t));
    for (int64_t i = 1; i <= nl; ++i)
        for (int64_t j = 1; j <= nr; ++j) {
            if (tokens_match(l, i - 1, r, j - 1)) dp[i * w + j] = dp[(i - 1) * w + j - 1] + 1;
            else dp[i * w + j] = imax(dp[(i - 1) * w + j], dp[i * w + j - 1]);
        }
    int64_t cnt = 0, i = nl, j = nr;
    while (i > 0 && j > 0) {
        if (tokens_match(l, i - 1, r, j - 1)) { ml[cnt] = i - 1; mr[cnt] = j - 1; ++cnt; --i; --j; continue; }
        if (dp[(i - 1) * w + j] > dp[i * w + j - 1]) --i; else --j;
    }
    free(dp);
    for (int64_t a = 0, b = cnt - 1; a < b; ++a, --b) {
        int64_t t = ml[a]; ml[a] = ml[b]; ml[b] = t;
        t = mr[a]; mr[a] = mr[b]; mr[b] = t;
    }
    return cnt;
}

/* merge.rs:105-140 */
static void merge_using_matches(const raw_t *l, const raw_t *r, const int64_t *ml, const int64_t *mr,
                                int64_t cnt, raw_t *out) {
    raw_extend(out, l, 0, ml[0]);
    for (int64_t m = 0; m < cnt; ++m) {
        raw_extend(out, l, ml[m], ml[m] + 1);
        if (m == cnt - 1) continue;
        int64_t left_gap = sat_sub(ml[m + 1], ml[m] + 1);
        int64_t right_gap = sat_sub(mr[m + 1], mr[m] + 1);
        if (right_gap > left_gap) raw_extend(out, r, mr[m] + 1, mr[m + 1]);
        else raw_extend(out, l, ml[m] + 1, ml[m + 1]);
    }
    raw_extend(out, r, mr[cnt - 1] + 1, r->n);
}

/* merge.rs:142-165 */
static void merge_by_midpoint(const raw_t *l, const raw_t *r, raw_t *out) {
    int64_t left_cutoff = l->n ? l->frm[l->n - 1] : 0;
    int64_t right_start = r->n ? r->frm[0] : left_cutoff;
    int64_t midpoint = (left_cutoff + right_start) / 2;
    for (int64_t i = 0; i < l->n; ++i) if (l->frm[i] < midpoint) raw_push(out, l, i);
    for (int64_t i = 0; i < r->n; ++i) if (r->frm[i] >= midpoint) raw_push(out, r, i);
}

/* merge.rs:15-34 */
static void merge_pair(raw_t *left, const raw_t *right) {
    if (right->n == 0) return;
    raw_t out; raw_init(&out);
    if (left->n == 0) { raw_extend(&out, right, 0, right->n); raw_free(left); *left = out; return; }
    int64_t cap = imin(left->n, right->n) + 1;
    int64_t *ml = (int64_t *)malloc(sizeof(int64_t) * (size_t)cap);
    int64_t *mr = (int64_t *)malloc(sizeof(int64_t) * (size_t)cap);
    int64_t cnt = contiguous_matches(left, right, ml, mr);
    if (cnt == 0) cnt = lcs_matches(left, right, ml, mr);
    if (cnt > 0) merge_using_matches(left, right, ml, mr, cnt, &out);
    else merge_by_midpoint(left, right, &out);
    free(ml); free(mr);
    raw_free(left);
    *left = out;
}

/*
 * merge.rs:3-13: left fold over windows, in order.  Windows are concatenated
 * in the input arrays; win_off[w]..win_off[w+1] delimits window w.  Returns
 * the merged length (-2 if out_cap is too small).
 */
int64_t sbo_merge_windows(const uint32_t *tok, const int64_t *frm, const int64_t *dur, const float *conf,
                          const int64_t *win_off, int64_t n_windows, uint32_t *otok, int64_t *ofrm,
                          int64_t *odur, float *oconf, int64_t out_cap) {
    raw_t merged; raw_init(&merged);
    for (int64_t w = 0; w < n_windows; ++w) {
        raw_t win;
        win.tok = (uint32_t *)tok + win_off[w]; win.frm = (int64_t *)frm + win_off[w];
        win.dur = (int64_t *)dur + win_off[w]; win.conf = (float *)conf + win_off[w];
        win.n = win_off[w + 1] - win_off[w]; win.cap = 0;
        if (w == 0) raw_extend(&merged, &win, 0, win.n);
        else merge_pair(&merged, &win);
    }
    int64_t n = merged.n;
    if (n > out_cap) { raw_free(&merged); return -2; }
    if (n) {
        memcpy(otok, merged.tok, sizeof(uint32_t) * (size_t)n);
        memcpy(ofrm, merged.frm, sizeof(int64_t) * (size_t)n);
        memcpy(odur, merged.dur, sizeof(int64_t) * (size_t)n);
        memcpy(oconf, merged.conf, sizeof(float) * (size_t)n);
    }
    raw_free(&merged);
    return n;
}
