/*
 * CPU oracle for the log-mel frontend.  TEST INFRASTRUCTURE ONLY: the product
 * library never links or calls this file; only the test-suite, the smoke check
 * and the CPU-baseline leg of the benchmark do.
 *
 * It restates, operation by operation, the reference's src/frontend.rs:
 *   hann_window            frontend.rs:161-165
 *   create_mel_filterbank  frontend.rs:167-223
 *   apply_preemphasis_into frontend.rs:150-159
 *   prepare_padded_audio   frontend.rs:59-65   (256 zeros each side)
 *   stft / process_frame   frontend.rs:67-85,120-147
 *   extract                frontend.rs:104-118
 *   normalize_columns      frontend.rs:225-241
 *
 * Every intermediate the reference keeps in f32 is kept in f32 here and no
 * multiply-add is contracted (build with -ffp-contract=off).  Two pieces of
 * the reference's arithmetic live in third-party crates that are not part of
 * the reference tree (realfft 3.5.0 -> rustfft 6.4.1 for the 512-point real
 * FFT; ndarray 0.17.2 -> matrixmultiply 0.3.10 for the [128x257]x[257xT]
 * product).  Their summation orders are unspecified, so in "gold" mode both
 * are evaluated in f64 and rounded once to f32, which is within the crates'
 * own rounding error of whatever order they use.  "port" mode (fft_f32 != 0)
 * runs an f32 FFT and an f32 dense product instead; it is what the CPU
 * baseline times, because it does the same amount of work in the same
 * precision as the reference.
 *
 * Parity status: the reference holds no numeric golden vectors for this path
 * (its three frontend tests are properties: peak bin 32 for a 1 kHz sine,
 * 128 columns, column-0 mean ~ 0).  Those three are checked in
 * tests/test_oracle_frontend.py; beyond them the numeric parity of this
 * restatement is unpinned and rests on following the source line by line.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define N_FFT 512
#define WIN 400
#define HOP 160
#define N_BINS 257
#define N_MELS 128
#define PAD 256

/* frontend.rs:161-165 — all arithmetic in f32, cos from libm. */
void sbo_hann_window(float *w, int n) {
    const float pi = 3.14159265358979323846f; /* std::f32::consts::PI */
    for (int i = 0; i < n; ++i) {
        float arg = (2.0f * pi * (float)i) / ((float)n - 1.0f);
        w[i] = 0.5f - 0.5f * cosf(arg);
    }
}

/* frontend.rs:167-186 */
static const double F_SP = 200.0 / 3.0;
static const double MIN_LOG_HZ = 1000.0;
static const double LOG_STEP = 0.06875177742094912;

static double hz_to_mel(double hz) {
    const double min_log_mel = MIN_LOG_HZ / F_SP;
    return hz < MIN_LOG_HZ ? hz / F_SP : min_log_mel + log(hz / MIN_LOG_HZ) / LOG_STEP;
}
static double mel_to_hz(double mel) {
    const double min_log_mel = MIN_LOG_HZ / F_SP;
    return mel < min_log_mel ? mel * F_SP : MIN_LOG_HZ * exp((mel - min_log_mel) * LOG_STEP);
}

/* frontend.rs:188-223 — triangles in f64, cast to f32, then scaled by the f32
 * cast of the Slaney area normalisation, the product taken in f32. */
void sbo_mel_filterbank(float *fb /* [n_mels x n_bins] */, int n_fft, int n_mels, int sample_rate) {
    int n_bins = n_fft / 2 + 1;
    double fmax = (double)sample_rate / 2.0;
    double mel_min = hz_to_mel(0.0), mel_max = hz_to_mel(fmax);
    double *pts = (double *)malloc(sizeof(double) * (size_t)(n_mels + 2));
    for (int i = 0; i <= n_mels + 1; ++i)
        pts[i] = mel_to_hz(mel_min + (mel_max - mel_min) * (double)i / (double)(n_mels + 1));
    for (int m = 0; m < n_mels; ++m) {
        double d0 = pts[m + 1] - pts[m], d1 = pts[m + 2] - pts[m + 1];
        for (int k = 0; k < n_bins; ++k) {
            double f = (double)k * (double)sample_rate / (double)n_fft;
            double lower = (f - pts[m]) / d0;
            double upper = (pts[m + 2] - f) / d1;
            double v = lower < upper ? lower : upper;
            fb[m * n_bins + k] = (float)(v > 0.0 ? v : 0.0);
        }
    }
    for (int m = 0; m < n_mels; ++m) {
        float enorm = (float)(2.0 / (pts[m + 2] - pts[m]));
        for (int k = 0; k < n_bins; ++k) fb[m * n_bins + k] *= enorm;
    }
    free(pts);
}

/* Twiddles exp(-2*pi*i*k/512), computed once in f64. */
static double TW_RE[N_FFT / 2], TW_IM[N_FFT / 2];
static float TW_RE32[N_FFT / 2], TW_IM32[N_FFT / 2];
static int tw_ready = 0;
static void init_twiddles(void) {
    if (tw_ready) return;
    for (int k = 0; k < N_FFT / 2; ++k) {
        double ang = -2.0 * 3.14159265358979323846 * (double)k / (double)N_FFT;
        TW_RE[k] = cos(ang); TW_IM[k] = sin(ang);
        TW_RE32[k] = (float)TW_RE[k]; TW_IM32[k] = (float)TW_IM[k];
    }
    tw_ready = 1;
}

/* In-place iterative radix-2 FFT of length 512, forward sign, instantiated for
 * f64 (gold) and f32 (timed port). */
#define DEFINE_FFT(NAME, T, WR, WI)                                                \
    static void NAME(T *re, T *im) {                                               \
        const int n = N_FFT;                                                       \
        for (int i = 1, j = 0; i < n; ++i) {                                       \
            int bit = n >> 1;                                                      \
            for (; j & bit; bit >>= 1) j ^= bit;                                   \
            j ^= bit;                                                              \
            if (i < j) {                                                           \
                T t = re[i]; re[i] = re[j]; re[j] = t;                             \
                t = im[i]; im[i] = im[j]; im[j] = t;                               \
            }                                                                      \
        }                                                                          \
        for (int len = 2; len <= n; len <<= 1) {                                   \
            int half = len >> 1, step = n / len;                                   \
            for (int s0 = 0; s0 < n; s0 += len) {                                  \
                for (int k = 0; k < half; ++k) {                                   \
                    T wr = WR[k * step], wi = WI[k * step];                        \
                    int s = s0 + k, b = s + half;                                  \
                    T xr = re[b] * wr - im[b] * wi;                                \
                    T xi = re[b] * wi + im[b] * wr;                                \
                    re[b] = re[s] - xr; im[b] = im[s] - xi;                        \
                    re[s] = re[s] + xr; im[s] = im[s] + xi;                        \
                }                                                                  \
            }                                                                      \
        }                                                                          \
    }
DEFINE_FFT(fft_f64, double, TW_RE, TW_IM)
DEFINE_FFT(fft_f32, float, TW_RE32, TW_IM32)

/* Power spectrogram, frontend.rs:120-147.  power: [n_bins x T] bin-major like
 * the reference's Array2 (spectrogram[[bin, frame]]).  Returns T. */
static int64_t stft_power(const float *audio, int64_t n, float preemph, const float *window,
                          int fft_f32_mode, float *power, int64_t t_cap) {
    int64_t padded_len = n + 2 * PAD;
    int64_t T = (padded_len - N_FFT) / HOP + 1; /* frontend.rs:127 */
    if (T > t_cap) return -1;
    init_twiddles();
    float *padded = (float *)calloc((size_t)padded_len, sizeof(float));
    /* frontend.rs:150-159: y[0] = x[0]; y[i] = x[i] - c*x[i-1], product rounded first. */
    padded[PAD] = audio[0];
    for (int64_t i = 1; i < n; ++i) {
        float prod = preemph * audio[i - 1];
        padded[PAD + i] = audio[i] - prod;
    }
    double re64[N_FFT], im64[N_FFT];
    float re32[N_FFT], im32[N_FFT];
    for (int64_t t = 0; t < T; ++t) {
        int64_t start = t * HOP;
        /* frontend.rs:74-77: window is left-aligned in the 512 buffer. */
        for (int j = 0; j < N_FFT; ++j) {
            float v = j < WIN ? padded[start + j] * window[j] : 0.0f;
            re64[j] = (double)v; im64[j] = 0.0;
            re32[j] = v; im32[j] = 0.0f;
        }
        if (fft_f32_mode) fft_f32(re32, im32);
        else fft_f64(re64, im64);
        for (int k = 0; k < N_BINS; ++k) {
            float r = fft_f32_mode ? re32[k] : (float)re64[k];
            float i = fft_f32_mode ? im32[k] : (float)im64[k];
            float rr = r * r, ii = i * i; /* norm_sqr: re*re + im*im in f32 */
            power[(int64_t)k * T + t] = rr + ii;
        }
    }
    free(padded);
    return T;
}

/* frontend.rs:225-241 — strictly sequential f32 sums, left to right. */
static void normalize_columns(float *feat /* [T x 128] */, int64_t T) {
    for (int f = 0; f < N_MELS; ++f) {
        float sum = 0.0f;
        for (int64_t t = 0; t < T; ++t) sum = sum + feat[t * N_MELS + f];
        float mean = sum / (float)T;
        float acc = 0.0f;
        for (int64_t t = 0; t < T; ++t) {
            float d = feat[t * N_MELS + f] - mean;
            float sq = d * d;
            acc = acc + sq;
        }
        float variance = acc / ((float)T - 1.0f);
        float std = sqrtf(variance) + 1e-5f;
        for (int64_t t = 0; t < T; ++t) feat[t * N_MELS + f] = (feat[t * N_MELS + f] - mean) / std;
    }
}

/*
 * Full extract(), frontend.rs:104-118.
 *   audio[n]       mono 16 kHz f32
 *   feats          [T x 128] row-major (the reference's output orientation)
 *   raw_logmel     optional [T x 128]: ln(mel + 2^-24) before normalisation
 *   power_out      optional [257 x T] bin-major power spectrogram
 *   fft_f32        0 = gold (f64 FFT and f64-accumulated mel product),
 *                  1 = port (f32 FFT, f32 dense product; the timed baseline)
 * Returns T (= n/160 + 1) or a negative code: -1 empty audio (frontend.rs:105),
 * -2 capacity too small.
 */
int64_t sbo_frontend_extract(const float *audio, int64_t n, float preemph, int fft_f32,
                             float *feats, int64_t t_cap, float *raw_logmel, float *power_out) {
    if (n <= 0) return -1;
    int64_t T = (n + 2 * PAD - N_FFT) / HOP + 1;
    if (T > t_cap) return -2;
    static float window[WIN];
    static float fb[N_MELS * N_BINS];
    static int tables_ready = 0;
    if (!tables_ready) {
        sbo_hann_window(window, WIN);
        sbo_mel_filterbank(fb, N_FFT, N_MELS, 16000);
        tables_ready = 1;
    }
    float *power = (float *)malloc(sizeof(float) * (size_t)N_BINS * (size_t)T);
    stft_power(audio, n, preemph, window, fft_f32, power, T);
    if (power_out) memcpy(power_out, power, sizeof(float) * (size_t)N_BINS * (size_t)T);
    const float guard = 5.9604644775390625e-08f; /* 2^-24, frontend.rs:111 */
    /* frontend.rs:110-115: mel = fb . power, then ln(mel + 2^-24), transposed.
     * The k loop is outermost per mel row so that the inner loop is contiguous
     * in t; the order of accumulation over k is ascending in both modes. */
    double *acc64 = (double *)malloc(sizeof(double) * (size_t)T);
    float *acc32 = (float *)malloc(sizeof(float) * (size_t)T);
    for (int m = 0; m < N_MELS; ++m) {
        const float *row = fb + m * N_BINS;
        if (fft_f32) {
            for (int64_t t = 0; t < T; ++t) acc32[t] = 0.0f;
            for (int k = 0; k < N_BINS; ++k) {
                const float w = row[k];
                const float *p = power + (int64_t)k * T;
                for (int64_t t = 0; t < T; ++t) {
                    float prod = w * p[t];
                    acc32[t] = acc32[t] + prod;
                }
            }
        } else {
            for (int64_t t = 0; t < T; ++t) acc64[t] = 0.0;
            for (int k = 0; k < N_BINS; ++k) {
                if (row[k] == 0.0f) continue;
                const double w = (double)row[k];
                const float *p = power + (int64_t)k * T;
                for (int64_t t = 0; t < T; ++t) acc64[t] += w * (double)p[t];
            }
        }
        for (int64_t t = 0; t < T; ++t) {
            float mel = fft_f32 ? acc32[t] : (float)acc64[t];
            float shifted = mel + guard;
            feats[t * N_MELS + m] = logf(shifted);
        }
    }
    free(acc64);
    free(acc32);
    free(power);
    if (raw_logmel) memcpy(raw_logmel, feats, sizeof(float) * (size_t)T * N_MELS);
    normalize_columns(feats, T);
    return T;
}

/* Batch helper for the timed baseline: clips laid out back to back, equal length. */
int64_t sbo_frontend_batch(const float *audio, int64_t n_per_clip, int64_t n_clips, float preemph,
                           int fft_f32, float *feats) {
    int64_t T = (n_per_clip + 2 * PAD - N_FFT) / HOP + 1;
    for (int64_t c = 0; c < n_clips; ++c) {
        int64_t r = sbo_frontend_extract(audio + c * n_per_clip, n_per_clip, preemph, fft_f32,
                                         feats + c * T * N_MELS, T, NULL, NULL);
        if (r < 0) return r;
    }
    return T;
}
