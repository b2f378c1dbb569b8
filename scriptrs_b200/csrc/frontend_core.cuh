// Per-frame arithmetic of the log-mel frontend, written so that the same functions run on the device (sixteen
// lanes of a warp work on one frame) and, for index-arithmetic checks, on the host with the lanes run one after
// another.  One frame: 400 windowed samples in a 512-point real FFT -> 257 power bins -> 128 mel rows -> ln.
//
// The 512-point real transform is a 256-point complex transform of z[n] = x[2n] + i x[2n+1] followed by the
// usual untangling.  The complex transform is two radix-16 passes (256 = 16 x 16) that stay in registers, with
// one transpose through shared memory between them:
//   pass 1   lane n2 holds z[16 n1 + n2], n1 = 0..15 (zero from n = 200 on): DFT-16 over n1 -> A[k1]
//   twiddle  A[k1] *= W256^(n2 k1), then B[k1][n2] = A[k1] goes to shared memory (row stride 17: conflict-free)
//   pass 2   lane k1 reads row k1: DFT-16 over n2 -> Z[k1 + 16 k2]
// Z then goes back to shared memory (k-indexed); each lane untangles eight (k, 256 - k) pairs into power bins,
// and finally sums its eight mel rows (row 16 g + lane) over their contiguous tap runs.
#pragma once
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "frontend.h"

#if defined(__CUDACC__)
#define SB_HD __host__ __device__ __forceinline__
#else
#define SB_HD inline
#endif

namespace sb {
namespace fe {

constexpr int kRow = 17;                    // float2 per row of the 16 x 16 transpose buffer
constexpr int kFrameScratch = 280;          // float2 per frame (>= 16 * kRow = 272): transpose buffer, then Z[0..255], then
                                            // the power bins.  560 words = 16 (mod 32), so that the 4-byte accesses of the
                                            // two frames of a warp fall into different banks

SB_HD float2 cadd(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
SB_HD float2 csub(float2 a, float2 b) { return make_float2(a.x - b.x, a.y - b.y); }
SB_HD float2 cmul(float2 a, float2 b) { return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x); }

// Forward 4-point DFT in place: (x0, x1, x2, x3) -> (X0, X1, X2, X3).
SB_HD void dft4(float2& x0, float2& x1, float2& x2, float2& x3) {
    const float2 t0 = cadd(x0, x2), t1 = csub(x0, x2), t2 = cadd(x1, x3), t3 = csub(x1, x3);
    x0 = cadd(t0, t2);
    x2 = csub(t0, t2);
    x1 = make_float2(t1.x + t3.y, t1.y - t3.x);  // t1 - i t3
    x3 = make_float2(t1.x - t3.y, t1.y + t3.x);  // t1 + i t3
}
// Same with x3 = 0 (the first pass of a frame: samples from 2 * 208 on are zero padding).
SB_HD void dft4_x3zero(float2& x0, float2& x1, float2& x2, float2& x3) {
    const float2 t0 = cadd(x0, x2), t1 = csub(x0, x2);
    x0 = cadd(t0, x1);
    x2 = csub(t0, x1);
    const float2 y1 = make_float2(t1.x + x1.y, t1.y - x1.x);
    x3 = make_float2(t1.x - x1.y, t1.y + x1.x);
    x1 = y1;
}

// Forward 16-point DFT in place.  Input a[n] in natural order; output X[k] is left at a[4 (k & 3) + (k >> 2)]
// (read it through dft16_slot).  n = 4 a + b, k = c + 4 d:  X[c + 4d] = sum_b W4^(bd) W16^(bc) sum_a x[4a + b] W4^(ac).
SB_HD constexpr int dft16_slot(int k) { return 4 * (k & 3) + (k >> 2); }

template <bool TAIL_ZERO>
SB_HD void dft16(float2 (&a)[16]) {
    const float c1 = 0.92387953251128673848f, s1 = 0.38268343236508978178f, h = 0.70710678118654752440f;
    dft4(a[0], a[4], a[8], a[12]);
    if (TAIL_ZERO) {
        dft4_x3zero(a[1], a[5], a[9], a[13]);
        dft4_x3zero(a[2], a[6], a[10], a[14]);
        dft4_x3zero(a[3], a[7], a[11], a[15]);
    } else {
        dft4(a[1], a[5], a[9], a[13]);
        dft4(a[2], a[6], a[10], a[14]);
        dft4(a[3], a[7], a[11], a[15]);
    }
    // a[4c + b] *= W16^(bc), W16 = exp(-2 pi i / 16)
    a[5] = cmul(a[5], make_float2(c1, -s1));                         // b = 1, c = 1: W^1
    a[6] = make_float2((a[6].x + a[6].y) * h, (a[6].y - a[6].x) * h);  // b = 2, c = 1: W^2 = (1 - i) / sqrt 2
    a[7] = cmul(a[7], make_float2(s1, -c1));                         // b = 3, c = 1: W^3
    a[9] = make_float2((a[9].x + a[9].y) * h, (a[9].y - a[9].x) * h);  // b = 1, c = 2: W^2
    a[10] = make_float2(a[10].y, -a[10].x);                          // b = 2, c = 2: W^4 = -i
    a[11] = make_float2((a[11].y - a[11].x) * h, -(a[11].x + a[11].y) * h);  // b = 3, c = 2: W^6 = (-1 - i) / sqrt 2
    a[13] = cmul(a[13], make_float2(s1, -c1));                       // b = 1, c = 3: W^3
    a[14] = make_float2((a[14].y - a[14].x) * h, -(a[14].x + a[14].y) * h);  // b = 2, c = 3: W^6
    a[15] = cmul(a[15], make_float2(-c1, s1));                       // b = 3, c = 3: W^9
    dft4(a[0], a[1], a[2], a[3]);
    dft4(a[4], a[5], a[6], a[7]);
    dft4(a[8], a[9], a[10], a[11]);
    dft4(a[12], a[13], a[14], a[15]);
}

#if defined(__CUDA_ARCH__)
#define SB_MUL_RN(a, b) __fmul_rn((a), (b))
#define SB_ADD_RN(a, b) __fadd_rn((a), (b))
#else
#define SB_MUL_RN(a, b) ((a) * (b))
#define SB_ADD_RN(a, b) ((a) + (b))
#endif

// Pass 1 of one frame for lane p (0..15).  ys: the frame's 400 pre-emphasised samples (8-byte aligned);
// window: Hann[400]; twid: the 256 inter-pass twiddles; B: this frame's transpose buffer.
SB_HD void pass1(int p, const float* ys, const float* window, const float2* twid, float2* B) {
    float2 a[16];
#pragma unroll
    for (int n1 = 0; n1 < 13; ++n1) {
        const int n = 16 * n1 + p;
        if (n1 < 12 || p < 8) {  // n < 200
            const float2 v = *reinterpret_cast<const float2*>(ys + 2 * n);
            const float2 w = *reinterpret_cast<const float2*>(window + 2 * n);
            a[n1] = make_float2(SB_MUL_RN(v.x, w.x), SB_MUL_RN(v.y, w.y));  // frontend.rs:74-77
        } else {
            a[n1] = make_float2(0.0f, 0.0f);
        }
    }
    a[13] = a[14] = a[15] = make_float2(0.0f, 0.0f);
    dft16<true>(a);
    B[p] = a[0];
#pragma unroll
    for (int k1 = 1; k1 < 16; ++k1) B[k1 * kRow + p] = cmul(a[dft16_slot(k1)], twid[k1 * 16 + p]);
}

// Pass 2 for lane p = k1: reads row p of B (after all lanes' pass 1), returns Z[p + 16 k2] at z[dft16_slot(k2)].
SB_HD void pass2(int p, const float2* B, float2 (&z)[16]) {
#pragma unroll
    for (int n2 = 0; n2 < 16; ++n2) z[n2] = B[p * kRow + n2];
    dft16<false>(z);
}

// After every lane finished reading B: Z goes to the same buffer, k-indexed.
SB_HD void store_z(int p, const float2 (&z)[16], float2* Z) {
#pragma unroll
    for (int k2 = 0; k2 < 16; ++k2) Z[p + 16 * k2] = z[dft16_slot(k2)];
}

// Real-FFT untangling and power for bins k and 256 - k, k = 1 + p + 16 m (m = 0..7), plus DC / Nyquist (lane 0).
//   E = (Z[k] + conj(Z[256-k])) / 2,  O = -i (Z[k] - conj(Z[256-k])) / 2,  X[k] = E + W512^k O,  X[256-k] = conj(E - W512^k O)
// The halves are left out: with tw_post[k] = W512^k the code forms 2 X, so the stored value is 4 |X|^2 (an exact
// scaling), and the filterbank taps carry the factor 1/4 (frontend.rs:142, norm_sqr, then :110).
// Two steps so that the power bins may overwrite the buffer Z was read from: every lane first loads its sixteen Z
// values (untangle_load), the warp synchronises, then the bins are written (untangle_store).
SB_HD void untangle_load(int p, const float2* Z, float2 (&zk)[8], float2 (&zc)[8], float2& z0) {
#pragma unroll
    for (int m = 0; m < 8; ++m) {
        const int k = 1 + p + 16 * m;
        zk[m] = Z[k];
        zc[m] = Z[256 - k];
    }
    z0 = Z[0];
}
SB_HD void untangle_store(int p, const float2 (&zk)[8], const float2 (&zc)[8], float2 z0, const float2* tw_post, float* pw) {
#pragma unroll
    for (int m = 0; m < 8; ++m) {
        const int k = 1 + p + 16 * m, kc = 256 - k;
        const float2 e = make_float2(zk[m].x + zc[m].x, zk[m].y - zc[m].y);
        const float2 d = make_float2(zk[m].x - zc[m].x, zk[m].y + zc[m].y);  // Z[k] - conj(Z[256-k])
        const float2 t = cmul(make_float2(d.y, -d.x), tw_post[k]);            // (-i d) * W
        const float2 xp = cadd(e, t), xm = csub(e, t);
        pw[k] = fmaf(xp.x, xp.x, xp.y * xp.y);
        pw[kc] = fmaf(xm.x, xm.x, xm.y * xm.y);
    }
    if (p == 0) {
        const float dc = 2.0f * (z0.x + z0.y), ny = 2.0f * (z0.x - z0.y);
        pw[0] = dc * dc;
        pw[256] = ny * ny;
    }
}

// kGroupTaps / kGroupTapOffset as functions (device code cannot index a host constexpr array)
SB_HD constexpr int group_taps(int g) {
    return g < 3 ? 2 : (g == 3 ? 3 : (g == 4 ? 4 : (g == 5 ? 6 : (g == 6 ? 9 : 12))));
}
SB_HD constexpr int group_tap_offset(int g) {
    return g == 0 ? 0 : (g == 1 ? 2 : (g == 2 ? 4 : (g == 3 ? 6 : (g == 4 ? 9 : (g == 5 ? 13 : (g == 6 ? 19 : 28))))));
}

SB_HD float log_mel(float acc, float log_floor) {
    // frontend.rs:111: ln(mel + 2^-24).  An empty cell (silence) is exactly 2^-24: its logarithm comes from the
    // table so that it carries the host library's rounding; everything else goes through the hardware logarithm
    // (absolute error below 3 ulp of the result, far inside the 1e-4 parity bound).
    if (acc == 0.0f) return log_floor;
#if defined(__CUDA_ARCH__)
    return __logf(SB_ADD_RN(acc, 5.9604644775390625e-08f));
#else
    return logf(acc + 5.9604644775390625e-08f);
#endif
}

// Mel rows 16 g + p, g = 0..7, of one frame: out[16 g + p] = ln(sum_t w[t] * pw[start + t] + 2^-24); pw holds four
// times the power and the taps a quarter of the filterbank value (both exact).  Taps past a row's run are zero and
// meet power bins of index <= 255, which always hold finite values.  The lane's 40 taps live in registers
// (load_mel_taps, once per kernel).
SB_HD void load_mel_taps(int p, const float* melw, float (&w)[kMelTapRows]) {
#pragma unroll
    for (int i = 0; i < kMelTapRows; ++i) w[i] = melw[i * 16 + p];
}
SB_HD void mel_rows(int p, const float* pw, const float (&w)[kMelTapRows], const int16_t* mel_start, float log_floor,
                    float* out) {
#pragma unroll
    for (int g = 0; g < kMelGroups; ++g) {
        const int m = 16 * g + p;
        const int st = mel_start[m];
        float acc = 0.0f;
#pragma unroll
        for (int t = 0; t < group_taps(g); ++t) acc = fmaf(w[group_tap_offset(g) + t], pw[st + t], acc);
        out[m] = log_mel(acc, log_floor);
    }
}

// 16-bit PCM sample -> f32 as the reference's WAV reader does it: value / 32767 in f32, correctly rounded
// (examples/transcribe_wav.rs:341-347).  Quotient from the rounded reciprocal plus one exact-remainder correction;
// equal to the IEEE division for every 16-bit value (checked exhaustively by the host-side tests).
SB_HD float pcm16_to_f32(int v) {
    const float x = (float)v;
    const float r = 3.0518509447574615e-05f;  // RN(1 / 32767)
    const float q = SB_MUL_RN(x, r);
    const float rem = fmaf(-q, 32767.0f, x);
    return fmaf(rem, r, q);
}

}  // namespace fe
}  // namespace sb
