// Host-side constant tables of the log-mel frontend: Hann window, Slaney mel
// filterbank (dense and as per-row tap runs) and the real-FFT untangling twiddles.
// Follows the table construction of the reference's feature extractor
// (src/frontend.rs:161-223): window in f32, filterbank triangles in f64 cast to
// f32 and scaled in f32.  Compiled with floating-point contraction off.
#include <algorithm>
#include <cmath>
#include <vector>

#include "frontend.h"

namespace sb {

void hann_window_host(float* w, int n) {
    const float pi = 3.14159265358979323846f;
    const float denom = static_cast<float>(n) - 1.0f;
    for (int i = 0; i < n; ++i) {
        const float phase = (2.0f * pi * static_cast<float>(i)) / denom;
        w[i] = 0.5f - 0.5f * std::cos(phase);  // f32 cos
    }
}

namespace {
constexpr double kFsp = 200.0 / 3.0;
constexpr double kMinLogHz = 1000.0;
constexpr double kMinLogMel = kMinLogHz / kFsp;
constexpr double kLogStep = 0.06875177742094912;

double slaney_mel(double hz) { return hz < kMinLogHz ? hz / kFsp : kMinLogMel + std::log(hz / kMinLogHz) / kLogStep; }
double slaney_hz(double mel) {
    return mel < kMinLogMel ? mel * kFsp : kMinLogHz * std::exp((mel - kMinLogMel) * kLogStep);
}
}  // namespace

void mel_filterbank_host(float* fb, int n_fft, int n_mels, int sample_rate) {
    const int bins = n_fft / 2 + 1;
    const double lo = slaney_mel(0.0), hi = slaney_mel(sample_rate / 2.0);
    std::vector<double> edge(n_mels + 2);
    for (int i = 0; i < n_mels + 2; ++i) edge[i] = slaney_hz(lo + (hi - lo) * i / static_cast<double>(n_mels + 1));
    for (int m = 0; m < n_mels; ++m) {
        const double rise = edge[m + 1] - edge[m], fall = edge[m + 2] - edge[m + 1];
        const float area = static_cast<float>(2.0 / (edge[m + 2] - edge[m]));
        for (int k = 0; k < bins; ++k) {
            const double hz = static_cast<double>(k) * sample_rate / static_cast<double>(n_fft);
            const double tri = std::fmax(0.0, std::fmin((hz - edge[m]) / rise, (edge[m + 2] - hz) / fall));
            fb[m * bins + k] = static_cast<float>(tri) * area;  // f32 product
        }
    }
}

bool build_frontend_tables(FrontendTables* t, float* dense_fb) {
    const double pi = 3.14159265358979323846;
    hann_window_host(t->window, kWin);
    for (int k = 0; k < 132; ++k) {
        const double ang = -2.0 * pi * k / 512.0;
        t->tw_post[k] = make_float2(static_cast<float>(std::cos(ang)), static_cast<float>(std::sin(ang)));
    }
    for (int k1 = 0; k1 < 16; ++k1)
        for (int n2 = 0; n2 < 16; ++n2) {
            const double ang = -2.0 * pi * (n2 * k1) / 256.0;
            t->twid[k1 * 16 + n2] = make_float2(static_cast<float>(std::cos(ang)), static_cast<float>(std::sin(ang)));
        }
    t->log_floor = std::log(5.9604644775390625e-08f);  // f32 logarithm of 2^-24, frontend.rs:111
    std::vector<float> fb(static_cast<size_t>(kMels) * kBins);
    mel_filterbank_host(fb.data(), kNfft, kMels, kSampleRate);
    if (dense_fb) std::copy(fb.begin(), fb.end(), dense_fb);
    for (int i = 0; i < kMelTapRows * 16; ++i) t->melw[i] = 0.0f;
    for (int m = 0; m < kMels; ++m) {
        int first = -1, last = -1, nonzero = 0;
        for (int k = 0; k < kBins; ++k)
            if (fb[m * kBins + k] != 0.0f) {
                if (first < 0) first = k;
                last = k;
                ++nonzero;
            }
        if (first < 0) { first = 0; last = -1; }
        const int cnt = last - first + 1;
        const int g = m / 16, lane = m % 16;
        if (cnt > kGroupTaps[g] || cnt > kMaxTaps || nonzero != cnt) return false;
        // a quarter of the tap: the kernel's power bins are 4 |X|^2 (scaling by a power of two is exact)
        for (int j = 0; j < cnt; ++j) t->melw[(kGroupTapOffset[g] + j) * 16 + lane] = 0.25f * fb[m * kBins + first + j];
        t->mel_start[m] = static_cast<int16_t>(first);
    }
    return true;
}

}  // namespace sb
