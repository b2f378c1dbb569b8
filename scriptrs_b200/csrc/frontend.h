// Internal interface of the log-mel frontend (see frontend.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace sb {

constexpr int kSampleRate = 16000;
constexpr int kNfft = 512;
constexpr int kWin = 400;
constexpr int kHop = 160;
constexpr int kPad = kNfft / 2;
constexpr int kBins = kNfft / 2 + 1;
constexpr int kMels = 128;
constexpr int kMaxTaps = 12;  // most non-zero filterbank taps in one mel row (asserted when tables are built)

// Device-resident constant tables, built once on the host.
struct FrontendTables {
    float window[kWin];             // Hann, frontend.rs:161-165
    float2 tw_post[132];            // 0.5 * exp(-2*pi*i*k/512), k = 0..128
    float melw[kMaxTaps * kMels];   // non-zero taps of the [128 x 257] Slaney filterbank, tap-major
    int16_t mel_start[kMels];       // first non-zero bin of each row
    int16_t mel_cnt[kMels];         // number of non-zero taps of each row
};

// Host-side table construction (frontend_tables.cpp).  `dense_fb`, if not null,
// receives the dense [128 x 257] filterbank.  Returns false if a row has more
// than kMaxTaps taps or taps that are not contiguous.
bool build_frontend_tables(FrontendTables* t, float* dense_fb);
void hann_window_host(float* w, int n);
void mel_filterbank_host(float* fb, int n_fft, int n_mels, int sample_rate);

inline int64_t frames_for_samples(int64_t n) { return (n + 2 * kPad - kNfft) / kHop + 1; }  // frontend.rs:127

size_t frontend_smem_bytes();
cudaError_t frontend_configure();
// Clip i is pcm[d_clip_start[i] .. + d_clip_len[i]) (clips may overlap in the PCM buffer); its features are
// written at row d_frame_off[i] of feats.
cudaError_t frontend_launch(const float* pcm, const int64_t* d_clip_start, const int64_t* d_clip_len,
                            const int64_t* d_frame_off, int n_clips,
                            int max_frames, float preemph, const FrontendTables* d_tables, float* feats,
                            float* d_mean, float* d_std, bool normalize, cudaStream_t stream);

}  // namespace sb
