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

// The kernel walks the mel rows in 8 groups of 16 (row m = 16 g + lane); kGroupTaps[g] is the largest tap count
// of a row in group g for the 16 kHz / 512-point / 128-bin Slaney filterbank.  The table builder checks the
// filterbank it computes against these bounds, so the kernel can unroll its tap loops completely.
constexpr int kMelGroups = 8;
constexpr int kGroupTaps[kMelGroups] = {2, 2, 2, 3, 4, 6, 9, 12};
constexpr int kGroupTapOffset[kMelGroups + 1] = {0, 2, 4, 6, 9, 13, 19, 28, 40};
constexpr int kMelTapRows = 40;  // sum of kGroupTaps

// Device-resident constant tables, built once on the host.
struct FrontendTables {
    float window[kWin];               // Hann, frontend.rs:161-165
    float2 tw_post[132];              // exp(-2*pi*i*k/512), k = 0..128
    float2 twid[256];                 // exp(-2*pi*i*n2*k1/256) at [k1 * 16 + n2]: twiddles between the two radix-16 passes
    float melw[kMelTapRows * 16];     // [kGroupTapOffset[g] + t][lane] = tap t of row 16 g + lane, times 1/4 (0 past its run)
    int16_t mel_start[kMels];         // first non-zero bin of each row
    float log_floor;                  // ln(2^-24) as the host's logf rounds it: the log-mel value of an empty mel cell
};

// Host-side table construction (frontend_tables.cpp).  `dense_fb`, if not null,
// receives the dense [128 x 257] filterbank.  Returns false if a row has more
// taps than its group's bound or taps that are not contiguous.
bool build_frontend_tables(FrontendTables* t, float* dense_fb);
void hann_window_host(float* w, int n);
void mel_filterbank_host(float* fb, int n_fft, int n_mels, int sample_rate);

inline int64_t frames_for_samples(int64_t n) { return (n + 2 * kPad - kNfft) / kHop + 1; }  // frontend.rs:127

enum SampleFormat : int {
    kSampleF32 = 0,  // mono f32 in [-1, 1], the reference's input contract (src/lib.rs:62-65)
    kSampleI16 = 1,  // 16-bit PCM; converted as value / 32767 in f32 (examples/transcribe_wav.rs:341-347)
};

size_t frontend_smem_bytes();
cudaError_t frontend_configure();
// Clip i is samples [d_clip_start[i], d_clip_start[i] + d_clip_len[i]) of `pcm` (clips may overlap in the PCM
// buffer); its features are written at row d_frame_off[i] of feats.  One launch: a CTA per clip computes the
// log-mel rows and, if `normalize`, the per-feature statistics and the normalised values.
cudaError_t frontend_launch(const void* pcm, SampleFormat fmt, const int64_t* d_clip_start, const int64_t* d_clip_len,
                            const int64_t* d_frame_off, int n_clips, float preemph, const FrontendTables* d_tables,
                            float* feats, bool normalize, cudaStream_t stream);

}  // namespace sb
