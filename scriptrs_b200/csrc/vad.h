// Streaming voice-activity network of the VAD long-form mode (vad.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "context.h"

namespace sb {

constexpr int kVadWindow = 512;    // new samples per step, constants.rs:7
constexpr int kVadContext = 64;    // samples of the window before, constants.rs:9
constexpr int kVadState = 128;     // LSTM width, constants.rs:11
constexpr int kVadInput = kVadWindow + kVadContext;  // 576, coreml.rs:195
constexpr int kVadPadded = kVadInput + 64;           // reflected on the right
constexpr int kVadFilter = 256;    // STFT filter length, stride 128 -> 4 frames per window
constexpr int kVadBins = 129;
constexpr int kVadFrames = 4;
constexpr int kVadGates = 4 * kVadState;

// Device copies of the weights in the layouts the kernels read.
struct VadModel {
    float* basis = nullptr;   // [258 x 256]: rows 0..128 real, 129..257 imaginary
    float* w1 = nullptr;      // [129 x 3 x 128]  (in channel, tap, out channel)
    float* b1 = nullptr;      // [128]
    float* w2 = nullptr;      // [128 x 3 x 64]
    float* b2 = nullptr;      // [64]
    float* w3 = nullptr;      // [64 x 3 x 64]
    float* b3 = nullptr;      // [64]
    float* w4 = nullptr;      // [64 x 128]: centre tap only, the one that meets data when the sequence has one step
    float* b4 = nullptr;      // [128]
    float* wih = nullptr;     // [128 x 512]: (input, gate row'), row' = 4 * unit + gate
    float* bsum = nullptr;    // [512]: bias_ih + bias_hh, rows permuted the same way
    float* whh = nullptr;     // [512 x 128]: rows permuted the same way
    float* wout = nullptr;    // [128]
    float bout = 0.0f;
    // work buffers for one segment of windows, and the state carried between segments
    Buffer gx[2], hout, state, audio, prob;  // gate inputs of a pass (two, so that a pass can be prepared while the one before recurs)
    Buffer host_prob;  // pinned: the probabilities on their way to the planner
    void release();
};

int32_t vad_load(sb_ctx* c, const sb_tensor* tensors, int64_t n_tensors);
cudaError_t vad_configure();
// One probability per window of d_audio[0, n_samples) into d_prob (device pointers), on the context's stream.
int32_t vad_process_device(sb_ctx* c, const float* d_audio, int64_t n_samples, float* d_prob);
// The same in passes chosen by the caller.  vad_begin sizes the work buffers for the largest pass and zeroes the
// recurrent state (stream-ordered on st).  vad_encode_pass computes the gate inputs of windows [first, first + n)
// into buffer `buf`; vad_recur_pass runs the recurrence over that buffer and writes d_prob[first, first + n).  The
// recurrences must run in window order on one stream; an encode pass may run on another stream while the pass before
// it recurs, if the caller orders it after the recurrence that last read its buffer.
int32_t vad_begin(sb_ctx* c, int64_t max_pass_windows, cudaStream_t st, bool two_buffers);
int32_t vad_encode_pass(sb_ctx* c, cudaStream_t st, const float* d_audio, int64_t n_samples, int64_t first, int n, int buf);
int32_t vad_recur_pass(sb_ctx* c, cudaStream_t st, int64_t first, int n, int buf, float* d_prob);
// The device copy of the recording that the last sb_vad_process call on this context made (null if none).
const float* vad_resident_audio(const sb_ctx* c);

}  // namespace sb
