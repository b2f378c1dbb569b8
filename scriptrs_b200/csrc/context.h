// Per-GPU context: stream, constant tables, grow-only workspaces, error reporting.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/scriptrs_b200.h"
#include "frontend.h"

namespace sb {

// Thread-local last-error message (sb_last_error()).
void set_error(const std::string& msg);
int32_t fail(sb_status st, const std::string& msg);
int32_t cuda_fail(cudaError_t e, const char* what);

#define SB_CUDA(expr)                                       \
    do {                                                    \
        cudaError_t _e = (expr);                            \
        if (_e != cudaSuccess) return ::sb::cuda_fail(_e, #expr); \
    } while (0)

// Device (or pinned host) buffer that only ever grows.
struct Buffer {
    void* p = nullptr;
    size_t cap = 0;
    bool pinned_host = false;
    cudaError_t ensure(size_t bytes);
    void release();
    template <typename T>
    T* as() const { return static_cast<T*>(p); }
};

// Optional in-situ timing: CUDA events around kernel launches, summed per label.
struct Profiler {
    bool on = false;
    std::vector<cudaEvent_t> pool;
    size_t used = 0;
    struct Rec { const char* name; cudaEvent_t a, b; };
    std::vector<Rec> recs;
    cudaEvent_t take();
    void begin(const char* name, cudaStream_t st);
    void end(cudaStream_t st);
    std::string report();  // synchronises; "name ms launches" per line, then resets
    void release();
};

struct Model;             // encoder + predictor + joint weights (model.h)
struct EncoderWorkspace;  // encoder.h
struct DecodeWorkspace;   // pipeline.cu
struct VadModel;          // vad.h
int32_t model_load(sb_ctx* c, const sb_model_desc* desc, const sb_tensor* tensors, int64_t n_tensors);
// Reads (after the stream `st` has drained up to here) the flag that a kernel raises when a bounded wait runs out;
// clears it and fails with SB_TIMEOUT if it was set.
int32_t take_device_error(sb_ctx* c, cudaStream_t st);

}  // namespace sb

struct sb_ctx {
    int device = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    cudaStream_t copy_stream = nullptr;     // host-to-device PCM pieces, ahead of the kernels that read them
    std::vector<cudaEvent_t> copy_events;  // one per piece, plus one that orders the copies after earlier work
    int sm_count = 0;
    int64_t launches = 0;
    sb::FrontendTables* d_tables = nullptr;
    int* d_error = nullptr;  // set by a kernel whose bounded wait ran out
    // frontend workspaces
    sb::Buffer clip_off, frame_off, pcm_stage, feat_stage, enc_stage;
    sb::Model* model = nullptr;
    sb::VadModel* vad = nullptr;  // voice-activity network of the VAD long-form mode
    int vad_cluster = 8;          // CTAs in the cluster that runs the VAD recurrence (4 or 8)
    cudaStream_t vad_stream = nullptr;       // high priority: the VAD network's recurrences beside the transcription
    cudaStream_t vad_feed_stream = nullptr;  // sample copies and gate inputs of the pass after the one that recurs
    std::vector<cudaEvent_t> vad_events;    // three per pass, plus one that orders the passes after earlier work
    int vad_stream_pass_windows = 49152;   // streamed VAD mode: largest pass (26 minutes of audio)
    int64_t vad_rows_cap = 0;              // streamed VAD mode: encoder frames kept for one decoder run (0 = sized from the recording)
    bool vad_unstreamed = false;           // VAD mode: run the whole network before the first transcription kernel (tests)
    int vad_segment_windows = 131072;  // windows per pass of the VAD network (268 MB of gate inputs)
    sb::Profiler prof;
    bool fp8 = false;             // FP8 e4m3 GEMMs in the Conformer blocks (needs fp8 weights)
    int fp8_mask = 8;             // which GEMMs take the FP8 path: 1 ff up, 2 ff down, 4 QKV, 8 first pointwise
                                  // (default: the subset that keeps the encoder within 5e-2 of the fp32 oracle)
    bool fp8_hidden_amax = false; // FP8 feed-forward: quantise the hidden row by its true maximum (one more pass) instead of a bound
    bool simt_decode = false;     // fp32 CUDA-core decoder (one persistent kernel) instead of the tensor-core steps
    bool simt_attention = false;  // reference implementation of the attention kernel on CUDA cores (tests)
    bool simt_subsample = false;  // fp32 CUDA-core version of the first two sub-sampling stages (tests)
    sb::EncoderWorkspace* enc_ws = nullptr;
    sb::DecodeWorkspace* dec_ws = nullptr;
    size_t workspace_budget = (size_t)48 << 30;  // bytes of encoder intermediates per group of clips (8 h of chunks fit one group)
};
