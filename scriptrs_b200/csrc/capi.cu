// extern "C" layer: context management and the frontend entry points.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <algorithm>
#include <vector>

#include "context.h"
#include "encoder.h"
#include "gemm.h"
#include "host/weights_file.h"
#include "model.h"
#include "pipeline.h"
#include "vad.h"

namespace sb {

static thread_local std::string g_last_error;

void set_error(const std::string& msg) { g_last_error = msg; }

int32_t fail(sb_status st, const std::string& msg) {
    g_last_error = msg;
    return static_cast<int32_t>(st);
}

int32_t cuda_fail(cudaError_t e, const char* what) {
    g_last_error = std::string("CUDA error: ") + cudaGetErrorString(e) + " at " + what;
    return SB_CUDA_ERROR;
}

cudaError_t Buffer::ensure(size_t bytes) {
    if (bytes <= cap) return cudaSuccess;
    if (p) {
        cudaError_t e = pinned_host ? cudaFreeHost(p) : cudaFree(p);
        p = nullptr;
        cap = 0;
        if (e != cudaSuccess) return e;
    }
    size_t want = bytes + bytes / 8 + 256;
    cudaError_t e = pinned_host ? cudaMallocHost(&p, want) : cudaMalloc(&p, want);
    if (e == cudaSuccess) cap = want;
    return e;
}

void Buffer::release() {
    if (p) {
        if (pinned_host) cudaFreeHost(p);
        else cudaFree(p);
    }
    p = nullptr;
    cap = 0;
}

cudaEvent_t Profiler::take() {
    if (used == pool.size()) {
        cudaEvent_t e;
        cudaEventCreate(&e);
        pool.push_back(e);
    }
    return pool[used++];
}
void Profiler::begin(const char* name, cudaStream_t st) {
    if (!on) return;
    Rec r{name, take(), take()};
    cudaEventRecord(r.a, st);
    recs.push_back(r);
}
void Profiler::end(cudaStream_t st) {
    if (!on || recs.empty()) return;
    cudaEventRecord(recs.back().b, st);
}
std::string Profiler::report() {
    std::map<std::string, std::pair<double, long>> sum;
    if (!recs.empty()) cudaEventSynchronize(recs.back().b);
    for (const Rec& r : recs) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) {
            sum[r.name].first += ms;
            sum[r.name].second += 1;
        }
    }
    recs.clear();
    used = 0;
    std::string out;
    char line[160];
    for (auto& kv : sum) {
        std::snprintf(line, sizeof line, "%s %.4f %ld\n", kv.first.c_str(), kv.second.first, kv.second.second);
        out += line;
    }
    return out;
}
void Profiler::release() {
    for (cudaEvent_t e : pool) cudaEventDestroy(e);
    pool.clear();
    recs.clear();
    used = 0;
}

}  // namespace sb

using namespace sb;

void sb_model_free_internal(sb_ctx*);

namespace sb {

// Shared by the public frontend entry points and the chunk pipeline.  Asynchronous on the stream.
int32_t frontend_run(sb_ctx* c, const void* d_pcm, SampleFormat fmt, const int64_t* clip_start, const int64_t* clip_len,
                     int64_t n_clips, float preemphasis, bool normalize, float* d_feats, int64_t* frame_offsets) {
    if (n_clips > (int64_t)1 << 30) return fail(SB_INVALID_ARGUMENT, "too many clips in one call");
    const size_t n1 = static_cast<size_t>(n_clips) + 1;
    std::vector<int64_t> meta(3 * n1);  // starts | lens | frame prefix sums
    int64_t* fo = meta.data() + 2 * n1;
    fo[0] = 0;
    for (int64_t i = 0; i < n_clips; ++i) {
        if (clip_len[i] <= 0) return fail(SB_EMPTY_AUDIO, "audio input was empty");  // frontend.rs:105
        meta[i] = clip_start[i];
        meta[n1 + i] = clip_len[i];
        const int64_t t = frames_for_samples(clip_len[i]);
        if (t > INT32_MAX / 2) return fail(SB_INVALID_ARGUMENT, "clip too long");
        fo[i + 1] = fo[i] + t;
    }
    if (frame_offsets) std::memcpy(frame_offsets, fo, sizeof(int64_t) * n1);
    SB_CUDA(cudaSetDevice(c->device));
    SB_CUDA(c->clip_off.ensure(sizeof(int64_t) * 3 * n1));
    // pageable source: the copy is staged before the call returns, so the vector may go out of scope
    SB_CUDA(cudaMemcpyAsync(c->clip_off.p, meta.data(), sizeof(int64_t) * 3 * n1, cudaMemcpyHostToDevice, c->stream));
    const int64_t* d_meta = c->clip_off.as<int64_t>();
    c->prof.begin("frontend", c->stream);
    cudaError_t e = frontend_launch(d_pcm, fmt, d_meta, d_meta + n1, d_meta + 2 * n1, (int)n_clips, preemphasis,
                                    c->d_tables, d_feats, normalize, c->stream);
    c->prof.end(c->stream);
    if (e == cudaErrorMisalignedAddress)
        return fail(SB_INVALID_ARGUMENT, "the feature buffer must be 16-byte aligned and the PCM buffer aligned to its sample type");
    SB_CUDA(e);
    c->launches += 1;
    return SB_OK;
}

int32_t take_device_error(sb_ctx* c, cudaStream_t st) {
    int err = 0;
    SB_CUDA(cudaMemcpyAsync(&err, c->d_error, sizeof(int), cudaMemcpyDeviceToHost, st));
    SB_CUDA(cudaStreamSynchronize(st));
    if (err) {
        SB_CUDA(cudaMemsetAsync(c->d_error, 0, sizeof(int), st));
        return fail(SB_TIMEOUT, "a bounded device-side wait ran out (kernel aborted cleanly)");
    }
    return SB_OK;
}

}  // namespace sb

extern "C" {

const char* sb_last_error(void) { return g_last_error.c_str(); }

const char* sb_status_string(int32_t status) {
    switch (status) {
        case SB_OK: return "ok";
        case SB_EMPTY_AUDIO: return "audio input was empty";
        case SB_AUDIO_TOO_LONG: return "audio exceeds the single-chunk limit";
        case SB_MISSING_MODEL_ASSET: return "missing model asset";
        case SB_IO: return "i/o error";
        case SB_INVALID_VOCABULARY: return "invalid vocabulary";
        case SB_INVALID_MODEL_OUTPUT: return "invalid model output";
        case SB_BACKEND: return "backend failure";
        case SB_UNSUPPORTED_PLATFORM: return "unsupported platform";
        case SB_CUDA_ERROR: return "CUDA error";
        case SB_TIMEOUT: return "device-side wait timed out";
        case SB_INVALID_ARGUMENT: return "invalid argument";
        case SB_BUFFER_TOO_SMALL: return "buffer too small";
        default: return "unknown status";
    }
}

void sb_default_transcription_config(sb_transcription_config* c) {
    c->sample_rate = 16000;
    c->feature_size = 128;
    c->n_fft = 512;
    c->win_length = 400;
    c->hop_length = 160;
    c->preemphasis = 0.97f;
    c->max_audio_samples = 240000;
    c->samples_per_encoder_frame = 1280;
}

void sb_default_overlap_config(sb_overlap_config* c) {
    c->overlap_seconds = 2.0;
    c->context_samples = 1280;
    c->max_model_samples = 240000;
}

void sb_default_vad_config(sb_vad_config* c) { c->default_threshold = 0.85f; }

void sb_default_vad_segmentation_config(sb_vad_segmentation_config* c) {
    c->min_speech_duration = 0.15;
    c->min_silence_duration = 0.75;
    c->max_speech_duration = 14.0;
    c->speech_padding = 0.1;
    c->silence_threshold_for_split = 0.3f;
    c->has_negative_threshold = 0;
    c->negative_threshold = 0.0f;
    c->negative_threshold_offset = 0.15f;
    c->min_silence_at_max_speech = 0.098;
    c->use_max_possible_silence_at_max_speech = 1;
}

void sb_default_longform_config(sb_longform_config* c) {
    c->mode = 0;
    c->worker_count = 4;
    sb_default_transcription_config(&c->transcription);
    sb_default_vad_config(&c->vad);
    sb_default_vad_segmentation_config(&c->segmentation);
    sb_default_overlap_config(&c->overlap);
}

int32_t sb_ctx_create(int32_t device, sb_ctx** out) {
    if (!out) return fail(SB_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return fail(SB_UNSUPPORTED_PLATFORM, "no CUDA device: this library has no CPU fallback");
    if (device < 0 || device >= count) return fail(SB_INVALID_ARGUMENT, "device index out of range");
    SB_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    SB_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return fail(SB_UNSUPPORTED_PLATFORM, "kernels are built for sm_100a only");
    sb_ctx* c = new sb_ctx();
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    c->pcm_stage.pinned_host = false;
    // any failure from here on destroys the half-built context (sb_ctx_destroy tolerates null members)
    auto bail = [&](int32_t st) {
        sb_ctx_destroy(c);
        return st;
    };
#define SB_CREATE_CUDA(expr)                                            \
    do {                                                                \
        cudaError_t _e = (expr);                                        \
        if (_e != cudaSuccess) return bail(::sb::cuda_fail(_e, #expr)); \
    } while (0)
    SB_CREATE_CUDA(cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking));
    c->stream = c->own_stream;
    FrontendTables host_tables;
    if (!build_frontend_tables(&host_tables, nullptr))
        return bail(fail(SB_INVALID_MODEL_OUTPUT, "mel filterbank rows exceed the tap budget"));
    SB_CREATE_CUDA(cudaMalloc(&c->d_tables, sizeof(FrontendTables)));
    SB_CREATE_CUDA(cudaMemcpy(c->d_tables, &host_tables, sizeof(FrontendTables), cudaMemcpyHostToDevice));
    SB_CREATE_CUDA(frontend_configure());
    SB_CREATE_CUDA(cudaMalloc(&c->d_error, sizeof(int)));
    SB_CREATE_CUDA(cudaMemset(c->d_error, 0, sizeof(int)));
    const char* why = nullptr;
    cudaError_t ge = gemm_configure(&why);
    if (ge != cudaSuccess)
        return bail(fail(SB_CUDA_ERROR, std::string("GEMM set-up failed: ") + (why ? why : cudaGetErrorString(ge))));
    SB_CREATE_CUDA(encoder_configure());
#undef SB_CREATE_CUDA
    c->enc_ws = new EncoderWorkspace();
    *out = c;
    return SB_OK;
}

void sb_ctx_destroy(sb_ctx* c) {
    if (!c) return;
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
    sb_model_free_internal(c);
    if (c->vad) {
        c->vad->release();
        delete c->vad;
    }
    c->clip_off.release();
    c->frame_off.release();
    c->pcm_stage.release();
    c->feat_stage.release();
    c->enc_stage.release();
    if (c->d_tables) cudaFree(c->d_tables);
    if (c->d_error) cudaFree(c->d_error);
    c->prof.release();
    for (cudaEvent_t e : c->copy_events) cudaEventDestroy(e);
    for (cudaEvent_t e : c->vad_events) cudaEventDestroy(e);
    if (c->vad_stream) cudaStreamDestroy(c->vad_stream);
    if (c->vad_feed_stream) cudaStreamDestroy(c->vad_feed_stream);
    if (c->copy_stream) cudaStreamDestroy(c->copy_stream);
    if (c->own_stream) cudaStreamDestroy(c->own_stream);
    delete c;
}

int32_t sb_ctx_set_stream(sb_ctx* c, void* stream) {
    if (!c) return fail(SB_INVALID_ARGUMENT, "ctx is null");
    c->stream = stream ? static_cast<cudaStream_t>(stream) : c->own_stream;
    return SB_OK;
}

int32_t sb_ctx_synchronize(sb_ctx* c) {
    if (!c) return fail(SB_INVALID_ARGUMENT, "ctx is null");
    SB_CUDA(cudaSetDevice(c->device));
    SB_CUDA(cudaStreamSynchronize(c->stream));
    int err = 0;
    SB_CUDA(cudaMemcpy(&err, c->d_error, sizeof(int), cudaMemcpyDeviceToHost));
    if (err) {
        SB_CUDA(cudaMemset(c->d_error, 0, sizeof(int)));
        return fail(SB_TIMEOUT, "a bounded device-side wait ran out (kernel aborted cleanly)");
    }
    return SB_OK;
}

int64_t sb_ctx_kernel_launches(const sb_ctx* c) { return c ? c->launches : 0; }

int32_t sb_ctx_set_option(sb_ctx* c, const char* name, int64_t value) {
    if (!c || !name) return fail(SB_INVALID_ARGUMENT, "null argument");
    const std::string n(name);
    if (n == "simt_attention") c->simt_attention = value != 0;
    else if (n == "simt_subsample") c->simt_subsample = value != 0;
    else if (n == "simt_decode") c->simt_decode = value != 0;
    else if (n == "vad_segment_windows") {
        if (value < 1 || value > (1 << 22)) return fail(SB_INVALID_ARGUMENT, "vad_segment_windows must be in [1, 4194304]");
        c->vad_segment_windows = (int)value;
    }
    else if (n == "vad_unstreamed") c->vad_unstreamed = value != 0;
    else if (n == "vad_stream_pass_windows") {
        if (value < 1 || value > (1 << 22)) return fail(SB_INVALID_ARGUMENT, "vad_stream_pass_windows must be in [1, 4194304]");
        c->vad_stream_pass_windows = (int)value;
    }
    else if (n == "vad_rows_cap") c->vad_rows_cap = value < 0 ? 0 : value;
    else if (n == "vad_cluster") {
        if (value != 4 && value != 8) return fail(SB_INVALID_ARGUMENT, "vad_cluster must be 4 or 8");
        c->vad_cluster = (int)value;
    }
    else if (n == "gemm_pair_tiles") sb::gemm_set_pair_tiles((int)(value < 0 ? 0 : (value > 2 ? 2 : value)));
    else if (n == "fp8") {
        if (value && (!c->model || !c->model->has_fp8))
            return fail(SB_MISSING_MODEL_ASSET, "the model was loaded without fp8 weights");
        c->fp8 = value != 0;
    }
    else if (n == "fp8_mask") c->fp8_mask = (int)(value & 15);
    else if (n == "fp8_hidden_amax") c->fp8_hidden_amax = value != 0;
    else if (n == "test_raise_device_error") {
        // host-side fault injection for tests: sets the flag a kernel would set when a bounded wait runs out
        SB_CUDA(cudaSetDevice(c->device));
        SB_CUDA(cudaMemsetAsync(c->d_error, value ? 1 : 0, sizeof(int), c->stream));
    }
    else if (n == "workspace_budget_mb" && value > 0) c->workspace_budget = (size_t)value << 20;
    else return fail(SB_INVALID_ARGUMENT, "unknown option: " + n);
    return SB_OK;
}

int32_t sb_ctx_set_profiling(sb_ctx* c, int32_t on) {
    if (!c) return fail(SB_INVALID_ARGUMENT, "ctx is null");
    c->prof.on = on != 0;
    return SB_OK;
}

int64_t sb_ctx_profile_report(sb_ctx* c, char* buf, int64_t cap) {
    if (!c) return 0;
    cudaSetDevice(c->device);
    const std::string r = c->prof.report();
    if (buf && cap > 0) {
        const size_t n = std::min<size_t>(r.size(), (size_t)cap - 1);
        std::memcpy(buf, r.data(), n);
        buf[n] = 0;
    }
    return (int64_t)r.size();
}

int32_t sb_frontend_tables(float* window, float* filterbank) {
    if (window) hann_window_host(window, kWin);
    if (filterbank) mel_filterbank_host(filterbank, kNfft, kMels, kSampleRate);
    return SB_OK;
}

int64_t sb_frontend_num_frames(int64_t n_samples) { return n_samples <= 0 ? 0 : frames_for_samples(n_samples); }

static int32_t frontend_device_any(sb_ctx* c, const void* d_pcm, SampleFormat fmt, const int64_t* clip_offsets,
                                   int64_t n_clips, float preemphasis, int32_t normalize, float* d_feats,
                                   int64_t* frame_offsets) {
    if (!c || !clip_offsets || !d_pcm || !d_feats) return fail(SB_INVALID_ARGUMENT, "null argument");
    if (n_clips <= 0) return fail(SB_EMPTY_AUDIO, "audio input was empty");
    std::vector<int64_t> start(static_cast<size_t>(n_clips)), len(static_cast<size_t>(n_clips));
    for (int64_t i = 0; i < n_clips; ++i) {
        start[i] = clip_offsets[i];
        len[i] = clip_offsets[i + 1] - clip_offsets[i];
    }
    return frontend_run(c, d_pcm, fmt, start.data(), len.data(), n_clips, preemphasis, normalize != 0, d_feats,
                        frame_offsets);
}

int32_t sb_frontend_device(sb_ctx* c, const float* d_pcm, const int64_t* clip_offsets, int64_t n_clips,
                           float preemphasis, int32_t normalize, float* d_feats, int64_t* frame_offsets) {
    return frontend_device_any(c, d_pcm, kSampleF32, clip_offsets, n_clips, preemphasis, normalize, d_feats, frame_offsets);
}

int32_t sb_frontend_device_i16(sb_ctx* c, const int16_t* d_pcm, const int64_t* clip_offsets, int64_t n_clips,
                               float preemphasis, int32_t normalize, float* d_feats, int64_t* frame_offsets) {
    return frontend_device_any(c, d_pcm, kSampleI16, clip_offsets, n_clips, preemphasis, normalize, d_feats, frame_offsets);
}

int32_t sb_frontend_host(sb_ctx* c, const float* pcm, const int64_t* clip_offsets, int64_t n_clips,
                         float preemphasis, int32_t normalize, float* feats, int64_t* frame_offsets) {
    if (!c || !clip_offsets || !pcm || !feats) return fail(SB_INVALID_ARGUMENT, "null argument");
    if (n_clips <= 0) return fail(SB_EMPTY_AUDIO, "audio input was empty");
    const int64_t base = clip_offsets[0];
    const int64_t total = clip_offsets[n_clips] - base;
    if (total <= 0) return fail(SB_EMPTY_AUDIO, "audio input was empty");
    int64_t frames = 0;
    std::vector<int64_t> rel(static_cast<size_t>(n_clips) + 1);
    for (int64_t i = 0; i <= n_clips; ++i) rel[i] = clip_offsets[i] - base;
    for (int64_t i = 0; i < n_clips; ++i) {
        const int64_t n = rel[i + 1] - rel[i];
        if (n <= 0) return fail(SB_EMPTY_AUDIO, "audio input was empty");
        frames += frames_for_samples(n);
    }
    SB_CUDA(cudaSetDevice(c->device));
    SB_CUDA(c->pcm_stage.ensure(sizeof(float) * static_cast<size_t>(total)));
    SB_CUDA(c->feat_stage.ensure(sizeof(float) * kMels * static_cast<size_t>(frames)));
    SB_CUDA(cudaMemcpyAsync(c->pcm_stage.p, pcm + base, sizeof(float) * static_cast<size_t>(total),
                            cudaMemcpyHostToDevice, c->stream));
    int32_t st = sb_frontend_device(c, c->pcm_stage.as<float>(), rel.data(), n_clips, preemphasis, normalize,
                                    c->feat_stage.as<float>(), frame_offsets);
    if (st != SB_OK) return st;
    SB_CUDA(cudaMemcpyAsync(feats, c->feat_stage.p, sizeof(float) * kMels * static_cast<size_t>(frames),
                            cudaMemcpyDeviceToHost, c->stream));
    SB_CUDA(cudaStreamSynchronize(c->stream));
    return SB_OK;
}

int32_t sb_model_load(sb_ctx* c, const sb_model_desc* desc, const sb_tensor* tensors, int64_t n_tensors) {
    return model_load(c, desc, tensors, n_tensors);
}

int32_t sb_model_load_file(sb_ctx* c, const sb_model_desc* desc, const char* path, const char* name_prefix) {
    if (!c || !desc || !path) return fail(SB_INVALID_ARGUMENT, "null argument");
    WeightFile wf;
    bool missing = false;
    const std::string err = weight_file_open(path, &wf, &missing);
    if (!err.empty()) return fail(missing ? SB_MISSING_MODEL_ASSET : SB_IO, err);  // models.rs:53-66
    const std::string prefix = name_prefix ? name_prefix : "";
    std::vector<std::string> names;
    std::vector<sb_tensor> tensors;
    names.reserve(wf.entries.size());
    int max_layer = -1;
    for (auto& kv : wf.entries) {
        if (kv.first.compare(0, prefix.size(), prefix) != 0) continue;
        names.push_back(kv.first.substr(prefix.size()));
        const std::string& n = names.back();
        if (n.compare(0, 7, "layers.") == 0) max_layer = std::max(max_layer, std::atoi(n.c_str() + 7));
    }
    size_t k = 0;
    for (auto& kv : wf.entries) {
        if (kv.first.compare(0, prefix.size(), prefix) != 0) continue;
        const float* data = wf.as_f32(kv.first);
        tensors.push_back(sb_tensor{names[k].c_str(), data, kv.second.numel()});
        ++k;
    }
    sb_model_desc d = *desc;
    if (d.encoder_layers < 0) d.encoder_layers = max_layer + 1;  // as many Conformer blocks as the file holds
    return model_load(c, &d, tensors.data(), (int64_t)tensors.size());
}

int32_t sb_vad_load(sb_ctx* c, const sb_tensor* tensors, int64_t n_tensors) {
    if (!c || n_tensors < 0 || (n_tensors > 0 && !tensors)) return fail(SB_INVALID_ARGUMENT, "null argument");
    return vad_load(c, tensors, n_tensors);
}

int32_t sb_vad_load_file(sb_ctx* c, const char* path) {
    if (!c || !path) return fail(SB_INVALID_ARGUMENT, "null argument");
    WeightFile wf;
    bool missing = false;
    const std::string err = weight_file_open(path, &wf, &missing);
    if (!err.empty()) return fail(missing ? SB_MISSING_MODEL_ASSET : SB_IO, err);  // models.rs:68-78
    std::vector<sb_tensor> tensors;
    for (auto& kv : wf.entries) tensors.push_back(sb_tensor{kv.first.c_str(), wf.as_f32(kv.first), kv.second.numel()});
    return vad_load(c, tensors.data(), (int64_t)tensors.size());
}

int32_t sb_vad_process_device(sb_ctx* c, const float* d_audio, int64_t n_samples, float* d_prob) {
    if (!c || n_samples < 0 || (n_samples > 0 && (!d_audio || !d_prob))) return fail(SB_INVALID_ARGUMENT, "null argument");
    return vad_process_device(c, d_audio, n_samples, d_prob);
}

int32_t sb_vad_process(sb_ctx* c, const float* audio, int64_t n_samples, float* prob, int64_t cap, int64_t* n_prob) {
    if (!c || !n_prob || n_samples < 0 || (n_samples > 0 && !audio)) return fail(SB_INVALID_ARGUMENT, "null argument");
    if (!c->vad) return fail(SB_MISSING_MODEL_ASSET, "missing model asset: vad network (sb_vad_load)");
    const int64_t n = n_samples > 0 ? (n_samples + kVadWindow - 1) / kVadWindow : 0;
    *n_prob = n;
    if (n == 0) return SB_OK;  // vad.rs:65-67
    if (!prob || cap < n) return fail(SB_BUFFER_TOO_SMALL, "probability buffer too small");
    SB_CUDA(cudaSetDevice(c->device));
    VadModel& m = *c->vad;
    SB_CUDA(m.audio.ensure(sizeof(float) * (size_t)n_samples));
    SB_CUDA(m.prob.ensure(sizeof(float) * (size_t)n));
    SB_CUDA(cudaMemcpyAsync(m.audio.p, audio, sizeof(float) * (size_t)n_samples, cudaMemcpyHostToDevice, c->stream));
    const int32_t s = vad_process_device(c, m.audio.as<float>(), n_samples, m.prob.as<float>());
    if (s != SB_OK) return s;
    SB_CUDA(cudaMemcpyAsync(prob, m.prob.p, sizeof(float) * (size_t)n, cudaMemcpyDeviceToHost, c->stream));
    return take_device_error(c, c->stream);  // synchronises; a recurrence that gave up waiting fails the call
}

int64_t sb_weights_file_list(const char* path, char* buf, int64_t cap) {
    if (!path) return -(int64_t)fail(SB_INVALID_ARGUMENT, "null argument");
    WeightFile wf;
    bool missing = false;
    const std::string err = weight_file_open(path, &wf, &missing);
    if (!err.empty()) return -(int64_t)fail(missing ? SB_MISSING_MODEL_ASSET : SB_IO, err);
    std::string out;
    for (auto& kv : wf.entries) {
        out += kv.first + " " + kv.second.dtype + " ";
        for (size_t i = 0; i < kv.second.shape.size(); ++i) out += (i ? "x" : "") + std::to_string(kv.second.shape[i]);
        if (kv.second.shape.empty()) out += "scalar";
        out += "\n";
    }
    if (buf && cap > 0) {
        const size_t n = std::min<size_t>(out.size(), (size_t)cap - 1);
        std::memcpy(buf, out.data(), n);
        buf[n] = 0;
    }
    return (int64_t)out.size();
}

int64_t sb_encoder_num_frames(int64_t feature_frames) {
    return feature_frames <= 0 ? 0 : encoder_out_frames((int)feature_frames);
}

int32_t sb_encode_device(sb_ctx* c, const float* d_feats, const int64_t* frame_offsets, int64_t n_clips,
                         float* d_out, int64_t* enc_offsets) {
    if (!c || !d_feats || !frame_offsets || !d_out) return fail(SB_INVALID_ARGUMENT, "null argument");
    if (!c->model || !c->model->has_encoder) return fail(SB_MISSING_MODEL_ASSET, "no encoder weights loaded");
    if (n_clips <= 0) return fail(SB_EMPTY_AUDIO, "audio input was empty");
    if (n_clips > 65535) return fail(SB_INVALID_ARGUMENT, "at most 65535 clips per call");
    for (int64_t i = 0; i < n_clips; ++i) {
        const int64_t t = frame_offsets[i + 1] - frame_offsets[i];
        if (t <= 0) return fail(SB_EMPTY_AUDIO, "clip without feature frames");
        if (t > 1501)  // model.rs:259-264: feature frames beyond the encoder's window
            return fail(SB_INVALID_MODEL_OUTPUT, "feature frame count " + std::to_string(t) + " exceeded encoder target 1501");
    }
    SB_CUDA(cudaSetDevice(c->device));
    std::vector<int> eo(static_cast<size_t>(n_clips) + 1);
    cudaError_t e = encoder_forward(c, *c->model, d_feats, frame_offsets, (int)n_clips, d_out, eo.data(), *c->enc_ws,
                                    c->workspace_budget);
    SB_CUDA(e);
    if (enc_offsets)
        for (int64_t i = 0; i <= n_clips; ++i) enc_offsets[i] = eo[i];
    return SB_OK;
}

int32_t sb_gemm(sb_ctx* c, const void* d_a, const void* d_w, const float* d_bias, const float* d_row_scale,
                const float* d_col_scale, void* d_out, int64_t M, int64_t N, int64_t K, int32_t fp8, int32_t act,
                int32_t out_mode, float alpha) {
    if (!c || !d_a || !d_w || !d_out) return fail(SB_INVALID_ARGUMENT, "null argument");
    if (M < 0 || N <= 0 || K <= 0 || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX)
        return fail(SB_INVALID_ARGUMENT, "bad GEMM shape");
    SB_CUDA(cudaSetDevice(c->device));
    GemmArgs g{};
    g.a = d_a; g.w = d_w; g.bias = d_bias; g.row_scale = d_row_scale; g.col_scale = d_col_scale; g.out = d_out;
    g.M = (int)M; g.N = (int)N; g.K = (int)K; g.ldo = (int)N; g.act = act; g.out_mode = out_mode; g.alpha = alpha;
    g.fp8 = fp8 != 0;
    cudaError_t e = gemm_launch(g, c->sm_count, c->d_error, c->stream);
    if (e == cudaErrorInvalidValue) return fail(SB_INVALID_ARGUMENT, "GEMM shape or alignment not supported");
    SB_CUDA(e);
    if (M > 0) c->launches += 1;
    return SB_OK;
}

}  // extern "C"
