// extern "C" layer, part 2: host logic (planner, offsets, merge, text), result objects and the
// chunk / single-chunk / long-form pipelines.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "context.h"
#include "encoder.h"
#include "host/longform.h"
#include "model.h"
#include "pipeline.h"
#include "vad.h"

struct sb_vocab { sb::Vocabulary v; };
struct sb_result { sb::TranscriptionResult r; };
struct sb_raw_batch { std::vector<sb::RawTokens> items; };

namespace sb {

namespace {

RawTokens raw_from_arrays(const uint32_t* tok, const int64_t* frm, const int64_t* dur, const float* conf, int64_t a,
                          int64_t b) {
    RawTokens r;
    r.token_ids.assign(tok + a, tok + b);
    r.frame_indices.assign(frm + a, frm + b);
    r.durations.assign(dur + a, dur + b);
    r.confidences.assign(conf + a, conf + b);
    return r;
}

// Frontend -> encoder -> decoder for a set of tasks over one host PCM buffer; the reference's
// transcribe_task (src/long_form.rs:584-592) for a whole batch at once.
int32_t transcribe_tasks(sb_ctx* c, const void* pcm_any, int64_t n_samples, const sb_chunk_task* tasks, int64_t n_tasks,
                         const sb_transcription_config& cfg, std::vector<RawTokens>* out, bool pcm_on_device = false,
                         SampleFormat fmt = kSampleF32) {
    const size_t esz = fmt == kSampleI16 ? sizeof(int16_t) : sizeof(float);
    const char* pcm = static_cast<const char*>(pcm_any);
    out->clear();
    if (n_tasks == 0) return SB_OK;
    if (!c->model || !c->model->has_encoder || !c->model->has_decoder)
        return fail(SB_MISSING_MODEL_ASSET, "encoder and decoder weights must be loaded first");
    int64_t lo = n_samples, hi = 0;
    for (int64_t i = 0; i < n_tasks; ++i) {
        const sb_chunk_task& t = tasks[i];
        if (t.audio_start < 0 || t.audio_end > n_samples || t.audio_end < t.audio_start)
            return fail(SB_INVALID_ARGUMENT, "task range outside the audio");
        const int64_t len = t.audio_end - t.audio_start;
        if (len == 0) return fail(SB_EMPTY_AUDIO, "audio input was empty");  // pipeline.rs:202
        if (len > cfg.max_audio_samples) {                                      // pipeline.rs:205-210
            char msg[160];
            std::snprintf(msg, sizeof msg, "audio exceeds the single-chunk limit: actual=%.2fs max=%.2fs",
                          (double)len / (double)cfg.sample_rate, (double)cfg.max_audio_samples / (double)cfg.sample_rate);
            return fail(SB_AUDIO_TOO_LONG, msg);
        }
        lo = std::min(lo, t.audio_start);
        hi = std::max(hi, t.audio_end);
    }
    SB_CUDA(cudaSetDevice(c->device));
    cudaStream_t st = c->stream;
    std::vector<int64_t> start(n_tasks), len(n_tasks), fo(n_tasks + 1), eo(n_tasks + 1);
    int64_t frames = 0, enc_rows = 0, max_enc = 0;
    bool ordered = true;  // tasks run left to right through the audio (what the planner produces)
    for (int64_t i = 0; i < n_tasks; ++i) {
        start[i] = tasks[i].audio_start - lo;
        len[i] = tasks[i].audio_end - tasks[i].audio_start;
        const int64_t t = frames_for_samples(len[i]);
        frames += t;
        const int64_t e = encoder_out_frames((int)t);
        enc_rows += e;
        max_enc = std::max(max_enc, e);
        if (i > 0 && (tasks[i].audio_start < tasks[i - 1].audio_start || tasks[i].audio_end < tasks[i - 1].audio_end))
            ordered = false;
    }
    SB_CUDA(c->feat_stage.ensure(sizeof(float) * kMels * (size_t)frames));
    SB_CUDA(c->enc_stage.ensure(sizeof(float) * kDModel * (size_t)enc_rows));
    if (n_tasks > 65535) return fail(SB_INVALID_ARGUMENT, "more than 65535 tasks in one batch");
    // Host PCM goes to the device in pieces on a second stream, so that all but the first piece's copy overlaps the
    // kernels of the pieces before it; frontend and encoder run piece by piece, the decoder once over everything.
    // The first piece is small (1/16 or 1/8 of the tasks: little copy time exposed), the last one large (3/4 or 7/8:
    // the GEMMs keep their large row counts); at PCIe rates each later copy finishes well inside the earlier pieces'
    // compute.
    const void* d_pcm = pcm + (size_t)lo * esz;
    int n_pieces = 1;
    if (!pcm_on_device) {
        SB_CUDA(c->pcm_stage.ensure(esz * (size_t)(hi - lo)));
        d_pcm = c->pcm_stage.p;
        // three pieces for large batches, two (1/8 + 7/8) for medium ones: at 280 tasks the single copy of 230 MB is
        // 4-5 ms of exposed time, the second set of launches costs about 1 ms
        if (ordered && n_tasks >= 512) n_pieces = 3;
        else if (ordered && n_tasks >= 64) n_pieces = 2;
        if (!c->copy_stream) SB_CUDA(cudaStreamCreateWithFlags(&c->copy_stream, cudaStreamNonBlocking));
        while ((int)c->copy_events.size() < n_pieces + 1) {
            cudaEvent_t ev;
            SB_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
            c->copy_events.push_back(ev);
        }
        // the staging buffer may still be read by kernels of an earlier call
        SB_CUDA(cudaEventRecord(c->copy_events[n_pieces], st));
        SB_CUDA(cudaStreamWaitEvent(c->copy_stream, c->copy_events[n_pieces], 0));
    }
    std::vector<int> eoi(n_tasks + 1);
    fo[0] = 0;
    eo[0] = 0;
    int64_t copied_to = lo;
    for (int p = 0; p < n_pieces; ++p) {
        // piece boundaries at 0, 1/16, 4/16, 1 of the task list (one piece: everything)
        static const int kCut3[4] = {0, 1, 4, 16}, kCut2[3] = {0, 2, 16}, kCut1[2] = {0, 16};
        const int* cut = n_pieces == 3 ? kCut3 : (n_pieces == 2 ? kCut2 : kCut1);
        const int64_t i0 = n_tasks * cut[p] / 16;
        const int64_t i1 = n_tasks * cut[p + 1] / 16;
        if (i1 <= i0) continue;
        if (!pcm_on_device) {
            const int64_t end = (p == n_pieces - 1) ? hi : tasks[i1 - 1].audio_end;
            if (end > copied_to)
                SB_CUDA(cudaMemcpyAsync(c->pcm_stage.as<char>() + (size_t)(copied_to - lo) * esz, pcm + (size_t)copied_to * esz,
                                        esz * (size_t)(end - copied_to), cudaMemcpyHostToDevice, c->copy_stream));
            copied_to = std::max(copied_to, end);
            SB_CUDA(cudaEventRecord(c->copy_events[p], c->copy_stream));
            SB_CUDA(cudaStreamWaitEvent(st, c->copy_events[p], 0));
        }
        std::vector<int64_t> rel(i1 - i0 + 1);
        int32_t s = frontend_run(c, d_pcm, fmt, start.data() + i0, len.data() + i0, i1 - i0, cfg.preemphasis, true,
                                 c->feat_stage.as<float>() + (size_t)fo[i0] * kMels, rel.data());
        if (s != SB_OK) return s;
        for (int64_t k = 1; k <= i1 - i0; ++k) fo[i0 + k] = fo[i0] + rel[k];
        cudaError_t e = encoder_forward(c, *c->model, c->feat_stage.as<float>() + (size_t)fo[i0] * kMels, rel.data(),
                                        (int)(i1 - i0), c->enc_stage.as<float>() + (size_t)eo[i0] * kDModel,
                                        eoi.data() + i0, *c->enc_ws, c->workspace_budget);
        SB_CUDA(e);
        // encoder_forward writes offsets relative to its first clip
        const int64_t ebase = eo[i0];
        for (int64_t k = 1; k <= i1 - i0; ++k) eo[i0 + k] = ebase + eoi[i0 + k];
    }
    const int64_t max_tokens = std::max<int64_t>(1, kMaxSymbols * max_enc);
    std::vector<uint32_t> tok((size_t)n_tasks * max_tokens);
    std::vector<int64_t> frm((size_t)n_tasks * max_tokens), dur((size_t)n_tasks * max_tokens), cnt(n_tasks);
    std::vector<float> conf((size_t)n_tasks * max_tokens);
    int32_t s = tdt_decode(c, c->enc_stage.as<float>(), eo.data(), n_tasks, max_tokens, tok.data(), frm.data(),
                           dur.data(), conf.data(), cnt.data(), nullptr, 0, nullptr);
    if (s != SB_OK) return s;
    out->resize(n_tasks);
    for (int64_t i = 0; i < n_tasks; ++i) {
        const int64_t o = i * max_tokens;
        (*out)[i] = raw_from_arrays(tok.data(), frm.data(), dur.data(), conf.data(), o, o + cnt[i]);
        // pipeline.rs:132-136
        apply_time_offsets((*out)[i], tasks[i].global_sample_offset / cfg.samples_per_encoder_frame,
                           tasks[i].context_samples / cfg.samples_per_encoder_frame);
    }
    return SB_OK;
}

// Tasks that arrive in pieces over one recording that is resident on the GPU: every piece goes through the
// frontend and the encoder as it arrives (asynchronously on the context's stream), the decoder runs once over all
// pieces' encoder frames at the end.  transcribe_tasks for a plan that is still growing.
struct PieceRun {
    sb_ctx* c;
    const float* d_pcm;  // the whole recording, device memory
    int64_t n_samples;
    sb_transcription_config cfg;
    std::vector<sb_chunk_task> tasks;  // all tasks so far
    std::vector<RawTokens> raws;       // decoded tasks, in task order (a prefix of `tasks`)
    std::vector<int64_t> eo{0};        // encoder frame offsets of the tasks that wait for the decoder
    int64_t max_enc = 0, cap_rows = 0;

    int32_t begin(int64_t rows_hint) {
        cap_rows = rows_hint;
        SB_CUDA(cudaSetDevice(c->device));
        SB_CUDA(c->enc_stage.ensure(sizeof(float) * kDModel * (size_t)cap_rows));
        return SB_OK;
    }

    int32_t decode_pending() {
        const int64_t n = (int64_t)eo.size() - 1;
        if (n == 0) return SB_OK;
        const int64_t first = (int64_t)raws.size();
        const int64_t max_tokens = std::max<int64_t>(1, kMaxSymbols * max_enc);
        std::vector<uint32_t> tok((size_t)n * max_tokens);
        std::vector<int64_t> frm((size_t)n * max_tokens), dur((size_t)n * max_tokens), cnt(n);
        std::vector<float> conf((size_t)n * max_tokens);
        int32_t s = tdt_decode(c, c->enc_stage.as<float>(), eo.data(), n, max_tokens, tok.data(), frm.data(), dur.data(),
                               conf.data(), cnt.data(), nullptr, 0, nullptr);
        if (s != SB_OK) return s;
        for (int64_t i = 0; i < n; ++i) {
            const int64_t o = i * max_tokens;
            raws.push_back(raw_from_arrays(tok.data(), frm.data(), dur.data(), conf.data(), o, o + cnt[i]));
            const sb_chunk_task& t = tasks[(size_t)(first + i)];
            apply_time_offsets(raws.back(), t.global_sample_offset / cfg.samples_per_encoder_frame,
                               t.context_samples / cfg.samples_per_encoder_frame);  // pipeline.rs:132-136
        }
        eo.assign(1, 0);
        max_enc = 0;
        return SB_OK;
    }

    int32_t add(const sb_chunk_task* t, int64_t n) {
        if (n == 0) return SB_OK;
        if (!c->model || !c->model->has_encoder || !c->model->has_decoder)
            return fail(SB_MISSING_MODEL_ASSET, "encoder and decoder weights must be loaded first");
        std::vector<int64_t> start(n), len(n), rel(n + 1);
        int64_t frames = 0, rows = 0;
        for (int64_t i = 0; i < n; ++i) {
            if (t[i].audio_start < 0 || t[i].audio_end > n_samples || t[i].audio_end < t[i].audio_start)
                return fail(SB_INVALID_ARGUMENT, "task range outside the audio");
            start[i] = t[i].audio_start;
            len[i] = t[i].audio_end - t[i].audio_start;
            if (len[i] == 0) return fail(SB_EMPTY_AUDIO, "audio input was empty");  // pipeline.rs:202
            if (len[i] > cfg.max_audio_samples) {                                    // pipeline.rs:205-210
                char msg[160];
                std::snprintf(msg, sizeof msg, "audio exceeds the single-chunk limit: actual=%.2fs max=%.2fs",
                              (double)len[i] / (double)cfg.sample_rate, (double)cfg.max_audio_samples / (double)cfg.sample_rate);
                return fail(SB_AUDIO_TOO_LONG, msg);
            }
            const int64_t f = frames_for_samples(len[i]);
            frames += f;
            const int64_t e = encoder_out_frames((int)f);
            rows += e;
            max_enc = std::max(max_enc, e);
        }
        if (n > 65535) return fail(SB_INVALID_ARGUMENT, "more than 65535 tasks in one piece");
        SB_CUDA(cudaSetDevice(c->device));
        if (eo.back() + rows > cap_rows) {  // the encoder frames kept for the decoder are full: decode what is there
            int32_t s = decode_pending();
            if (s != SB_OK) return s;
            for (int64_t i = 0; i < n; ++i) max_enc = std::max<int64_t>(max_enc, encoder_out_frames((int)frames_for_samples(len[i])));
            if (rows > cap_rows) {
                cap_rows = rows;
                SB_CUDA(c->enc_stage.ensure(sizeof(float) * kDModel * (size_t)cap_rows));
            }
        }
        SB_CUDA(c->feat_stage.ensure(sizeof(float) * kMels * (size_t)frames));
        int32_t s = frontend_run(c, d_pcm, kSampleF32, start.data(), len.data(), n, cfg.preemphasis, true,
                                 c->feat_stage.as<float>(), rel.data());
        if (s != SB_OK) return s;
        std::vector<int> eoi(n + 1);
        SB_CUDA(encoder_forward(c, *c->model, c->feat_stage.as<float>(), rel.data(), (int)n,
                                c->enc_stage.as<float>() + (size_t)eo.back() * kDModel, eoi.data(), *c->enc_ws,
                                c->workspace_budget));
        const int64_t base = eo.back();
        for (int64_t k = 1; k <= n; ++k) eo.push_back(base + eoi[k]);
        tasks.insert(tasks.end(), t, t + n);
        return SB_OK;
    }
};

int32_t check_config(const sb_transcription_config& t) {
    if (t.sample_rate != 16000 || t.feature_size != 128 || t.n_fft != 512 || t.win_length != 400 ||
        t.hop_length != 160 || t.samples_per_encoder_frame != 1280 || t.max_audio_samples > 240000 ||
        t.max_audio_samples <= 0)
        return fail(SB_INVALID_ARGUMENT,
                    "the kernels are specialised for 16 kHz / 128 mels / n_fft 512 / win 400 / hop 160 / 1280 samples "
                    "per encoder frame and at most 240000 samples per chunk");
    return SB_OK;
}

}  // namespace
}  // namespace sb

using namespace sb;

extern "C" {

// ------------------------------------------------------------------ planner / offsets / merge
int64_t sb_overlap_chunk_samples(const sb_overlap_config* c) { return c ? overlap_chunk_samples(*c) : 0; }
int64_t sb_overlap_overlap_samples(const sb_overlap_config* c) { return c ? overlap_overlap_samples(*c) : 0; }
int64_t sb_overlap_stride_samples(const sb_overlap_config* c) { return c ? overlap_stride_samples(*c) : 0; }

int32_t sb_plan_fast(const sb_overlap_config* cfg, int64_t audio_len, sb_chunk_task* tasks, int64_t cap,
                     int64_t* n_tasks) {
    if (!cfg || !n_tasks) return fail(SB_INVALID_ARGUMENT, "null argument");
    const std::vector<sb_chunk_task> t = plan_fast_tasks(audio_len, *cfg);
    *n_tasks = (int64_t)t.size();
    if (!tasks) return SB_OK;
    if (cap < (int64_t)t.size()) return fail(SB_BUFFER_TOO_SMALL, "task buffer too small");
    std::copy(t.begin(), t.end(), tasks);
    return SB_OK;
}

int64_t sb_parallel_worker_count(int64_t task_count, int64_t requested) {
    return parallel_worker_count(task_count, requested);
}

int32_t sb_apply_time_offsets(uint32_t* tok, int64_t* frm, int64_t* dur, float* conf, int64_t n, int64_t frame_offset,
                              int64_t context_frames, int64_t* n_out) {
    if (n < 0 || !n_out || (n > 0 && (!tok || !frm || !dur || !conf))) return fail(SB_INVALID_ARGUMENT, "null argument");
    RawTokens r = raw_from_arrays(tok, frm, dur, conf, 0, n);
    apply_time_offsets(r, frame_offset, context_frames);
    const size_t k = r.token_ids.size();
    std::copy(r.token_ids.begin(), r.token_ids.end(), tok);
    std::copy(r.frame_indices.begin(), r.frame_indices.end(), frm);
    std::copy(r.durations.begin(), r.durations.end(), dur);
    std::copy(r.confidences.begin(), r.confidences.end(), conf);
    *n_out = (int64_t)k;
    return SB_OK;
}

int32_t sb_merge_windows(const uint32_t* tok, const int64_t* frm, const int64_t* dur, const float* conf,
                         const int64_t* win_off, int64_t n_windows, uint32_t* otok, int64_t* ofrm, int64_t* odur,
                         float* oconf, int64_t out_cap, int64_t* n_out) {
    if (!win_off || !n_out || n_windows < 0) return fail(SB_INVALID_ARGUMENT, "null argument");
    OverlapMerger m;
    for (int64_t w = 0; w < n_windows; ++w) m.push(RawView{tok + win_off[w], frm + win_off[w], dur + win_off[w], conf + win_off[w], (size_t)(win_off[w + 1] - win_off[w])});
    const RawTokens& r = m.merged();
    *n_out = (int64_t)r.token_ids.size();
    if (*n_out > out_cap) return fail(SB_BUFFER_TOO_SMALL, "merge output buffer too small");
    std::copy(r.token_ids.begin(), r.token_ids.end(), otok);
    std::copy(r.frame_indices.begin(), r.frame_indices.end(), ofrm);
    std::copy(r.durations.begin(), r.durations.end(), odur);
    std::copy(r.confidences.begin(), r.confidences.end(), oconf);
    return SB_OK;
}

// ------------------------------------------------------------------ VAD planning
int64_t sb_vad_num_windows(int64_t n_samples) {
    return n_samples > 0 ? (n_samples + kVadWindowSamples - 1) / kVadWindowSamples : 0;
}

int32_t sb_vad_detect_speech_regions(const float* prob, int64_t n_prob, int64_t audio_len, float threshold,
                                     const sb_vad_segmentation_config* cfg, sb_sample_range* regions, int64_t cap,
                                     int64_t* n_regions) {
    if (!n_regions || n_prob < 0 || (n_prob > 0 && !prob)) return fail(SB_INVALID_ARGUMENT, "null argument");
    sb_vad_segmentation_config sc;
    if (cfg) sc = *cfg; else sb_default_vad_segmentation_config(&sc);
    const std::vector<sb_sample_range> r = detect_speech_regions(prob, n_prob, audio_len, threshold, sc);
    *n_regions = (int64_t)r.size();
    if (!regions) return SB_OK;
    if (cap < (int64_t)r.size()) return fail(SB_BUFFER_TOO_SMALL, "region buffer too small");
    std::copy(r.begin(), r.end(), regions);
    return SB_OK;
}

int32_t sb_vad_plan_region_subsegments(const sb_sample_range* region, const float* prob, int64_t n_prob,
                                       const sb_vad_segmentation_config* cfg, int64_t max_chunk_samples,
                                       sb_sample_range* segments, int64_t cap, int64_t* n_segments) {
    if (!region || !n_segments || n_prob < 0 || (n_prob > 0 && !prob)) return fail(SB_INVALID_ARGUMENT, "null argument");
    sb_vad_segmentation_config sc;
    if (cfg) sc = *cfg; else sb_default_vad_segmentation_config(&sc);
    std::vector<sb_sample_range> parts;
    if (!plan_region_subsegments(*region, prob, n_prob, sc, max_chunk_samples, &parts)) {
        *n_segments = -1;
        return SB_OK;
    }
    *n_segments = (int64_t)parts.size();
    if (!segments) return SB_OK;
    if (cap < (int64_t)parts.size()) return fail(SB_BUFFER_TOO_SMALL, "segment buffer too small");
    std::copy(parts.begin(), parts.end(), segments);
    return SB_OK;
}

int32_t sb_plan_vad(const sb_longform_config* cfg, const sb_sample_range* regions, int64_t n_regions, const float* prob,
                    int64_t n_prob, sb_chunk_task* tasks, int64_t task_cap, int64_t* n_tasks, sb_region_task* region_tasks,
                    int64_t region_cap) {
    if (!n_tasks || n_regions < 0 || (n_regions > 0 && !regions) || n_prob < 0 || (n_prob > 0 && !prob))
        return fail(SB_INVALID_ARGUMENT, "null argument");
    sb_longform_config lc;
    if (cfg) lc = *cfg; else sb_default_longform_config(&lc);
    const ExecutionPlan plan =
        build_vad_plan(std::vector<sb_sample_range>(regions, regions + n_regions), prob, n_prob, lc);
    *n_tasks = (int64_t)plan.tasks.size();
    if (tasks) {
        if (task_cap < (int64_t)plan.tasks.size()) return fail(SB_BUFFER_TOO_SMALL, "task buffer too small");
        std::copy(plan.tasks.begin(), plan.tasks.end(), tasks);
    }
    if (region_tasks) {
        if (region_cap < n_regions) return fail(SB_BUFFER_TOO_SMALL, "region task buffer too small");
        std::copy(plan.regions.begin(), plan.regions.end(), region_tasks);
    }
    return SB_OK;
}

// ------------------------------------------------------------------ vocabulary / text / results
int32_t sb_vocab_load(const char* path, sb_vocab** out) {
    if (!path || !out) return fail(SB_INVALID_ARGUMENT, "null argument");
    sb_vocab* v = new sb_vocab();
    bool io = false;
    const std::string err = vocabulary_from_file(path, &v->v, &io);
    if (!err.empty()) {
        delete v;
        return fail(io ? SB_IO : SB_INVALID_VOCABULARY, err);
    }
    *out = v;
    return SB_OK;
}

int32_t sb_vocab_from_text(const char* text, int64_t len, sb_vocab** out) {
    if (!text || !out || len < 0) return fail(SB_INVALID_ARGUMENT, "null argument");
    sb_vocab* v = new sb_vocab();
    const std::string err = vocabulary_from_text(std::string(text, (size_t)len), &v->v);
    if (!err.empty()) {
        delete v;
        return fail(SB_INVALID_VOCABULARY, err);
    }
    *out = v;
    return SB_OK;
}

void sb_vocab_free(sb_vocab* v) { delete v; }
int64_t sb_vocab_size(const sb_vocab* v) { return v ? (int64_t)v->v.id_to_token.size() : 0; }
int64_t sb_vocab_blank_id(const sb_vocab* v) { return v ? v->v.blank_id : -1; }

int32_t sb_text_decode(const sb_vocab* vocab, const uint32_t* tok, const int64_t* frm, const float* conf, int64_t n,
                       int64_t n_conf, double duration_seconds, sb_result** out) {
    if (!vocab || !out || n < 0 || (n > 0 && (!tok || !frm))) return fail(SB_INVALID_ARGUMENT, "null argument");
    RawTokens r;
    r.token_ids.assign(tok, tok + n);
    r.frame_indices.assign(frm, frm + n);
    r.durations.assign((size_t)n, 0);
    if (conf && n_conf > 0) r.confidences.assign(conf, conf + n_conf);
    sb_result* res = new sb_result();
    res->r = decode_tokens(vocab->v, r, duration_seconds);
    *out = res;
    return SB_OK;
}

const char* sb_result_text(const sb_result* r) { return r ? r->r.text.c_str() : ""; }
double sb_result_duration(const sb_result* r) { return r ? r->r.duration_seconds : 0.0; }
int64_t sb_result_num_tokens(const sb_result* r) { return r ? (int64_t)r->r.tokens.size() : 0; }
int64_t sb_result_num_chunks(const sb_result* r) { return r ? (int64_t)r->r.chunks.size() : 0; }

int32_t sb_result_token(const sb_result* r, int64_t i, uint32_t* token_id, const char** text, double* start,
                        double* end, float* confidence) {
    if (!r || i < 0 || i >= (int64_t)r->r.tokens.size()) return fail(SB_INVALID_ARGUMENT, "token index out of range");
    const TimedToken& t = r->r.tokens[(size_t)i];
    if (token_id) *token_id = t.token_id;
    if (text) *text = t.text.c_str();
    if (start) *start = t.start;
    if (end) *end = t.end;
    if (confidence) *confidence = t.confidence;
    return SB_OK;
}

int32_t sb_result_chunk(const sb_result* r, int64_t i, double* start, double* end, const char** text) {
    if (!r || i < 0 || i >= (int64_t)r->r.chunks.size()) return fail(SB_INVALID_ARGUMENT, "chunk index out of range");
    const TranscriptChunk& c = r->r.chunks[(size_t)i];
    if (start) *start = c.start;
    if (end) *end = c.end;
    if (text) *text = c.text.c_str();
    return SB_OK;
}

int32_t sb_result_tokens_bulk(const sb_result* r, uint32_t* token_ids, double* starts, double* ends,
                              float* confidences, int64_t* text_offsets, char* text_buf, int64_t text_cap,
                              int64_t* text_len) {
    if (!r) return fail(SB_INVALID_ARGUMENT, "result is null");
    const auto& tk = r->r.tokens;
    int64_t total = 0;
    for (const auto& t : tk) total += (int64_t)t.text.size();
    if (text_len) *text_len = total;
    if (text_buf && text_cap < total) return fail(SB_BUFFER_TOO_SMALL, "token text buffer too small");
    int64_t off = 0;
    for (size_t i = 0; i < tk.size(); ++i) {
        if (token_ids) token_ids[i] = tk[i].token_id;
        if (starts) starts[i] = tk[i].start;
        if (ends) ends[i] = tk[i].end;
        if (confidences) confidences[i] = tk[i].confidence;
        if (text_offsets) text_offsets[i] = off;
        if (text_buf) std::memcpy(text_buf + off, tk[i].text.data(), tk[i].text.size());
        off += (int64_t)tk[i].text.size();
    }
    if (text_offsets) text_offsets[tk.size()] = off;
    return SB_OK;
}

void sb_result_free(sb_result* r) { delete r; }

int64_t sb_raw_batch_size(const sb_raw_batch* b) { return b ? (int64_t)b->items.size() : 0; }

int32_t sb_raw_batch_get(const sb_raw_batch* b, int64_t i, int64_t* n, const uint32_t** tok, const int64_t** frm,
                         const int64_t** dur, const float** conf) {
    if (!b || i < 0 || i >= (int64_t)b->items.size()) return fail(SB_INVALID_ARGUMENT, "batch index out of range");
    const RawTokens& r = b->items[(size_t)i];
    if (n) *n = (int64_t)r.token_ids.size();
    if (tok) *tok = r.token_ids.data();
    if (frm) *frm = r.frame_indices.data();
    if (dur) *dur = r.durations.data();
    if (conf) *conf = r.confidences.data();
    return SB_OK;
}

int64_t sb_raw_batch_total(const sb_raw_batch* b) {
    int64_t n = 0;
    if (b)
        for (const auto& r : b->items) n += (int64_t)r.token_ids.size();
    return n;
}

int32_t sb_raw_batch_flatten(const sb_raw_batch* b, int64_t* offsets, uint32_t* tok, int64_t* frm, int64_t* dur,
                             float* conf) {
    if (!b || !offsets) return fail(SB_INVALID_ARGUMENT, "null argument");
    int64_t off = 0;
    for (size_t i = 0; i < b->items.size(); ++i) {
        const RawTokens& r = b->items[i];
        const size_t k = r.token_ids.size();
        offsets[i] = off;
        if (k) {
            if (tok) std::memcpy(tok + off, r.token_ids.data(), k * sizeof(uint32_t));
            if (frm) std::memcpy(frm + off, r.frame_indices.data(), k * sizeof(int64_t));
            if (dur) std::memcpy(dur + off, r.durations.data(), k * sizeof(int64_t));
            if (conf) std::memcpy(conf + off, r.confidences.data(), k * sizeof(float));
        }
        off += (int64_t)k;
    }
    offsets[b->items.size()] = off;
    return SB_OK;
}

void sb_raw_batch_free(sb_raw_batch* b) { delete b; }

// ------------------------------------------------------------------ pipelines
int32_t sb_transcribe_chunks(sb_ctx* c, const float* pcm, int64_t n_samples, const sb_chunk_task* tasks,
                             int64_t n_tasks, const sb_transcription_config* cfg, sb_raw_batch** out) {
    if (!c || !pcm || !out || (n_tasks > 0 && !tasks) || n_tasks < 0) return fail(SB_INVALID_ARGUMENT, "null argument");
    sb_transcription_config t;
    if (cfg) t = *cfg; else sb_default_transcription_config(&t);
    int32_t s = check_config(t);
    if (s != SB_OK) return s;
    sb_raw_batch* b = new sb_raw_batch();
    s = transcribe_tasks(c, pcm, n_samples, tasks, n_tasks, t, &b->items);
    if (s != SB_OK) {
        delete b;
        return s;
    }
    *out = b;
    return SB_OK;
}

int32_t sb_transcribe_chunks_i16(sb_ctx* c, const int16_t* pcm, int64_t n_samples, const sb_chunk_task* tasks,
                                 int64_t n_tasks, const sb_transcription_config* cfg, sb_raw_batch** out) {
    if (!c || !pcm || !out || (n_tasks > 0 && !tasks) || n_tasks < 0) return fail(SB_INVALID_ARGUMENT, "null argument");
    sb_transcription_config t;
    if (cfg) t = *cfg; else sb_default_transcription_config(&t);
    int32_t s = check_config(t);
    if (s != SB_OK) return s;
    sb_raw_batch* b = new sb_raw_batch();
    s = transcribe_tasks(c, pcm, n_samples, tasks, n_tasks, t, &b->items, false, kSampleI16);
    if (s != SB_OK) {
        delete b;
        return s;
    }
    *out = b;
    return SB_OK;
}

int32_t sb_transcribe_chunks_device(sb_ctx* c, const float* d_audio, int64_t n_samples, const sb_chunk_task* tasks,
                                    int64_t n_tasks, const sb_transcription_config* cfg, sb_raw_batch** out) {
    if (!c || !d_audio || !out || (n_tasks > 0 && !tasks) || n_tasks < 0) return fail(SB_INVALID_ARGUMENT, "null argument");
    sb_transcription_config t;
    if (cfg) t = *cfg; else sb_default_transcription_config(&t);
    int32_t s = check_config(t);
    if (s != SB_OK) return s;
    sb_raw_batch* b = new sb_raw_batch();
    s = transcribe_tasks(c, d_audio, n_samples, tasks, n_tasks, t, &b->items, true);
    if (s != SB_OK) {
        delete b;
        return s;
    }
    *out = b;
    return SB_OK;
}

int32_t sb_pipeline_run(sb_ctx* c, const sb_vocab* vocab, const float* audio, int64_t n_samples,
                        const sb_transcription_config* cfg, sb_result** out) {
    if (!c || !vocab || !out) return fail(SB_INVALID_ARGUMENT, "null argument");
    sb_transcription_config t;
    if (cfg) t = *cfg; else sb_default_transcription_config(&t);
    int32_t s = check_config(t);
    if (s != SB_OK) return s;
    if (n_samples <= 0 || !audio) return fail(SB_EMPTY_AUDIO, "audio input was empty");  // pipeline.rs:150
    const sb_chunk_task task{0, n_samples, 0, 0};
    std::vector<RawTokens> raw;
    s = transcribe_tasks(c, audio, n_samples, &task, 1, t, &raw);  // AudioTooLong is raised inside
    if (s != SB_OK) return s;
    sb_result* res = new sb_result();
    res->r = decode_tokens(vocab->v, raw[0], (double)n_samples / (double)t.sample_rate);
    *out = res;
    return SB_OK;
}

int32_t sb_longform_finish(const sb_vocab* vocab, int64_t audio_len, const uint32_t* tok, const int64_t* frm,
                           const int64_t* dur, const float* conf, const int64_t* win_off, int64_t n_windows,
                           sb_result** out) {
    if (!vocab || !out || !win_off || n_windows < 0) return fail(SB_INVALID_ARGUMENT, "null argument");
    OverlapMerger m;
    for (int64_t w = 0; w < n_windows; ++w) m.push(RawView{tok + win_off[w], frm + win_off[w], dur + win_off[w], conf + win_off[w], (size_t)(win_off[w + 1] - win_off[w])});
    // long_form.rs:404-419: decode the merged stream against the whole recording's duration
    std::string joined;
    TranscriptionResult merged = decode_tokens(vocab->v, m.merged(), (double)audio_len / 16000.0, &joined);
    sb_result* res = new sb_result();
    res->r = long_form_result(std::move(merged.tokens), joined, audio_len);
    *out = res;
    return SB_OK;
}

int32_t sb_longform_finish_regions(const sb_vocab* vocab, int64_t audio_len, const sb_chunk_task* tasks, int64_t n_tasks,
                                   const sb_region_task* region_tasks, int64_t n_regions, const uint32_t* tok,
                                   const int64_t* frm, const int64_t* dur, const float* conf, const int64_t* win_off,
                                   sb_result** out) {
    if (!vocab || !out || n_tasks < 0 || n_regions < 0 || (n_tasks > 0 && (!tasks || !win_off)) ||
        (n_regions > 0 && !region_tasks))
        return fail(SB_INVALID_ARGUMENT, "null argument");
    for (int64_t r = 0; r < n_regions; ++r)
        if (region_tasks[r].first_task < 0 || region_tasks[r].n_tasks < 0 ||
            region_tasks[r].first_task + region_tasks[r].n_tasks > n_tasks)
            return fail(SB_INVALID_ARGUMENT, "region task outside the task list");
    std::vector<RawTokens> raw((size_t)n_tasks);
    for (int64_t i = 0; i < n_tasks; ++i) raw[(size_t)i] = raw_from_arrays(tok, frm, dur, conf, win_off[i], win_off[i + 1]);
    sb_result* res = new sb_result();
    res->r = build_plan_result(vocab->v, audio_len, tasks, region_tasks, n_regions, raw);
    *out = res;
    return SB_OK;
}

namespace {

// execute_plan (src/long_form.rs:232-245): the tasks go to min(worker_count, n_ctx, tasks) GPU shards in
// contiguous blocks (run_parallel_regions, long_form.rs:266-314); build_parallel_result joins them.
// d_audio0, if not null, is the recording in the memory of ctxs[0]'s GPU (the VAD network left it there): the
// first shard then reads it in place instead of copying its part from the host again.
int32_t execute_plan(sb_ctx** ctxs, int64_t n_ctx, const sb_vocab* vocab, const float* audio, int64_t n_samples,
                     const sb_longform_config& lc, const ExecutionPlan& plan, sb_result** out,
                     const float* d_audio0 = nullptr) {
    sb_result* res = new sb_result();
    const int64_t n_tasks = (int64_t)plan.tasks.size();
    if (n_tasks == 0) {  // TranscriptionResult::empty
        res->r.duration_seconds = (double)n_samples / 16000.0;
        *out = res;
        return SB_OK;
    }
    const int64_t shards = parallel_worker_count(n_tasks, std::min<int64_t>(lc.worker_count, n_ctx));
    std::vector<std::vector<RawTokens>> parts((size_t)shards);
    std::vector<int32_t> status((size_t)shards, SB_OK);
    std::vector<std::string> errors((size_t)shards);
    auto work = [&](int64_t k) {
        const int64_t a = n_tasks * k / shards, b = n_tasks * (k + 1) / shards;
        const bool resident = k == 0 && d_audio0;
        // a batch holds at most 65535 tasks (a plan of very short regions over a long recording can hold more)
        for (int64_t i = a; i < b && status[k] == SB_OK; i += 32768) {
            std::vector<RawTokens> some;
            status[k] = transcribe_tasks(ctxs[k], resident ? d_audio0 : audio, n_samples, plan.tasks.data() + i,
                                         std::min<int64_t>(32768, b - i), lc.transcription, &some, resident);
            for (auto& r : some) parts[k].push_back(std::move(r));
        }
        if (status[k] != SB_OK) errors[k] = sb_last_error();
    };
    if (shards == 1) {
        work(0);
    } else {
        std::vector<std::thread> th;
        for (int64_t k = 0; k < shards; ++k) th.emplace_back(work, k);
        for (auto& t : th) t.join();
    }
    for (int64_t k = 0; k < shards; ++k)  // the first failing shard aborts the call (long_form.rs:328-332)
        if (status[k] != SB_OK) {
            delete res;
            return fail((sb_status)status[k], errors[k]);
        }
    std::vector<RawTokens> raw;
    raw.reserve((size_t)n_tasks);
    for (auto& p : parts)
        for (auto& r : p) raw.push_back(std::move(r));
    res->r = build_plan_result(vocab->v, n_samples, plan.tasks.data(), plan.regions.data(), (int64_t)plan.regions.size(), raw);
    *out = res;
    return SB_OK;
}

int32_t run_vad_plan(sb_ctx** ctxs, int64_t n_ctx, const sb_vocab* vocab, const float* audio, int64_t n_samples,
                     const sb_longform_config& lc, const float* prob, int64_t n_prob, sb_result** out,
                     const float* d_audio0 = nullptr) {
    // long_form.rs:200-216; VadSegmentationConfig::threshold returns the VadConfig's value (planner.rs:71-73)
    const std::vector<sb_sample_range> regions =
        detect_speech_regions(prob, n_prob, n_samples, lc.vad.default_threshold, lc.segmentation);
    return execute_plan(ctxs, n_ctx, vocab, audio, n_samples, lc, build_vad_plan(regions, prob, n_prob, lc), out, d_audio0);
}

// The VAD mode on one GPU with the voice-activity network and the transcription overlapped.  The recording goes
// to the GPU in passes on a second, high-priority stream: copy, network, probabilities back to the host.  The
// recurrence of the network occupies one 8-CTA cluster for as long as the rest of the GPU needs to transcribe a
// comparable stretch of audio, so the host plans the regions that pass k made final (SpeechRegionStream) and
// sends their tasks through the frontend and the encoder on the context's stream while pass k + 1 runs beside
// them.  Passes start short (the first one is exposed) and double up to "vad_stream_pass_windows" (or "vad_segment_windows", if smaller).  The decoder runs
// once at the end.  Regions, tasks and results equal those of the unstreamed path.
int32_t run_vad_streamed(sb_ctx* c, const sb_vocab* vocab, const float* audio, int64_t n_samples,
                         const sb_longform_config& lc, sb_result** out) {
    VadModel& m = *c->vad;
    SB_CUDA(cudaSetDevice(c->device));
    const int64_t n_win = sb_vad_num_windows(n_samples);
    // passes of 8192, 16384, 32768, then 49152 windows (26 minutes of audio; measured on an 8 h recording with 76 % sound,
    // largest pass 131072 / 65536 / 49152 / 32768 / 24576 windows: 456 / 425 / 422 / 433 / 472 ms: longer passes leave a
    // longer stretch to transcribe after the last recurrence, shorter ones make the pieces' kernels small)
    const int64_t pass_cap = std::min<int64_t>(c->vad_segment_windows, c->vad_stream_pass_windows);
    std::vector<int64_t> cut{0};  // pass boundaries, in windows
    for (int64_t w = 8192; cut.back() < n_win; w = std::min<int64_t>(2 * w, pass_cap))
        cut.push_back(std::min(n_win, cut.back() + std::min<int64_t>(w, pass_cap)));
    const int n_pass = (int)cut.size() - 1;
    int64_t max_pass = 0;
    for (int k = 0; k < n_pass; ++k) max_pass = std::max(max_pass, cut[k + 1] - cut[k]);
    SB_CUDA(m.audio.ensure(sizeof(float) * (size_t)n_samples));
    SB_CUDA(m.prob.ensure(sizeof(float) * (size_t)n_win));
    m.host_prob.pinned_host = true;
    SB_CUDA(m.host_prob.ensure(sizeof(float) * (size_t)n_win));
    if (!c->vad_stream) {
        int least = 0, greatest = 0;
        SB_CUDA(cudaDeviceGetStreamPriorityRange(&least, &greatest));
        SB_CUDA(cudaStreamCreateWithPriority(&c->vad_stream, cudaStreamNonBlocking, greatest));
        SB_CUDA(cudaStreamCreateWithPriority(&c->vad_feed_stream, cudaStreamNonBlocking, greatest));
    }
    // events per pass: probabilities on the host | gate inputs ready | recurrence done; plus one that orders the passes
    // after earlier work
    while ((int)c->vad_events.size() < 3 * n_pass + 1) {
        cudaEvent_t ev;
        SB_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        c->vad_events.push_back(ev);
    }
    PieceRun run{c, m.audio.as<float>(), n_samples, lc.transcription};
    // room for the encoder frames of the whole recording windowed with overlap, plus a margin for short regions
    int32_t s = run.begin(c->vad_rows_cap > 0 ? c->vad_rows_cap : (int64_t)(1.2 * (double)n_samples / 1280.0) + 16384);
    if (s != SB_OK) return s;
    // Two streams feed the network: `fs` copies a pass's samples in and computes its gate inputs, `vs` runs the
    // recurrences one after another; the gate inputs alternate between two buffers, so pass k + 1 is prepared while
    // pass k recurs.
    cudaStream_t vs = c->vad_stream, fs = c->vad_feed_stream;
    cudaEvent_t* ev_host = c->vad_events.data();           // [k]: pass k's probabilities are in host memory
    cudaEvent_t* ev_fed = c->vad_events.data() + n_pass;   // [k]: pass k's gate inputs are ready
    cudaEvent_t* ev_rec = c->vad_events.data() + 2 * n_pass;  // [k]: pass k's recurrence has ended
    cudaEvent_t ev_prior = c->vad_events[3 * n_pass];
    // work of an earlier call on the context's stream may still read the buffers that the passes overwrite
    SB_CUDA(cudaEventRecord(ev_prior, c->stream));
    SB_CUDA(cudaStreamWaitEvent(vs, ev_prior, 0));
    s = vad_begin(c, max_pass, vs, true);
    if (s != SB_OK) return s;
    SB_CUDA(cudaEventRecord(ev_prior, vs));
    SB_CUDA(cudaStreamWaitEvent(fs, ev_prior, 0));
    float* h_prob = m.host_prob.as<float>();
    auto enqueue = [&](int k) -> int32_t {
        const int64_t a = cut[k] * kVadWindow, b = std::min(n_samples, cut[k + 1] * kVadWindow);
        const int n = (int)(cut[k + 1] - cut[k]);
        if (k >= 2) SB_CUDA(cudaStreamWaitEvent(fs, ev_rec[k - 2], 0));  // the buffer's last reader
        SB_CUDA(cudaMemcpyAsync(m.audio.as<float>() + a, audio + a, sizeof(float) * (size_t)(b - a), cudaMemcpyHostToDevice, fs));
        int32_t r = vad_encode_pass(c, fs, m.audio.as<float>(), n_samples, cut[k], n, k & 1);
        if (r != SB_OK) return r;
        SB_CUDA(cudaEventRecord(ev_fed[k], fs));
        SB_CUDA(cudaStreamWaitEvent(vs, ev_fed[k], 0));
        r = vad_recur_pass(c, vs, cut[k], n, k & 1, m.prob.as<float>());
        if (r != SB_OK) return r;
        SB_CUDA(cudaEventRecord(ev_rec[k], vs));
        SB_CUDA(cudaMemcpyAsync(h_prob + cut[k], m.prob.as<float>() + cut[k], sizeof(float) * (size_t)n, cudaMemcpyDeviceToHost, vs));
        SB_CUDA(cudaEventRecord(ev_host[k], vs));
        return SB_OK;
    };
    // The recurrence kernel holds one SM per CTA of its cluster for the length of a pass, and the GEMM and attention
    // kernels (one CTA per SM, each with a fixed share of the tiles, nearly all of the SM's shared memory) cannot sit
    // beside it: launched over all SMs, the CTAs that find their SM taken would run as a second wave.  So while passes
    // are in flight those kernels are sized for the SMs that are left.
    const int all_sms = c->sm_count;
    c->sm_count = std::max(8, all_sms - c->vad_cluster);
    auto bail = [&](int32_t code) {
        const std::string msg = sb_last_error();
        cudaStreamSynchronize(fs);
        cudaStreamSynchronize(vs);
        cudaStreamSynchronize(c->stream);
        c->sm_count = all_sms;
        return fail((sb_status)code, msg);
    };
    s = enqueue(0);
    if (s != SB_OK) return bail(s);
    SpeechRegionStream regions(n_samples, lc.vad.default_threshold, lc.segmentation);
    ExecutionPlan plan;
    size_t planned = 0;
    for (int k = 0; k < n_pass; ++k) {
        if (k + 1 < n_pass && (s = enqueue(k + 1)) != SB_OK) return bail(s);
        cudaError_t e = cudaEventSynchronize(ev_host[k]);
        if (e != cudaSuccess) return bail(cuda_fail(e, "cudaEventSynchronize(vad pass)"));
        regions.push(h_prob + cut[k], cut[k + 1] - cut[k]);
        if (k + 1 == n_pass) regions.finish();
        const size_t first_task = plan.tasks.size();
        for (; planned < regions.regions().size(); ++planned)
            append_region_plan(&plan, regions.regions()[planned], h_prob, cut[k + 1], lc);
        if ((s = run.add(plan.tasks.data() + first_task, (int64_t)(plan.tasks.size() - first_task))) != SB_OK) return bail(s);
    }
    c->sm_count = all_sms;  // every pass has ended
    if ((s = take_device_error(c, vs)) != SB_OK) return bail(s);  // a recurrence that gave up waiting
    sb_result* res = new sb_result();
    if (plan.tasks.empty()) {  // TranscriptionResult::empty (long_form.rs:206-208)
        res->r.duration_seconds = (double)n_samples / 16000.0;
        *out = res;
        return SB_OK;
    }
    if ((s = run.decode_pending()) != SB_OK) {
        delete res;
        return bail(s);
    }
    res->r = build_plan_result(vocab->v, n_samples, plan.tasks.data(), plan.regions.data(), (int64_t)plan.regions.size(), run.raws);
    *out = res;
    return SB_OK;
}

}  // namespace

int32_t sb_longform_run_with_probabilities(sb_ctx** ctxs, int64_t n_ctx, const sb_vocab* vocab, const float* audio,
                                           int64_t n_samples, const sb_longform_config* cfg, const float* prob,
                                           int64_t n_prob, sb_result** out) {
    if (!ctxs || n_ctx <= 0 || !vocab || !out || n_prob < 0 || (n_prob > 0 && !prob))
        return fail(SB_INVALID_ARGUMENT, "null argument");
    sb_longform_config lc;
    if (cfg) lc = *cfg; else sb_default_longform_config(&lc);
    int32_t s = check_config(lc.transcription);
    if (s != SB_OK) return s;
    if (n_samples <= 0 || !audio) return fail(SB_EMPTY_AUDIO, "audio input was empty");  // long_form.rs:158
    if (n_samples <= lc.transcription.max_audio_samples)                                 // long_form.rs:161-163
        return sb_pipeline_run(ctxs[0], vocab, audio, n_samples, &lc.transcription, out);
    return run_vad_plan(ctxs, n_ctx, vocab, audio, n_samples, lc, prob, n_prob, out);
}

int32_t sb_longform_run_multi(sb_ctx** ctxs, int64_t n_ctx, const sb_vocab* vocab, const float* audio,
                              int64_t n_samples, const sb_longform_config* cfg, sb_result** out) {
    if (!ctxs || n_ctx <= 0 || !vocab || !out) return fail(SB_INVALID_ARGUMENT, "null argument");
    sb_longform_config lc;
    if (cfg) lc = *cfg; else sb_default_longform_config(&lc);
    if (lc.mode != 0 && lc.mode != 1) return fail(SB_INVALID_ARGUMENT, "long-form mode must be 0 (Fast) or 1 (Vad)");
    int32_t s = check_config(lc.transcription);
    if (s != SB_OK) return s;
    if (n_samples <= 0 || !audio) return fail(SB_EMPTY_AUDIO, "audio input was empty");  // long_form.rs:158
    if (n_samples <= lc.transcription.max_audio_samples)                                 // long_form.rs:161-163
        return sb_pipeline_run(ctxs[0], vocab, audio, n_samples, &lc.transcription, out);
    if (lc.mode == 0) return execute_plan(ctxs, n_ctx, vocab, audio, n_samples, lc, build_fast_plan(n_samples, lc), out);
    // long_form.rs:193-200: the VAD network is needed only when the mode asks for it
    if (!ctxs[0]->vad) return fail(SB_MISSING_MODEL_ASSET, "missing model asset: vad/silero-vad (load it with sb_vad_load)");
    // one GPU: the network and the transcription overlap; several: the network first, then the tasks in shards
    if (std::min<int64_t>(lc.worker_count, n_ctx) <= 1 && !ctxs[0]->vad_unstreamed)
        return run_vad_streamed(ctxs[0], vocab, audio, n_samples, lc, out);
    std::vector<float> prob((size_t)sb_vad_num_windows(n_samples));
    int64_t n_prob = 0;
    s = sb_vad_process(ctxs[0], audio, n_samples, prob.data(), (int64_t)prob.size(), &n_prob);
    if (s != SB_OK) return s;
    return run_vad_plan(ctxs, n_ctx, vocab, audio, n_samples, lc, prob.data(), n_prob, out, vad_resident_audio(ctxs[0]));
}

int32_t sb_longform_run(sb_ctx* c, const sb_vocab* vocab, const float* audio, int64_t n_samples,
                        const sb_longform_config* cfg, sb_result** out) {
    if (!c) return fail(SB_INVALID_ARGUMENT, "ctx is null");
    sb_ctx* one[1] = {c};
    return sb_longform_run_multi(one, 1, vocab, audio, n_samples, cfg, out);
}

}  // extern "C"
