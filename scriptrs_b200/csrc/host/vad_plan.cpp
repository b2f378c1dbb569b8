// Host-side planning of the VAD long-form mode: speech regions from per-window probabilities, silence splits of
// long regions, and the execution plan of region tasks.  Logic of the reference, restated for the host driver:
//   VadSegmentationConfig::effective_negative_threshold          src/long_form/planner.rs:75-80
//   detect_speech_regions                                        src/long_form/planner.rs:139-233
//     (as a stream: windows go in as the network produces them, a region comes out as soon as nothing later can
//      change it, which is when the speech span after it has closed)
//   region_probability_slice                                     src/long_form/planner.rs:235-240
//   plan_region_subsegments / silence_spans                      src/long_form/planner.rs:242-315
//   build_execution_plan / build_region_plan / push_*_task       src/long_form.rs:421-459,508-582
//   build_parallel_result / decode_*_tasks / offset_tokens       src/long_form.rs:344-419,649-661
#include <algorithm>
#include <cmath>

#include "longform.h"

namespace sb {

namespace {
constexpr double kRate = 16000.0;

inline int64_t sat_sub(int64_t a, int64_t b) { return a > b ? a - b : 0; }
inline int64_t div_ceil(int64_t a, int64_t b) { return (a + b - 1) / b; }

// `(seconds * SAMPLE_RATE as f64) as usize`: the cast saturates (negative and NaN give 0)
inline int64_t seconds_to_samples(double seconds) {
    const double v = seconds * kRate;
    if (!(v > 0.0)) return 0;
    if (v >= 9.2e18) return INT64_MAX;
    return static_cast<int64_t>(v);
}

inline float negative_threshold(const sb_vad_segmentation_config& c, float base) {
    if (c.has_negative_threshold) return c.negative_threshold;
    const float v = base - c.negative_threshold_offset;
    return v > 0.01f ? v : 0.01f;  // f32::max: a NaN difference gives 0.01
}

// planner.rs:286-315
std::vector<sb_sample_range> silence_spans(sb_sample_range region, const float* prob, int64_t n, float threshold) {
    const int64_t first_window = region.start / kVadWindowSamples;
    std::vector<sb_sample_range> spans;
    bool open = false;
    int64_t open_at = 0;
    for (int64_t i = 0; i < n; ++i) {
        const int64_t sample = (first_window + i) * kVadWindowSamples;
        if (prob[i] <= threshold) {
            if (!open) { open = true; open_at = sample; }
            continue;
        }
        if (open) {
            spans.push_back({std::max(open_at, region.start), std::min(sample, region.end)});
            open = false;
        }
    }
    if (open) spans.push_back({std::max(open_at, region.start), region.end});
    return spans;
}

sb_chunk_task segment_task(sb_sample_range s) { return sb_chunk_task{s.start, s.end, 0, 0}; }  // long_form.rs:550-564

sb_chunk_task overlap_task(sb_sample_range chunk, const sb_overlap_config& o) {  // long_form.rs:566-582
    const int64_t ctx_start = sat_sub(chunk.start, o.context_samples);
    return sb_chunk_task{ctx_start, chunk.end, chunk.start, chunk.start - ctx_start};
}

// OverlapChunkConfig::plan over an arbitrary range (planner.rs:124-136)
std::vector<sb_sample_range> overlap_plan(sb_sample_range range, const sb_overlap_config& o) {
    std::vector<sb_sample_range> chunks;
    const int64_t chunk = overlap_chunk_samples(o), stride = overlap_stride_samples(o);
    int64_t start = range.start;
    while (start < range.end) {
        const int64_t end = std::min(start + chunk, range.end);
        chunks.push_back({start, end});
        if (end == range.end) break;
        start += stride;
    }
    return chunks;
}
}  // namespace

SpeechRegionStream::SpeechRegionStream(int64_t audio_len, float threshold, const sb_vad_segmentation_config& cfg)
    : audio_len_(audio_len),
      min_speech_(seconds_to_samples(cfg.min_speech_duration)),
      min_silence_(seconds_to_samples(cfg.min_silence_duration)),
      pad_(seconds_to_samples(cfg.speech_padding)),
      threshold_(threshold),
      negative_(negative_threshold(cfg, threshold)) {}

// A raw speech span has closed.  Its start is final once the gap to the span before it is shared out; its end once
// the span after it is known: so the span before it leaves now, and this one waits.
void SpeechRegionStream::on_speech(sb_sample_range s) {
    if (!has_pending_) {
        s.start = sat_sub(s.start, pad_);  // first region: padding towards the start of the recording
        pending_ = s;
        has_pending_ = true;
        return;
    }
    const int64_t gap = sat_sub(s.start, pending_.end);
    const int64_t grow = gap < 2 * pad_ ? gap / 2 : pad_;
    pending_.end = std::min(pending_.end + grow, audio_len_);
    s.start = sat_sub(s.start, grow);
    if (pending_.end > pending_.start) regions_.push_back(pending_);
    pending_ = s;
}

void SpeechRegionStream::push(const float* prob, int64_t n) {
    if (audio_len_ <= 0) return;
    for (int64_t i = 0; i < n; ++i, ++window_) {
        const int64_t at = window_ * kVadWindowSamples;
        const float p = prob[i];
        if (p >= threshold_) {
            silence_open_ = false;
            if (!triggered_) { triggered_ = true; speech_start_ = at; }
            continue;
        }
        if (p < negative_ && triggered_) {
            if (!silence_open_) { silence_open_ = true; silence_start_ = at; }
            if (sat_sub(at, silence_start_) >= min_silence_) {
                if (sat_sub(silence_start_, speech_start_) >= min_speech_) on_speech({speech_start_, silence_start_});
                triggered_ = false;
                silence_open_ = false;
            }
        }
    }
}

void SpeechRegionStream::finish() {
    if (audio_len_ <= 0 || window_ == 0) return;
    if (triggered_ && sat_sub(audio_len_, speech_start_) >= min_speech_) on_speech({speech_start_, audio_len_});
    triggered_ = false;
    if (has_pending_) {
        pending_.end = std::min(pending_.end + pad_, audio_len_);
        if (pending_.end > pending_.start) regions_.push_back(pending_);
        has_pending_ = false;
    }
}

std::vector<sb_sample_range> detect_speech_regions(const float* prob, int64_t n_prob, int64_t audio_len, float threshold,
                                                   const sb_vad_segmentation_config& cfg) {
    // fed in pieces, the way the streamed mode feeds it pass by pass (the result does not depend on the pieces)
    SpeechRegionStream stream(audio_len, threshold, cfg);
    for (int64_t at = 0; at < n_prob; at += 1000) stream.push(prob + at, std::min<int64_t>(1000, n_prob - at));
    stream.finish();
    return stream.regions();
}

bool plan_region_subsegments(sb_sample_range region, const float* region_prob, int64_t n_prob,
                             const sb_vad_segmentation_config& cfg, int64_t max_chunk_samples,
                             std::vector<sb_sample_range>* out) {
    out->clear();
    if (sat_sub(region.end, region.start) <= max_chunk_samples) {
        out->push_back(region);
        return true;
    }
    const int64_t min_silence = seconds_to_samples(cfg.min_silence_at_max_speech);
    std::vector<sb_sample_range> spans = silence_spans(region, region_prob, n_prob, cfg.silence_threshold_for_split);
    spans.erase(std::remove_if(spans.begin(), spans.end(),
                               [&](const sb_sample_range& s) { return sat_sub(s.end, s.start) < min_silence; }),
                spans.end());
    int64_t cursor = region.start;
    while (sat_sub(region.end, cursor) > max_chunk_samples) {
        const int64_t search_end = cursor + max_chunk_samples;
        // Iterator::max_by_key keeps the LAST of several equally long spans
        bool found = false;
        sb_sample_range best{0, 0};
        for (const sb_sample_range& s : spans) {
            if (!(s.start > cursor && s.start < search_end)) continue;
            if (!found || sat_sub(s.end, s.start) >= sat_sub(best.end, best.start)) { best = s; found = true; }
        }
        if (!found) { out->clear(); return false; }
        out->push_back({cursor, best.start});
        cursor = best.end;
    }
    if (cursor < region.end) out->push_back({cursor, region.end});
    return true;
}

void append_region_plan(ExecutionPlan* plan, sb_sample_range region, const float* prob, int64_t n_prob,
                        const sb_longform_config& cfg) {
    const int64_t max_chunk = cfg.transcription.max_audio_samples;
    sb_region_task rt{1, (int64_t)plan->tasks.size(), 0};
    if (sat_sub(region.end, region.start) <= max_chunk) {
        plan->tasks.push_back(segment_task(region));
    } else {
        // region_probability_slice
        const int64_t w0 = std::min(region.start / kVadWindowSamples, n_prob);
        const int64_t w1 = std::min(div_ceil(region.end, kVadWindowSamples), n_prob);
        std::vector<sb_sample_range> parts;
        if (plan_region_subsegments(region, prob + w0, std::max<int64_t>(w1 - w0, 0), cfg.segmentation, max_chunk, &parts)) {
            for (const sb_sample_range& s : parts) plan->tasks.push_back(segment_task(s));
        } else {
            rt.kind = 0;
            for (const sb_sample_range& s : overlap_plan(region, cfg.overlap)) plan->tasks.push_back(overlap_task(s, cfg.overlap));
        }
    }
    rt.n_tasks = (int64_t)plan->tasks.size() - rt.first_task;
    plan->regions.push_back(rt);
}

ExecutionPlan build_vad_plan(const std::vector<sb_sample_range>& regions, const float* prob, int64_t n_prob,
                             const sb_longform_config& cfg) {
    ExecutionPlan plan;
    for (const sb_sample_range& region : regions) append_region_plan(&plan, region, prob, n_prob, cfg);
    return plan;
}

ExecutionPlan build_fast_plan(int64_t audio_len, const sb_longform_config& cfg) {
    ExecutionPlan plan;
    plan.tasks = plan_fast_tasks(audio_len, cfg.overlap);
    plan.regions.push_back(sb_region_task{0, 0, (int64_t)plan.tasks.size()});
    return plan;
}

TranscriptionResult build_plan_result(const Vocabulary& vocab, int64_t audio_len, const sb_chunk_task* tasks,
                                      const sb_region_task* regions, int64_t n_regions, std::vector<RawTokens>& raw) {
    TranscriptionResult res;
    res.duration_seconds = static_cast<double>(audio_len) / kRate;
    for (int64_t r = 0; r < n_regions; ++r) {
        const sb_region_task& rt = regions[r];
        std::vector<TimedToken> tokens;
        std::string joined, part_text;  // the region's token texts, concatenated (join_token_text, long_form.rs:613-620)
        if (rt.kind == 1) {
            for (int64_t i = rt.first_task; i < rt.first_task + rt.n_tasks; ++i) {
                const int64_t len = sat_sub(tasks[i].audio_end, tasks[i].audio_start);
                TranscriptionResult part = decode_tokens(vocab, raw[(size_t)i], static_cast<double>(len) / kRate, &part_text);
                joined += part_text;
                const double shift = static_cast<double>(tasks[i].audio_start) / kRate;
                for (TimedToken& t : part.tokens) {
                    t.start += shift;
                    t.end += shift;
                    tokens.push_back(std::move(t));
                }
            }
        } else {
            OverlapMerger m;
            for (int64_t i = rt.first_task; i < rt.first_task + rt.n_tasks; ++i) m.push(raw[(size_t)i]);
            tokens = decode_tokens(vocab, m.merged(), res.duration_seconds, &joined).tokens;
        }
        if (tokens.empty()) continue;  // build_chunk returns None
        res.chunks.push_back(TranscriptChunk{tokens.front().start, tokens.back().end, trim_whitespace(joined)});
        for (TimedToken& t : tokens) res.tokens.push_back(std::move(t));
    }
    for (size_t i = 0; i < res.chunks.size(); ++i) {
        if (i) res.text += " ";
        res.text += res.chunks[i].text;
    }
    return res;
}

}  // namespace sb
