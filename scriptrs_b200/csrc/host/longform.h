// Host-side long-form logic (longform.cpp) and text decoding (text.cpp).
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

#include "../../../include/scriptrs_b200.h"
#include "../pipeline.h"

namespace sb {

int64_t overlap_chunk_samples(const sb_overlap_config& c);
int64_t overlap_overlap_samples(const sb_overlap_config& c);
int64_t overlap_stride_samples(const sb_overlap_config& c);
std::vector<sb_chunk_task> plan_fast_tasks(int64_t audio_len, const sb_overlap_config& c);
int64_t parallel_worker_count(int64_t task_count, int64_t requested);
void apply_time_offsets(RawTokens& raw, int64_t frame_offset, int64_t context_frames);

// Left fold of the reference's overlap merge, one window at a time, in cost proportional to the
// overlap rather than to the transcript so far.
// One window's token stream where it lies (no copy).
struct RawView {
    const uint32_t* token_ids;
    const int64_t* frame_indices;
    const int64_t* durations;
    const float* confidences;
    size_t n;
};

class OverlapMerger {
  public:
    void push(const RawView& window);
    void push(const RawTokens& w) {
        push(RawView{w.token_ids.data(), w.frame_indices.data(), w.durations.data(), w.confidences.data(), w.token_ids.size()});
    }
    RawTokens take() { prefix_max_.clear(); return std::move(m_); }
    const RawTokens& merged() const { return m_; }

  private:
    void append(const RawView& src, size_t from, size_t to);
    void truncate(size_t n);
    RawTokens m_;
    std::vector<int64_t> prefix_max_;  // running maximum of m_.frame_indices
    std::vector<uint32_t> near_;       // scratch: the right window's tokens that can match at all
};

RawTokens merge_overlapping_windows(const std::vector<RawTokens>& windows);

// ------------------------------------------------------------------ VAD planning (vad_plan.cpp)
constexpr int64_t kVadWindowSamples = 512;   // constants.rs:7
constexpr int64_t kVadContextSamples = 64;   // constants.rs:9
constexpr int64_t kVadStateSize = 128;       // constants.rs:11

// planner.rs:139-233
std::vector<sb_sample_range> detect_speech_regions(const float* prob, int64_t n_prob, int64_t audio_len, float threshold,
                                                   const sb_vad_segmentation_config& cfg);
// The same computation fed window by window.  regions() grows as regions become final: a region's end depends on
// where the next kept speech span starts (the gap between them is shared out as padding), so a region is final when
// the span after it has closed, and the last one when finish() is called.
class SpeechRegionStream {
  public:
    SpeechRegionStream(int64_t audio_len, float threshold, const sb_vad_segmentation_config& cfg);
    void push(const float* prob, int64_t n);
    void finish();
    const std::vector<sb_sample_range>& regions() const { return regions_; }
    int64_t windows_seen() const { return window_; }

  private:
    void on_speech(sb_sample_range s);
    int64_t audio_len_, min_speech_, min_silence_, pad_;
    float threshold_, negative_;
    bool triggered_ = false, silence_open_ = false, has_pending_ = false;
    int64_t speech_start_ = 0, silence_start_ = 0, window_ = 0;
    sb_sample_range pending_{0, 0};
    std::vector<sb_sample_range> regions_;
};
// planner.rs:242-284; returns false where the reference returns None
bool plan_region_subsegments(sb_sample_range region, const float* region_prob, int64_t n_prob,
                             const sb_vad_segmentation_config& cfg, int64_t max_chunk_samples,
                             std::vector<sb_sample_range>* out);
// long_form.rs:421-437,508-582
struct ExecutionPlan {
    std::vector<sb_chunk_task> tasks;
    std::vector<sb_region_task> regions;
};
void append_region_plan(ExecutionPlan* plan, sb_sample_range region, const float* prob, int64_t n_prob,
                        const sb_longform_config& cfg);  // build_region_plan, long_form.rs:508-548
ExecutionPlan build_vad_plan(const std::vector<sb_sample_range>& regions, const float* prob, int64_t n_prob,
                             const sb_longform_config& cfg);
ExecutionPlan build_fast_plan(int64_t audio_len, const sb_longform_config& cfg);  // long_form.rs:439-459

// ------------------------------------------------------------------ text
struct Vocabulary {
    std::vector<std::string> id_to_token;
    int64_t blank_id = 0;
    // what the text decoder needs of every token, worked out once when the vocabulary is read
    struct Shown {
        std::string display;  // the token with the word-boundary mark turned into a space (decode.rs:64)
        bool special;         // <...> other than <unk> (decode.rs:110-112)
        bool digits;          // only ASCII digits (true for the empty token, as in the reference)
    };
    std::vector<Shown> shown;
};

struct TimedToken {
    uint32_t token_id;
    std::string text;
    double start, end;
    float confidence;
};

struct TranscriptChunk {
    double start, end;
    std::string text;
};

struct TranscriptionResult {
    std::string text;
    std::vector<TranscriptChunk> chunks;
    std::vector<TimedToken> tokens;
    double duration_seconds = 0.0;
};

// vocab.rs:15-52.  Returns an empty string on success, else the error text; *io_error is set when the
// file could not be read.
std::string vocabulary_from_file(const std::string& path, Vocabulary* out, bool* io_error);
std::string vocabulary_from_text(const std::string& text, Vocabulary* out);
// str::trim (Unicode White_Space) as join_token_text applies it, long_form.rs:613-620
std::string trim_whitespace(const std::string& s);
// decode.rs:39-104.  untrimmed, if not null, receives the text before its final trim (the concatenation of the
// token texts, which is what the long-form chunks are rebuilt from, long_form.rs:613-620).
TranscriptionResult decode_tokens(const Vocabulary& vocab, const RawTokens& raw, double duration_seconds,
                                  std::string* untrimmed = nullptr);
// long_form.rs:344-374,602-647 for the single Overlap region of the Fast mode; `joined` is the concatenation of the
// tokens' texts (decode_tokens' untrimmed text)
TranscriptionResult long_form_result(std::vector<TimedToken> tokens, const std::string& joined, int64_t audio_len);
// long_form.rs:344-419,602-661: the result of an execution plan from its tasks' token streams (raw[i] is consumed)
TranscriptionResult build_plan_result(const Vocabulary& vocab, int64_t audio_len, const sb_chunk_task* tasks,
                                      const sb_region_task* regions, int64_t n_regions, std::vector<RawTokens>& raw);

}  // namespace sb
