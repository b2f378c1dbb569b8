// Host-side long-form logic: overlap chunk planning, task building, time offsets and the
// overlap merge.  Integer logic of the reference, restated for the host driver:
//   OverlapChunkConfig::{chunk,overlap,stride}_samples, plan   src/long_form/planner.rs:104-137
//   push_overlap_task                                          src/long_form.rs:566-582
//   parallel_worker_count                                      src/long_form.rs:594-600
//   apply_time_offsets                                         src/pipeline.rs:219-252
//   merge_overlapping_windows / merge_pair / ...               src/long_form/merge.rs:3-200
//
// The merge gives the reference's result but never scans the whole accumulated transcript:
// two tokens can only match if their frames differ by at most 25, so only the part of the left
// transcript from its first token with frame >= min(right frames) - 25 can take part; that index is
// found by binary search on the running prefix maximum of the left frames (which makes it exact even
// if the frames are not monotone).  Every match is a diagonal run of length >= 1, so when the
// contiguous search finds nothing the reference's LCS fallback finds nothing either and the
// midpoint cut decides; and for a contiguous run the gaps between anchors are empty, so the merged
// transcript is left[.. run end) + right[run end ..).
#include "longform.h"

#include <algorithm>
#include <cstdlib>

namespace sb {

namespace {
constexpr int64_t kRateHz = 16000;
constexpr int64_t kHopSamples = 160;
constexpr int64_t kEncFrameSamples = 1280;
constexpr int64_t kMatchFrames = 25;  // merge.rs:102

inline int64_t sat_sub(int64_t a, int64_t b) { return a > b ? a - b : 0; }
}  // namespace

int64_t overlap_chunk_samples(const sb_overlap_config& c) {
    const int64_t max_actual = sat_sub(c.max_model_samples, c.context_samples);
    const int64_t raw = std::max(sat_sub(max_actual, kHopSamples), kEncFrameSamples);
    return raw / kEncFrameSamples * kEncFrameSamples;
}

int64_t overlap_overlap_samples(const sb_overlap_config& c) {
    const double want = c.overlap_seconds * static_cast<double>(kRateHz);
    const int64_t requested = want > 0.0 ? static_cast<int64_t>(want) : 0;  // `as usize` saturates at 0
    const int64_t capped = std::min(requested, overlap_chunk_samples(c) / 2);
    return capped / kEncFrameSamples * kEncFrameSamples;
}

int64_t overlap_stride_samples(const sb_overlap_config& c) {
    const int64_t raw = sat_sub(overlap_chunk_samples(c), overlap_overlap_samples(c));
    return std::max(raw, kEncFrameSamples) / kEncFrameSamples * kEncFrameSamples;
}

std::vector<sb_chunk_task> plan_fast_tasks(int64_t audio_len, const sb_overlap_config& c) {
    std::vector<sb_chunk_task> tasks;
    const int64_t chunk = overlap_chunk_samples(c), stride = overlap_stride_samples(c);
    int64_t start = 0;
    while (start < audio_len) {
        const int64_t end = std::min(start + chunk, audio_len);
        const int64_t ctx_start = sat_sub(start, c.context_samples);
        tasks.push_back(sb_chunk_task{ctx_start, end, start, start - ctx_start});
        if (end == audio_len) break;
        start += stride;
    }
    return tasks;
}

int64_t parallel_worker_count(int64_t task_count, int64_t requested) {
    if (task_count <= 1) return 1;
    return std::min(std::max<int64_t>(requested, 1), task_count);
}

void apply_time_offsets(RawTokens& raw, int64_t frame_offset, int64_t context_frames) {
    if (context_frames == 0) {
        for (auto& f : raw.frame_indices) f += frame_offset;
        return;
    }
    size_t k = 0;
    for (size_t i = 0; i < raw.token_ids.size(); ++i) {
        if (raw.frame_indices[i] < context_frames) continue;
        raw.token_ids[k] = raw.token_ids[i];
        raw.frame_indices[k] = raw.frame_indices[i] - context_frames + frame_offset;
        raw.durations[k] = raw.durations[i];
        raw.confidences[k] = raw.confidences[i];
        ++k;
    }
    raw.token_ids.resize(k);
    raw.frame_indices.resize(k);
    raw.durations.resize(k);
    raw.confidences.resize(k);
}

// ---------------------------------------------------------------------------- merge
void OverlapMerger::append(const RawView& src, size_t from, size_t to) {
    for (size_t i = from; i < to; ++i) {
        m_.token_ids.push_back(src.token_ids[i]);
        m_.frame_indices.push_back(src.frame_indices[i]);
        m_.durations.push_back(src.durations[i]);
        m_.confidences.push_back(src.confidences[i]);
        const int64_t f = src.frame_indices[i];
        prefix_max_.push_back(prefix_max_.empty() ? f : std::max(prefix_max_.back(), f));
    }
}

void OverlapMerger::truncate(size_t n) {
    m_.token_ids.resize(n);
    m_.frame_indices.resize(n);
    m_.durations.resize(n);
    m_.confidences.resize(n);
    prefix_max_.resize(n);
}

void OverlapMerger::push(const RawView& right) {
    const size_t nr = right.n;
    if (nr == 0) return;                       // merge.rs:19-21
    const size_t nl = m_.token_ids.size();
    if (nl == 0) { append(right, 0, nr); return; }  // merge.rs:16-18

    // first left index that can match anything in `right`
    int64_t min_r = right.frame_indices[0];
    for (size_t i = 1; i < nr; ++i) min_r = std::min(min_r, right.frame_indices[i]);
    const int64_t threshold = min_r - kMatchFrames;
    const size_t lo = std::lower_bound(prefix_max_.begin(), prefix_max_.end(), threshold) - prefix_max_.begin();

    auto match = [&](size_t li, size_t ri) {
        return m_.token_ids[li] == right.token_ids[ri] &&
               std::llabs(m_.frame_indices[li] - right.frame_indices[ri]) <= kMatchFrames;
    };
    // merge.rs:36-60: first strictly-longest diagonal run in (left, right) scan order
    // right tokens later than every left frame + 25 cannot match either: only the others are visited
    const int64_t left_reach = prefix_max_.back() + kMatchFrames;
    std::vector<uint32_t>& near = near_;
    near.clear();
    for (size_t ri = 0; ri < nr; ++ri)
        if (right.frame_indices[ri] <= left_reach) near.push_back((uint32_t)ri);
    size_t best = 0, bl = 0, br = 0;
    for (size_t li = lo; li < nl; ++li)
        for (const uint32_t ri : near) {
            if (!match(li, ri)) continue;
            // the tail of a run that began one step up the diagonal: that run was met first and is longer
            if (li > lo && ri > 0 && match(li - 1, ri - 1)) continue;
            size_t a = li, b = ri, len = 0;
            while (a < nl && b < nr && match(a, b)) { ++a; ++b; ++len; }
            if (len > best) { best = len; bl = li; br = ri; }
        }
    if (best > 0) {
        // merge.rs:105-140 with contiguous anchors: left[.. bl + best) then right[br + best ..)
        truncate(bl + best);
        append(right, br + best, nr);
        return;
    }
    // merge.rs:142-165: cut at the midpoint between the last left and the first right frame
    const int64_t midpoint = (m_.frame_indices[nl - 1] + right.frame_indices[0]) / 2;
    const size_t first_ge = std::lower_bound(prefix_max_.begin(), prefix_max_.end(), midpoint) - prefix_max_.begin();
    // everything before first_ge is < midpoint; filter the (short) rest
    RawTokens tail;
    for (size_t i = first_ge; i < nl; ++i) {
        if (m_.frame_indices[i] >= midpoint) continue;
        tail.token_ids.push_back(m_.token_ids[i]);
        tail.frame_indices.push_back(m_.frame_indices[i]);
        tail.durations.push_back(m_.durations[i]);
        tail.confidences.push_back(m_.confidences[i]);
    }
    truncate(first_ge);
    append(RawView{tail.token_ids.data(), tail.frame_indices.data(), tail.durations.data(), tail.confidences.data(),
                   tail.token_ids.size()},
           0, tail.token_ids.size());
    for (size_t i = 0; i < nr; ++i)
        if (right.frame_indices[i] >= midpoint) append(right, i, i + 1);
}

RawTokens merge_overlapping_windows(const std::vector<RawTokens>& windows) {
    OverlapMerger m;
    for (const auto& w : windows) m.push(w);
    return m.take();
}

}  // namespace sb
