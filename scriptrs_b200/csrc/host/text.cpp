// Token ids -> text with timestamps, and the vocabulary file parser.  Restates on the host
//   Vocabulary::from_file           src/vocab.rs:15-52
//   ParakeetTdtDecoder::decode      src/decode.rs:39-104
//   frame_to_seconds                src/decode.rs:106-108
//   is_special_token                src/decode.rs:110-112
//   needs_digit_spacing             src/decode.rs:114-134
//   join_token_text / build_chunk / build_result   src/long_form.rs:602-647
// Strings are UTF-8.  `char::is_alphabetic` is the Unicode derived property Alphabetic; it is evaluated from a
// generated table of that property's code-point ranges (unicode_alpha_table.h, written by make_alpha_table.py from
// Unicode 17.0 tables; a Rust toolchain on an older Unicode version differs only on code points assigned later).
#include <algorithm>
#include <cstdio>
#include <fstream>
#include <sstream>
#include <utility>

#include "longform.h"
#include "unicode_alpha_table.h"

namespace sb {

namespace {

constexpr double kSecondsPerFrame = 1280.0 / 16000.0;

// binary search in the generated table (sorted, non-overlapping ranges)
bool is_alphabetic(uint32_t cp) {
    int lo = 0, hi = kAlphaRangeCount - 1;
    while (lo <= hi) {
        const int mid = (lo + hi) / 2;
        if (cp < kAlphaRanges[mid].lo) hi = mid - 1;
        else if (cp > kAlphaRanges[mid].hi) lo = mid + 1;
        else return true;
    }
    return false;
}

bool is_whitespace(uint32_t cp) {
    return (cp >= 0x09 && cp <= 0x0D) || cp == 0x20 || cp == 0x85 || cp == 0xA0 || cp == 0x1680 ||
           (cp >= 0x2000 && cp <= 0x200A) || cp == 0x2028 || cp == 0x2029 || cp == 0x202F || cp == 0x205F ||
           cp == 0x3000;
}

// Decodes the code point that ends at byte `end` (exclusive); returns its first byte index.
size_t prev_char(const std::string& s, size_t end, uint32_t* cp) {
    size_t i = end - 1;
    while (i > 0 && (static_cast<unsigned char>(s[i]) & 0xC0) == 0x80) --i;
    const unsigned char b0 = static_cast<unsigned char>(s[i]);
    uint32_t v = b0;
    const size_t n = end - i;
    if (n == 2) v = b0 & 0x1F;
    else if (n == 3) v = b0 & 0x0F;
    else if (n == 4) v = b0 & 0x07;
    for (size_t k = 1; k < n; ++k) v = (v << 6) | (static_cast<unsigned char>(s[i + k]) & 0x3F);
    *cp = v;
    return i;
}

size_t next_char(const std::string& s, size_t i, uint32_t* cp) {
    const unsigned char b0 = static_cast<unsigned char>(s[i]);
    size_t n = 1;
    uint32_t v = b0;
    if (b0 >= 0xF0) { n = 4; v = b0 & 0x07; }
    else if (b0 >= 0xE0) { n = 3; v = b0 & 0x0F; }
    else if (b0 >= 0xC0) { n = 2; v = b0 & 0x1F; }
    for (size_t k = 1; k < n && i + k < s.size(); ++k) v = (v << 6) | (static_cast<unsigned char>(s[i + k]) & 0x3F);
    *cp = v;
    return i + n;
}

std::string trim(const std::string& s) {
    size_t a = 0, b = s.size();
    while (a < b) {
        uint32_t cp;
        const size_t nx = next_char(s, a, &cp);
        if (!is_whitespace(cp)) break;
        a = nx;
    }
    while (b > a) {
        uint32_t cp;
        const size_t pv = prev_char(s, b, &cp);
        if (!is_whitespace(cp)) break;
        b = pv;
    }
    return s.substr(a, b - a);
}

double frame_to_seconds(int64_t frame) { return static_cast<double>(frame * 160 * 8) / 16000.0; }

bool is_special_token(const std::string& t) {
    return !t.empty() && t.front() == '<' && t.back() == '>' && t != "<unk>";
}

// needs_digit_spacing (decode.rs:114-134) for a display string known to hold only digits and no leading space
bool digits_need_space(const std::string& existing) {
    if (existing.empty()) return false;
    size_t trailing = 0, end = existing.size();
    while (end > 0) {
        uint32_t cp;
        const size_t pv = prev_char(existing, end, &cp);
        if (!is_alphabetic(cp)) break;
        ++trailing;
        end = pv;
    }
    const bool is_article_a = trailing == 1 && existing.back() == 'a';
    return trailing > 1 || is_article_a;
}

std::string replace_underline(const std::string& t) {
    std::string out;
    out.reserve(t.size());
    for (size_t i = 0; i < t.size();) {
        if (i + 2 < t.size() && static_cast<unsigned char>(t[i]) == 0xE2 &&
            static_cast<unsigned char>(t[i + 1]) == 0x96 && static_cast<unsigned char>(t[i + 2]) == 0x81) {
            out.push_back(' ');
            i += 3;
        } else {
            out.push_back(t[i]);
            ++i;
        }
    }
    return out;
}

}  // namespace

std::string vocabulary_from_text(const std::string& text, Vocabulary* out) {
    out->id_to_token.clear();
    bool have_blank = false;
    int64_t blank = 0;
    size_t pos = 0;
    while (pos <= text.size()) {
        size_t nl = text.find('\n', pos);
        if (nl == std::string::npos) nl = text.size();
        std::string line = text.substr(pos, nl - pos);
        pos = nl + 1;
        if (!line.empty() && line.back() == '\r') line.pop_back();
        const size_t sp = line.find(' ');
        if (sp == std::string::npos) { if (nl == text.size()) break; continue; }
        const std::string token = line.substr(0, sp), idtxt = line.substr(sp + 1);
        size_t d = 0;
        if (!idtxt.empty() && idtxt[0] == '+') d = 1;
        bool ok = d < idtxt.size();
        for (size_t i = d; i < idtxt.size() && ok; ++i) ok = idtxt[i] >= '0' && idtxt[i] <= '9';
        if (!ok || idtxt.size() - d > 18) return "invalid token id `" + idtxt + "`";
        const int64_t id = std::stoll(idtxt.substr(d));
        if (id >= static_cast<int64_t>(out->id_to_token.size())) out->id_to_token.resize(id + 1);
        out->id_to_token[id] = token;
        if (token == "<blk>" || token == "<blank>") { blank = id; have_blank = true; }
        if (nl == text.size()) break;
    }
    if (out->id_to_token.empty()) return "vocabulary was empty";
    out->blank_id = have_blank ? blank : static_cast<int64_t>(out->id_to_token.size()) - 1;
    out->shown.clear();
    out->shown.reserve(out->id_to_token.size());
    for (const std::string& tok : out->id_to_token) {
        Vocabulary::Shown sh{replace_underline(tok), is_special_token(tok), true};
        for (char ch : sh.display)
            if (ch < '0' || ch > '9') sh.digits = false;
        out->shown.push_back(std::move(sh));
    }
    return "";
}

std::string vocabulary_from_file(const std::string& path, Vocabulary* out, bool* io_error) {
    *io_error = false;
    std::ifstream f(path, std::ios::binary);
    if (!f) { *io_error = true; return "cannot open " + path; }
    std::stringstream ss;
    ss << f.rdbuf();
    return vocabulary_from_text(ss.str(), out);
}

TranscriptionResult decode_tokens(const Vocabulary& vocab, const RawTokens& raw, double duration_seconds,
                                  std::string* untrimmed) {
    TranscriptionResult res;
    res.duration_seconds = duration_seconds;
    if (untrimmed) untrimmed->clear();
    if (raw.token_ids.empty()) return res;
    std::string text;
    res.tokens.reserve(raw.token_ids.size());
    text.reserve(raw.token_ids.size() * 4);
    const size_t n = raw.token_ids.size();
    for (size_t index = 0; index < n; ++index) {
        const uint32_t id = raw.token_ids[index];
        if (id >= vocab.shown.size()) continue;
        const Vocabulary::Shown& sh = vocab.shown[id];
        if (sh.special) continue;
        const double start = frame_to_seconds(raw.frame_indices[index]);
        double end;
        if (index + 1 < n) end = frame_to_seconds(raw.frame_indices[index + 1]);
        else end = std::min(start + kSecondsPerFrame, duration_seconds);
        const float conf = index < raw.confidences.size() ? raw.confidences[index] : 0.0f;
        // a digit token directly after a word gets a space in front (decode.rs:66-68)
        if (sh.digits && digits_need_space(text)) {
            text += ' ';
            text += sh.display;
            res.tokens.push_back(TimedToken{id, " " + sh.display, start, end, conf});
        } else {
            text += sh.display;
            res.tokens.push_back(TimedToken{id, sh.display, start, end, conf});
        }
    }
    res.text = trim(text);
    if (!res.text.empty() && !res.tokens.empty())
        res.chunks.push_back(TranscriptChunk{res.tokens.front().start, res.tokens.back().end, res.text});
    if (untrimmed) *untrimmed = std::move(text);
    return res;
}

std::string trim_whitespace(const std::string& s) { return trim(s); }

TranscriptionResult long_form_result(std::vector<TimedToken> tokens, const std::string& joined, int64_t audio_len) {
    TranscriptionResult res;
    res.duration_seconds = static_cast<double>(audio_len) / 16000.0;
    if (!tokens.empty()) {
        res.chunks.push_back(TranscriptChunk{tokens.front().start, tokens.back().end, trim(joined)});
        res.tokens = std::move(tokens);
    }
    for (size_t i = 0; i < res.chunks.size(); ++i) {
        if (i) res.text += " ";
        res.text += res.chunks[i].text;
    }
    return res;
}

}  // namespace sb
