// Host half of the sampling path: the thinking-budget control and the
// helpers that emit the token groups it asks for. A from-scratch C++
// restatement of the behaviour of the reference's src/thinking.rs and
// src/generate.rs:121-169, behind the C ABI of include/lily_thinking.h.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "../../include/lily_thinking.h"
#include "unicode_tables.h"

namespace {

// ------------------------------------------------------------ characters --

bool in_ranges(const uint32_t (*table)[2], unsigned count, uint32_t cp) {
    unsigned lo = 0, hi = count;
    while (lo < hi) {
        const unsigned mid = (lo + hi) / 2;
        if (cp < table[mid][0]) {
            hi = mid;
        } else if (cp > table[mid][1]) {
            lo = mid + 1;
        } else {
            return true;
        }
    }
    return false;
}

// Rust's char::is_whitespace / char::is_alphanumeric.
bool is_whitespace(uint32_t cp) { return in_ranges(kWhiteSpace, kWhiteSpace_count, cp); }
bool is_alphanumeric(uint32_t cp) { return in_ranges(kAlphanumeric, kAlphanumeric_count, cp); }

// Decodes one scalar value of well-formed UTF-8 (malformed bytes come out as
// U+FFFD, one per byte).
uint32_t next_char(const std::string &s, size_t &i) {
    const unsigned char b0 = (unsigned char)s[i];
    auto cont = [&](size_t k) { return i + k < s.size() && ((unsigned char)s[i + k] & 0xC0) == 0x80; };
    if (b0 < 0x80) {
        i += 1;
        return b0;
    }
    if ((b0 & 0xE0) == 0xC0 && cont(1)) {
        const uint32_t cp = ((b0 & 0x1Fu) << 6) | ((unsigned char)s[i + 1] & 0x3Fu);
        i += 2;
        return cp;
    }
    if ((b0 & 0xF0) == 0xE0 && cont(1) && cont(2)) {
        const uint32_t cp = ((b0 & 0x0Fu) << 12) | (((unsigned char)s[i + 1] & 0x3Fu) << 6) |
                            ((unsigned char)s[i + 2] & 0x3Fu);
        i += 3;
        return cp;
    }
    if ((b0 & 0xF8) == 0xF0 && cont(1) && cont(2) && cont(3)) {
        const uint32_t cp = ((b0 & 0x07u) << 18) | (((unsigned char)s[i + 1] & 0x3Fu) << 12) |
                            (((unsigned char)s[i + 2] & 0x3Fu) << 6) |
                            ((unsigned char)s[i + 3] & 0x3Fu);
        i += 4;
        return cp;
    }
    i += 1;
    return 0xFFFD;
}

void append_utf8(std::string &out, uint32_t cp) {
    if (cp < 0x80) {
        out.push_back((char)cp);
    } else if (cp < 0x800) {
        out.push_back((char)(0xC0 | (cp >> 6)));
        out.push_back((char)(0x80 | (cp & 0x3F)));
    } else if (cp < 0x10000) {
        out.push_back((char)(0xE0 | (cp >> 12)));
        out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
        out.push_back((char)(0x80 | (cp & 0x3F)));
    } else {
        out.push_back((char)(0xF0 | (cp >> 18)));
        out.push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
        out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
        out.push_back((char)(0x80 | (cp & 0x3F)));
    }
}

// str::trim: White_Space off both ends.
std::string trim(const std::string &s) {
    size_t begin = 0, end = s.size();
    while (begin < end) {
        size_t j = begin;
        if (!is_whitespace(next_char(s, j))) {
            break;
        }
        begin = j;
    }
    while (end > begin) {
        size_t j = end - 1;
        while (j > begin && ((unsigned char)s[j] & 0xC0) == 0x80) {
            --j;
        }
        size_t k = j;
        if (!is_whitespace(next_char(s, k))) {
            break;
        }
        end = j;
    }
    return s.substr(begin, end - begin);
}

bool ends_with(const std::string &s, const char *suffix) {
    const size_t n = std::strlen(suffix);
    return s.size() >= n && std::memcmp(s.data() + s.size() - n, suffix, n) == 0;
}

// ------------------------------------------------- src/thinking.rs:648-844 --

const char *kToolStart = "<tool_call>";
const char *kToolEnd = "</tool_call>";

struct Fence {
    uint32_t ch = 0;
    size_t len = 0;
};

// The whitespace CommonMark allows after a closing fence (src/thinking.rs:661).
bool blank_char(uint32_t c) { return c == ' ' || c == '\t' || c == '\r'; }

// What the current line starts with, for the fence rules (src/thinking.rs:666-722).
struct Lead {
    enum Kind { Indent, Run, After, Text } kind = Indent;
    unsigned indent = 0;
    Fence run;
    bool blank = false, tick = false;

    static Lead text() {
        Lead l;
        l.kind = Text;
        return l;
    }

    Lead next(uint32_t c) const {
        Lead out = *this;
        switch (kind) {
        case Indent:
            if (c == ' ' && indent < 3) {
                out.indent = indent + 1;
            } else if (c == '`' || c == '~') {
                out.kind = Run;
                out.run.ch = c;
                out.run.len = 1;
            } else {
                out = text();
            }
            return out;
        case Run:
            if (c == run.ch) {
                out.run.len = run.len + 1;
            } else if (run.len >= 3) {
                out.kind = After;
                out.blank = blank_char(c);
                out.tick = c == '`';
            } else {
                out = text();
            }
            return out;
        case After:
            out.blank = blank && blank_char(c);
            out.tick = tick || c == '`';
            return out;
        case Text:
        default:
            return text();
        }
    }

    // The fence this line opens, if it ends here.
    bool opens(Fence *f) const {
        if (kind == Run && run.len >= 3) {
            *f = run;
            return true;
        }
        if (kind == After && !(run.ch == '`' && tick)) {
            *f = run;
            return true;
        }
        return false;
    }

    // Whether this line closes `open`, if it ends here.
    bool closes(const Fence &open) const {
        if (kind == Run || (kind == After && blank)) {
            return run.ch == open.ch && run.len >= open.len;
        }
        return false;
    }
};

// Where a reasoning text stands, character by character (src/thinking.rs:731-844).
class ReasoningScan {
  public:
    void feed(const std::string &text) {
        size_t i = 0;
        while (i < text.size()) {
            push(next_char(text, i));
        }
    }

    size_t trailing_newlines() const { return trailing_newlines_; }
    bool has_last() const { return has_last_; }
    uint32_t last_char() const { return last_; }
    bool in_call() const { return in_call_; }

    bool in_fence() const {
        if (has_fence_) {
            return !lead_.closes(fence_);
        }
        Fence f;
        return !in_call_ && lead_.opens(&f);
    }

    bool call_may_start() const { return trailing_newlines_ > 0 && !has_fence_ && !in_call_; }

  private:
    void push(uint32_t c) {
        has_last_ = true;
        last_ = c;
        append_utf8(tail_, c);
        const size_t keep = std::strlen(kToolEnd);
        if (tail_.size() > keep) {
            size_t cut = tail_.size() - keep;
            while (cut < tail_.size() && ((unsigned char)tail_[cut] & 0xC0) == 0x80) {
                ++cut;
            }
            tail_.erase(0, cut);
        }
        if (c == '\n') {
            trailing_newlines_ += 1;
            if (!in_call_) {
                if (has_fence_) {
                    if (lead_.closes(fence_)) {
                        has_fence_ = false;
                    }
                } else {
                    Fence f;
                    if (lead_.opens(&f)) {
                        has_fence_ = true;
                        fence_ = f;
                    }
                }
            }
            lead_ = Lead();
            line_len_ = 0;
            return;
        }
        trailing_newlines_ = 0;
        line_len_ += 1;
        if (in_call_) {
            if (ends_with(tail_, kToolEnd)) {
                in_call_ = false;
            }
            return;
        }
        if (!has_fence_ && line_len_ == std::strlen(kToolStart) && ends_with(tail_, kToolStart)) {
            in_call_ = true;
            lead_ = Lead::text();
            return;
        }
        lead_ = lead_.next(c);
    }

    size_t trailing_newlines_ = 1;  // the prompt's "<think>\n" ended a line
    bool has_last_ = false;
    uint32_t last_ = 0;
    size_t line_len_ = 0;
    Lead lead_;
    bool has_fence_ = false;
    Fence fence_;
    bool in_call_ = false;
    std::string tail_;
};

// ------------------------------------------------- src/thinking.rs:182-326 --

struct Insert {
    std::vector<uint32_t> ids;
    std::string text;
};

enum class Seam { LineStart, Word, Symbol };

struct Placed {
    Insert line_start, word, symbol;
    const Insert &at(Seam s) const {
        return s == Seam::LineStart ? line_start : (s == Seam::Word ? word : symbol);
    }
};

struct NudgeLevelTokens {
    double at = 0;
    std::vector<Placed> variants;
};

struct Texts {
    std::vector<std::string> close;
    std::vector<std::pair<double, std::vector<std::string>>> nudges;
};

Texts builtin_texts() {
    Texts t;
    t.close = {
        "I've thought enough; time to act: make the next tool call or give the answer.",
        "That is enough thinking. Now I act: the next tool call, or the answer.",
        "Time to stop thinking and act: make the next tool call or give the answer.",
    };
    t.nudges = {
        {0.5,
         {"I should start converging on a decision.", "Time to start converging on a decision.",
          "I should begin narrowing this down to a decision."}},
        {0.75,
         {"I need to wrap up my thinking and decide the next action.",
          "I need to wrap this up and settle on the next action.",
          "Time to wrap up and decide what to do next."}},
        {0.9,
         {"I must stop deliberating now.", "I must stop deliberating and act now.",
          "No more deliberation: I must act now."}},
    };
    return t;
}

}  // namespace

struct lily_thinking_tokens {
    uint32_t think_end = 0, tool_call = 0, tool_call_end = 0;
    std::vector<uint32_t> close_tag;
    std::vector<Placed> closes;
    Placed bare_close;
    std::vector<NudgeLevelTokens> nudges;
};

namespace {

struct Encoder {
    lily_encode_fn encode;
    lily_is_added_fn is_added;
    void *user;

    bool run(const std::string &s, std::vector<uint32_t> *out, std::string *err) const {
        std::vector<uint32_t> buf(s.size() + 8);
        int32_t n = encode(user, s.data(), (uint32_t)s.size(), buf.data(), (uint32_t)buf.size());
        if (n > (int32_t)buf.size()) {
            buf.resize((size_t)n);
            n = encode(user, s.data(), (uint32_t)s.size(), buf.data(), (uint32_t)buf.size());
        }
        if (n < 0 || n > (int32_t)buf.size()) {
            *err = "the tokenizer failed to encode a thinking text";
            return false;
        }
        buf.resize((size_t)n);
        *out = std::move(buf);
        return true;
    }
};

std::string quoted(const std::string &s) {
    std::string out = "\"";
    for (char ch : s) {
        if (ch == '"' || ch == '\\') {
            out.push_back('\\');
        }
        if (ch == '\n') {
            out += "\\n";
        } else {
            out.push_back(ch);
        }
    }
    return out + "\"";
}

// `text` on a line of its own after each kind of seam, then `end` and `tail`
// (src/thinking.rs:264-287).
bool place(const lily_thinking_tokens &t, const Encoder &enc, const std::string &raw,
           const char *end, const std::vector<uint32_t> &tail_ids, const char *tail_text,
           Placed *out, std::string *err) {
    const std::string text = trim(raw);
    auto with = [&](const char *lead, const char *empty, Insert *ins) {
        const std::string s = text.empty() ? std::string(empty) : std::string(lead) + text + end;
        std::vector<uint32_t> ids;
        if (!s.empty() && !enc.run(s, &ids, err)) {
            return false;
        }
        for (uint32_t id : ids) {
            if (enc.is_added(enc.user, id) || id == t.think_end || id == t.tool_call ||
                id == t.tool_call_end) {
                *err = "the thinking text " + quoted(text) +
                       " encodes a special or added token (such as </think>, a tool call tag or "
                       "<|im_end|>)";
                return false;
            }
        }
        ids.insert(ids.end(), tail_ids.begin(), tail_ids.end());
        if (ids.empty()) {
            *err = "an inserted text encodes to nothing";
            return false;
        }
        ins->ids = std::move(ids);
        ins->text = s + tail_text;
        return true;
    };
    return with("", "", &out->line_start) && with("\n\n", "\n", &out->word) &&
           with(" \n\n", " \n", &out->symbol);
}

int32_t build_tokens(uint32_t think_end, uint32_t tool_call, uint32_t tool_call_end,
                     const Texts &texts, const Encoder &enc, lily_thinking_tokens_t **out,
                     std::string *err) {
    auto t = std::make_unique<lily_thinking_tokens>();
    t->think_end = think_end;
    t->tool_call = tool_call;
    t->tool_call_end = tool_call_end;
    std::vector<uint32_t> paragraph;
    if (!enc.run("\n\n", &paragraph, err)) {
        return 1;
    }
    if (paragraph.empty()) {
        *err = "\"\\n\\n\" encodes to nothing";
        return 1;
    }
    t->close_tag.push_back(think_end);
    t->close_tag.insert(t->close_tag.end(), paragraph.begin(), paragraph.end());
    const char *close_text = "</think>\n\n";
    for (const std::string &c : texts.close) {
        Placed p;
        if (!place(*t, enc, c, "\n", t->close_tag, close_text, &p, err)) {
            return 1;
        }
        t->closes.push_back(std::move(p));
    }
    if (!place(*t, enc, "", "\n", t->close_tag, close_text, &t->bare_close, err)) {
        return 1;
    }
    double previous = 0.0;
    for (const auto &level : texts.nudges) {
        if (!(level.first > previous && level.first < 1.0)) {
            char buf[128];
            std::snprintf(buf, sizeof buf,
                          "nudge levels must be ascending fractions of the budget in (0, 1), got %g",
                          level.first);
            *err = buf;
            return 1;
        }
        previous = level.first;
        NudgeLevelTokens lt;
        lt.at = level.first;
        for (const std::string &text : level.second) {
            if (trim(text).empty()) {
                continue;
            }
            Placed p;
            if (!place(*t, enc, text, "\n\n", {}, "", &p, err)) {
                return 1;
            }
            lt.variants.push_back(std::move(p));
        }
        if (lt.variants.empty()) {
            char buf[96];
            std::snprintf(buf, sizeof buf, "the nudge level at %g has no text", level.first);
            *err = buf;
            return 1;
        }
        t->nudges.push_back(std::move(lt));
    }
    *out = t.release();
    return 0;
}

void write_err(const std::string &msg, char *err, uint32_t cap) {
    if (err != nullptr && cap > 0) {
        std::snprintf(err, cap, "%s", msg.c_str());
    }
}

// ------------------------------------------------------------- tiny JSON --
// Just enough for {"close": [...], "nudges": [{"at": n, "texts": [...]}]},
// with unknown fields refused as the reference's serde attributes do.

struct Json {
    const char *p, *end;
    std::string err;

    void ws() {
        while (p < end && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r')) {
            ++p;
        }
    }
    bool eat(char ch) {
        ws();
        if (p < end && *p == ch) {
            ++p;
            return true;
        }
        return false;
    }
    bool fail(const char *what) {
        if (err.empty()) {
            err = std::string("parsing thinking texts: ") + what;
        }
        return false;
    }
    bool string(std::string *out) {
        ws();
        if (p >= end || *p != '"') {
            return fail("expected a string");
        }
        ++p;
        out->clear();
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) {
                    return fail("unterminated escape");
                }
                switch (*p) {
                case 'n': out->push_back('\n'); break;
                case 't': out->push_back('\t'); break;
                case 'r': out->push_back('\r'); break;
                case 'b': out->push_back('\b'); break;
                case 'f': out->push_back('\f'); break;
                case '/': out->push_back('/'); break;
                case '\\': out->push_back('\\'); break;
                case '"': out->push_back('"'); break;
                case 'u': {
                    auto hex4 = [&](uint32_t *v) {
                        if (end - p < 5) {
                            return false;
                        }
                        *v = 0;
                        for (int i = 1; i <= 4; ++i) {
                            const char h = p[i];
                            uint32_t d;
                            if (h >= '0' && h <= '9') {
                                d = h - '0';
                            } else if (h >= 'a' && h <= 'f') {
                                d = h - 'a' + 10;
                            } else if (h >= 'A' && h <= 'F') {
                                d = h - 'A' + 10;
                            } else {
                                return false;
                            }
                            *v = *v * 16 + d;
                        }
                        p += 4;
                        return true;
                    };
                    uint32_t cp;
                    if (!hex4(&cp)) {
                        return fail("bad \\u escape");
                    }
                    if (cp >= 0xD800 && cp < 0xDC00 && end - p >= 7 && p[1] == '\\' && p[2] == 'u') {
                        p += 2;
                        uint32_t lo;
                        if (!hex4(&lo) || lo < 0xDC00 || lo > 0xDFFF) {
                            return fail("bad surrogate pair");
                        }
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    append_utf8(*out, cp);
                    break;
                }
                default: return fail("unknown escape");
                }
                ++p;
            } else {
                out->push_back(*p++);
            }
        }
        if (p >= end) {
            return fail("unterminated string");
        }
        ++p;
        return true;
    }
    bool number(double *out) {
        ws();
        char *stop = nullptr;
        std::string tmp(p, (size_t)(end - p) < 64 ? (size_t)(end - p) : 64);
        *out = std::strtod(tmp.c_str(), &stop);
        if (stop == tmp.c_str()) {
            return fail("expected a number");
        }
        p += stop - tmp.c_str();
        return true;
    }
    bool strings(std::vector<std::string> *out) {
        if (!eat('[')) {
            return fail("expected an array");
        }
        if (eat(']')) {
            return true;
        }
        do {
            std::string s;
            if (!string(&s)) {
                return false;
            }
            out->push_back(std::move(s));
        } while (eat(','));
        return eat(']') || fail("expected ] or ,");
    }
};

bool parse_texts(const char *json, uint32_t len, Texts *out, std::string *err) {
    Json j{json, json + len, {}};
    auto done = [&](bool ok) {
        if (!ok) {
            *err = j.err.empty() ? "parsing thinking texts failed" : j.err;
        }
        return ok;
    };
    if (!j.eat('{')) {
        return done(j.fail("expected an object"));
    }
    if (!j.eat('}')) {
        do {
            std::string key;
            if (!j.string(&key) || !j.eat(':')) {
                return done(j.fail("expected a field"));
            }
            if (key == "close") {
                if (!j.strings(&out->close)) {
                    return done(false);
                }
            } else if (key == "nudges") {
                if (!j.eat('[')) {
                    return done(j.fail("expected an array"));
                }
                if (!j.eat(']')) {
                    do {
                        if (!j.eat('{')) {
                            return done(j.fail("expected a nudge level"));
                        }
                        double at = 0;
                        bool has_at = false, has_texts = false;
                        std::vector<std::string> texts;
                        do {
                            std::string k2;
                            if (!j.string(&k2) || !j.eat(':')) {
                                return done(j.fail("expected a field"));
                            }
                            if (k2 == "at") {
                                has_at = j.number(&at);
                                if (!has_at) {
                                    return done(false);
                                }
                            } else if (k2 == "texts") {
                                has_texts = j.strings(&texts);
                                if (!has_texts) {
                                    return done(false);
                                }
                            } else {
                                return done(j.fail("unknown field in a nudge level"));
                            }
                        } while (j.eat(','));
                        if (!j.eat('}') || !has_at || !has_texts) {
                            return done(j.fail("a nudge level needs \"at\" and \"texts\""));
                        }
                        out->nudges.emplace_back(at, std::move(texts));
                    } while (j.eat(','));
                    if (!j.eat(']')) {
                        return done(j.fail("expected ] or ,"));
                    }
                }
            } else {
                return done(j.fail("unknown field"));
            }
        } while (j.eat(','));
        if (!j.eat('}')) {
            return done(j.fail("expected } or ,"));
        }
    }
    j.ws();
    return done(j.p == j.end || j.fail("trailing characters"));
}

}  // namespace

// ------------------------------------------------- src/thinking.rs:397-646 --

struct lily_thinking_control {
    const lily_thinking_tokens *tokens = nullptr;
    lily_thinking_settings_t settings{};
    bool open = false;
    size_t counted = 0;
    size_t level = 0;
    size_t nudged = 0;
    ReasoningScan scan;
    bool has_closed = false;
    int32_t closed_by = 0;
    size_t closed_tokens = 0;
    std::vector<uint32_t> action_ids;

    bool has_budget() const { return settings.budget >= 0; }

    bool tool_call_would_close() const {
        return settings.tool_call_ends_thinking != 0 && scan.call_may_start();
    }

    // Where an insertion lands if it lands now; false mid-line right after
    // whitespace, where no seam is clean.
    bool seam(Seam *out) const {
        if (scan.trailing_newlines() > 0 || !scan.has_last()) {
            *out = Seam::LineStart;
            return true;
        }
        const uint32_t c = scan.last_char();
        if (is_whitespace(c)) {
            return false;
        }
        *out = is_alphanumeric(c) ? Seam::Word : Seam::Symbol;
        return true;
    }

    bool nudge_at(size_t lvl, size_t *at) const {
        if (!has_budget() || settings.nudges == 0 || lvl >= tokens->nudges.size()) {
            return false;
        }
        const double x = std::ceil(tokens->nudges[lvl].at * (double)settings.budget);
        const size_t v = x <= 0 ? 0 : (size_t)x;
        *at = v < 1 ? 1 : v;
        return true;
    }

    size_t pick(size_t offset, size_t len) const {
        return (size_t)((settings.seed + (uint64_t)offset) % (uint64_t)len);
    }

    bool close_seam(size_t over, Seam *out) const {
        if (scan.in_call() || scan.in_fence()) {
            return false;
        }
        Seam s;
        if (!seam(&s)) {
            return false;
        }
        const size_t grace = (size_t)settings.grace;
        const uint32_t last = scan.has_last() ? scan.last_char() : 0;
        const bool sentence_end = scan.has_last() && (last == '.' || last == '!' || last == '?');
        if (over >= 2 * grace || s == Seam::LineStart || (over >= grace && sentence_end)) {
            *out = s;
            return true;
        }
        return false;
    }

    enum class Place { Wait, Here, Never };

    Place nudge_place(size_t over) const {
        const size_t grace = (size_t)settings.grace;
        if (over <= grace && scan.trailing_newlines() > 0 && !scan.in_fence() && !scan.in_call()) {
            return Place::Here;
        }
        return over >= grace ? Place::Never : Place::Wait;
    }

    int32_t act(int32_t kind, const std::vector<uint32_t> &ids) {
        action_ids = ids;
        return kind;
    }

    int32_t decide(uint32_t token, const std::string &text) {
        action_ids.clear();
        if (!open) {
            return LILY_ACTION_KEEP;
        }
        if (token == tokens->think_end) {
            open = false;  // closed by the model itself
            return LILY_ACTION_KEEP;
        }
        if (token == tokens->tool_call && tool_call_would_close()) {
            open = false;
            has_closed = true;
            closed_by = LILY_CLOSED_TOOL_CALL;
            closed_tokens = counted;
            return act(LILY_ACTION_BEFORE, tokens->close_tag);
        }
        counted += 1;
        scan.feed(text);
        if (!has_budget()) {
            return LILY_ACTION_KEEP;
        }
        const size_t budget = (size_t)settings.budget;
        if (counted >= budget) {
            Seam s;
            if (close_seam(counted - budget, &s)) {
                open = false;
                has_closed = true;
                closed_by = LILY_CLOSED_BUDGET;
                closed_tokens = counted;
                const Placed &p = tokens->closes.empty()
                                      ? tokens->bare_close
                                      : tokens->closes[pick(0, tokens->closes.size())];
                return act(LILY_ACTION_AFTER, p.at(s).ids);
            }
            return LILY_ACTION_KEEP;
        }
        size_t at = 0;
        if (!nudge_at(level, &at) || counted < at) {
            return LILY_ACTION_KEEP;
        }
        switch (nudge_place(counted - at)) {
        case Place::Wait:
            return LILY_ACTION_KEEP;
        case Place::Never:
            level += 1;
            return LILY_ACTION_KEEP;
        case Place::Here:
        default: {
            const auto &variants = tokens->nudges[level].variants;
            const Insert &insert = variants[pick(level, variants.size())].at(Seam::LineStart);
            level += 1;
            nudged += 1;
            scan.feed(insert.text);  // read like the model's own text
            return act(LILY_ACTION_AFTER, insert.ids);
        }
        }
    }

    int32_t decide_stop() {
        action_ids.clear();
        if (!open || !has_budget()) {
            return LILY_ACTION_KEEP;
        }
        open = false;
        has_closed = true;
        closed_by = LILY_CLOSED_END_OF_TURN;
        closed_tokens = counted;
        Seam s;
        if (!seam(&s)) {
            s = Seam::Word;  // no clean seam after whitespace: take the break
        }
        return act(LILY_ACTION_REPLACE, tokens->bare_close.at(s).ids);
    }
};

extern "C" {

int32_t lily_thinking_tokens_create(uint32_t think_end, uint32_t tool_call, uint32_t tool_call_end,
                                    const lily_thinking_texts_t *texts, lily_encode_fn encode,
                                    lily_is_added_fn is_added, void *user,
                                    lily_thinking_tokens_t **out, char *err, uint32_t err_cap) {
    if (out == nullptr || encode == nullptr || is_added == nullptr) {
        write_err("null argument", err, err_cap);
        return 1;
    }
    *out = nullptr;
    Texts t;
    if (texts == nullptr) {
        t = builtin_texts();
    } else {
        for (uint32_t i = 0; i < texts->n_close; ++i) {
            t.close.emplace_back(texts->close[i]);
        }
        for (uint32_t i = 0; i < texts->n_nudges; ++i) {
            std::vector<std::string> v;
            for (uint32_t j = 0; j < texts->nudges[i].n_texts; ++j) {
                v.emplace_back(texts->nudges[i].texts[j]);
            }
            t.nudges.emplace_back(texts->nudges[i].at, std::move(v));
        }
    }
    std::string msg;
    const int32_t st =
        build_tokens(think_end, tool_call, tool_call_end, t, Encoder{encode, is_added, user}, out, &msg);
    if (st != 0) {
        write_err(msg, err, err_cap);
    }
    return st;
}

int32_t lily_thinking_tokens_create_json(uint32_t think_end, uint32_t tool_call,
                                         uint32_t tool_call_end, const char *json, uint32_t json_len,
                                         lily_encode_fn encode, lily_is_added_fn is_added,
                                         void *user, lily_thinking_tokens_t **out, char *err,
                                         uint32_t err_cap) {
    if (out == nullptr || encode == nullptr || is_added == nullptr || json == nullptr) {
        write_err("null argument", err, err_cap);
        return 1;
    }
    *out = nullptr;
    Texts t;
    std::string msg;
    if (!parse_texts(json, json_len, &t, &msg)) {
        write_err(msg, err, err_cap);
        return 1;
    }
    const int32_t st =
        build_tokens(think_end, tool_call, tool_call_end, t, Encoder{encode, is_added, user}, out, &msg);
    if (st != 0) {
        write_err(msg, err, err_cap);
    }
    return st;
}

void lily_thinking_tokens_destroy(lily_thinking_tokens_t *t) { delete t; }

int32_t lily_thinking_settings_any(const lily_thinking_settings_t *s) {
    return s != nullptr && (s->budget >= 0 || s->tool_call_ends_thinking != 0);
}

lily_thinking_control_t *lily_thinking_control_create(const lily_thinking_tokens_t *tokens,
                                                      const lily_thinking_settings_t *settings,
                                                      int32_t opens_thinking) {
    if (tokens == nullptr || settings == nullptr) {
        return nullptr;
    }
    auto *c = new lily_thinking_control();
    c->tokens = tokens;
    c->settings = *settings;
    c->open = opens_thinking != 0;
    return c;
}

void lily_thinking_control_destroy(lily_thinking_control_t *c) { delete c; }

int32_t lily_thinking_is_open(const lily_thinking_control_t *c) { return c && c->open; }

int32_t lily_thinking_closed(const lily_thinking_control_t *c, int32_t *by,
                             uint64_t *thinking_tokens) {
    if (c == nullptr || !c->has_closed) {
        return 0;
    }
    if (by) {
        *by = c->closed_by;
    }
    if (thinking_tokens) {
        *thinking_tokens = c->closed_tokens;
    }
    return 1;
}

int32_t lily_thinking_close_emitted(const lily_thinking_control_t *c, const uint32_t *generated,
                                    uint64_t n) {
    if (c == nullptr || !c->has_closed) {
        return 0;
    }
    for (uint64_t i = 0; i < n; ++i) {
        if (generated[i] == c->tokens->think_end) {
            return 1;
        }
    }
    return 0;
}

uint64_t lily_thinking_nudged(const lily_thinking_control_t *c) { return c ? c->nudged : 0; }

uint64_t lily_thinking_tokens_counted(const lily_thinking_control_t *c) {
    return c ? c->counted : 0;
}

int32_t lily_thinking_may_act_next(const lily_thinking_control_t *c) {
    return c && c->open && (c->has_budget() || c->tool_call_would_close());
}

int32_t lily_thinking_decide(lily_thinking_control_t *c, uint32_t token, const char *text_utf8,
                             uint32_t len) {
    if (c == nullptr) {
        return LILY_ACTION_KEEP;
    }
    return c->decide(token, std::string(text_utf8 ? text_utf8 : "", text_utf8 ? len : 0));
}

int32_t lily_thinking_decide_stop(lily_thinking_control_t *c) {
    return c ? c->decide_stop() : LILY_ACTION_KEEP;
}

void lily_thinking_action_ids(const lily_thinking_control_t *c, const uint32_t **ids, uint32_t *n) {
    if (ids) {
        *ids = c ? c->action_ids.data() : nullptr;
    }
    if (n) {
        *n = c ? (uint32_t)c->action_ids.size() : 0;
    }
}

int32_t lily_opens_thinking(const char *prompt_tail, uint32_t len) {
    const char *want = "<think>\n";
    const size_t n = std::strlen(want);
    return prompt_tail != nullptr && len >= n && std::memcmp(prompt_tail + len - n, want, n) == 0;
}

// ------------------------------------------------ src/generate.rs:121-169 --

int32_t lily_push_group(uint32_t *tokens, uint64_t *n, uint64_t cap, const uint32_t *group,
                        uint64_t n_group, uint64_t max_tokens, lily_on_token_fn on_token,
                        void *user, int32_t *finish) {
    if (tokens == nullptr || n == nullptr || finish == nullptr || on_token == nullptr ||
        (group == nullptr && n_group > 0)) {
        return 1;
    }
    int32_t end = LILY_FINISH_NONE;
    for (uint64_t i = 0; i < n_group; ++i) {
        if (*n >= max_tokens) {
            break;
        }
        if (*n >= cap) {
            return 2;
        }
        tokens[(*n)++] = group[i];
        const int32_t go = on_token(user, group[i]);
        if (go < 0) {
            return 3;
        }
        if (go == 0 && end == LILY_FINISH_NONE) {
            end = LILY_FINISH_CALLBACK;
        }
    }
    if (*n >= max_tokens && end == LILY_FINISH_NONE) {
        end = LILY_FINISH_LENGTH;
    }
    *finish = end;
    return 0;
}

int32_t lily_emit_acted(int32_t action, const uint32_t *group, uint64_t n_group, uint32_t drawn,
                        uint32_t *tokens, uint64_t *n, uint64_t cap, uint64_t max_tokens,
                        lily_on_token_fn on_token, void *user, int32_t *finish) {
    if (tokens == nullptr || n == nullptr || finish == nullptr || on_token == nullptr) {
        return 1;
    }
    switch (action) {
    case LILY_ACTION_BEFORE: {
        std::vector<uint32_t> whole(group, group + n_group);
        whole.push_back(drawn);
        return lily_push_group(tokens, n, cap, whole.data(), whole.size(), max_tokens, on_token,
                               user, finish);
    }
    case LILY_ACTION_REPLACE:
        return lily_push_group(tokens, n, cap, group, n_group, max_tokens, on_token, user, finish);
    case LILY_ACTION_AFTER: {
        if (*n >= cap) {
            return 2;
        }
        tokens[(*n)++] = drawn;
        const int32_t go = on_token(user, drawn);
        if (go < 0) {
            return 3;
        }
        int32_t rest = LILY_FINISH_NONE;
        const int32_t st =
            lily_push_group(tokens, n, cap, group, n_group, max_tokens, on_token, user, &rest);
        if (st != 0) {
            return st;
        }
        *finish = go == 0 ? LILY_FINISH_CALLBACK : rest;
        return 0;
    }
    default:
        return 4;  // emit_acted with nothing to insert
    }
}

}  // extern "C"
