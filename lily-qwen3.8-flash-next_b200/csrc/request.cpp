// Host side of include/lily_request.h: an OpenAI-style request's sampling and
// thinking fields resolved over the server's defaults, as the reference's
// serving layer does (src/serve/api.rs:436-457, 498-708, 798-888;
// src/serve.rs:1762-1835). Pure host code: no CUDA here.
#include <cerrno>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../../include/lily_request.h"

namespace {

// ---- a small JSON reader: enough to pick typed members out of an object and
// to skip everything else.

struct Json {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    double num = 0.0;
    bool integral = false;   // the number was written without fraction or exponent
    long long i64 = 0;       // its value when integral and in range
    bool i64_ok = false;
    unsigned long long u64 = 0;
    bool u64_ok = false;
    std::string str;
    std::vector<Json> items;
    std::vector<std::pair<std::string, Json>> members;

    const Json *get(const char *key) const {
        if (kind != Object) {
            return nullptr;
        }
        const Json *found = nullptr;
        for (const auto &m : members) {
            if (m.first == key) {
                found = &m.second;  // the last duplicate wins, as serde_json's map does
            }
        }
        return found;
    }
};

struct Parser {
    const char *p, *end;
    std::string error;

    bool fail(const char *what) {
        if (error.empty()) {
            error = what;
        }
        return false;
    }
    void ws() {
        while (p < end && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r')) {
            ++p;
        }
    }
    bool literal(const char *text) {
        const size_t n = std::strlen(text);
        if ((size_t)(end - p) < n || std::memcmp(p, text, n) != 0) {
            return fail("invalid JSON literal");
        }
        p += n;
        return true;
    }
    bool string(std::string &out) {
        if (p >= end || *p != '"') {
            return fail("expected a JSON string");
        }
        ++p;
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) {
                    return fail("unterminated JSON string");
                }
                switch (*p) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'u': {
                        if (end - p < 5) {
                            return fail("bad \\u escape");
                        }
                        unsigned cp = 0;
                        for (int k = 1; k <= 4; ++k) {
                            const char ch = p[k];
                            cp <<= 4;
                            if (ch >= '0' && ch <= '9') cp |= (unsigned)(ch - '0');
                            else if (ch >= 'a' && ch <= 'f') cp |= (unsigned)(ch - 'a' + 10);
                            else if (ch >= 'A' && ch <= 'F') cp |= (unsigned)(ch - 'A' + 10);
                            else return fail("bad \\u escape");
                        }
                        p += 4;
                        // Keys and values this layer reads are ASCII; others are kept as UTF-8
                        // of the code unit (surrogate pairs are not joined: never compared).
                        if (cp < 0x80) {
                            out += (char)cp;
                        } else if (cp < 0x800) {
                            out += (char)(0xC0 | (cp >> 6));
                            out += (char)(0x80 | (cp & 0x3F));
                        } else {
                            out += (char)(0xE0 | (cp >> 12));
                            out += (char)(0x80 | ((cp >> 6) & 0x3F));
                            out += (char)(0x80 | (cp & 0x3F));
                        }
                        break;
                    }
                    default: out += *p; break;  // \" \\ \/
                }
                ++p;
            } else {
                out += *p++;
            }
        }
        if (p >= end) {
            return fail("unterminated JSON string");
        }
        ++p;
        return true;
    }
    bool number(Json &v) {
        const char *s = p;
        if (p < end && *p == '-') {
            ++p;
        }
        bool digits = false, integral = true;
        while (p < end && *p >= '0' && *p <= '9') {
            ++p;
            digits = true;
        }
        if (p < end && *p == '.') {
            integral = false;
            ++p;
            while (p < end && *p >= '0' && *p <= '9') {
                ++p;
            }
        }
        if (p < end && (*p == 'e' || *p == 'E')) {
            integral = false;
            ++p;
            if (p < end && (*p == '+' || *p == '-')) {
                ++p;
            }
            while (p < end && *p >= '0' && *p <= '9') {
                ++p;
            }
        }
        if (!digits) {
            return fail("invalid JSON number");
        }
        const std::string text(s, p);
        v.kind = Json::Number;
        v.num = std::strtod(text.c_str(), nullptr);
        v.integral = integral;
        if (integral) {
            errno = 0;
            char *e = nullptr;
            const long long i = std::strtoll(text.c_str(), &e, 10);
            v.i64_ok = errno == 0 && e && *e == '\0';
            v.i64 = i;
            if (text[0] != '-') {
                errno = 0;
                const unsigned long long u = std::strtoull(text.c_str(), &e, 10);
                v.u64_ok = errno == 0 && e && *e == '\0';
                v.u64 = u;
            }
        }
        return true;
    }
    bool value(Json &v, int depth) {
        if (depth > 64) {
            return fail("JSON nested too deeply");
        }
        ws();
        if (p >= end) {
            return fail("unexpected end of JSON");
        }
        switch (*p) {
            case 'n': v.kind = Json::Null; return literal("null");
            case 't': v.kind = Json::Bool; v.b = true; return literal("true");
            case 'f': v.kind = Json::Bool; v.b = false; return literal("false");
            case '"': v.kind = Json::String; return string(v.str);
            case '[': {
                v.kind = Json::Array;
                ++p;
                ws();
                if (p < end && *p == ']') {
                    ++p;
                    return true;
                }
                for (;;) {
                    v.items.emplace_back();
                    if (!value(v.items.back(), depth + 1)) {
                        return false;
                    }
                    ws();
                    if (p < end && *p == ',') {
                        ++p;
                        continue;
                    }
                    if (p < end && *p == ']') {
                        ++p;
                        return true;
                    }
                    return fail("expected , or ] in a JSON array");
                }
            }
            case '{': {
                v.kind = Json::Object;
                ++p;
                ws();
                if (p < end && *p == '}') {
                    ++p;
                    return true;
                }
                for (;;) {
                    ws();
                    std::string key;
                    if (!string(key)) {
                        return false;
                    }
                    ws();
                    if (p >= end || *p != ':') {
                        return fail("expected : in a JSON object");
                    }
                    ++p;
                    v.members.emplace_back(std::move(key), Json());
                    if (!value(v.members.back().second, depth + 1)) {
                        return false;
                    }
                    ws();
                    if (p < end && *p == ',') {
                        ++p;
                        continue;
                    }
                    if (p < end && *p == '}') {
                        ++p;
                        return true;
                    }
                    return fail("expected , or } in a JSON object");
                }
            }
            default: return number(v);
        }
    }
};

bool parse_json(const char *text, uint32_t len, Json &out, std::string &error) {
    Parser ps{text, text + len, {}};
    if (!ps.value(out, 0)) {
        error = ps.error;
        return false;
    }
    ps.ws();
    if (ps.p != ps.end) {
        error = "trailing characters after the JSON value";
        return false;
    }
    return true;
}

int32_t refuse(char *err, uint32_t cap, int32_t code, const std::string &msg) {
    if (err != nullptr && cap > 0) {
        std::snprintf(err, cap, "%s", msg.c_str());
    }
    return code;
}

// src/kernels/sample.rs:57-79 SamplingParams::validate.
bool params_valid(const lily_sampling_params_t &p, std::string &why) {
    if (!(std::isfinite(p.temperature) && p.temperature >= 0.0f)) {
        why = "temperature must be finite and >= 0";
    } else if (!(std::isfinite(p.top_p) && p.top_p > 0.0f && p.top_p <= 1.0f)) {
        why = "top_p must be in (0, 1]";
    } else if (!(std::isfinite(p.min_p) && p.min_p >= 0.0f && p.min_p <= 1.0f)) {
        why = "min_p must be in [0, 1]";
    } else if (!(std::isfinite(p.repetition_penalty) && p.repetition_penalty > 0.0f)) {
        why = "repetition_penalty must be finite and > 0";
    } else if (!std::isfinite(p.presence_penalty) || !std::isfinite(p.frequency_penalty)) {
        why = "presence_penalty and frequency_penalty must be finite";
    } else {
        return true;
    }
    return false;
}

uint32_t clamp_top_k(unsigned long long k) { return k > 0xFFFFFFFFull ? 0xFFFFFFFFu : (uint32_t)k; }

// A member that must be a number (or null / absent): Option<f32>.
bool opt_f32(const Json &obj, const char *key, uint32_t bit, uint32_t &present, float &slot, std::string &error) {
    const Json *v = obj.get(key);
    if (v == nullptr || v->kind == Json::Null) {
        return true;
    }
    if (v->kind != Json::Number) {
        error = std::string(key) + " must be a number";
        return false;
    }
    slot = (float)v->num;
    present |= bit;
    return true;
}

// Option<i64>: an integer in range, written as one.
bool opt_i64(const Json &obj, const char *key, const char *prefix, uint32_t bit, uint32_t &present,
             int64_t &slot, std::string &error) {
    const Json *v = obj.get(key);
    if (v == nullptr || v->kind == Json::Null) {
        return true;
    }
    if (v->kind != Json::Number || !v->integral || !v->i64_ok) {
        error = std::string(prefix) + key + " must be an integer";
        return false;
    }
    slot = v->i64;
    present |= bit;
    return true;
}

bool opt_bool(const Json &obj, const char *key, const char *prefix, uint32_t bit, uint32_t &present,
              int32_t &slot, std::string &error) {
    const Json *v = obj.get(key);
    if (v == nullptr || v->kind == Json::Null) {
        return true;
    }
    if (v->kind != Json::Bool) {
        error = std::string(prefix) + key + " must be a boolean";
        return false;
    }
    slot = v->b ? 1 : 0;
    present |= bit;
    return true;
}

std::string trim(const std::string &s) {
    size_t a = 0, b = s.size();
    while (a < b && std::isspace((unsigned char)s[a])) {
        ++a;
    }
    while (b > a && std::isspace((unsigned char)s[b - 1])) {
        --b;
    }
    return s.substr(a, b - a);
}

// Rust's str::parse::<usize>: optional '+', decimal digits only.
bool parse_usize(const std::string &text, unsigned long long &out) {
    size_t i = 0;
    if (i < text.size() && text[i] == '+') {
        ++i;
    }
    if (i >= text.size()) {
        return false;
    }
    unsigned long long v = 0;
    for (; i < text.size(); ++i) {
        if (text[i] < '0' || text[i] > '9') {
            return false;
        }
        const unsigned d = (unsigned)(text[i] - '0');
        if (v > (0xFFFFFFFFFFFFFFFFull - d) / 10ull) {
            return false;
        }
        v = v * 10ull + d;
    }
    out = v;
    return true;
}

}  // namespace

extern "C" {

int32_t lily_sampling_defaults(const char *generation_config_json, uint32_t len,
                               const lily_sampling_overrides_t *overrides, int32_t validate,
                               lily_sampling_params_t *out, char *err, uint32_t err_cap) {
    if (out == nullptr) {
        return refuse(err, err_cap, LILY_ERR_ARG, "out is null");
    }
    lily_sampling_params_t p;
    std::memset(&p, 0, sizeof p);
    p.temperature = 1.0f;
    p.top_k = 0;
    p.top_p = 1.0f;
    p.min_p = 0.0f;
    p.repetition_penalty = 1.0f;
    if (generation_config_json != nullptr) {
        Json cfg;
        std::string error;
        if (!parse_json(generation_config_json, len, cfg, error)) {
            return refuse(err, err_cap, LILY_ERR_ARG, "parsing generation_config.json: " + error);
        }
        auto f = [&](const char *key, float &slot) {
            const Json *v = cfg.get(key);
            if (v != nullptr && v->kind == Json::Number) {
                slot = (float)v->num;
            }
        };
        const Json *ds = cfg.get("do_sample");
        if (ds != nullptr && ds->kind == Json::Bool && !ds->b) {
            p.temperature = 0.0f;
        }
        f("temperature", p.temperature);
        f("top_p", p.top_p);
        const Json *k = cfg.get("top_k");
        if (k != nullptr && k->kind == Json::Number && k->integral && k->u64_ok) {
            p.top_k = clamp_top_k(k->u64);
        }
        f("min_p", p.min_p);
        f("repetition_penalty", p.repetition_penalty);
        f("presence_penalty", p.presence_penalty);
    }
    if (overrides != nullptr) {
        const lily_sampling_overrides_t &o = *overrides;
        if (o.present & LILY_HAS_TEMPERATURE) p.temperature = o.temperature;
        if (o.present & LILY_HAS_TOP_K) p.top_k = clamp_top_k(o.top_k);
        if (o.present & LILY_HAS_TOP_P) p.top_p = o.top_p;
        if (o.present & LILY_HAS_MIN_P) p.min_p = o.min_p;
        if (o.present & LILY_HAS_PRESENCE) p.presence_penalty = o.presence_penalty;
        if (o.present & LILY_HAS_FREQUENCY) p.frequency_penalty = o.frequency_penalty;
        if (o.present & LILY_HAS_REPETITION) p.repetition_penalty = o.repetition_penalty;
    }
    std::string why;
    if (validate && !params_valid(p, why)) {
        return refuse(err, err_cap, LILY_ERR_PARAMS, why);
    }
    *out = p;
    return LILY_OK;
}

int32_t lily_request_fields_from_json(const char *body, uint32_t len, lily_request_fields_t *out,
                                      char *err, uint32_t err_cap) {
    if (body == nullptr || out == nullptr) {
        return refuse(err, err_cap, LILY_ERR_ARG, "body or out is null");
    }
    Json req;
    std::string error;
    if (!parse_json(body, len, req, error)) {
        return refuse(err, err_cap, LILY_ERR_ARG, error);
    }
    if (req.kind != Json::Object) {
        return refuse(err, err_cap, LILY_ERR_ARG, "a request is a JSON object");
    }
    lily_request_fields_t f;
    std::memset(&f, 0, sizeof f);
    bool ok = opt_f32(req, "temperature", LILY_HAS_TEMPERATURE, f.present, f.temperature, error) &&
              opt_f32(req, "top_p", LILY_HAS_TOP_P, f.present, f.top_p, error) &&
              opt_i64(req, "top_k", "", LILY_HAS_TOP_K, f.present, f.top_k, error) &&
              opt_f32(req, "min_p", LILY_HAS_MIN_P, f.present, f.min_p, error) &&
              opt_i64(req, "seed", "", LILY_HAS_SEED, f.present, f.seed, error) &&
              opt_f32(req, "presence_penalty", LILY_HAS_PRESENCE, f.present, f.presence_penalty, error) &&
              opt_f32(req, "frequency_penalty", LILY_HAS_FREQUENCY, f.present, f.frequency_penalty, error) &&
              opt_f32(req, "repetition_penalty", LILY_HAS_REPETITION, f.present, f.repetition_penalty,
                      error) &&
              opt_i64(req, "thinking_budget", "", LILY_HAS_THINKING_BUDGET, f.present, f.thinking_budget,
                      error) &&
              opt_bool(req, "thinking_nudges", "", LILY_HAS_THINKING_NUDGES, f.present, f.thinking_nudges,
                       error) &&
              opt_bool(req, "tool_call_ends_thinking", "", LILY_HAS_TOOL_CALL_ENDS_THINKING, f.present,
                       f.tool_call_ends_thinking, error);
    if (!ok) {
        return refuse(err, err_cap, LILY_ERR_ARG, error);
    }
    if ((f.present & LILY_HAS_THINKING_BUDGET) && f.thinking_budget == 0) {
        return refuse(err, err_cap, LILY_ERR_ARG,
                      "thinking_budget must be a positive token count, or negative to turn the server's "
                      "default off; got 0");
    }
    // chat_template_kwargs win over the top-level fields (from_kwargs, then `or`).
    const Json *kw = req.get("chat_template_kwargs");
    if (kw != nullptr && kw->kind == Json::Object) {
        lily_request_fields_t k;
        std::memset(&k, 0, sizeof k);
        const char *pre = "chat_template_kwargs.";
        ok = opt_i64(*kw, "thinking_budget", pre, LILY_HAS_THINKING_BUDGET, k.present, k.thinking_budget,
                     error) &&
             opt_bool(*kw, "thinking_nudges", pre, LILY_HAS_THINKING_NUDGES, k.present, k.thinking_nudges,
                      error) &&
             opt_bool(*kw, "tool_call_ends_thinking", pre, LILY_HAS_TOOL_CALL_ENDS_THINKING, k.present,
                      k.tool_call_ends_thinking, error);
        if (!ok) {
            return refuse(err, err_cap, LILY_ERR_ARG, error);
        }
        if ((k.present & LILY_HAS_THINKING_BUDGET) && k.thinking_budget == 0) {
            return refuse(err, err_cap, LILY_ERR_ARG,
                          "chat_template_kwargs.thinking_budget must be a positive token count, or "
                          "negative to turn the server's default off; got 0");
        }
        if (k.present & LILY_HAS_THINKING_BUDGET) {
            f.thinking_budget = k.thinking_budget;
            f.present |= LILY_HAS_THINKING_BUDGET;
        }
        if (k.present & LILY_HAS_THINKING_NUDGES) {
            f.thinking_nudges = k.thinking_nudges;
            f.present |= LILY_HAS_THINKING_NUDGES;
        }
        if (k.present & LILY_HAS_TOOL_CALL_ENDS_THINKING) {
            f.tool_call_ends_thinking = k.tool_call_ends_thinking;
            f.present |= LILY_HAS_TOOL_CALL_ENDS_THINKING;
        }
    }
    *out = f;
    return LILY_OK;
}

int32_t lily_resolve_sampling(const lily_request_fields_t *fields,
                              const lily_sampling_params_t *defaults, uint64_t entropy,
                              lily_sampling_params_t *out, char *err, uint32_t err_cap) {
    if (fields == nullptr || defaults == nullptr || out == nullptr) {
        return refuse(err, err_cap, LILY_ERR_ARG, "fields, defaults or out is null");
    }
    const lily_request_fields_t &f = *fields;
    lily_sampling_params_t p = *defaults;
    if (f.present & LILY_HAS_TOP_K) {
        p.top_k = f.top_k < 0 ? 0u : clamp_top_k((unsigned long long)f.top_k);
    }
    p.seed = (f.present & LILY_HAS_SEED) ? (uint64_t)f.seed : entropy;
    if (f.present & LILY_HAS_TEMPERATURE) p.temperature = f.temperature;
    if (f.present & LILY_HAS_TOP_P) p.top_p = f.top_p;
    if (f.present & LILY_HAS_MIN_P) p.min_p = f.min_p;
    if (f.present & LILY_HAS_PRESENCE) p.presence_penalty = f.presence_penalty;
    if (f.present & LILY_HAS_FREQUENCY) p.frequency_penalty = f.frequency_penalty;
    if (f.present & LILY_HAS_REPETITION) p.repetition_penalty = f.repetition_penalty;
    p.reserved = 0;
    std::string why;
    if (!params_valid(p, why)) {
        return refuse(err, err_cap, LILY_ERR_PARAMS, why);
    }
    *out = p;
    return LILY_OK;
}

int32_t lily_thinking_budgets_parse(const char *text_, lily_thinking_budgets_t *out, char *err,
                                    uint32_t err_cap) {
    if (text_ == nullptr || out == nullptr) {
        return refuse(err, err_cap, LILY_ERR_ARG, "text or out is null");
    }
    lily_thinking_budgets_t b = {-1, -1, -1};
    const std::string text = trim(text_);
    if (text == "off") {
        *out = b;
        return LILY_OK;
    }
    unsigned long long all = 0;
    if (parse_usize(text, all)) {
        if (all == 0) {
            return refuse(err, err_cap, LILY_ERR_ARG, "a thinking budget must be a positive token count");
        }
        if (all > LILY_MAX_THINKING_TOKENS) {
            return refuse(err, err_cap, LILY_ERR_ARG, "a thinking budget must be at most 1048576 tokens");
        }
        b.low = b.medium = b.xhigh = (int64_t)all;
        *out = b;
        return LILY_OK;
    }
    size_t at = 0;
    while (at <= text.size()) {
        const size_t comma = text.find(',', at);
        const std::string part = trim(text.substr(at, comma == std::string::npos ? std::string::npos : comma - at));
        at = comma == std::string::npos ? text.size() + 1 : comma + 1;
        if (part.empty()) {
            continue;
        }
        const size_t eq = part.find('=');
        if (eq == std::string::npos) {
            return refuse(err, err_cap, LILY_ERR_ARG,
                          "thinking budget \"" + part + "\" is not level=tokens or a number");
        }
        const std::string level = trim(part.substr(0, eq)), value = trim(part.substr(eq + 1));
        unsigned long long v = 0;
        if (!parse_usize(value, v)) {
            return refuse(err, err_cap, LILY_ERR_ARG,
                          "thinking budget \"" + part + "\": \"" + value + "\" is not a token count");
        }
        if (v == 0) {
            return refuse(err, err_cap, LILY_ERR_ARG,
                          "thinking budget \"" + part + "\": a budget must be a positive token count");
        }
        if (v > LILY_MAX_THINKING_TOKENS) {
            return refuse(err, err_cap, LILY_ERR_ARG,
                          "thinking budget \"" + part + "\": a budget must be at most 1048576 tokens");
        }
        if (level == "low") {
            b.low = (int64_t)v;
        } else if (level == "medium") {
            b.medium = (int64_t)v;
        } else if (level == "high" || level == "xhigh") {
            b.xhigh = (int64_t)v;
        } else {
            return refuse(err, err_cap, LILY_ERR_ARG,
                          "unknown reasoning effort \"" + level + "\" in the thinking budget (low, medium, xhigh)");
        }
    }
    *out = b;
    return LILY_OK;
}

int64_t lily_thinking_budgets_at(const lily_thinking_budgets_t *b, const char *effort) {
    if (b == nullptr) {
        return -1;
    }
    if (effort != nullptr && std::strcmp(effort, "low") == 0) {
        return b->low < 0 ? -1 : b->low;
    }
    if (effort != nullptr && std::strcmp(effort, "medium") == 0) {
        return b->medium < 0 ? -1 : b->medium;
    }
    return b->xhigh < 0 ? -1 : b->xhigh;
}

const char *lily_template_effort(const char *value) {
    if (value == nullptr) {
        return nullptr;
    }
    if (std::strcmp(value, "low") == 0) {
        return "low";
    }
    if (std::strcmp(value, "medium") == 0) {
        return "medium";
    }
    if (std::strcmp(value, "high") == 0 || std::strcmp(value, "xhigh") == 0 || std::strcmp(value, "max") == 0) {
        return "xhigh";
    }
    return nullptr;
}

void lily_thinking_defaults_init(lily_thinking_defaults_t *d) {
    if (d == nullptr) {
        return;
    }
    d->budgets.low = d->budgets.medium = d->budgets.xhigh = -1;
    d->tool_turn_factor = 1.0;
    d->nudges = 0;
    d->tool_call_ends_thinking = 0;
    d->grace = LILY_THINKING_DEFAULT_GRACE;
}

int32_t lily_thinking_defaults_validate(const lily_thinking_defaults_t *d, char *err, uint32_t err_cap) {
    if (d == nullptr) {
        return refuse(err, err_cap, LILY_ERR_ARG, "defaults is null");
    }
    const double f = d->tool_turn_factor;
    if (!(std::isfinite(f) && f > 0.0 && f <= LILY_MAX_TOOL_TURN_FACTOR)) {
        return refuse(err, err_cap, LILY_ERR_ARG,
                      "--thinking-budget-tool-turn-factor must be a positive number of at most 100");
    }
    if (d->grace > LILY_MAX_THINKING_TOKENS) {
        return refuse(err, err_cap, LILY_ERR_ARG, "--thinking-budget-grace must be at most 1048576 tokens");
    }
    return LILY_OK;
}

int64_t lily_thinking_defaults_budget(const lily_thinking_defaults_t *d, const char *effort,
                                      int32_t tool_turn) {
    if (d == nullptr) {
        return -1;
    }
    const int64_t budget = lily_thinking_budgets_at(&d->budgets, effort);
    if (budget < 0) {
        return -1;
    }
    if (!tool_turn) {
        return budget;
    }
    // f64::round: half away from zero.
    const double scaled = std::round((double)budget * d->tool_turn_factor);
    const int64_t v = scaled < 0.0 ? 0 : (int64_t)scaled;
    return v < 1 ? 1 : v;
}

void lily_thinking_resolve(const lily_request_fields_t *fields, const lily_thinking_defaults_t *defaults,
                           int64_t default_budget, uint64_t seed, lily_thinking_settings_t *out) {
    if (fields == nullptr || defaults == nullptr || out == nullptr) {
        return;
    }
    int64_t budget = default_budget < 0 ? -1 : default_budget;
    if (fields->present & LILY_HAS_THINKING_BUDGET) {
        budget = fields->thinking_budget < 0 ? -1 : fields->thinking_budget;
    }
    const bool nudges = (fields->present & LILY_HAS_THINKING_NUDGES) ? fields->thinking_nudges != 0
                                                                     : defaults->nudges != 0;
    out->budget = budget;
    out->grace = defaults->grace;
    out->nudges = (budget >= 0 && nudges) ? 1 : 0;
    out->tool_call_ends_thinking = (fields->present & LILY_HAS_TOOL_CALL_ENDS_THINKING)
                                       ? (fields->tool_call_ends_thinking != 0)
                                       : (defaults->tool_call_ends_thinking != 0);
    out->seed = seed;
}

}  // extern "C"
