// Minimal JSON reader (objects, arrays, strings, numbers, true / false / null) for config.json, safetensors headers and
// the step lines of trace sessions. Host only; numbers are kept as double (and their text, for 64-bit integers).
#pragma once
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace b200 {

struct Json {
    enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
    bool b = false;
    double num = 0;
    std::string str;                 // Str: the text; Num: the literal
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;   // in file order

    bool is_null() const { return kind == Null; }
    const Json* get(const std::string& k) const {
        if (kind != Obj) return nullptr;
        for (auto& kv : obj)
            if (kv.first == k) return &kv.second;
        return nullptr;
    }
    bool has(const std::string& k) const { const Json* j = get(k); return j && !j->is_null(); }
    double number(const std::string& k, double dflt) const { const Json* j = get(k); return j && j->kind == Num ? j->num : dflt; }
    long long integer(const std::string& k, long long dflt) const {
        const Json* j = get(k);
        return j && j->kind == Num ? std::strtoll(j->str.c_str(), nullptr, 10) : dflt;
    }
    std::string text(const std::string& k, const std::string& dflt = "") const {
        const Json* j = get(k);
        return j && j->kind == Str ? j->str : dflt;
    }
};

class JsonParser {
public:
    // returns false and sets err on malformed input
    static bool parse(const char* s, size_t n, Json& out, std::string& err) {
        JsonParser p(s, s + n);
        if (!p.value(out)) { err = "json: " + p.err_ + " at byte " + std::to_string(p.p_ - s); return false; }
        p.ws();
        if (p.p_ != p.e_) { err = "json: trailing characters"; return false; }
        return true;
    }

private:
    JsonParser(const char* b, const char* e) : p_(b), e_(e) {}
    const char* p_;
    const char* e_;
    std::string err_;
    int depth_ = 0;
    void ws() { while (p_ < e_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_; }
    bool fail(const char* m) { err_ = m; return false; }
    bool lit(const char* w) {
        size_t n = strlen(w);
        if ((size_t)(e_ - p_) < n || strncmp(p_, w, n) != 0) return fail("bad literal");
        p_ += n;
        return true;
    }
    bool string(std::string& out) {
        if (p_ >= e_ || *p_ != '"') return fail("expected string");
        ++p_;
        out.clear();
        while (p_ < e_ && *p_ != '"') {
            if (*p_ == '\\') {
                if (++p_ >= e_) return fail("bad escape");
                switch (*p_) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'u': {
                        if (e_ - p_ < 5) return fail("bad \\u");
                        unsigned cp = (unsigned)std::strtoul(std::string(p_ + 1, p_ + 5).c_str(), nullptr, 16);
                        p_ += 4;
                        if (cp < 0x80) out += (char)cp;
                        else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
                        else { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
                        break;
                    }
                    default: out += *p_;
                }
                ++p_;
            } else
                out += *p_++;
        }
        if (p_ >= e_) return fail("unterminated string");
        ++p_;
        return true;
    }
    bool value(Json& out) {
        if (++depth_ > 64) return fail("too deep");
        ws();
        if (p_ >= e_) return fail("unexpected end");
        bool ok = true;
        const char c = *p_;
        if (c == '{') {
            out.kind = Json::Obj;
            ++p_;
            ws();
            if (p_ < e_ && *p_ == '}') ++p_;
            else
                for (;;) {
                    ws();
                    std::string k;
                    if (!string(k)) return false;
                    ws();
                    if (p_ >= e_ || *p_ != ':') return fail("expected ':'");
                    ++p_;
                    out.obj.emplace_back(k, Json());
                    if (!value(out.obj.back().second)) return false;
                    ws();
                    if (p_ < e_ && *p_ == ',') { ++p_; continue; }
                    if (p_ < e_ && *p_ == '}') { ++p_; break; }
                    return fail("expected ',' or '}'");
                }
        } else if (c == '[') {
            out.kind = Json::Arr;
            ++p_;
            ws();
            if (p_ < e_ && *p_ == ']') ++p_;
            else
                for (;;) {
                    out.arr.emplace_back();
                    if (!value(out.arr.back())) return false;
                    ws();
                    if (p_ < e_ && *p_ == ',') { ++p_; continue; }
                    if (p_ < e_ && *p_ == ']') { ++p_; break; }
                    return fail("expected ',' or ']'");
                }
        } else if (c == '"') {
            out.kind = Json::Str;
            ok = string(out.str);
        } else if (c == 't') { out.kind = Json::Bool; out.b = true; ok = lit("true"); }
        else if (c == 'f') { out.kind = Json::Bool; out.b = false; ok = lit("false"); }
        else if (c == 'n') { out.kind = Json::Null; ok = lit("null"); }
        else {
            const char* s = p_;
            while (p_ < e_ && (strchr("+-.eE", *p_) || (*p_ >= '0' && *p_ <= '9'))) ++p_;
            if (p_ == s) return fail("unexpected character");
            out.kind = Json::Num;
            out.str.assign(s, p_);
            out.num = std::strtod(out.str.c_str(), nullptr);
        }
        --depth_;
        return ok;
    }
};

}  // namespace b200
