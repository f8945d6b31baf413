// A small JSON reader: enough for an .nx header (objects, arrays, strings, numbers, booleans, null).
#pragma once
#include <cmath>
#include <cstring>
#include <cstdlib>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace b2 {

struct JValue {
    enum Type { Null, Bool, Num, Str, Arr, Obj } type = Null;
    bool b = false;
    double num = 0;
    std::string str;
    std::vector<JValue> arr;
    std::vector<std::pair<std::string, JValue>> obj;

    const JValue* get(const std::string& key) const {
        if (type != Obj) return nullptr;
        for (auto& kv : obj) if (kv.first == key) return &kv.second;
        return nullptr;
    }
    bool is_num() const { return type == Num; }
};

class JParser {
public:
    JParser(const char* s, size_t n) : p_(s), end_(s + n) {}
    bool parse(JValue& out, std::string& err) {
        if (!value(out, 0)) { err = err_.empty() ? "bad JSON" : err_; return false; }
        ws();
        if (p_ != end_) { err = "trailing characters after JSON value"; return false; }
        return true;
    }

private:
    const char *p_, *end_;
    std::string err_;
    void ws() { while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) p_++; }
    bool fail(const char* m) { if (err_.empty()) err_ = m; return false; }
    bool lit(const char* w) {
        size_t n = strlen(w);
        if ((size_t)(end_ - p_) < n || strncmp(p_, w, n) != 0) return fail("bad literal");
        p_ += n;
        return true;
    }
    bool string(std::string& out) {
        if (p_ >= end_ || *p_ != '"') return fail("expected string");
        p_++;
        while (p_ < end_ && *p_ != '"') {
            char c = *p_++;
            if (c == '\\') {
                if (p_ >= end_) return fail("bad escape");
                char e = *p_++;
                switch (e) {
                case 'n': out += '\n'; break;
                case 't': out += '\t'; break;
                case 'r': out += '\r'; break;
                case 'b': out += '\b'; break;
                case 'f': out += '\f'; break;
                case 'u': {
                    if (end_ - p_ < 4) return fail("bad \\u escape");
                    unsigned cp = (unsigned)strtoul(std::string(p_, 4).c_str(), nullptr, 16);
                    p_ += 4;
                    if (cp < 0x80) out += (char)cp;
                    else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
                    else { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
                } break;
                default: out += e;
                }
            } else out += c;
        }
        if (p_ >= end_) return fail("unterminated string");
        p_++;
        return true;
    }
    bool value(JValue& v, int depth) {
        if (depth > 64) return fail("JSON nested too deeply");
        ws();
        if (p_ >= end_) return fail("unexpected end of JSON");
        char c = *p_;
        if (c == '{') {
            v.type = JValue::Obj;
            p_++;
            ws();
            if (p_ < end_ && *p_ == '}') { p_++; return true; }
            while (true) {
                ws();
                std::string k;
                if (!string(k)) return false;
                ws();
                if (p_ >= end_ || *p_ != ':') return fail("expected ':'");
                p_++;
                v.obj.emplace_back(std::move(k), JValue());
                if (!value(v.obj.back().second, depth + 1)) return false;
                ws();
                if (p_ < end_ && *p_ == ',') { p_++; continue; }
                if (p_ < end_ && *p_ == '}') { p_++; return true; }
                return fail("expected ',' or '}'");
            }
        }
        if (c == '[') {
            v.type = JValue::Arr;
            p_++;
            ws();
            if (p_ < end_ && *p_ == ']') { p_++; return true; }
            while (true) {
                v.arr.emplace_back();
                if (!value(v.arr.back(), depth + 1)) return false;
                ws();
                if (p_ < end_ && *p_ == ',') { p_++; continue; }
                if (p_ < end_ && *p_ == ']') { p_++; return true; }
                return fail("expected ',' or ']'");
            }
        }
        if (c == '"') { v.type = JValue::Str; return string(v.str); }
        if (c == 't') { v.type = JValue::Bool; v.b = true; return lit("true"); }
        if (c == 'f') { v.type = JValue::Bool; v.b = false; return lit("false"); }
        if (c == 'n') { v.type = JValue::Null; return lit("null"); }
        // number (also accepts Python's Infinity / NaN spellings as errors)
        char* e = nullptr;
        std::string tmp(p_, (size_t)std::min<ptrdiff_t>(end_ - p_, 64));
        double d = strtod(tmp.c_str(), &e);
        if (e == tmp.c_str()) return fail("bad number");
        p_ += (e - tmp.c_str());
        v.type = JValue::Num;
        v.num = d;
        return true;
    }
};

}  // namespace b2
