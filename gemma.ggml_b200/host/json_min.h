// json_min.h — a small JSON reader for model configurations and safetensors headers: objects keep the order of
// their keys, numbers are doubles, no streaming, errors as a message.  Header-only.
#pragma once

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <string>
#include <utility>
#include <vector>

struct json_value {
    enum kind_t { NUL, BOOL, NUM, STR, ARR, OBJ } kind = NUL;
    bool b = false;
    double num = 0.0;
    std::string str;
    std::vector<json_value> arr;
    std::vector<std::pair<std::string, json_value>> obj;

    bool is_null() const { return kind == NUL; }
    const json_value *find(const std::string &key) const {
        if (kind != OBJ) return nullptr;
        for (const auto &kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    // present and not null
    const json_value *get(const std::string &key) const {
        const json_value *v = find(key);
        return v && !v->is_null() ? v : nullptr;
    }
    double number(const std::string &key, double dflt) const {
        const json_value *v = get(key);
        return v && v->kind == NUM ? v->num : dflt;
    }
    long long integer(const std::string &key, long long dflt) const { return (long long)std::llround(number(key, (double)dflt)); }
    std::string string(const std::string &key, const std::string &dflt) const {
        const json_value *v = get(key);
        return v && v->kind == STR ? v->str : dflt;
    }
};

class json_parser {
  public:
    json_parser(const char *p, size_t n) : p_(p), end_(p + n) {}
    bool parse(json_value *out, std::string *err) {
        if (!value(out) || (ws(), p_ != end_)) {
            if (err) *err = err_.empty() ? "trailing characters after the JSON value" : err_;
            return false;
        }
        return true;
    }

  private:
    const char *p_, *end_;
    std::string err_;
    int depth_ = 0;
    void ws() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) p_++;
    }
    bool fail(const char *m) {
        if (err_.empty()) err_ = m;
        return false;
    }
    bool lit(const char *s) {
        const char *q = p_;
        while (*s) {
            if (q >= end_ || *q != *s) return false;
            q++, s++;
        }
        p_ = q;
        return true;
    }
    bool string_(std::string *out) {
        if (p_ >= end_ || *p_ != '"') return fail("expected a string");
        p_++;
        out->clear();
        while (p_ < end_ && *p_ != '"') {
            char c = *p_++;
            if (c == '\\') {
                if (p_ >= end_) return fail("unfinished escape");
                c = *p_++;
                switch (c) {
                case 'n': out->push_back('\n'); break;
                case 't': out->push_back('\t'); break;
                case 'r': out->push_back('\r'); break;
                case 'b': out->push_back('\b'); break;
                case 'f': out->push_back('\f'); break;
                case 'u': {
                    if (end_ - p_ < 4) return fail("unfinished \\u escape");
                    unsigned cp = (unsigned)strtoul(std::string(p_, p_ + 4).c_str(), nullptr, 16);
                    p_ += 4;
                    if (cp < 0x80) out->push_back((char)cp);
                    else if (cp < 0x800) { out->push_back((char)(0xC0 | (cp >> 6))); out->push_back((char)(0x80 | (cp & 0x3F))); }
                    else { out->push_back((char)(0xE0 | (cp >> 12))); out->push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out->push_back((char)(0x80 | (cp & 0x3F))); }
                    break;
                }
                default: out->push_back(c);
                }
            } else {
                out->push_back(c);
            }
        }
        if (p_ >= end_) return fail("unfinished string");
        p_++;
        return true;
    }
    bool value(json_value *v) {
        if (++depth_ > 64) return fail("nesting too deep");
        ws();
        if (p_ >= end_) return fail("unexpected end");
        bool ok = true;
        if (*p_ == '{') {
            p_++;
            v->kind = json_value::OBJ;
            ws();
            if (p_ < end_ && *p_ == '}') p_++;
            else
                for (;;) {
                    ws();
                    std::string k;
                    json_value e;
                    if (!string_(&k)) { ok = false; break; }
                    ws();
                    if (p_ >= end_ || *p_++ != ':') { ok = fail("expected ':'"); break; }
                    if (!value(&e)) { ok = false; break; }
                    v->obj.emplace_back(std::move(k), std::move(e));
                    ws();
                    if (p_ < end_ && *p_ == ',') { p_++; continue; }
                    if (p_ < end_ && *p_ == '}') { p_++; break; }
                    ok = fail("expected ',' or '}'");
                    break;
                }
        } else if (*p_ == '[') {
            p_++;
            v->kind = json_value::ARR;
            ws();
            if (p_ < end_ && *p_ == ']') p_++;
            else
                for (;;) {
                    json_value e;
                    if (!value(&e)) { ok = false; break; }
                    v->arr.push_back(std::move(e));
                    ws();
                    if (p_ < end_ && *p_ == ',') { p_++; continue; }
                    if (p_ < end_ && *p_ == ']') { p_++; break; }
                    ok = fail("expected ',' or ']'");
                    break;
                }
        } else if (*p_ == '"') {
            v->kind = json_value::STR;
            ok = string_(&v->str);
        } else if (lit("true")) {
            v->kind = json_value::BOOL, v->b = true;
        } else if (lit("false")) {
            v->kind = json_value::BOOL, v->b = false;
        } else if (lit("null")) {
            v->kind = json_value::NUL;
        } else {
            const std::string tmp(p_, (size_t)std::min<ptrdiff_t>(end_ - p_, 64));
            char *e = nullptr;
            v->num = strtod(tmp.c_str(), &e);
            if (e == tmp.c_str()) ok = fail("unexpected character");
            else { v->kind = json_value::NUM; p_ += e - tmp.c_str(); }
        }
        depth_--;
        return ok;
    }
};
