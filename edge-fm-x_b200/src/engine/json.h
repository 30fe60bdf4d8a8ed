// Minimal JSON reader for the engine config and the HF config.json / safetensors header.
// (The reference uses nlohmann::json, which is not vendored here.)  Parses RFC 8259 text into
// a small DOM; numbers are kept as double plus an exact int64 when the literal is integral.
#pragma once
#include <cstdint>
#include <cstdlib>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace edge_fm {
namespace json {

struct Value {
    enum Type { Null, Bool, Number, String, Array, Object } type = Null;
    bool b = false;
    double num = 0.0;
    int64_t inum = 0;
    bool is_int = false;
    std::string str;
    std::vector<Value> arr;
    std::vector<std::pair<std::string, Value>> obj;   // insertion order kept

    bool is_null() const { return type == Null; }
    bool is_object() const { return type == Object; }
    bool is_array() const { return type == Array; }
    bool is_string() const { return type == String; }
    bool is_number() const { return type == Number; }
    bool is_bool() const { return type == Bool; }

    const Value* find(const std::string& key) const {
        if (type != Object) return nullptr;
        for (const auto& kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    bool contains(const std::string& key) const { return find(key) != nullptr; }
    void set(const std::string& key, const Value& v) {
        type = Object;
        for (auto& kv : obj)
            if (kv.first == key) { kv.second = v; return; }
        obj.emplace_back(key, v);
    }
    // typed getters with defaults
    int64_t get_int(const std::string& key, int64_t dflt) const {
        const Value* v = find(key);
        return v != nullptr && v->type == Number ? (v->is_int ? v->inum : (int64_t)v->num) : dflt;
    }
    double get_double(const std::string& key, double dflt) const {
        const Value* v = find(key);
        return v != nullptr && v->type == Number ? v->num : dflt;
    }
    bool get_bool(const std::string& key, bool dflt) const {
        const Value* v = find(key);
        return v != nullptr && v->type == Bool ? v->b : dflt;
    }
    std::string get_string(const std::string& key, const std::string& dflt) const {
        const Value* v = find(key);
        return v != nullptr && v->type == String ? v->str : dflt;
    }
};

class Parser {
public:
    explicit Parser(const std::string& text) : s_(text) {}
    Value parse() {
        Value v = value();
        ws();
        if (i_ != s_.size()) fail("trailing characters");
        return v;
    }

private:
    const std::string& s_;
    size_t i_ = 0;

    [[noreturn]] void fail(const char* what) const {
        throw std::runtime_error(std::string("JSON: ") + what + " at offset " + std::to_string(i_));
    }
    void ws() {
        while (i_ < s_.size() && (s_[i_] == ' ' || s_[i_] == '\n' || s_[i_] == '\t' || s_[i_] == '\r')) ++i_;
    }
    bool lit(const char* w) {
        size_t n = 0;
        while (w[n] != 0) ++n;
        if (s_.compare(i_, n, w) == 0) { i_ += n; return true; }
        return false;
    }
    Value value() {
        ws();
        if (i_ >= s_.size()) fail("unexpected end");
        const char c = s_[i_];
        Value v;
        if (c == '{') {
            v.type = Value::Object;
            ++i_;
            ws();
            if (i_ < s_.size() && s_[i_] == '}') { ++i_; return v; }
            for (;;) {
                ws();
                if (i_ >= s_.size() || s_[i_] != '"') fail("expected key");
                std::string k = string();
                ws();
                if (i_ >= s_.size() || s_[i_] != ':') fail("expected ':'");
                ++i_;
                v.obj.emplace_back(std::move(k), value());
                ws();
                if (i_ < s_.size() && s_[i_] == ',') { ++i_; continue; }
                if (i_ < s_.size() && s_[i_] == '}') { ++i_; return v; }
                fail("expected ',' or '}'");
            }
        }
        if (c == '[') {
            v.type = Value::Array;
            ++i_;
            ws();
            if (i_ < s_.size() && s_[i_] == ']') { ++i_; return v; }
            for (;;) {
                v.arr.push_back(value());
                ws();
                if (i_ < s_.size() && s_[i_] == ',') { ++i_; continue; }
                if (i_ < s_.size() && s_[i_] == ']') { ++i_; return v; }
                fail("expected ',' or ']'");
            }
        }
        if (c == '"') { v.type = Value::String; v.str = string(); return v; }
        if (lit("true")) { v.type = Value::Bool; v.b = true; return v; }
        if (lit("false")) { v.type = Value::Bool; v.b = false; return v; }
        if (lit("null")) return v;
        if (c == '-' || (c >= '0' && c <= '9')) {
            const size_t start = i_;
            bool integral = true;
            if (s_[i_] == '-') ++i_;
            while (i_ < s_.size()) {
                const char d = s_[i_];
                if (d >= '0' && d <= '9') { ++i_; continue; }
                if (d == '.' || d == 'e' || d == 'E' || d == '+' || d == '-') { integral = false; ++i_; continue; }
                break;
            }
            const std::string tok = s_.substr(start, i_ - start);
            v.type = Value::Number;
            v.num = std::strtod(tok.c_str(), nullptr);
            v.is_int = integral;
            v.inum = integral ? std::strtoll(tok.c_str(), nullptr, 10) : (int64_t)v.num;
            return v;
        }
        fail("unexpected character");
    }
    std::string string() {
        std::string out;
        ++i_;   // opening quote
        while (i_ < s_.size()) {
            const char c = s_[i_++];
            if (c == '"') return out;
            if (c != '\\') { out.push_back(c); continue; }
            if (i_ >= s_.size()) break;
            const char e = s_[i_++];
            switch (e) {
                case 'n': out.push_back('\n'); break;
                case 't': out.push_back('\t'); break;
                case 'r': out.push_back('\r'); break;
                case 'b': out.push_back('\b'); break;
                case 'f': out.push_back('\f'); break;
                case 'u': {
                    if (i_ + 4 > s_.size()) fail("bad \\u escape");
                    const unsigned cp = (unsigned)std::strtoul(s_.substr(i_, 4).c_str(), nullptr, 16);
                    i_ += 4;
                    if (cp < 0x80) out.push_back((char)cp);
                    else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
                    else { out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
                    break;
                }
                default: out.push_back(e);
            }
        }
        fail("unterminated string");
    }
};

inline Value parse(const std::string& text) { return Parser(text).parse(); }

}  // namespace json
}  // namespace edge_fm
