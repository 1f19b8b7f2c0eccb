// Minimal JSON reader used to load the ISA table (no third-party JSON library is available).
//
// Objects keep their members in file order; `get()` returns the LAST member with a given
// name, which is what serde_json does when a key is repeated (the reference parses the
// table with serde_json 1.x, reference src/table.rs:270,347).
#pragma once
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace cubit_json {

struct Value;
using Member = std::pair<std::string, Value>;

struct Value {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    bool is_integer = false;   // number had no fraction / exponent
    bool is_negative = false;
    uint64_t mag = 0;          // |integer| when is_integer
    double num = 0.0;
    std::string str;
    std::vector<Value> arr;
    std::vector<Member> obj;

    bool is_object() const { return kind == Object; }
    bool is_array() const { return kind == Array; }
    bool is_string() const { return kind == String; }
    const Value* get(const std::string& name) const {
        if (kind != Object) return nullptr;
        for (size_t i = obj.size(); i-- > 0;)
            if (obj[i].first == name) return &obj[i].second;
        return nullptr;
    }
};

class Parser {
public:
    Parser(const char* data, size_t len) : p_(data), end_(data + len), begin_(data) {}

    Value parse_document() {
        Value v = parse_value(0);
        skip_ws();
        if (p_ != end_) fail("trailing characters after JSON document");
        return v;
    }

private:
    const char* p_;
    const char* end_;
    const char* begin_;

    [[noreturn]] void fail(const std::string& why) const {
        throw std::runtime_error("invalid JSON at byte " + std::to_string(p_ - begin_) + ": " + why);
    }
    void skip_ws() {
        while (p_ != end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\r' || *p_ == '\t')) ++p_;
    }
    bool consume(const char* lit) {
        const char* q = p_;
        while (*lit) {
            if (q == end_ || *q != *lit) return false;
            ++q; ++lit;
        }
        p_ = q;
        return true;
    }
    static void put_utf8(std::string& out, uint32_t cp) {
        if (cp < 0x80) out.push_back(char(cp));
        else if (cp < 0x800) { out.push_back(char(0xC0 | (cp >> 6))); out.push_back(char(0x80 | (cp & 0x3F))); }
        else if (cp < 0x10000) {
            out.push_back(char(0xE0 | (cp >> 12))); out.push_back(char(0x80 | ((cp >> 6) & 0x3F)));
            out.push_back(char(0x80 | (cp & 0x3F)));
        } else {
            out.push_back(char(0xF0 | (cp >> 18))); out.push_back(char(0x80 | ((cp >> 12) & 0x3F)));
            out.push_back(char(0x80 | ((cp >> 6) & 0x3F))); out.push_back(char(0x80 | (cp & 0x3F)));
        }
    }
    uint32_t hex4() {
        if (end_ - p_ < 4) fail("truncated \\u escape");
        uint32_t v = 0;
        for (int i = 0; i < 4; ++i) {
            char c = *p_++;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= uint32_t(c - '0');
            else if (c >= 'a' && c <= 'f') v |= uint32_t(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= uint32_t(c - 'A' + 10);
            else fail("bad hex digit in \\u escape");
        }
        return v;
    }
    std::string parse_string() {
        // *p_ == '"'
        ++p_;
        std::string out;
        for (;;) {
            if (p_ == end_) fail("unterminated string");
            unsigned char c = (unsigned char)*p_++;
            if (c == '"') return out;
            if (c < 0x20) fail("control character in string");
            if (c != '\\') { out.push_back(char(c)); continue; }
            if (p_ == end_) fail("unterminated escape");
            char e = *p_++;
            switch (e) {
                case '"': out.push_back('"'); break;
                case '\\': out.push_back('\\'); break;
                case '/': out.push_back('/'); break;
                case 'b': out.push_back('\b'); break;
                case 'f': out.push_back('\f'); break;
                case 'n': out.push_back('\n'); break;
                case 'r': out.push_back('\r'); break;
                case 't': out.push_back('\t'); break;
                case 'u': {
                    uint32_t cp = hex4();
                    if (cp >= 0xD800 && cp <= 0xDBFF) {
                        if (!consume("\\u")) fail("lone surrogate");
                        uint32_t lo = hex4();
                        if (lo < 0xDC00 || lo > 0xDFFF) fail("bad low surrogate");
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    put_utf8(out, cp);
                    break;
                }
                default: fail("unknown escape");
            }
        }
    }
    Value parse_number() {
        Value v;
        v.kind = Value::Number;
        const char* s = p_;
        if (p_ != end_ && *p_ == '-') { v.is_negative = true; ++p_; }
        if (p_ == end_ || *p_ < '0' || *p_ > '9') fail("bad number");
        bool overflow = false;
        uint64_t mag = 0;
        while (p_ != end_ && *p_ >= '0' && *p_ <= '9') {
            uint64_t d = uint64_t(*p_ - '0');
            if (mag > (UINT64_MAX - d) / 10) overflow = true; else mag = mag * 10 + d;
            ++p_;
        }
        bool integral = true;
        if (p_ != end_ && *p_ == '.') {
            integral = false; ++p_;
            if (p_ == end_ || *p_ < '0' || *p_ > '9') fail("bad fraction");
            while (p_ != end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        if (p_ != end_ && (*p_ == 'e' || *p_ == 'E')) {
            integral = false; ++p_;
            if (p_ != end_ && (*p_ == '+' || *p_ == '-')) ++p_;
            if (p_ == end_ || *p_ < '0' || *p_ > '9') fail("bad exponent");
            while (p_ != end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        v.num = std::stod(std::string(s, p_));
        v.is_integer = integral && !overflow;
        v.mag = mag;
        return v;
    }
    Value parse_value(int depth) {
        if (depth > 128) fail("nesting too deep");
        skip_ws();
        if (p_ == end_) fail("unexpected end of input");
        Value v;
        char c = *p_;
        if (c == '{') {
            ++p_;
            v.kind = Value::Object;
            skip_ws();
            if (p_ != end_ && *p_ == '}') { ++p_; return v; }
            for (;;) {
                skip_ws();
                if (p_ == end_ || *p_ != '"') fail("expected member name");
                std::string name = parse_string();
                skip_ws();
                if (p_ == end_ || *p_ != ':') fail("expected ':'");
                ++p_;
                Value child = parse_value(depth + 1);
                v.obj.emplace_back(std::move(name), std::move(child));
                skip_ws();
                if (p_ == end_) fail("unterminated object");
                if (*p_ == ',') { ++p_; continue; }
                if (*p_ == '}') { ++p_; return v; }
                fail("expected ',' or '}'");
            }
        }
        if (c == '[') {
            ++p_;
            v.kind = Value::Array;
            skip_ws();
            if (p_ != end_ && *p_ == ']') { ++p_; return v; }
            for (;;) {
                v.arr.push_back(parse_value(depth + 1));
                skip_ws();
                if (p_ == end_) fail("unterminated array");
                if (*p_ == ',') { ++p_; continue; }
                if (*p_ == ']') { ++p_; return v; }
                fail("expected ',' or ']'");
            }
        }
        if (c == '"') { v.kind = Value::String; v.str = parse_string(); return v; }
        if (c == 't') { if (!consume("true")) fail("bad literal"); v.kind = Value::Bool; v.b = true; return v; }
        if (c == 'f') { if (!consume("false")) fail("bad literal"); v.kind = Value::Bool; v.b = false; return v; }
        if (c == 'n') { if (!consume("null")) fail("bad literal"); v.kind = Value::Null; return v; }
        return parse_number();
    }
};

inline Value parse(const std::string& text) {
    Parser p(text.data(), text.size());
    return p.parse_document();
}

}  // namespace cubit_json
