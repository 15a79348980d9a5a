// A small JSON reader for the host runtime: values keep the order of an object's members and repeated names (a
// safetensors header that names a tensor twice must be refused, not silently merged), integers stay exact 64-bit
// integers and are told apart from other numbers.  Errors are reported by position.
#pragma once

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace mmjson {

struct Value {
    enum Kind { Null, Bool, Int, Number, String, Array, Object } kind = Null;
    bool b = false;
    long long i = 0;          // Int
    double d = 0.0;           // Int and Number
    std::string s;            // String
    std::vector<Value> items;                                // Array
    std::vector<std::pair<std::string, Value>> members;      // Object, in file order, repeats kept

    const Value* find(const std::string& key) const {
        for (auto& m : members)
            if (m.first == key) return &m.second;
        return nullptr;
    }
    bool is_int() const { return kind == Int; }
};

class Parser {
  public:
    Parser(const char* p, size_t n) : p_(p), end_(p + n), begin_(p) {}
    // false with `error` set when the text is not one JSON value (followed by blanks only)
    bool parse(Value& out, std::string& error) {
        try {
            skip();
            value(out, 0);
            skip();
            if (p_ != end_) fail("text after the value");
            return true;
        } catch (const std::string& e) {
            error = e;
            return false;
        }
    }

  private:
    const char *p_, *end_, *begin_;
    [[noreturn]] void fail(const std::string& what) { throw what + " at byte " + std::to_string(p_ - begin_); }
    void skip() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\t' || *p_ == '\n' || *p_ == '\r')) ++p_;
    }
    bool eat(const char* word) {
        const size_t n = strlen_(word);
        if ((size_t)(end_ - p_) >= n && std::equal(word, word + n, p_)) {
            p_ += n;
            return true;
        }
        return false;
    }
    static size_t strlen_(const char* s) {
        size_t n = 0;
        while (s[n]) ++n;
        return n;
    }
    void value(Value& v, int depth) {
        if (depth > 64) fail("nesting too deep");
        if (p_ >= end_) fail("unexpected end");
        const char c = *p_;
        if (c == '{') {
            ++p_;
            v.kind = Value::Object;
            skip();
            if (p_ < end_ && *p_ == '}') { ++p_; return; }
            while (true) {
                skip();
                if (p_ >= end_ || *p_ != '"') fail("expected a member name");
                std::string key;
                string(key);
                skip();
                if (p_ >= end_ || *p_ != ':') fail("expected ':'");
                ++p_;
                skip();
                v.members.emplace_back(std::move(key), Value());
                value(v.members.back().second, depth + 1);
                skip();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == '}') { ++p_; return; }
                fail("expected ',' or '}'");
            }
        } else if (c == '[') {
            ++p_;
            v.kind = Value::Array;
            skip();
            if (p_ < end_ && *p_ == ']') { ++p_; return; }
            while (true) {
                skip();
                v.items.emplace_back();
                value(v.items.back(), depth + 1);
                skip();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == ']') { ++p_; return; }
                fail("expected ',' or ']'");
            }
        } else if (c == '"') {
            v.kind = Value::String;
            string(v.s);
        } else if (eat("true")) {
            v.kind = Value::Bool;
            v.b = true;
        } else if (eat("false")) {
            v.kind = Value::Bool;
            v.b = false;
        } else if (eat("null")) {
            v.kind = Value::Null;
        } else if (c == '-' || (c >= '0' && c <= '9')) {
            number(v);
        } else {
            fail("unexpected character");
        }
    }
    void number(Value& v) {
        const char* s = p_;
        if (*p_ == '-') ++p_;
        if (p_ >= end_ || *p_ < '0' || *p_ > '9') fail("bad number");
        while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        bool integral = true;
        if (p_ < end_ && *p_ == '.') {
            integral = false;
            ++p_;
            if (p_ >= end_ || *p_ < '0' || *p_ > '9') fail("bad number");
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        if (p_ < end_ && (*p_ == 'e' || *p_ == 'E')) {
            integral = false;
            ++p_;
            if (p_ < end_ && (*p_ == '+' || *p_ == '-')) ++p_;
            if (p_ >= end_ || *p_ < '0' || *p_ > '9') fail("bad number");
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        const std::string text(s, p_);
        v.d = std::strtod(text.c_str(), nullptr);
        if (integral && text.size() <= 18) {
            v.kind = Value::Int;
            v.i = std::strtoll(text.c_str(), nullptr, 10);
        } else {
            v.kind = Value::Number;
        }
    }
    void string(std::string& out) {
        ++p_;   // opening quote
        while (true) {
            if (p_ >= end_) fail("unterminated string");
            const unsigned char c = (unsigned char)*p_++;
            if (c == '"') return;
            if (c < 0x20) fail("control character in a string");
            if (c != '\\') {
                out.push_back((char)c);
                continue;
            }
            if (p_ >= end_) fail("unterminated escape");
            const char e = *p_++;
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
                    unsigned cp = hex4();
                    if (cp >= 0xD800 && cp <= 0xDBFF && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
                        p_ += 2;
                        const unsigned lo = hex4();
                        if (lo >= 0xDC00 && lo <= 0xDFFF) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                        else fail("bad surrogate pair");
                    }
                    if (cp >= 0xD800 && cp <= 0xDFFF) fail("half of a surrogate pair");      // not a character: it has no UTF-8 form
                    utf8(out, cp);
                    break;
                }
                default: fail("bad escape");
            }
        }
    }
    unsigned hex4() {
        if (end_ - p_ < 4) fail("bad \\u escape");
        unsigned v = 0;
        for (int k = 0; k < 4; ++k) {
            const char c = *p_++;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= c - '0';
            else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
            else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
            else fail("bad \\u escape");
        }
        return v;
    }
    static void utf8(std::string& out, unsigned cp) {
        if (cp < 0x80) out.push_back((char)cp);
        else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
        else if (cp < 0x10000) { out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
        else { out.push_back((char)(0xF0 | (cp >> 18))); out.push_back((char)(0x80 | ((cp >> 12) & 0x3F))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
    }
};

// JSON text of a string (quotes and escapes)
inline std::string quote(const std::string& s) {
    std::string out = "\"";
    for (unsigned char c : s) {
        switch (c) {
            case '"': out += "\\\""; break;
            case '\\': out += "\\\\"; break;
            case '\n': out += "\\n"; break;
            case '\r': out += "\\r"; break;
            case '\t': out += "\\t"; break;
            default:
                if (c < 0x20) {
                    char buf[8];
                    snprintf(buf, sizeof(buf), "\\u%04x", c);
                    out += buf;
                } else {
                    out.push_back((char)c);
                }
        }
    }
    out.push_back('"');
    return out;
}

}  // namespace mmjson
