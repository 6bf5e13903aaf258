// Minimal JSON reader/writer for the host runtime (tokenizer.json, config.json, safetensors headers).
// Values keep object key order (safetensors headers and vocab files are order-sensitive for round trips).
#pragma once
#include <cstdint>
#include <cstdlib>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace sg {

struct Json {
    enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
    bool b = false;
    double num = 0.0;
    int64_t inum = 0;
    bool is_int = false;
    std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;

    bool is_null() const { return kind == Null; }
    const Json* find(const std::string& key) const {
        if (kind != Obj) return nullptr;
        for (auto& kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    const Json& at(const std::string& key) const {
        const Json* j = find(key);
        if (!j) throw std::runtime_error("json: missing key '" + key + "'");
        return *j;
    }
    int64_t as_int(int64_t dflt = 0) const { return kind == Num ? (is_int ? inum : static_cast<int64_t>(num)) : dflt; }
    double as_double(double dflt = 0) const { return kind == Num ? (is_int ? static_cast<double>(inum) : num) : dflt; }
    const std::string& as_str() const {
        if (kind != Str) throw std::runtime_error("json: not a string");
        return str;
    }
};

class JsonParser {
public:
    JsonParser(const char* p, size_t n) : p_(p), end_(p + n) {}
    Json parse() {
        Json j = value();
        ws();
        return j;
    }

private:
    const char* p_;
    const char* end_;
    [[noreturn]] void fail(const char* what) { throw std::runtime_error(std::string("json: ") + what); }
    void ws() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_;
    }
    static void put_utf8(std::string& out, uint32_t cp) {
        if (cp < 0x80) out.push_back(static_cast<char>(cp));
        else if (cp < 0x800) { out.push_back(static_cast<char>(0xC0 | (cp >> 6))); out.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
        else if (cp < 0x10000) {
            out.push_back(static_cast<char>(0xE0 | (cp >> 12)));
            out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
            out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
        } else {
            out.push_back(static_cast<char>(0xF0 | (cp >> 18)));
            out.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
            out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
            out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
        }
    }
    uint32_t hex4() {
        if (end_ - p_ < 4) fail("bad \\u escape");
        uint32_t v = 0;
        for (int i = 0; i < 4; ++i) {
            char c = *p_++;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= c - '0';
            else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
            else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
            else fail("bad hex digit");
        }
        return v;
    }
    std::string string() {
        if (*p_ != '"') fail("expected string");
        ++p_;
        std::string out;
        while (p_ < end_ && *p_ != '"') {
            char c = *p_++;
            if (c != '\\') { out.push_back(c); continue; }
            if (p_ >= end_) fail("bad escape");
            char e = *p_++;
            switch (e) {
                case 'n': out.push_back('\n'); break;
                case 't': out.push_back('\t'); break;
                case 'r': out.push_back('\r'); break;
                case 'b': out.push_back('\b'); break;
                case 'f': out.push_back('\f'); break;
                case 'u': {
                    uint32_t cp = hex4();
                    if (cp >= 0xD800 && cp < 0xDC00 && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
                        p_ += 2;
                        uint32_t lo = hex4();
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    put_utf8(out, cp);
                    break;
                }
                default: out.push_back(e);
            }
        }
        if (p_ >= end_) fail("unterminated string");
        ++p_;
        return out;
    }
    Json value() {
        ws();
        if (p_ >= end_) fail("unexpected end");
        Json j;
        char c = *p_;
        if (c == '{') {
            j.kind = Json::Obj;
            ++p_;
            ws();
            if (p_ < end_ && *p_ == '}') { ++p_; return j; }
            while (true) {
                ws();
                std::string k = string();
                ws();
                if (p_ >= end_ || *p_ != ':') fail("expected ':'");
                ++p_;
                j.obj.emplace_back(std::move(k), value());
                ws();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == '}') { ++p_; break; }
                fail("expected ',' or '}'");
            }
        } else if (c == '[') {
            j.kind = Json::Arr;
            ++p_;
            ws();
            if (p_ < end_ && *p_ == ']') { ++p_; return j; }
            while (true) {
                j.arr.push_back(value());
                ws();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == ']') { ++p_; break; }
                fail("expected ',' or ']'");
            }
        } else if (c == '"') {
            j.kind = Json::Str;
            j.str = string();
        } else if (c == 't' && end_ - p_ >= 4 && std::string(p_, 4) == "true") { j.kind = Json::Bool; j.b = true; p_ += 4; }
        else if (c == 'f' && end_ - p_ >= 5 && std::string(p_, 5) == "false") { j.kind = Json::Bool; p_ += 5; }
        else if (c == 'n' && end_ - p_ >= 4 && std::string(p_, 4) == "null") { p_ += 4; }
        else {
            const char* s = p_;
            bool integral = true;
            while (p_ < end_ && (*p_ == '-' || *p_ == '+' || (*p_ >= '0' && *p_ <= '9') || *p_ == '.' || *p_ == 'e' || *p_ == 'E')) {
                if (*p_ == '.' || *p_ == 'e' || *p_ == 'E') integral = false;
                ++p_;
            }
            if (s == p_) fail("unexpected character");
            std::string t(s, p_);
            j.kind = Json::Num;
            j.is_int = integral;
            if (integral) j.inum = std::strtoll(t.c_str(), nullptr, 10);
            j.num = std::strtod(t.c_str(), nullptr);
        }
        return j;
    }
};

inline Json parse_json(const std::string& s) { return JsonParser(s.data(), s.size()).parse(); }

inline void json_escape(std::string& out, const std::string& s) {
    out.push_back('"');
    for (unsigned char c : s) {
        switch (c) {
            case '"': out += "\\\""; break;
            case '\\': out += "\\\\"; break;
            case '\n': out += "\\n"; break;
            case '\t': out += "\\t"; break;
            case '\r': out += "\\r"; break;
            default:
                if (c < 0x20) { char buf[8]; snprintf(buf, sizeof buf, "\\u%04x", c); out += buf; }
                else out.push_back(static_cast<char>(c));
        }
    }
    out.push_back('"');
}

}  // namespace sg
