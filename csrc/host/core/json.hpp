// A small self-contained JSON value with parser and serialiser. Objects keep their
// keys sorted (std::map), integers keep 64-bit precision (addresses and rkeys travel
// as JSON numbers), and doubles print with enough digits to round-trip.
#pragma once

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace slime {

class Json {
public:
    enum class Type { Null, Bool, Int, UInt, Double, String, Array, Object };
    using Array  = std::vector<Json>;
    using Object = std::map<std::string, Json>;

    Json(): type_(Type::Null) {}
    Json(std::nullptr_t): type_(Type::Null) {}
    Json(bool b): type_(Type::Bool) { u_.b = b; }
    Json(int v): type_(Type::Int) { u_.i = v; }
    Json(long v): type_(Type::Int) { u_.i = v; }
    Json(long long v): type_(Type::Int) { u_.i = v; }
    Json(unsigned v): type_(Type::UInt) { u_.u = v; }
    Json(unsigned long v): type_(Type::UInt) { u_.u = v; }
    Json(unsigned long long v): type_(Type::UInt) { u_.u = v; }
    Json(double v): type_(Type::Double) { u_.d = v; }
    Json(const char* s): type_(Type::String), str_(s ? s : "") {}
    Json(const std::string& s): type_(Type::String), str_(s) {}
    Json(std::string&& s): type_(Type::String), str_(std::move(s)) {}
    Json(const Array& a): type_(Type::Array), arr_(a) {}
    Json(Array&& a): type_(Type::Array), arr_(std::move(a)) {}
    Json(const Object& o): type_(Type::Object), obj_(o) {}
    Json(Object&& o): type_(Type::Object), obj_(std::move(o)) {}

    static Json array() { Json j; j.type_ = Type::Array; return j; }
    static Json object() { Json j; j.type_ = Type::Object; return j; }

    Type type() const { return type_; }
    bool is_null() const { return type_ == Type::Null; }
    bool is_bool() const { return type_ == Type::Bool; }
    bool is_number() const { return type_ == Type::Int || type_ == Type::UInt || type_ == Type::Double; }
    bool is_integer() const { return type_ == Type::Int || type_ == Type::UInt; }
    bool is_string() const { return type_ == Type::String; }
    bool is_array() const { return type_ == Type::Array; }
    bool is_object() const { return type_ == Type::Object; }

    bool as_bool(bool dflt = false) const
    {
        if (type_ == Type::Bool) return u_.b;
        if (is_integer()) return as_int() != 0;
        return dflt;
    }
    int64_t as_int(int64_t dflt = 0) const
    {
        switch (type_) {
            case Type::Int: return u_.i;
            case Type::UInt: return static_cast<int64_t>(u_.u);
            case Type::Double: return static_cast<int64_t>(u_.d);
            case Type::Bool: return u_.b ? 1 : 0;
            case Type::String: {
                char* end = nullptr;
                long long v = std::strtoll(str_.c_str(), &end, 10);
                return (end && *end == 0 && !str_.empty()) ? v : dflt;
            }
            default: return dflt;
        }
    }
    uint64_t as_uint(uint64_t dflt = 0) const
    {
        switch (type_) {
            case Type::Int: return static_cast<uint64_t>(u_.i);
            case Type::UInt: return u_.u;
            case Type::Double: return static_cast<uint64_t>(u_.d);
            case Type::String: {
                char* end = nullptr;
                unsigned long long v = std::strtoull(str_.c_str(), &end, 10);
                return (end && *end == 0 && !str_.empty()) ? v : dflt;
            }
            default: return dflt;
        }
    }
    double as_double(double dflt = 0.0) const
    {
        switch (type_) {
            case Type::Int: return static_cast<double>(u_.i);
            case Type::UInt: return static_cast<double>(u_.u);
            case Type::Double: return u_.d;
            default: return dflt;
        }
    }
    const std::string& as_string() const
    {
        static const std::string empty;
        return type_ == Type::String ? str_ : empty;
    }
    std::string string_or(const std::string& dflt) const { return type_ == Type::String ? str_ : dflt; }

    const Array& items() const { return arr_; }
    Array&       items() { return arr_; }
    const Object& fields() const { return obj_; }
    Object&       fields() { return obj_; }

    size_t size() const { return type_ == Type::Array ? arr_.size() : type_ == Type::Object ? obj_.size() : 0; }
    bool   contains(const std::string& k) const { return type_ == Type::Object && obj_.count(k) != 0; }

    // object access; a missing key on a const value yields a shared null
    const Json& operator[](const std::string& k) const
    {
        static const Json null_value;
        if (type_ != Type::Object) return null_value;
        auto it = obj_.find(k);
        return it == obj_.end() ? null_value : it->second;
    }
    Json& operator[](const std::string& k)
    {
        if (type_ == Type::Null) type_ = Type::Object;
        if (type_ != Type::Object) throw std::runtime_error("json: value is not an object");
        return obj_[k];
    }
    const Json& operator[](size_t i) const
    {
        static const Json null_value;
        return (type_ == Type::Array && i < arr_.size()) ? arr_[i] : null_value;
    }
    void push_back(Json v)
    {
        if (type_ == Type::Null) type_ = Type::Array;
        if (type_ != Type::Array) throw std::runtime_error("json: value is not an array");
        arr_.push_back(std::move(v));
    }
    void erase(const std::string& k) { obj_.erase(k); }

    bool operator==(const Json& o) const
    {
        if (is_number() && o.is_number()) {
            if (is_integer() && o.is_integer()) return as_int() == o.as_int() && as_uint() == o.as_uint();
            return as_double() == o.as_double();
        }
        if (type_ != o.type_) return false;
        switch (type_) {
            case Type::Null: return true;
            case Type::Bool: return u_.b == o.u_.b;
            case Type::String: return str_ == o.str_;
            case Type::Array: return arr_ == o.arr_;
            case Type::Object: return obj_ == o.obj_;
            default: return false;
        }
    }
    bool operator!=(const Json& o) const { return !(*this == o); }

    // ------------------------------------------------------------------ dump
    std::string dump(int indent = -1) const
    {
        std::string out;
        dump_to(out, indent, 0);
        return out;
    }

    // ------------------------------------------------------------------ parse
    static Json parse(const std::string& text)
    {
        Parser p{text.data(), text.data() + text.size()};
        Json   v = p.value();
        p.skip_ws();
        if (p.cur != p.end) p.fail("trailing characters");
        return v;
    }
    static bool try_parse(const std::string& text, Json& out)
    {
        try {
            out = parse(text);
            return true;
        }
        catch (const std::exception&) {
            return false;
        }
    }

    static void escape_to(std::string& out, const std::string& s)
    {
        out.push_back('"');
        for (unsigned char c : s) {
            switch (c) {
                case '"': out += "\\\""; break;
                case '\\': out += "\\\\"; break;
                case '\n': out += "\\n"; break;
                case '\r': out += "\\r"; break;
                case '\t': out += "\\t"; break;
                case '\b': out += "\\b"; break;
                case '\f': out += "\\f"; break;
                default:
                    if (c < 0x20) {
                        char buf[8];
                        snprintf(buf, sizeof(buf), "\\u%04x", c);
                        out += buf;
                    }
                    else {
                        out.push_back(static_cast<char>(c));
                    }
            }
        }
        out.push_back('"');
    }

private:
    struct Parser {
        const char* cur;
        const char* end;

        [[noreturn]] void fail(const char* what) const { throw std::runtime_error(std::string("json parse error: ") + what); }
        void skip_ws()
        {
            while (cur != end && (*cur == ' ' || *cur == '\n' || *cur == '\t' || *cur == '\r')) ++cur;
        }
        bool consume(const char* lit)
        {
            size_t n = strlen(lit);
            if (static_cast<size_t>(end - cur) >= n && memcmp(cur, lit, n) == 0) {
                cur += n;
                return true;
            }
            return false;
        }
        Json value()
        {
            skip_ws();
            if (cur == end) fail("unexpected end");
            switch (*cur) {
                case '{': return object();
                case '[': return array();
                case '"': return Json(string());
                case 't': if (consume("true")) return Json(true); fail("bad literal");
                case 'f': if (consume("false")) return Json(false); fail("bad literal");
                case 'n': if (consume("null")) return Json(); fail("bad literal");
                default: return number();
            }
        }
        Json object()
        {
            Json j = Json::object();
            ++cur;
            skip_ws();
            if (cur != end && *cur == '}') {
                ++cur;
                return j;
            }
            while (true) {
                skip_ws();
                if (cur == end || *cur != '"') fail("expected string key");
                std::string k = string();
                skip_ws();
                if (cur == end || *cur != ':') fail("expected ':'");
                ++cur;
                j.obj_[std::move(k)] = value();
                skip_ws();
                if (cur == end) fail("unterminated object");
                if (*cur == ',') {
                    ++cur;
                    continue;
                }
                if (*cur == '}') {
                    ++cur;
                    return j;
                }
                fail("expected ',' or '}'");
            }
        }
        Json array()
        {
            Json j = Json::array();
            ++cur;
            skip_ws();
            if (cur != end && *cur == ']') {
                ++cur;
                return j;
            }
            while (true) {
                j.arr_.push_back(value());
                skip_ws();
                if (cur == end) fail("unterminated array");
                if (*cur == ',') {
                    ++cur;
                    continue;
                }
                if (*cur == ']') {
                    ++cur;
                    return j;
                }
                fail("expected ',' or ']'");
            }
        }
        static void append_utf8(std::string& s, unsigned cp)
        {
            if (cp < 0x80) s.push_back(static_cast<char>(cp));
            else if (cp < 0x800) {
                s.push_back(static_cast<char>(0xC0 | (cp >> 6)));
                s.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
            }
            else if (cp < 0x10000) {
                s.push_back(static_cast<char>(0xE0 | (cp >> 12)));
                s.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
                s.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
            }
            else {
                s.push_back(static_cast<char>(0xF0 | (cp >> 18)));
                s.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
                s.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
                s.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
            }
        }
        unsigned hex4()
        {
            if (end - cur < 4) fail("bad \\u escape");
            unsigned v = 0;
            for (int i = 0; i < 4; ++i) {
                char c = *cur++;
                v <<= 4;
                if (c >= '0' && c <= '9') v |= c - '0';
                else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
                else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
                else fail("bad hex digit");
            }
            return v;
        }
        std::string string()
        {
            ++cur;  // opening quote
            std::string s;
            while (true) {
                if (cur == end) fail("unterminated string");
                char c = *cur++;
                if (c == '"') return s;
                if (c != '\\') {
                    s.push_back(c);
                    continue;
                }
                if (cur == end) fail("bad escape");
                char e = *cur++;
                switch (e) {
                    case '"': s.push_back('"'); break;
                    case '\\': s.push_back('\\'); break;
                    case '/': s.push_back('/'); break;
                    case 'b': s.push_back('\b'); break;
                    case 'f': s.push_back('\f'); break;
                    case 'n': s.push_back('\n'); break;
                    case 'r': s.push_back('\r'); break;
                    case 't': s.push_back('\t'); break;
                    case 'u': {
                        unsigned cp = hex4();
                        if (cp >= 0xD800 && cp < 0xDC00 && end - cur >= 6 && cur[0] == '\\' && cur[1] == 'u') {
                            cur += 2;
                            unsigned lo = hex4();
                            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                        }
                        append_utf8(s, cp);
                        break;
                    }
                    default: fail("unknown escape");
                }
            }
        }
        Json number()
        {
            const char* start = cur;
            bool        is_float = false;
            if (cur != end && (*cur == '-' || *cur == '+')) ++cur;
            while (cur != end && ((*cur >= '0' && *cur <= '9') || *cur == '.' || *cur == 'e' || *cur == 'E' || *cur == '-' || *cur == '+')) {
                if (*cur == '.' || *cur == 'e' || *cur == 'E') is_float = true;
                ++cur;
            }
            if (cur == start) fail("unexpected character");
            std::string tok(start, cur);
            if (is_float) return Json(std::strtod(tok.c_str(), nullptr));
            if (tok[0] == '-') return Json(static_cast<long long>(std::strtoll(tok.c_str(), nullptr, 10)));
            unsigned long long u = std::strtoull(tok.c_str(), nullptr, 10);
            if (u <= static_cast<unsigned long long>(INT64_MAX)) return Json(static_cast<long long>(u));
            return Json(u);
        }
    };

    void dump_to(std::string& out, int indent, int depth) const
    {
        auto newline = [&](int d) {
            if (indent >= 0) {
                out.push_back('\n');
                out.append(static_cast<size_t>(indent) * d, ' ');
            }
        };
        switch (type_) {
            case Type::Null: out += "null"; break;
            case Type::Bool: out += u_.b ? "true" : "false"; break;
            case Type::Int: out += std::to_string(u_.i); break;
            case Type::UInt: out += std::to_string(u_.u); break;
            case Type::Double: {
                if (!std::isfinite(u_.d)) {
                    out += "null";
                    break;
                }
                char buf[40];
                snprintf(buf, sizeof(buf), "%.17g", u_.d);
                out += buf;
                if (!strpbrk(buf, ".eE")) out += ".0";
                break;
            }
            case Type::String: escape_to(out, str_); break;
            case Type::Array: {
                out.push_back('[');
                bool first = true;
                for (const auto& v : arr_) {
                    if (!first) out.push_back(',');
                    first = false;
                    newline(depth + 1);
                    v.dump_to(out, indent, depth + 1);
                }
                if (!arr_.empty()) newline(depth);
                out.push_back(']');
                break;
            }
            case Type::Object: {
                out.push_back('{');
                bool first = true;
                for (const auto& kv : obj_) {
                    if (!first) out.push_back(',');
                    first = false;
                    newline(depth + 1);
                    escape_to(out, kv.first);
                    out.push_back(':');
                    if (indent >= 0) out.push_back(' ');
                    kv.second.dump_to(out, indent, depth + 1);
                }
                if (!obj_.empty()) newline(depth);
                out.push_back('}');
                break;
            }
        }
    }

    Type type_;
    union {
        bool     b;
        int64_t  i;
        uint64_t u;
        double   d;
    } u_{};
    std::string str_;
    Array       arr_;
    Object      obj_;
};

}  // namespace slime
