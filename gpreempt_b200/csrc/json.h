// Minimal JSON value, parser and writer (the reference links jsoncpp, which is an empty
// submodule in its tree).  Covers what the task configs (config/A.json) and the graph JSON
// (src/model.cpp:128-235) need: objects, arrays, strings, numbers, booleans, null.
#pragma once

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace gpx {

class Json {
public:
    enum Type { Null, Bool, Number, String, Array, Object };

    Json() : type_(Null) {}
    Json(bool b) : type_(Bool), num_(b ? 1 : 0) {}
    Json(double d) : type_(Number), num_(d) {}
    Json(int i) : type_(Number), num_(i) {}
    Json(long long i) : type_(Number), num_((double)i) {}
    Json(unsigned long long i) : type_(Number), num_((double)i) {}
    Json(const char *s) : type_(String), str_(s) {}
    Json(const std::string &s) : type_(String), str_(s) {}

    static Json array() {
        Json j;
        j.type_ = Array;
        return j;
    }
    static Json object() {
        Json j;
        j.type_ = Object;
        return j;
    }

    Type type() const { return type_; }
    bool is_null() const { return type_ == Null; }
    bool is_object() const { return type_ == Object; }
    bool is_array() const { return type_ == Array; }
    bool is_string() const { return type_ == String; }
    bool is_number() const { return type_ == Number; }

    bool as_bool(bool dflt = false) const {
        if (type_ == Bool || type_ == Number) return num_ != 0;
        return dflt;
    }
    double as_double(double dflt = 0) const {
        if (type_ == Number || type_ == Bool) return num_;
        if (type_ == String) return atof(str_.c_str());
        return dflt;
    }
    long long as_int(long long dflt = 0) const {
        if (type_ == Number || type_ == Bool) return (long long)num_;
        if (type_ == String) return atoll(str_.c_str());
        return dflt;
    }
    const std::string &as_string() const { return str_; }

    size_t size() const { return type_ == Array ? arr_.size() : type_ == Object ? keys_.size() : 0; }
    const Json &operator[](size_t i) const { return i < arr_.size() ? arr_[i] : null_value(); }
    bool has(const std::string &k) const { return type_ == Object && obj_.count(k); }
    const Json &operator[](const std::string &k) const {
        if (type_ != Object) return null_value();
        auto it = obj_.find(k);
        return it == obj_.end() ? null_value() : it->second;
    }
    const Json &operator[](const char *k) const { return (*this)[std::string(k)]; }
    const std::vector<std::string> &keys() const { return keys_; }

    void push(const Json &v) {
        if (type_ != Array) {
            *this = array();
        }
        arr_.push_back(v);
    }
    void set(const std::string &k, const Json &v) {
        if (type_ != Object) {
            *this = object();
        }
        if (!obj_.count(k)) keys_.push_back(k);
        obj_[k] = v;
    }

    // Returns false and fills *err on malformed input.
    static bool parse(const std::string &text, Json *out, std::string *err) {
        Parser p{text.c_str(), text.c_str() + text.size(), text.c_str(), ""};
        Json v;
        if (!p.value(&v)) {
            if (err) *err = p.err + " at offset " + std::to_string(p.cur - p.begin);
            return false;
        }
        p.ws();
        if (p.cur != p.end) {
            if (err) *err = "trailing characters at offset " + std::to_string(p.cur - p.begin);
            return false;
        }
        *out = v;
        return true;
    }

    std::string dump(int indent = -1) const {
        std::string s;
        write(s, indent, 0);
        return s;
    }

private:
    Type type_;
    double num_ = 0;
    std::string str_;
    std::vector<Json> arr_;
    std::map<std::string, Json> obj_;
    std::vector<std::string> keys_;  // insertion order

    static const Json &null_value() {
        static const Json n;
        return n;
    }

    static void write_string(std::string &s, const std::string &v) {
        s.push_back('"');
        for (unsigned char c : v) {
            switch (c) {
                case '"': s += "\\\""; break;
                case '\\': s += "\\\\"; break;
                case '\n': s += "\\n"; break;
                case '\t': s += "\\t"; break;
                case '\r': s += "\\r"; break;
                default:
                    if (c < 0x20) {
                        char buf[8];
                        snprintf(buf, sizeof(buf), "\\u%04x", c);
                        s += buf;
                    } else {
                        s.push_back((char)c);
                    }
            }
        }
        s.push_back('"');
    }

    void write(std::string &s, int indent, int depth) const {
        auto nl = [&](int d) {
            if (indent >= 0) {
                s.push_back('\n');
                s.append((size_t)indent * d, ' ');
            }
        };
        switch (type_) {
            case Null: s += "null"; break;
            case Bool: s += num_ != 0 ? "true" : "false"; break;
            case Number: {
                char buf[40];
                if (std::isfinite(num_) && num_ == std::floor(num_) && std::fabs(num_) < 9e15)
                    snprintf(buf, sizeof(buf), "%lld", (long long)num_);
                else if (std::isfinite(num_))
                    snprintf(buf, sizeof(buf), "%.9g", num_);
                else
                    snprintf(buf, sizeof(buf), "null");
                s += buf;
                break;
            }
            case String: write_string(s, str_); break;
            case Array:
                s.push_back('[');
                for (size_t i = 0; i < arr_.size(); ++i) {
                    if (i) s.push_back(',');
                    nl(depth + 1);
                    arr_[i].write(s, indent, depth + 1);
                }
                if (!arr_.empty()) nl(depth);
                s.push_back(']');
                break;
            case Object:
                s.push_back('{');
                for (size_t i = 0; i < keys_.size(); ++i) {
                    if (i) s.push_back(',');
                    nl(depth + 1);
                    write_string(s, keys_[i]);
                    s += indent >= 0 ? ": " : ":";
                    obj_.at(keys_[i]).write(s, indent, depth + 1);
                }
                if (!keys_.empty()) nl(depth);
                s.push_back('}');
                break;
        }
    }

    struct Parser {
        const char *cur, *end, *begin;
        std::string err;
        int depth = 0;

        void ws() {
            while (cur < end && (*cur == ' ' || *cur == '\n' || *cur == '\t' || *cur == '\r')) ++cur;
        }
        bool fail(const char *m) {
            err = m;
            return false;
        }
        bool lit(const char *w) {
            size_t n = strlen(w);
            if ((size_t)(end - cur) < n || strncmp(cur, w, n) != 0) return fail("bad literal");
            cur += n;
            return true;
        }
        bool string(std::string *out) {
            if (cur >= end || *cur != '"') return fail("expected string");
            ++cur;
            out->clear();
            while (cur < end && *cur != '"') {
                char c = *cur++;
                if (c == '\\') {
                    if (cur >= end) return fail("bad escape");
                    char e = *cur++;
                    switch (e) {
                        case 'n': out->push_back('\n'); break;
                        case 't': out->push_back('\t'); break;
                        case 'r': out->push_back('\r'); break;
                        case 'b': out->push_back('\b'); break;
                        case 'f': out->push_back('\f'); break;
                        case 'u': {
                            if (end - cur < 4) return fail("bad \\u escape");
                            unsigned cp = (unsigned)strtoul(std::string(cur, 4).c_str(), nullptr, 16);
                            cur += 4;
                            if (cp < 0x80) {
                                out->push_back((char)cp);
                            } else if (cp < 0x800) {
                                out->push_back((char)(0xC0 | (cp >> 6)));
                                out->push_back((char)(0x80 | (cp & 0x3F)));
                            } else {
                                out->push_back((char)(0xE0 | (cp >> 12)));
                                out->push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
                                out->push_back((char)(0x80 | (cp & 0x3F)));
                            }
                            break;
                        }
                        default: out->push_back(e);
                    }
                } else {
                    out->push_back(c);
                }
            }
            if (cur >= end) return fail("unterminated string");
            ++cur;
            return true;
        }
        bool value(Json *out) {
            if (++depth > 200) return fail("nesting too deep");
            ws();
            if (cur >= end) return fail("unexpected end");
            bool ok = true;
            char c = *cur;
            if (c == '{') {
                ++cur;
                *out = Json::object();
                ws();
                if (cur < end && *cur == '}') {
                    ++cur;
                } else {
                    for (;;) {
                        ws();
                        std::string k;
                        if (!string(&k)) return false;
                        ws();
                        if (cur >= end || *cur != ':') return fail("expected ':'");
                        ++cur;
                        Json v;
                        if (!value(&v)) return false;
                        out->set(k, v);
                        ws();
                        if (cur < end && *cur == ',') {
                            ++cur;
                            continue;
                        }
                        if (cur < end && *cur == '}') {
                            ++cur;
                            break;
                        }
                        return fail("expected ',' or '}'");
                    }
                }
            } else if (c == '[') {
                ++cur;
                *out = Json::array();
                ws();
                if (cur < end && *cur == ']') {
                    ++cur;
                } else {
                    for (;;) {
                        Json v;
                        if (!value(&v)) return false;
                        out->push(v);
                        ws();
                        if (cur < end && *cur == ',') {
                            ++cur;
                            continue;
                        }
                        if (cur < end && *cur == ']') {
                            ++cur;
                            break;
                        }
                        return fail("expected ',' or ']'");
                    }
                }
            } else if (c == '"') {
                std::string s;
                ok = string(&s);
                if (ok) *out = Json(s);
            } else if (c == 't') {
                ok = lit("true");
                if (ok) *out = Json(true);
            } else if (c == 'f') {
                ok = lit("false");
                if (ok) *out = Json(false);
            } else if (c == 'n') {
                ok = lit("null");
                if (ok) *out = Json();
            } else if (c == '-' || (c >= '0' && c <= '9')) {
                char *e = nullptr;
                double d = strtod(cur, &e);
                if (e == cur) return fail("bad number");
                cur = e;
                *out = Json(d);
            } else {
                return fail("unexpected character");
            }
            --depth;
            return ok;
        }
    };
};

}  // namespace gpx
