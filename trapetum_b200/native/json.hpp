// A small JSON reader and writer: what config.json, a safetensors header and a model spec need.
#pragma once
#include <cmath>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace tb {

struct Error : std::runtime_error {
    using std::runtime_error::runtime_error;
};

inline std::string fmt(const char* f, ...) __attribute__((format(printf, 1, 2)));
inline std::string fmt(const char* f, ...) {
    char buf[2048];
    va_list ap;
    va_start(ap, f);
    vsnprintf(buf, sizeof(buf), f, ap);
    va_end(ap);
    return buf;
}

class Json {
public:
    enum Kind { Null, Bool, Num, Str, Arr, Obj };
    Kind kind = Null;
    bool b = false;
    double num = 0;
    bool is_int = false;
    long long i = 0;
    std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;     // insertion order is kept (a safetensors header has one)

    bool is_null() const { return kind == Null; }
    bool has(const std::string& k) const { return find(k) != nullptr; }
    const Json* find(const std::string& k) const {
        if (kind != Obj) return nullptr;
        for (auto& kv : obj) if (kv.first == k) return &kv.second;
        return nullptr;
    }
    const Json& at(const std::string& k) const {
        const Json* v = find(k);
        if (!v) throw Error("key '" + k + "' is missing");
        return *v;
    }
    double number(const std::string& what) const {
        if (kind != Num) throw Error(what + " must be a number");
        return num;
    }
    long long integer(const std::string& what) const {
        if (kind != Num || !is_int) throw Error(what + " must be an integer");
        return i;
    }
    const std::string& string(const std::string& what) const {
        if (kind != Str) throw Error(what + " must be a string");
        return str;
    }
    // truthiness as Python's: null, false, 0, "" are false
    bool truthy() const {
        switch (kind) {
        case Null: return false;
        case Bool: return b;
        case Num: return num != 0;
        case Str: return !str.empty();
        case Arr: return !arr.empty();
        default: return !obj.empty();
        }
    }

    static Json parse(const std::string& text) {
        size_t p = 0;
        Json v = value(text, p);
        ws(text, p);
        if (p != text.size()) throw Error(fmt("JSON: trailing characters at offset %zu", p));
        return v;
    }

    static Json make_obj() { Json j; j.kind = Obj; return j; }
    static Json make_arr() { Json j; j.kind = Arr; return j; }
    static Json make_str(const std::string& s) { Json j; j.kind = Str; j.str = s; return j; }
    static Json make_int(long long v) { Json j; j.kind = Num; j.is_int = true; j.i = v; j.num = (double)v; return j; }
    static Json make_num(double v) { Json j; j.kind = Num; j.num = v; return j; }
    static Json make_bool(bool v) { Json j; j.kind = Bool; j.b = v; return j; }
    void set(const std::string& k, Json v) {
        kind = Obj;
        for (auto& kv : obj) if (kv.first == k) { kv.second = std::move(v); return; }
        obj.emplace_back(k, std::move(v));
    }

    std::string dump() const {
        std::string o;
        write(o);
        return o;
    }

private:
    static void ws(const std::string& s, size_t& p) {
        while (p < s.size() && (s[p] == ' ' || s[p] == '\n' || s[p] == '\t' || s[p] == '\r')) p++;
    }
    static Json value(const std::string& s, size_t& p) {
        ws(s, p);
        if (p >= s.size()) throw Error("JSON: unexpected end");
        Json v;
        char c = s[p];
        if (c == '{') {
            v.kind = Obj;
            p++;
            ws(s, p);
            if (p < s.size() && s[p] == '}') { p++; return v; }
            for (;;) {
                ws(s, p);
                if (p >= s.size() || s[p] != '"') throw Error(fmt("JSON: expected a key at offset %zu", p));
                std::string k = str_lit(s, p);
                ws(s, p);
                if (p >= s.size() || s[p] != ':') throw Error(fmt("JSON: expected ':' at offset %zu", p));
                p++;
                v.obj.emplace_back(std::move(k), value(s, p));
                ws(s, p);
                if (p < s.size() && s[p] == ',') { p++; continue; }
                if (p < s.size() && s[p] == '}') { p++; return v; }
                throw Error(fmt("JSON: expected ',' or '}' at offset %zu", p));
            }
        }
        if (c == '[') {
            v.kind = Arr;
            p++;
            ws(s, p);
            if (p < s.size() && s[p] == ']') { p++; return v; }
            for (;;) {
                v.arr.push_back(value(s, p));
                ws(s, p);
                if (p < s.size() && s[p] == ',') { p++; continue; }
                if (p < s.size() && s[p] == ']') { p++; return v; }
                throw Error(fmt("JSON: expected ',' or ']' at offset %zu", p));
            }
        }
        if (c == '"') { v.kind = Str; v.str = str_lit(s, p); return v; }
        if (s.compare(p, 4, "true") == 0) { p += 4; v.kind = Bool; v.b = true; return v; }
        if (s.compare(p, 5, "false") == 0) { p += 5; v.kind = Bool; v.b = false; return v; }
        if (s.compare(p, 4, "null") == 0) { p += 4; return v; }
        if (s.compare(p, 3, "NaN") == 0) { p += 3; v.kind = Num; v.num = NAN; return v; }
        if (s.compare(p, 8, "Infinity") == 0) { p += 8; v.kind = Num; v.num = INFINITY; return v; }
        // number
        size_t q = p;
        if (q < s.size() && (s[q] == '-' || s[q] == '+')) q++;
        bool integral = true;
        while (q < s.size() && (isdigit((unsigned char)s[q]) || s[q] == '.' || s[q] == 'e' || s[q] == 'E' || s[q] == '-' || s[q] == '+')) {
            if (s[q] == '.' || s[q] == 'e' || s[q] == 'E') integral = false;
            q++;
        }
        if (q == p) throw Error(fmt("JSON: unexpected character '%c' at offset %zu", c, p));
        std::string t = s.substr(p, q - p);
        v.kind = Num;
        v.num = strtod(t.c_str(), nullptr);
        if (integral) { v.is_int = true; v.i = strtoll(t.c_str(), nullptr, 10); }
        p = q;
        return v;
    }
    static std::string str_lit(const std::string& s, size_t& p) {
        std::string o;
        p++;                                   // opening quote
        while (p < s.size() && s[p] != '"') {
            char c = s[p++];
            if (c != '\\') { o += c; continue; }
            if (p >= s.size()) break;
            char e = s[p++];
            switch (e) {
            case 'n': o += '\n'; break;
            case 't': o += '\t'; break;
            case 'r': o += '\r'; break;
            case 'b': o += '\b'; break;
            case 'f': o += '\f'; break;
            case 'u': {
                unsigned cp = (unsigned)strtoul(s.substr(p, 4).c_str(), nullptr, 16);
                p += 4;
                if (cp < 0x80) o += (char)cp;
                else if (cp < 0x800) { o += (char)(0xC0 | (cp >> 6)); o += (char)(0x80 | (cp & 0x3F)); }
                else { o += (char)(0xE0 | (cp >> 12)); o += (char)(0x80 | ((cp >> 6) & 0x3F)); o += (char)(0x80 | (cp & 0x3F)); }
                break;
            }
            default: o += e;
            }
        }
        if (p >= s.size()) throw Error("JSON: unterminated string");
        p++;
        return o;
    }
    void write(std::string& o) const {
        switch (kind) {
        case Null: o += "null"; break;
        case Bool: o += b ? "true" : "false"; break;
        case Num:
            if (is_int) o += std::to_string(i);
            else { char buf[40]; snprintf(buf, sizeof buf, "%.17g", num); o += buf; }
            break;
        case Str:
            o += '"';
            for (char c : str) {
                if (c == '"' || c == '\\') { o += '\\'; o += c; }
                else if (c == '\n') o += "\\n";
                else if ((unsigned char)c < 0x20) { char buf[8]; snprintf(buf, sizeof buf, "\\u%04x", c); o += buf; }
                else o += c;
            }
            o += '"';
            break;
        case Arr:
            o += '[';
            for (size_t k = 0; k < arr.size(); k++) { if (k) o += ','; arr[k].write(o); }
            o += ']';
            break;
        case Obj:
            o += '{';
            for (size_t k = 0; k < obj.size(); k++) {
                if (k) o += ',';
                make_str(obj[k].first).write(o);
                o += ':';
                obj[k].second.write(o);
            }
            o += '}';
            break;
        }
    }
};

}  // namespace tb
