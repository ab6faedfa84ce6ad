#include "util/json.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <stdexcept>

namespace illm {

static const Json kNull;

bool Json::has(const std::string& key) const {
    for (auto& m : o_)
        if (m.first == key) return true;
    return false;
}
const Json& Json::at(const std::string& key) const {
    for (auto& m : o_)
        if (m.first == key) return m.second;
    return kNull;
}
void Json::set(const std::string& key, Json v) {
    if (kind_ != Object) { kind_ = Object; o_.clear(); }
    for (auto& m : o_)
        if (m.first == key) { m.second = std::move(v); return; }
    o_.emplace_back(key, std::move(v));
}

static void dump_string(const std::string& s, std::string& out) {
    out += '"';
    for (unsigned char c : s) {
        switch (c) {
            case '"': out += "\\\""; break;
            case '\\': out += "\\\\"; break;
            case '\n': out += "\\n"; break;
            case '\r': out += "\\r"; break;
            case '\t': out += "\\t"; break;
            default:
                if (c < 0x20) { char buf[8]; snprintf(buf, sizeof buf, "\\u%04x", c); out += buf; }
                else out += (char)c;
        }
    }
    out += '"';
}

void Json::dump_to(std::string& out, int indent, int depth) const {
    auto newline = [&](int d) {
        if (indent < 0) return;
        out += '\n';
        out.append((size_t)(indent * d), ' ');
    };
    switch (kind_) {
        case Null: out += "null"; break;
        case Bool: out += b_ ? "true" : "false"; break;
        case Int: out += std::to_string(i_); break;
        case Double: {
            if (!std::isfinite(d_)) { out += "null"; break; }
            char buf[40];
            snprintf(buf, sizeof buf, "%.17g", d_);
            // the shortest form that reads back as the same number
            for (int p = 1; p < 17; p++) {
                char b2[40];
                snprintf(b2, sizeof b2, "%.*g", p, d_);
                if (strtod(b2, nullptr) == d_) { snprintf(buf, sizeof buf, "%s", b2); break; }
            }
            std::string s = buf;
            if (s.find_first_of(".eEn") == std::string::npos) s += ".0";
            out += s;
            break;
        }
        case String: dump_string(s_, out); break;
        case Array:
            out += '[';
            for (size_t i = 0; i < a_.size(); i++) {
                if (i) out += indent < 0 ? ", " : ",";
                newline(depth + 1);
                a_[i].dump_to(out, indent, depth + 1);
            }
            if (!a_.empty()) newline(depth);
            out += ']';
            break;
        case Object:
            out += '{';
            for (size_t i = 0; i < o_.size(); i++) {
                if (i) out += indent < 0 ? ", " : ",";
                newline(depth + 1);
                dump_string(o_[i].first, out);
                out += ": ";
                o_[i].second.dump_to(out, indent, depth + 1);
            }
            if (!o_.empty()) newline(depth);
            out += '}';
            break;
    }
}

std::string Json::dump(int indent) const {
    std::string out;
    dump_to(out, indent, 0);
    return out;
}

std::string Json::repr() const {
    if (kind_ == String) return "'" + s_ + "'";
    std::string s = dump();
    if (s.size() > 60) s = s.substr(0, 57) + "...";
    return s;
}

namespace {
struct Parser {
    const std::string& t;
    size_t p = 0;
    explicit Parser(const std::string& text) : t(text) {}
    [[noreturn]] void fail(const std::string& what) {
        throw std::runtime_error(what + " at byte " + std::to_string(p));
    }
    void ws() {
        while (p < t.size() && (t[p] == ' ' || t[p] == '\n' || t[p] == '\t' || t[p] == '\r')) p++;
    }
    bool lit(const char* s) {
        size_t n = 0;
        while (s[n]) n++;
        if (t.compare(p, n, s) == 0) { p += n; return true; }
        return false;
    }
    static void utf8(unsigned cp, std::string& out) {
        if (cp < 0x80) out += (char)cp;
        else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
        else if (cp < 0x10000) {
            out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F));
        } else {
            out += (char)(0xF0 | (cp >> 18)); out += (char)(0x80 | ((cp >> 12) & 0x3F));
            out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F));
        }
    }
    unsigned hex4() {
        if (p + 4 > t.size()) fail("short \\u escape");
        unsigned v = 0;
        for (int i = 0; i < 4; i++) {
            char c = t[p++];
            v <<= 4;
            if (c >= '0' && c <= '9') v |= (unsigned)(c - '0');
            else if (c >= 'a' && c <= 'f') v |= (unsigned)(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= (unsigned)(c - 'A' + 10);
            else fail("bad \\u escape");
        }
        return v;
    }
    std::string str() {
        if (t[p] != '"') fail("expected a string");
        p++;
        std::string out;
        while (true) {
            if (p >= t.size()) fail("unterminated string");
            char c = t[p++];
            if (c == '"') break;
            if (c != '\\') { out += c; continue; }
            if (p >= t.size()) fail("unterminated string");
            char e = t[p++];
            switch (e) {
                case '"': out += '"'; break;
                case '\\': out += '\\'; break;
                case '/': out += '/'; break;
                case 'b': out += '\b'; break;
                case 'f': out += '\f'; break;
                case 'n': out += '\n'; break;
                case 'r': out += '\r'; break;
                case 't': out += '\t'; break;
                case 'u': {
                    unsigned cp = hex4();
                    if (cp >= 0xD800 && cp < 0xDC00 && t.compare(p, 2, "\\u") == 0) {
                        p += 2;
                        unsigned lo = hex4();
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    utf8(cp, out);
                    break;
                }
                default: fail("bad escape");
            }
        }
        return out;
    }
    Json value(int depth) {
        if (depth > 200) fail("nested too deeply");
        ws();
        if (p >= t.size()) fail("unexpected end");
        char c = t[p];
        if (c == '{') {
            p++;
            Json o = Json::object();
            ws();
            if (p < t.size() && t[p] == '}') { p++; return o; }
            while (true) {
                ws();
                if (p >= t.size()) fail("unterminated object");
                std::string k = str();
                ws();
                if (p >= t.size() || t[p] != ':') fail("expected ':'");
                p++;
                o.set(k, value(depth + 1));
                ws();
                if (p < t.size() && t[p] == ',') { p++; continue; }
                if (p < t.size() && t[p] == '}') { p++; return o; }
                fail("expected ',' or '}'");
            }
        }
        if (c == '[') {
            p++;
            Json a = Json::array();
            ws();
            if (p < t.size() && t[p] == ']') { p++; return a; }
            while (true) {
                a.push(value(depth + 1));
                ws();
                if (p < t.size() && t[p] == ',') { p++; continue; }
                if (p < t.size() && t[p] == ']') { p++; return a; }
                fail("expected ',' or ']'");
            }
        }
        if (c == '"') return Json(str());
        if (lit("true")) return Json(true);
        if (lit("false")) return Json(false);
        if (lit("null")) return Json();
        if (lit("NaN")) return Json(std::nan(""));
        if (lit("Infinity")) return Json(INFINITY);
        if (lit("-Infinity")) return Json(-INFINITY);
        size_t s = p;
        if (t[p] == '-') p++;
        bool is_int = true;
        while (p < t.size() && ((t[p] >= '0' && t[p] <= '9') || t[p] == '.' || t[p] == 'e' || t[p] == 'E' || t[p] == '+' ||
                                t[p] == '-')) {
            if (t[p] == '.' || t[p] == 'e' || t[p] == 'E') is_int = false;
            p++;
        }
        if (p == s || (p == s + 1 && t[s] == '-')) fail("unexpected character");
        std::string num = t.substr(s, p - s);
        if (is_int && num.size() < 19) return Json((long long)strtoll(num.c_str(), nullptr, 10));
        return Json(strtod(num.c_str(), nullptr));
    }
};
}  // namespace

Json Json::parse(const std::string& text) {
    Parser ps(text);
    Json v = ps.value(0);
    ps.ws();
    if (ps.p != text.size()) ps.fail("trailing characters");
    return v;
}

}  // namespace illm
