#include "json.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>

namespace hc {

static const Json kNullJson;

const Json &Json::operator[](const std::string &k) const
{
    if (type_ != OBJ) return kNullJson;
    auto it = obj_.find(k);
    return it == obj_.end() ? kNullJson : it->second;
}
const Json &Json::operator[](size_t i) const { return (type_ == ARR && i < arr_.size()) ? arr_[i] : kNullJson; }

bool Json::asInt(int64_t &out) const
{
    if (type_ == NUM) { out = (int64_t)num_; return true; }
    if (type_ == STR) {
        char *end = nullptr;
        long long v = strtoll(str_.c_str(), &end, 10);
        if (end == str_.c_str() || *end != '\0') return false;
        out = v;
        return true;
    }
    return false;
}

class JsonParser {
public:
    JsonParser(const std::string &t) : s_(t) {}
    bool Run(Json &out, std::string *err)
    {
        Ws();
        if (!Value(out)) { Fail(err); return false; }
        Ws();
        if (p_ != s_.size()) { msg_ = "trailing characters"; Fail(err); return false; }
        return true;
    }

private:
    const std::string &s_;
    size_t p_ = 0;
    std::string msg_;
    int depth_ = 0;

    void Fail(std::string *err)
    {
        if (!err) return;
        size_t line = 1, col = 1;
        for (size_t i = 0; i < p_ && i < s_.size(); ++i) {
            if (s_[i] == '\n') { ++line; col = 1; } else ++col;
        }
        *err = std::to_string(line) + ":" + std::to_string(col) + ": " + (msg_.empty() ? "syntax error" : msg_);
    }
    void Ws() { while (p_ < s_.size() && (s_[p_] == ' ' || s_[p_] == '\t' || s_[p_] == '\n' || s_[p_] == '\r')) ++p_; }
    bool Lit(const char *w) { size_t n = strlen_(w); if (s_.compare(p_, n, w) == 0) { p_ += n; return true; } return false; }
    static size_t strlen_(const char *w) { size_t n = 0; while (w[n]) ++n; return n; }

    bool Value(Json &out)
    {
        if (++depth_ > 64) { msg_ = "nesting too deep"; return false; }
        bool ok = ValueInner(out);
        --depth_;
        return ok;
    }
    bool ValueInner(Json &out)
    {
        if (p_ >= s_.size()) { msg_ = "unexpected end"; return false; }
        char c = s_[p_];
        if (c == '{') return Obj(out);
        if (c == '[') return Arr(out);
        if (c == '"') { out.type_ = Json::STR; return Str(out.str_); }
        if (Lit("true")) { out = Json(true); return true; }
        if (Lit("false")) { out = Json(false); return true; }
        if (Lit("null")) { out = Json(); return true; }
        return Num(out);
    }
    bool Num(Json &out)
    {
        const char *b = s_.c_str() + p_;
        char *e = nullptr;
        double v = strtod(b, &e);
        if (e == b) { msg_ = "bad number"; return false; }
        p_ += (size_t)(e - b);
        out = Json(v);
        return true;
    }
    bool Str(std::string &out)
    {
        ++p_;  // opening quote
        out.clear();
        while (p_ < s_.size()) {
            char c = s_[p_++];
            if (c == '"') return true;
            if (c == '\\') {
                if (p_ >= s_.size()) break;
                char e = s_[p_++];
                switch (e) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'u': {
                        if (p_ + 4 > s_.size()) { msg_ = "bad \\u escape"; return false; }
                        unsigned cp = (unsigned)strtoul(s_.substr(p_, 4).c_str(), nullptr, 16);
                        p_ += 4;
                        if (cp < 0x80) out += (char)cp;
                        else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
                        else { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
                        break;
                    }
                    default: out += e;
                }
            } else {
                out += c;
            }
        }
        msg_ = "unterminated string";
        return false;
    }
    bool Arr(Json &out)
    {
        ++p_;
        out = Json::Array();
        Ws();
        if (p_ < s_.size() && s_[p_] == ']') { ++p_; return true; }
        for (;;) {
            Json v;
            Ws();
            if (!Value(v)) return false;
            out.arr_.push_back(v);
            Ws();
            if (p_ < s_.size() && s_[p_] == ',') { ++p_; continue; }
            if (p_ < s_.size() && s_[p_] == ']') { ++p_; return true; }
            msg_ = "expected , or ]";
            return false;
        }
    }
    bool Obj(Json &out)
    {
        ++p_;
        out = Json::Object();
        Ws();
        if (p_ < s_.size() && s_[p_] == '}') { ++p_; return true; }
        for (;;) {
            Ws();
            if (p_ >= s_.size() || s_[p_] != '"') { msg_ = "expected key"; return false; }
            std::string k;
            if (!Str(k)) return false;
            Ws();
            if (p_ >= s_.size() || s_[p_] != ':') { msg_ = "expected :"; return false; }
            ++p_;
            Ws();
            Json v;
            if (!Value(v)) return false;
            if (!out.obj_.count(k)) out.keys_.push_back(k);
            out.obj_[k] = v;
            Ws();
            if (p_ < s_.size() && s_[p_] == ',') { ++p_; continue; }
            if (p_ < s_.size() && s_[p_] == '}') { ++p_; return true; }
            msg_ = "expected , or }";
            return false;
        }
    }
};

bool Json::Parse(const std::string &text, Json &out, std::string *err) { return JsonParser(text).Run(out, err); }

static void Escape(const std::string &s, std::string &o)
{
    o += '"';
    for (char c : s) {
        switch (c) {
            case '"': o += "\\\""; break;
            case '\\': o += "\\\\"; break;
            case '\n': o += "\\n"; break;
            case '\t': o += "\\t"; break;
            case '\r': o += "\\r"; break;
            default:
                if ((unsigned char)c < 0x20) { char b[8]; snprintf(b, sizeof(b), "\\u%04x", c); o += b; }
                else o += c;
        }
    }
    o += '"';
}

static void DumpRec(const Json &j, int indent, int level, std::string &o);

std::string Json::Dump(int indent) const
{
    std::string o;
    DumpRec(*this, indent, 0, o);
    return o;
}

static void Nl(int indent, int level, std::string &o)
{
    if (indent > 0) { o += '\n'; o.append((size_t)(indent * level), ' '); }
}

static void DumpRec(const Json &j, int indent, int level, std::string &o)
{
    switch (j.type()) {
        case Json::NUL: o += "null"; break;
        case Json::BOOL: o += j.boolean() ? "true" : "false"; break;
        case Json::NUM: {
            double d = j.num();
            char b[40];
            if (std::floor(d) == d && std::fabs(d) < 9e15) snprintf(b, sizeof(b), "%lld", (long long)d);
            else snprintf(b, sizeof(b), "%.9g", d);
            o += b;
            break;
        }
        case Json::STR: Escape(j.str(), o); break;
        case Json::ARR:
            o += '[';
            for (size_t i = 0; i < j.size(); ++i) {
                if (i) o += ',';
                Nl(indent, level + 1, o);
                DumpRec(j[i], indent, level + 1, o);
            }
            if (j.size()) Nl(indent, level, o);
            o += ']';
            break;
        case Json::OBJ: {
            o += '{';
            bool first = true;
            for (auto &k : j.keys()) {
                if (!first) o += ',';
                first = false;
                Nl(indent, level + 1, o);
                Escape(k, o);
                o += indent > 0 ? ": " : ":";
                DumpRec(j[k], indent, level + 1, o);
            }
            if (!first) Nl(indent, level, o);
            o += '}';
            break;
        }
    }
}

}  // namespace hc
