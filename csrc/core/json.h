// json.h - a small JSON value type with a recursive-descent parser and a writer.
// Used for rank tables, the tuning table and diagnostics; no external dependency.
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace hc {

class Json {
public:
    enum Type { NUL, BOOL, NUM, STR, ARR, OBJ };
    Json() : type_(NUL) {}
    explicit Json(bool b) : type_(BOOL), num_(b ? 1 : 0) {}
    explicit Json(double d) : type_(NUM), num_(d) {}
    explicit Json(int64_t i) : type_(NUM), num_((double)i) {}
    explicit Json(const std::string &s) : type_(STR), str_(s) {}
    static Json Array() { Json j; j.type_ = ARR; return j; }
    static Json Object() { Json j; j.type_ = OBJ; return j; }

    // Parses text; on failure returns false and describes the problem in *err ("line:col: message").
    static bool Parse(const std::string &text, Json &out, std::string *err);
    std::string Dump(int indent = 0) const;

    Type type() const { return type_; }
    bool isNull() const { return type_ == NUL; }
    bool isObject() const { return type_ == OBJ; }
    bool isArray() const { return type_ == ARR; }
    bool isString() const { return type_ == STR; }
    bool isNumber() const { return type_ == NUM; }
    bool has(const std::string &k) const { return type_ == OBJ && obj_.count(k) != 0; }
    const Json &operator[](const std::string &k) const;
    const Json &operator[](size_t i) const;
    Json &set(const std::string &k, const Json &v) { type_ = OBJ; obj_[k] = v; keys_.push_back(k); return *this; }
    Json &push(const Json &v) { type_ = ARR; arr_.push_back(v); return *this; }
    size_t size() const { return type_ == ARR ? arr_.size() : (type_ == OBJ ? obj_.size() : 0); }
    const std::vector<std::string> &keys() const { return keys_; }

    const std::string &str() const { return str_; }
    double num() const { return num_; }
    bool boolean() const { return num_ != 0; }
    // Rank tables write numbers both as 7 and as "7"; this accepts either.
    bool asInt(int64_t &out) const;
    int64_t intOr(int64_t def) const { int64_t v; return asInt(v) ? v : def; }
    std::string strOr(const std::string &def) const { return type_ == STR ? str_ : def; }

private:
    Type type_;
    double num_ = 0;
    std::string str_;
    std::vector<Json> arr_;
    std::map<std::string, Json> obj_;
    std::vector<std::string> keys_;
    friend class JsonParser;
};

}  // namespace hc
