// A small JSON value with a parser and a writer: config.json, the header of safetensors files, the
// trace of bin/trace_run and the binding's structured arguments.  Objects keep the order of their
// keys; numbers remember whether they were written as integers.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <utility>
#include <vector>

namespace illm {

class Json {
public:
    enum Kind { Null, Bool, Int, Double, String, Array, Object };
    Json() : kind_(Null) {}
    Json(std::nullptr_t) : kind_(Null) {}
    Json(bool b) : kind_(Bool), b_(b) {}
    Json(int v) : kind_(Int), i_(v) {}
    Json(long v) : kind_(Int), i_(v) {}
    Json(long long v) : kind_(Int), i_(v) {}
    Json(unsigned long v) : kind_(Int), i_((long long)v) {}
    Json(double v) : kind_(Double), d_(v) {}
    Json(const char* s) : kind_(String), s_(s) {}
    Json(const std::string& s) : kind_(String), s_(s) {}
    static Json array() { Json j; j.kind_ = Array; return j; }
    static Json object() { Json j; j.kind_ = Object; return j; }

    Kind kind() const { return kind_; }
    bool is_null() const { return kind_ == Null; }
    bool is_bool() const { return kind_ == Bool; }
    bool is_int() const { return kind_ == Int; }
    bool is_number() const { return kind_ == Int || kind_ == Double; }
    bool is_string() const { return kind_ == String; }
    bool is_array() const { return kind_ == Array; }
    bool is_object() const { return kind_ == Object; }

    bool as_bool() const { return b_; }
    long long as_int() const { return kind_ == Double ? (long long)d_ : i_; }
    double as_double() const { return kind_ == Int ? (double)i_ : d_; }
    const std::string& as_string() const { return s_; }

    // arrays
    size_t size() const { return kind_ == Array ? a_.size() : kind_ == Object ? o_.size() : 0; }
    const Json& operator[](size_t i) const { return a_[i]; }
    void push(Json v) { a_.push_back(std::move(v)); }
    const std::vector<Json>& items() const { return a_; }

    // objects
    bool has(const std::string& key) const;
    const Json& at(const std::string& key) const;          // a Null value if the key is absent
    void set(const std::string& key, Json v);
    const std::vector<std::pair<std::string, Json>>& members() const { return o_; }

    std::string dump(int indent = -1) const;
    // Throws std::runtime_error with the position of the fault.
    static Json parse(const std::string& text);
    // A short rendering for error messages ("found 3.5", "found 'x'").
    std::string repr() const;

private:
    void dump_to(std::string& out, int indent, int depth) const;
    Kind kind_;
    bool b_ = false;
    long long i_ = 0;
    double d_ = 0;
    std::string s_;
    std::vector<Json> a_;
    std::vector<std::pair<std::string, Json>> o_;
};

}  // namespace illm
