// A small JSON value with a parser and a writer: config.json, safetensors headers, model
// descriptions and the C interface's structured arguments all go through it.
#pragma once

#include <cstdint>
#include <map>
#include <string>
#include <utility>
#include <vector>

namespace sandy {

class Json {
public:
    enum class Type { Null, Bool, Int, Float, String, Array, Object };
    using Array = std::vector<Json>;
    using Member = std::pair<std::string, Json>;
    using Object = std::vector<Member>;      // members keep the order in which they were written

    Json() = default;
    Json(std::nullptr_t) {}
    Json(bool v) : type_(Type::Bool), bool_(v) {}
    Json(int v) : type_(Type::Int), int_(v) {}
    Json(long v) : type_(Type::Int), int_(v) {}
    Json(long long v) : type_(Type::Int), int_(v) {}
    Json(unsigned long v) : type_(Type::Int), int_((int64_t)v) {}
    Json(double v) : type_(Type::Float), float_(v) {}
    Json(const char* v) : type_(Type::String), string_(v) {}
    Json(std::string v) : type_(Type::String), string_(std::move(v)) {}
    Json(Array v) : type_(Type::Array), array_(std::move(v)) {}
    static Json object() { Json j; j.type_ = Type::Object; return j; }
    static Json array() { Json j; j.type_ = Type::Array; return j; }

    Type type() const { return type_; }
    bool is_null() const { return type_ == Type::Null; }
    bool is_bool() const { return type_ == Type::Bool; }
    bool is_int() const { return type_ == Type::Int; }
    bool is_number() const { return type_ == Type::Int || type_ == Type::Float; }
    bool is_string() const { return type_ == Type::String; }
    bool is_array() const { return type_ == Type::Array; }
    bool is_object() const { return type_ == Type::Object; }
    const char* type_name() const;

    bool as_bool() const;
    int64_t as_int() const;
    double as_double() const;
    const std::string& as_string() const;
    const Array& items() const;
    Array& items();
    const Object& members() const;

    // object access
    bool has(const std::string& key) const;
    const Json* find(const std::string& key) const;       // null if absent (or not an object)
    const Json& at(const std::string& key) const;         // throws if absent
    Json& operator[](const std::string& key);             // inserts a null member if absent
    void push(Json v);                                    // array append
    size_t size() const;

    std::string dump(int indent = -1) const;
    static Json parse(const std::string& text);           // throws ValueError with position and reason

private:
    void dump_to(std::string& out, int indent, int depth) const;
    Type type_ = Type::Null;
    bool bool_ = false;
    int64_t int_ = 0;
    double float_ = 0.0;
    std::string string_;
    Array array_;
    Object object_;
};

}  // namespace sandy
