#include "json.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "errors.h"

namespace sandy {

const char* Json::type_name() const {
    switch (type_) {
        case Type::Null: return "null";
        case Type::Bool: return "bool";
        case Type::Int: return "int";
        case Type::Float: return "float";
        case Type::String: return "str";
        case Type::Array: return "list";
        case Type::Object: return "object";
    }
    return "?";
}

bool Json::as_bool() const {
    if (type_ != Type::Bool) throw ValueError(std::string("JSON value is ") + type_name() + ", not a bool");
    return bool_;
}
int64_t Json::as_int() const {
    if (type_ == Type::Int) return int_;
    if (type_ == Type::Float && std::floor(float_) == float_ && std::fabs(float_) < 9e18) return (int64_t)float_;
    throw ValueError(std::string("JSON value is ") + type_name() + ", not an integer");
}
double Json::as_double() const {
    if (type_ == Type::Int) return (double)int_;
    if (type_ == Type::Float) return float_;
    throw ValueError(std::string("JSON value is ") + type_name() + ", not a number");
}
const std::string& Json::as_string() const {
    if (type_ != Type::String) throw ValueError(std::string("JSON value is ") + type_name() + ", not a string");
    return string_;
}
const Json::Array& Json::items() const {
    if (type_ != Type::Array) throw ValueError(std::string("JSON value is ") + type_name() + ", not a list");
    return array_;
}
Json::Array& Json::items() {
    if (type_ != Type::Array) throw ValueError(std::string("JSON value is ") + type_name() + ", not a list");
    return array_;
}
const Json::Object& Json::members() const {
    if (type_ != Type::Object) throw ValueError(std::string("JSON value is ") + type_name() + ", not an object");
    return object_;
}
bool Json::has(const std::string& key) const { return find(key) != nullptr; }
const Json* Json::find(const std::string& key) const {
    if (type_ != Type::Object) return nullptr;
    for (const auto& m : object_)
        if (m.first == key) return &m.second;
    return nullptr;
}
const Json& Json::at(const std::string& key) const {
    const Json* v = find(key);
    if (!v) throw ValueError("JSON object has no member '" + key + "'");
    return *v;
}
Json& Json::operator[](const std::string& key) {
    if (type_ == Type::Null) type_ = Type::Object;
    if (type_ != Type::Object) throw ValueError(std::string("JSON value is ") + type_name() + ", not an object");
    for (auto& m : object_)
        if (m.first == key) return m.second;
    object_.emplace_back(key, Json());
    return object_.back().second;
}
void Json::push(Json v) {
    if (type_ == Type::Null) type_ = Type::Array;
    if (type_ != Type::Array) throw ValueError(std::string("JSON value is ") + type_name() + ", not a list");
    array_.push_back(std::move(v));
}
size_t Json::size() const {
    if (type_ == Type::Array) return array_.size();
    if (type_ == Type::Object) return object_.size();
    return 0;
}

// ---- writer -------------------------------------------------------------------------------
static void dump_string(const std::string& s, std::string& out) {
    out.push_back('"');
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
                    std::snprintf(buf, sizeof buf, "\\u%04x", c);
                    out += buf;
                } else {
                    out.push_back((char)c);
                }
        }
    }
    out.push_back('"');
}

void Json::dump_to(std::string& out, int indent, int depth) const {
    auto newline = [&](int d) {
        if (indent < 0) return;
        out.push_back('\n');
        out.append((size_t)(indent * d), ' ');
    };
    switch (type_) {
        case Type::Null: out += "null"; break;
        case Type::Bool: out += bool_ ? "true" : "false"; break;
        case Type::Int: out += std::to_string(int_); break;
        case Type::Float: {
            if (!std::isfinite(float_)) { out += "null"; break; }
            char buf[40];
            std::snprintf(buf, sizeof buf, "%.17g", float_);
            out += buf;
            if (!std::strpbrk(buf, ".eEn")) out += ".0";
            break;
        }
        case Type::String: dump_string(string_, out); break;
        case Type::Array:
            out.push_back('[');
            for (size_t i = 0; i < array_.size(); i++) {
                if (i) out += indent < 0 ? "," : ",";
                newline(depth + 1);
                array_[i].dump_to(out, indent, depth + 1);
            }
            if (!array_.empty()) newline(depth);
            out.push_back(']');
            break;
        case Type::Object:
            out.push_back('{');
            for (size_t i = 0; i < object_.size(); i++) {
                if (i) out.push_back(',');
                newline(depth + 1);
                dump_string(object_[i].first, out);
                out += indent < 0 ? ":" : ": ";
                object_[i].second.dump_to(out, indent, depth + 1);
            }
            if (!object_.empty()) newline(depth);
            out.push_back('}');
            break;
    }
}

std::string Json::dump(int indent) const {
    std::string out;
    dump_to(out, indent, 0);
    return out;
}

// ---- parser -------------------------------------------------------------------------------
namespace {

struct Parser {
    const std::string& text;
    size_t pos = 0;
    int depth = 0;

    [[noreturn]] void fail(const std::string& why) const {
        throw ValueError("invalid JSON at byte " + std::to_string(pos) + ": " + why);
    }
    void skip() {
        while (pos < text.size() && (text[pos] == ' ' || text[pos] == '\n' || text[pos] == '\t' || text[pos] == '\r')) pos++;
    }
    char peek() {
        skip();
        if (pos >= text.size()) fail("unexpected end of text");
        return text[pos];
    }
    void expect(const char* word) {
        const size_t n = std::strlen(word);
        if (text.compare(pos, n, word) != 0) fail(std::string("expected '") + word + "'");
        pos += n;
    }
    static void utf8(unsigned cp, std::string& out) {
        if (cp < 0x80) out.push_back((char)cp);
        else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
        else if (cp < 0x10000) {
            out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
            out.push_back((char)(0x80 | (cp & 0x3F)));
        } else {
            out.push_back((char)(0xF0 | (cp >> 18))); out.push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
            out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F)));
        }
    }
    unsigned hex4() {
        if (pos + 4 > text.size()) fail("truncated \\u escape");
        unsigned v = 0;
        for (int i = 0; i < 4; i++) {
            const char c = text[pos++];
            v <<= 4;
            if (c >= '0' && c <= '9') v |= (unsigned)(c - '0');
            else if (c >= 'a' && c <= 'f') v |= (unsigned)(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= (unsigned)(c - 'A' + 10);
            else fail("bad \\u escape");
        }
        return v;
    }
    std::string string() {
        if (text[pos] != '"') fail("expected a string");
        pos++;
        std::string out;
        while (true) {
            if (pos >= text.size()) fail("unterminated string");
            const char c = text[pos++];
            if (c == '"') return out;
            if (c == '\\') {
                if (pos >= text.size()) fail("unterminated escape");
                const char e = text[pos++];
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
                        if (cp >= 0xD800 && cp < 0xDC00 && text.compare(pos, 2, "\\u") == 0) {
                            pos += 2;
                            const unsigned lo = hex4();
                            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                        }
                        utf8(cp, out);
                        break;
                    }
                    default: fail("unknown escape");
                }
            } else if ((unsigned char)c < 0x20) {
                fail("control character in a string");
            } else {
                out.push_back(c);
            }
        }
    }
    Json number() {
        const size_t start = pos;
        bool is_float = false;
        if (text[pos] == '-') pos++;
        if (pos >= text.size() || !(text[pos] >= '0' && text[pos] <= '9')) fail("expected a digit");
        while (pos < text.size() && text[pos] >= '0' && text[pos] <= '9') pos++;
        if (pos < text.size() && text[pos] == '.') {
            is_float = true;
            pos++;
            if (pos >= text.size() || !(text[pos] >= '0' && text[pos] <= '9')) fail("expected a digit after '.'");
            while (pos < text.size() && text[pos] >= '0' && text[pos] <= '9') pos++;
        }
        if (pos < text.size() && (text[pos] == 'e' || text[pos] == 'E')) {
            is_float = true;
            pos++;
            if (pos < text.size() && (text[pos] == '+' || text[pos] == '-')) pos++;
            if (pos >= text.size() || !(text[pos] >= '0' && text[pos] <= '9')) fail("expected a digit in the exponent");
            while (pos < text.size() && text[pos] >= '0' && text[pos] <= '9') pos++;
        }
        const std::string tok = text.substr(start, pos - start);
        if (!is_float && tok.size() <= 18) return Json((long long)std::strtoll(tok.c_str(), nullptr, 10));
        return Json(std::strtod(tok.c_str(), nullptr));
    }
    Json value() {
        if (++depth > 200) fail("nesting too deep");
        const char c = peek();
        Json out;
        if (c == '{') {
            pos++;
            out = Json::object();
            if (peek() == '}') { pos++; depth--; return out; }
            while (true) {
                skip();
                std::string key = string();
                if (peek() != ':') fail("expected ':'");
                pos++;
                out[key] = value();
                const char d = peek();
                pos++;
                if (d == '}') break;
                if (d != ',') fail("expected ',' or '}'");
            }
        } else if (c == '[') {
            pos++;
            out = Json::array();
            if (peek() == ']') { pos++; depth--; return out; }
            while (true) {
                out.push(value());
                const char d = peek();
                pos++;
                if (d == ']') break;
                if (d != ',') fail("expected ',' or ']'");
            }
        } else if (c == '"') {
            out = Json(string());
        } else if (c == 't') { expect("true"); out = Json(true); }
        else if (c == 'f') { expect("false"); out = Json(false); }
        else if (c == 'n') { expect("null"); }
        else if (c == 'N') { expect("NaN"); out = Json(std::nan("")); }              // as Python's json module writes them
        else if (c == 'I') { expect("Infinity"); out = Json((double)INFINITY); }
        else if (c == '-' && text.compare(pos, 9, "-Infinity") == 0) { pos += 9; out = Json(-(double)INFINITY); }
        else if (c == '-' || (c >= '0' && c <= '9')) out = number();
        else fail(std::string("unexpected character '") + c + "'");
        depth--;
        return out;
    }
};

}  // namespace

Json Json::parse(const std::string& text) {
    Parser p{text};
    Json v = p.value();
    p.skip();
    if (p.pos != text.size()) p.fail("text after the value");
    return v;
}

}  // namespace sandy
