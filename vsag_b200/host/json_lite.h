// A small JSON reader for the index / search parameter strings (objects, arrays, strings, numbers,
// booleans, null).  The reference parses the same strings with nlohmann-json behind JsonType
// (src/json_wrapper.cpp); only the subset the IVF / BruteForce parameters use is needed here.
#pragma once

#include <cctype>
#include <cstdlib>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace vsag_b200_host {

class Json {
public:
    enum class Kind { Null, Bool, Number, String, Object, Array };

    Kind kind = Kind::Null;
    bool boolean = false;
    double number = 0.0;
    bool is_integer = false;
    std::string text;
    std::vector<std::pair<std::string, Json>> members;  // insertion order kept for messages
    std::vector<Json> items;

    static Json
    Parse(const std::string& s) {
        size_t pos = 0;
        Json v = parse_value(s, pos);
        skip_ws(s, pos);
        if (pos != s.size()) {
            throw std::invalid_argument("trailing characters after JSON value");
        }
        return v;
    }

    bool IsObject() const { return kind == Kind::Object; }
    bool IsString() const { return kind == Kind::String; }
    bool IsBool() const { return kind == Kind::Bool; }
    bool IsNumber() const { return kind == Kind::Number; }
    bool IsInteger() const { return kind == Kind::Number && is_integer; }

    bool
    Contains(const std::string& key) const {
        return Find(key) != nullptr;
    }
    const Json*
    Find(const std::string& key) const {
        for (const auto& m : members) {
            if (m.first == key) {
                return &m.second;
            }
        }
        return nullptr;
    }
    const Json&
    At(const std::string& key) const {
        const Json* p = Find(key);
        if (p == nullptr) {
            throw std::invalid_argument("missing key " + key);
        }
        return *p;
    }

private:
    static void
    skip_ws(const std::string& s, size_t& pos) {
        while (pos < s.size() && std::isspace(static_cast<unsigned char>(s[pos]))) {
            ++pos;
        }
    }

    static std::string
    parse_string(const std::string& s, size_t& pos) {
        std::string out;
        ++pos;  // opening quote
        while (pos < s.size() && s[pos] != '"') {
            char c = s[pos++];
            if (c == '\\') {
                if (pos >= s.size()) {
                    break;
                }
                char e = s[pos++];
                switch (e) {
                    case 'n': out.push_back('\n'); break;
                    case 't': out.push_back('\t'); break;
                    case 'r': out.push_back('\r'); break;
                    case 'b': out.push_back('\b'); break;
                    case 'f': out.push_back('\f'); break;
                    case 'u':
                        // parameter strings are ASCII; keep the escape verbatim
                        out += "\\u";
                        break;
                    default: out.push_back(e); break;
                }
            } else {
                out.push_back(c);
            }
        }
        if (pos >= s.size()) {
            throw std::invalid_argument("unterminated string in JSON");
        }
        ++pos;  // closing quote
        return out;
    }

    static Json
    parse_value(const std::string& s, size_t& pos) {
        skip_ws(s, pos);
        if (pos >= s.size()) {
            throw std::invalid_argument("unexpected end of JSON");
        }
        Json v;
        char c = s[pos];
        if (c == '{') {
            v.kind = Kind::Object;
            ++pos;
            skip_ws(s, pos);
            if (pos < s.size() && s[pos] == '}') {
                ++pos;
                return v;
            }
            for (;;) {
                skip_ws(s, pos);
                if (pos >= s.size() || s[pos] != '"') {
                    throw std::invalid_argument("expected a string key in JSON object");
                }
                std::string key = parse_string(s, pos);
                skip_ws(s, pos);
                if (pos >= s.size() || s[pos] != ':') {
                    throw std::invalid_argument("expected ':' in JSON object");
                }
                ++pos;
                v.members.emplace_back(key, parse_value(s, pos));
                skip_ws(s, pos);
                if (pos < s.size() && s[pos] == ',') {
                    ++pos;
                    continue;
                }
                if (pos < s.size() && s[pos] == '}') {
                    ++pos;
                    return v;
                }
                throw std::invalid_argument("expected ',' or '}' in JSON object");
            }
        }
        if (c == '[') {
            v.kind = Kind::Array;
            ++pos;
            skip_ws(s, pos);
            if (pos < s.size() && s[pos] == ']') {
                ++pos;
                return v;
            }
            for (;;) {
                v.items.push_back(parse_value(s, pos));
                skip_ws(s, pos);
                if (pos < s.size() && s[pos] == ',') {
                    ++pos;
                    continue;
                }
                if (pos < s.size() && s[pos] == ']') {
                    ++pos;
                    return v;
                }
                throw std::invalid_argument("expected ',' or ']' in JSON array");
            }
        }
        if (c == '"') {
            v.kind = Kind::String;
            v.text = parse_string(s, pos);
            return v;
        }
        if (s.compare(pos, 4, "true") == 0) {
            v.kind = Kind::Bool;
            v.boolean = true;
            pos += 4;
            return v;
        }
        if (s.compare(pos, 5, "false") == 0) {
            v.kind = Kind::Bool;
            v.boolean = false;
            pos += 5;
            return v;
        }
        if (s.compare(pos, 4, "null") == 0) {
            pos += 4;
            return v;
        }
        // number
        size_t start = pos;
        bool integer = true;
        if (s[pos] == '-' || s[pos] == '+') {
            ++pos;
        }
        while (pos < s.size() && (std::isdigit(static_cast<unsigned char>(s[pos])) || s[pos] == '.' ||
                                  s[pos] == 'e' || s[pos] == 'E' || s[pos] == '-' || s[pos] == '+')) {
            if (s[pos] == '.' || s[pos] == 'e' || s[pos] == 'E') {
                integer = false;
            }
            ++pos;
        }
        if (pos == start) {
            throw std::invalid_argument(std::string("unexpected character '") + c + "' in JSON");
        }
        v.kind = Kind::Number;
        v.is_integer = integer;
        v.number = std::strtod(s.substr(start, pos - start).c_str(), nullptr);
        return v;
    }
};

}  // namespace vsag_b200_host
