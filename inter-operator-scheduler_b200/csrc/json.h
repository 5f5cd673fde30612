// Minimal JSON reader for the graph / block / stage wire format.
//
// The configs exchanged with the Python front-end only use objects, arrays, strings, integers,
// floats, booleans and null (python/ios/ir.py export_config methods), so a single recursive-descent
// pass into a tagged tree is all that is needed.  Object members keep their textual order (the
// stage profiler's input map relies on it).  Errors throw JsonError with a byte offset.
#pragma once
#include <cstdint>
#include <cstdlib>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace ios {

struct JsonError : std::runtime_error {
    explicit JsonError(const std::string &what) : std::runtime_error(what) {}
};

class Json {
public:
    enum Kind { Null, Bool, Number, String, Array, Object };

    Kind kind = Null;
    bool boolean = false;
    double number = 0.0;
    std::string text;
    std::vector<Json> items;                             // Array
    std::vector<std::pair<std::string, Json>> members;   // Object, in textual order

    bool is_null() const { return kind == Null; }
    bool is_array() const { return kind == Array; }
    bool is_object() const { return kind == Object; }
    bool is_string() const { return kind == String; }
    bool is_number() const { return kind == Number; }

    size_t size() const { return kind == Array ? items.size() : kind == Object ? members.size() : 0; }

    const Json &at(size_t i) const {
        if (kind != Array || i >= items.size()) throw JsonError("array index out of range");
        return items[i];
    }
    const Json *find(const std::string &key) const {
        if (kind != Object) return nullptr;
        for (const auto &m : members)
            if (m.first == key) return &m.second;
        return nullptr;
    }
    const Json &at(const std::string &key) const {
        const Json *p = find(key);
        if (!p) throw JsonError("missing key \"" + key + "\"");
        return *p;
    }
    int as_int() const {
        if (kind == Bool) return boolean ? 1 : 0;
        if (kind != Number) throw JsonError("expected a number");
        return static_cast<int>(number);
    }
    bool as_bool() const {
        if (kind == Bool) return boolean;
        if (kind == Number) return number != 0.0;
        throw JsonError("expected a boolean");
    }
    const std::string &as_string() const {
        if (kind != String) throw JsonError("expected a string");
        return text;
    }

    static Json parse(const char *src) {
        if (!src) throw JsonError("null JSON text");
        Reader r{src, src};
        Json v = r.value(0);
        r.skip_space();
        if (*r.p) r.fail("trailing characters");
        return v;
    }

private:
    struct Reader {
        const char *begin;
        const char *p;

        [[noreturn]] void fail(const std::string &why) const {
            throw JsonError("JSON: " + why + " at byte " + std::to_string(p - begin));
        }
        void skip_space() {
            while (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r') ++p;
        }
        bool take(char c) {
            skip_space();
            if (*p != c) return false;
            ++p;
            return true;
        }
        void expect_word(const char *word) {
            for (const char *w = word; *w; ++w, ++p)
                if (*p != *w) fail(std::string("expected '") + word + "'");
        }
        static void append_utf8(std::string &out, uint32_t cp) {
            if (cp < 0x80) {
                out += static_cast<char>(cp);
            } else if (cp < 0x800) {
                out += static_cast<char>(0xC0 | (cp >> 6));
                out += static_cast<char>(0x80 | (cp & 0x3F));
            } else if (cp < 0x10000) {
                out += static_cast<char>(0xE0 | (cp >> 12));
                out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F));
                out += static_cast<char>(0x80 | (cp & 0x3F));
            } else {
                out += static_cast<char>(0xF0 | (cp >> 18));
                out += static_cast<char>(0x80 | ((cp >> 12) & 0x3F));
                out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F));
                out += static_cast<char>(0x80 | (cp & 0x3F));
            }
        }
        uint32_t hex4() {
            uint32_t v = 0;
            for (int i = 0; i < 4; ++i, ++p) {
                char c = *p;
                v <<= 4;
                if (c >= '0' && c <= '9') v |= c - '0';
                else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
                else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
                else fail("bad \\u escape");
            }
            return v;
        }
        std::string string_body() {
            std::string out;
            for (;;) {
                char c = *p;
                if (c == '\0') fail("unterminated string");
                ++p;
                if (c == '"') return out;
                if (c != '\\') {
                    out += c;
                    continue;
                }
                char e = *p++;
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
                        uint32_t cp = hex4();
                        if (cp >= 0xD800 && cp < 0xDC00 && p[0] == '\\' && p[1] == 'u') {
                            p += 2;
                            uint32_t lo = hex4();
                            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                        }
                        append_utf8(out, cp);
                        break;
                    }
                    default: fail("bad escape");
                }
            }
        }
        Json value(int depth) {
            if (depth > 64) fail("nesting too deep");
            skip_space();
            Json v;
            char c = *p;
            if (c == '{') {
                ++p;
                v.kind = Object;
                if (take('}')) return v;
                do {
                    skip_space();
                    if (*p != '"') fail("expected a member name");
                    ++p;
                    std::string key = string_body();
                    if (!take(':')) fail("expected ':'");
                    v.members.emplace_back(std::move(key), value(depth + 1));
                } while (take(','));
                if (!take('}')) fail("expected '}'");
            } else if (c == '[') {
                ++p;
                v.kind = Array;
                if (take(']')) return v;
                do {
                    v.items.push_back(value(depth + 1));
                } while (take(','));
                if (!take(']')) fail("expected ']'");
            } else if (c == '"') {
                ++p;
                v.kind = String;
                v.text = string_body();
            } else if (c == 't') {
                expect_word("true");
                v.kind = Bool;
                v.boolean = true;
            } else if (c == 'f') {
                expect_word("false");
                v.kind = Bool;
            } else if (c == 'n') {
                expect_word("null");
            } else if (c == '-' || (c >= '0' && c <= '9')) {
                char *end = nullptr;
                v.kind = Number;
                v.number = std::strtod(p, &end);
                if (end == p) fail("bad number");
                p = end;
            } else {
                fail("unexpected character");
            }
            return v;
        }
    };
};

}  // namespace ios
