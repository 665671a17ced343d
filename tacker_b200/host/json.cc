#include "json.h"

#include <cstdarg>
#include <cstdlib>
#include <fstream>
#include <sstream>
#include <stdexcept>

#include "Logger.h"

namespace {

struct Parser {
    const std::string& t;
    size_t i = 0;
    explicit Parser(const std::string& text) : t(text) {}
    [[noreturn]] void fail(const std::string& what) {
        throw std::runtime_error("json: " + what + " at byte " + std::to_string(i));
    }
    void ws() {
        while (i < t.size() && (t[i] == ' ' || t[i] == '\n' || t[i] == '\t' || t[i] == '\r')) ++i;
    }
    std::string string_() {
        if (t[i] != '"') fail("expected string");
        ++i;
        std::string out;
        while (i < t.size() && t[i] != '"') {
            if (t[i] == '\\') {
                if (++i >= t.size()) fail("bad escape");
                switch (t[i]) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'u': {
                        if (i + 4 >= t.size()) fail("bad \\u escape");
                        unsigned cp = static_cast<unsigned>(std::strtoul(t.substr(i + 1, 4).c_str(), nullptr, 16));
                        i += 4;
                        if (cp < 0x80) out += static_cast<char>(cp);
                        else if (cp < 0x800) {
                            out += static_cast<char>(0xC0 | (cp >> 6));
                            out += static_cast<char>(0x80 | (cp & 0x3F));
                        } else {
                            out += static_cast<char>(0xE0 | (cp >> 12));
                            out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F));
                            out += static_cast<char>(0x80 | (cp & 0x3F));
                        }
                        break;
                    }
                    default: out += t[i];
                }
                ++i;
            } else {
                out += t[i++];
            }
        }
        if (i >= t.size()) fail("unterminated string");
        ++i;
        return out;
    }
    std::shared_ptr<JsonValue> value() {
        ws();
        if (i >= t.size()) fail("unexpected end");
        auto v = std::make_shared<JsonValue>();
        const char c = t[i];
        if (c == '{') {
            v->kind = JsonValue::Object;
            ++i;
            ws();
            if (i < t.size() && t[i] == '}') {
                ++i;
                return v;
            }
            for (;;) {
                ws();
                std::string key = string_();
                ws();
                if (i >= t.size() || t[i] != ':') fail("expected ':'");
                ++i;
                v->members.emplace_back(key, value());
                ws();
                if (i < t.size() && t[i] == ',') {
                    ++i;
                    continue;
                }
                if (i < t.size() && t[i] == '}') {
                    ++i;
                    return v;
                }
                fail("expected ',' or '}'");
            }
        }
        if (c == '[') {
            v->kind = JsonValue::Array;
            ++i;
            ws();
            if (i < t.size() && t[i] == ']') {
                ++i;
                return v;
            }
            for (;;) {
                v->items.push_back(value());
                ws();
                if (i < t.size() && t[i] == ',') {
                    ++i;
                    continue;
                }
                if (i < t.size() && t[i] == ']') {
                    ++i;
                    return v;
                }
                fail("expected ',' or ']'");
            }
        }
        if (c == '"') {
            v->kind = JsonValue::String;
            v->str = string_();
            return v;
        }
        if (t.compare(i, 4, "true") == 0) {
            v->kind = JsonValue::Bool;
            v->b = true;
            i += 4;
            return v;
        }
        if (t.compare(i, 5, "false") == 0) {
            v->kind = JsonValue::Bool;
            i += 5;
            return v;
        }
        if (t.compare(i, 4, "null") == 0) {
            i += 4;
            return v;
        }
        char* end = nullptr;
        const double d = std::strtod(t.c_str() + i, &end);
        if (end == t.c_str() + i) fail("unexpected character");
        v->kind = JsonValue::Number;
        v->num = d;
        i = static_cast<size_t>(end - t.c_str());
        return v;
    }
};

std::shared_ptr<JsonValue> g_model, g_common;

std::string slurp(const std::string& filename) {
    std::ifstream file(filename);
    if (!file.is_open()) throw std::runtime_error("Error: file not found: " + filename);
    std::stringstream ss;
    ss << file.rdbuf();
    return ss.str();
}

const JsonValue* field(const std::string& kernel_name, const std::string& key) {
    if (!g_model) return nullptr;
    const JsonValue* k = g_model->get(kernel_name);
    return k ? k->get(key) : nullptr;
}

}  // namespace

const JsonValue* JsonValue::get(const std::string& key) const {
    if (kind != Object) return nullptr;
    for (auto& m : members)
        if (m.first == key) return m.second.get();
    return nullptr;
}

std::shared_ptr<JsonValue> parse_json(const std::string& text) {
    Parser p(text);
    auto v = p.value();
    p.ws();
    if (p.i != text.size()) p.fail("trailing characters");
    return v;
}

std::string dump_json(const JsonValue& v, int indent) {
    std::ostringstream o;
    const std::string pad(indent + 4, ' '), pad0(indent, ' ');
    switch (v.kind) {
        case JsonValue::Null: o << "null"; break;
        case JsonValue::Bool: o << (v.b ? "true" : "false"); break;
        case JsonValue::Number:
            if (v.num == static_cast<long long>(v.num)) o << static_cast<long long>(v.num);
            else o << v.num;
            break;
        case JsonValue::String: o << '"' << v.str << '"'; break;
        case JsonValue::Array:
            o << "[";
            for (size_t i = 0; i < v.items.size(); ++i) o << (i ? ", " : "") << dump_json(*v.items[i], indent + 4);
            o << "]";
            break;
        case JsonValue::Object:
            o << "{\n";
            for (size_t i = 0; i < v.members.size(); ++i)
                o << pad << '"' << v.members[i].first << "\": " << dump_json(*v.members[i].second, indent + 4)
                  << (i + 1 < v.members.size() ? ",\n" : "\n");
            o << pad0 << "}";
            break;
    }
    return o.str();
}

void read_json(const std::string& filename) {
    g_model = parse_json(slurp(filename));
    logger.INFO("Read json file: " + filename);
}

void read_common_json(const std::string& filename) {
    g_common = parse_json(slurp(filename));
    logger.INFO("Read json file: " + filename);
}

int get_kernel_info(const std::string& kernel_name, const std::string& key) {
    const JsonValue* v = field(kernel_name, key);
    if (!v) return JSON_NOT_FOUND;
    if (v->kind == JsonValue::Number) return static_cast<int>(v->num);
    if (v->kind == JsonValue::String) return std::atoi(v->str.c_str());
    return JSON_NOT_FOUND;
}

float fget_kernel_info(const std::string& kernel_name, const std::string& key) {
    const JsonValue* v = field(kernel_name, key);
    if (!v) return static_cast<float>(JSON_NOT_FOUND);
    if (v->kind == JsonValue::Number) return static_cast<float>(v->num);
    if (v->kind == JsonValue::String) return static_cast<float>(std::atof(v->str.c_str()));
    return static_cast<float>(JSON_NOT_FOUND);
}

std::string sget_kernel_info(const std::string& kernel_name, const std::string& key) {
    const JsonValue* v = field(kernel_name, key);
    if (!v) return "";
    if (v->kind == JsonValue::String) return v->str;
    if (v->kind == JsonValue::Number) return dump_json(*v);
    return "";
}

void add_kernel_info(const std::string& kernel_name, const std::string& key, double value) {
    if (!g_model) {
        g_model = std::make_shared<JsonValue>();
        g_model->kind = JsonValue::Object;
    }
    JsonValue* k = const_cast<JsonValue*>(g_model->get(kernel_name));
    if (!k) {
        auto obj = std::make_shared<JsonValue>();
        obj->kind = JsonValue::Object;
        g_model->members.emplace_back(kernel_name, obj);
        k = obj.get();
    }
    JsonValue* f = const_cast<JsonValue*>(k->get(key));
    if (!f) {
        auto n = std::make_shared<JsonValue>();
        k->members.emplace_back(key, n);
        f = n.get();
    }
    f->kind = JsonValue::Number;
    f->num = value;
}

void build_json(const std::string& filename) {
    std::ofstream file(filename);
    if (!file.is_open()) throw std::runtime_error("Error: cannot write " + filename);
    if (g_model) file << dump_json(*g_model) << "\n";
}

long long geti(int count, const char* keys...) {
    va_list args;
    va_start(args, keys);
    const JsonValue* cur = g_common.get();
    std::string chain;
    for (int i = 0; i < count; ++i) {
        const char* key = (i == 0) ? keys : va_arg(args, const char*);
        chain += std::string(key) + " -> ";
        cur = cur ? cur->get(key) : nullptr;
        if (!cur) {
            va_end(args);
            throw std::runtime_error("key chain: " + chain + "END, not found!");
        }
    }
    va_end(args);
    if (cur->kind != JsonValue::Number) throw std::runtime_error("key chain: " + chain + "END is not a number");
    return static_cast<long long>(cur->num);
}
