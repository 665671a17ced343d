// json.h -- per-model kernel metadata (reference: src/json.h, src/json.cc:9-137; same function names
// and the same files/keys under config/).  The reference reads the files with Boost.PropertyTree; this
// is a small self-contained parser of the JSON subset those files use (objects, strings, numbers,
// booleans, arrays).
#pragma once
#include <map>
#include <memory>
#include <string>
#include <vector>

const int JSON_NOT_FOUND = -32767;  // -INT16_MAX, as in the reference

struct JsonValue {
    enum Kind { Null, Bool, Number, String, Object, Array } kind = Null;
    bool b = false;
    double num = 0.0;
    std::string str;
    std::vector<std::pair<std::string, std::shared_ptr<JsonValue>>> members;  // insertion order kept
    std::vector<std::shared_ptr<JsonValue>> items;
    const JsonValue* get(const std::string& key) const;
};

// throws std::runtime_error with the byte offset of the first syntax error
std::shared_ptr<JsonValue> parse_json(const std::string& text);
std::string dump_json(const JsonValue& v, int indent = 0);

void read_json(const std::string& filename);         // per-model file, e.g. config/kinfo-vgg16.json
void read_common_json(const std::string& filename);  // config/kinfo-common.json
int get_kernel_info(const std::string& kernel_name, const std::string& key);
float fget_kernel_info(const std::string& kernel_name, const std::string& key);
std::string sget_kernel_info(const std::string& kernel_name, const std::string& key);
void add_kernel_info(const std::string& kernel_name, const std::string& key, double value);
void build_json(const std::string& filename);
// geti(2, "vgg16", "MAX_BOTTOM"): walks the common file; throws when a key of the chain is missing
long long geti(int count, const char* keys...);
