// Process configuration: one strict JSON file, in the reference's manner (src/core/config/Config.hpp:362-415,
// config.example.json): a `models` list with `id` and `path` and a `defaultModel`, a `runtime` section
// (`maxContextTokens`), a `serving` section (`tokenBudget` 1..8192 default 512, `maxActiveRequests` 1..256 default 32,
// `blockSize` default 16) and a `diagnostics` section; an unknown key is an error, not a warning.  Keys the reference
// has for servers, other backends, speculative decoding or host governors do not exist here.  Beside the reference's:
// `runtime.dtype`, `runtime.cacheTokens` (size of the page pool in tokens; 0 sizes it from the free device memory,
// `runtime.cacheMemoryFraction` of it), `serving.prefillChunk`, and `models[].random` (a config.json object and a seed
// instead of a path).
//
// The answer is the whole configuration as JSON text, every key present with its value or default.
#include <cstdio>
#include <set>
#include <string>
#include <vector>

#include "json.h"

#define MMH_EXPORT extern "C" __attribute__((visibility("default")))

void mmh_set_error(const std::string& message);      // runtime.cpp

namespace {

using mmjson::Value;

struct Refused {
    std::string message;
};

enum Kind { INT, STR, BOOL, FLOAT, OBJECT };

struct Key {
    const char* name;
    Kind kind;
    const char* fallback;       // JSON text of the default
};

const Key MODEL_KEYS[] = {{"id", STR, "\"\""}, {"path", STR, "\"\""}, {"title", STR, "\"\""}, {"random", OBJECT, "null"}};
const Key RUNTIME_KEYS[] = {{"dtype", STR, "\"bfloat16\""}, {"maxContextTokens", INT, "8192"}, {"cacheTokens", INT, "0"}, {"cacheMemoryFraction", FLOAT, "0.9"}};
const Key SERVING_KEYS[] = {{"tokenBudget", INT, "512"}, {"maxActiveRequests", INT, "32"}, {"blockSize", INT, "16"}, {"prefillChunk", INT, "0"}};
// parityDump: prefix of the per-stage dump files of a prefill; traceDecodeFile: one JSON line per decode step (both are
// the reference's diagnostics keys); profile: the command line prints where a prefill and a decode step spend their time
const Key DIAGNOSTICS_KEYS[] = {{"parityDump", STR, "\"\""}, {"traceDecodeFile", STR, "\"\""}, {"profile", BOOL, "false"}};

template <size_t N>
std::string known_names(const Key (&keys)[N]) {
    std::string out;
    for (size_t i = 0; i < N; ++i) out += std::string(i ? ", " : "") + keys[i].name;
    return out;
}

// JSON text of a value as it was read (objects and lists member by member)
std::string text_of(const Value& v) {
    switch (v.kind) {
        case Value::Null: return "null";
        case Value::Bool: return v.b ? "true" : "false";
        case Value::Int: return std::to_string(v.i);
        case Value::Number: {
            char buf[40];
            snprintf(buf, sizeof(buf), "%.17g", v.d);
            return buf;
        }
        case Value::String: return mmjson::quote(v.s);
        case Value::Array: {
            std::string out = "[";
            for (size_t i = 0; i < v.items.size(); ++i) out += (i ? ", " : "") + text_of(v.items[i]);
            return out + "]";
        }
        default: {
            std::string out = "{";
            for (size_t i = 0; i < v.members.size(); ++i) out += (i ? ", " : "") + mmjson::quote(v.members[i].first) + ": " + text_of(v.members[i].second);
            return out + "}";
        }
    }
}

struct Section {
    std::vector<std::pair<std::string, std::string>> fields;      // key -> JSON text, in the order of the table
    const std::string& at(const std::string& key) const {
        for (auto& f : fields)
            if (f.first == key) return f.second;
        static const std::string none;
        return none;
    }
    std::string json() const {
        std::string out = "{";
        for (size_t i = 0; i < fields.size(); ++i) out += (i ? ", " : "") + mmjson::quote(fields[i].first) + ": " + fields[i].second;
        return out + "}";
    }
};

template <size_t N>
Section fill(const std::string& section, const Key (&keys)[N], const Value* obj) {
    Section s;
    for (size_t i = 0; i < N; ++i) s.fields.emplace_back(keys[i].name, keys[i].fallback);
    if (obj == nullptr) return s;
    if (obj->kind != Value::Object) throw Refused{"'" + section + "' must be an object"};
    for (auto& m : obj->members) {
        const Key* key = nullptr;
        for (size_t i = 0; i < N; ++i)
            if (m.first == keys[i].name) key = &keys[i];
        if (key == nullptr) throw Refused{"unknown key '" + section + "." + m.first + "' (known: " + known_names(keys) + ")"};
        const Value& v = m.second;
        const std::string name = "'" + section + "." + m.first + "'";
        switch (key->kind) {
            case OBJECT:
                if (v.kind != Value::Null && v.kind != Value::Object) throw Refused{name + " must be an object"};
                break;
            case BOOL:
                if (v.kind != Value::Bool) throw Refused{name + " must be true or false"};
                break;
            case INT:
                if (!v.is_int()) throw Refused{name + " must be an integer"};
                break;
            case STR:
                if (v.kind != Value::String) throw Refused{name + " must be a string"};
                break;
            case FLOAT:
                if (v.kind != Value::Int && v.kind != Value::Number) throw Refused{name + " must be a number"};
                break;
        }
        for (auto& f : s.fields)
            if (f.first == m.first) f.second = text_of(v);
    }
    return s;
}

long long as_int(const std::string& text) { return std::strtoll(text.c_str(), nullptr, 10); }
double as_float(const std::string& text) { return std::strtod(text.c_str(), nullptr); }

std::string parse_engine(const Value& obj) {
    if (obj.kind != Value::Object) throw Refused{"configuration must be a JSON object"};
    std::string default_model = "\"\"";
    std::vector<Section> models;
    const Value *runtime_obj = nullptr, *serving_obj = nullptr, *diagnostics_obj = nullptr;
    for (auto& m : obj.members) {
        if (m.first == "defaultModel") {
            if (m.second.kind != Value::String) throw Refused{"'defaultModel' must be a string"};
            default_model = mmjson::quote(m.second.s);
        } else if (m.first == "models") {
            if (m.second.kind != Value::Array) throw Refused{"'models' must be a list"};
            models.clear();
            for (size_t i = 0; i < m.second.items.size(); ++i) models.push_back(fill("models[" + std::to_string(i) + "]", MODEL_KEYS, &m.second.items[i]));
        } else if (m.first == "runtime") {
            runtime_obj = &m.second;
        } else if (m.first == "serving") {
            serving_obj = &m.second;
        } else if (m.first == "diagnostics") {
            diagnostics_obj = &m.second;
        } else {
            throw Refused{"unknown key '" + m.first + "' (known: defaultModel, models, runtime, serving, diagnostics)"};
        }
    }
    const Section runtime = fill("runtime", RUNTIME_KEYS, runtime_obj);
    const Section serving = fill("serving", SERVING_KEYS, serving_obj);
    const Section diagnostics = fill("diagnostics", DIAGNOSTICS_KEYS, diagnostics_obj);

    // ranges of the reference (src/core/config/Config.hpp:285-351)
    const long long budget = as_int(serving.at("tokenBudget")), active = as_int(serving.at("maxActiveRequests")), block = as_int(serving.at("blockSize"));
    if (budget < 1 || budget > 8192) throw Refused{"serving.tokenBudget must be in 1..8192"};
    if (active < 1 || active > 256) throw Refused{"serving.maxActiveRequests must be in 1..256"};
    if (block != 8 && block != 16 && block != 32 && block != 64) throw Refused{"serving.blockSize must be 8, 16, 32 or 64"};
    if (as_int(serving.at("prefillChunk")) < 0) throw Refused{"serving.prefillChunk must be >= 0"};
    const std::string& dtype = runtime.at("dtype");
    if (dtype != "\"bfloat16\"" && dtype != "\"float32\"") throw Refused{"runtime.dtype must be bfloat16 or float32"};
    if (as_int(runtime.at("maxContextTokens")) < 1) throw Refused{"runtime.maxContextTokens must be positive"};
    if (as_int(runtime.at("cacheTokens")) < 0) throw Refused{"runtime.cacheTokens must be >= 0"};
    const double fraction = as_float(runtime.at("cacheMemoryFraction"));
    if (!(fraction > 0.0 && fraction <= 1.0)) throw Refused{"runtime.cacheMemoryFraction must be in (0, 1]"};
    std::set<std::string> ids;
    for (auto& m : models) {
        const std::string& id = m.at("id");
        if (id == "\"\"") throw Refused{"every model needs an 'id'"};
        if (!ids.insert(id).second) throw Refused{"model ids must be unique"};
    }
    for (auto& m : models) {
        const bool has_path = m.at("path") != "\"\"";
        const std::string& random = m.at("random");
        const bool has_random = random != "null" && random != "{}";
        if (has_path == has_random) throw Refused{"model '" + m.at("id").substr(1, m.at("id").size() - 2) + "' needs either 'path' or 'random'"};
    }

    std::string out = "{\"defaultModel\": " + default_model + ", \"models\": [";
    for (size_t i = 0; i < models.size(); ++i) out += (i ? ", " : "") + models[i].json();
    out += "], \"runtime\": " + runtime.json() + ", \"serving\": " + serving.json() + ", \"diagnostics\": " + diagnostics.json() + "}";
    return out;
}

thread_local std::string g_answer;

}  // namespace

// The process configuration from the text of its JSON file: every key with its value or default as JSON text (valid
// until this thread's next call), or null with the reason in mmh_last_error().  `where` (or null) goes before a syntax error.
MMH_EXPORT const char* mmh_engine_config(const char* text, long long n, const char* where) {
    try {
        Value obj;
        std::string err;
        mmjson::Parser parser(text, (size_t)n);
        if (!parser.parse(obj, err)) throw Refused{std::string(where ? where : "configuration") + ": not valid JSON (" + err + ")"};
        g_answer = parse_engine(obj);
        return g_answer.c_str();
    } catch (const Refused& e) {
        mmh_set_error(e.message);
        return nullptr;
    }
}
