// Typed model configuration from a model folder's config.json: the Qwen2.5 dense decoder's own keys.
//
// The reference fills one architecture-agnostic configuration from container metadata with "required key throws /
// optional key takes a logged default" helpers (src/model/LlmConfig.cpp:64-93) and has an HF config.json reader of the
// same style for another architecture (src/runtime/nvfp4/Qwen3_5MoeConfig.cpp:20-114).  This is that mechanism for
// this architecture's keys.  Nothing here knows a model size: every number comes from the file.
//
// The answer is the typed configuration as JSON text with every field present (defaults filled in and listed in
// "defaults_used"), which the Python face turns into its dataclass; an error is one sentence that names the file and the key.
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "json.h"

#define MMH_EXPORT extern "C" __attribute__((visibility("default")))

void mmh_set_error(const std::string& message);      // runtime.cpp

namespace {

using mmjson::Value;

struct ConfigError {
    std::string message;
};

// how a value reads in a message: strings quoted, the rest as written
std::string shown(const Value& v) {
    switch (v.kind) {
        case Value::Null: return "null";
        case Value::Bool: return v.b ? "true" : "false";
        case Value::Int: return std::to_string(v.i);
        case Value::Number: {
            char buf[40];
            snprintf(buf, sizeof(buf), "%.17g", v.d);
            return buf;
        }
        case Value::String: return "'" + v.s + "'";
        case Value::Array: return "a list";
        default: return "an object";
    }
}

std::string num(double d) {
    char buf[40];
    snprintf(buf, sizeof(buf), "%.17g", d);
    return buf;
}

// required / optional typed access to a JSON object, collecting the defaults that were used
class Reader {
  public:
    Reader(const Value& obj, std::string where) : obj_(obj), where_(std::move(where)) {
        if (obj.kind != Value::Object) throw ConfigError{where_ + ": not a JSON object"};
    }
    const Value* get(const char* key) const {
        const Value* v = obj_.find(key);
        return (v != nullptr && v->kind == Value::Null) ? nullptr : v;
    }
    bool has(const char* key) const { return obj_.find(key) != nullptr; }
    long long req_int(const char* key, long long minimum = 1) {
        const Value* v = get(key);
        if (v == nullptr || !v->is_int()) throw ConfigError{where_ + ": missing required integer '" + key + "'"};
        if (v->i < minimum) throw ConfigError{where_ + ": '" + key + "' = " + std::to_string(v->i) + " must be >= " + std::to_string(minimum)};
        return v->i;
    }
    // false: absent (the default stands and is noted)
    bool opt_int(const char* key, long long* out, long long minimum = 0) {
        const Value* v = get(key);
        if (v == nullptr) {
            defaults_used.push_back(key);
            return false;
        }
        if (!v->is_int()) throw ConfigError{where_ + ": '" + key + "' must be an integer, got " + shown(*v)};
        if (v->i < minimum) throw ConfigError{where_ + ": '" + key + "' = " + std::to_string(v->i) + " must be >= " + std::to_string(minimum)};
        *out = v->i;
        return true;
    }
    double opt_float(const char* key, double fallback) {
        const Value* v = get(key);
        if (v == nullptr) {
            defaults_used.push_back(key);
            return fallback;
        }
        if (v->kind != Value::Int && v->kind != Value::Number) throw ConfigError{where_ + ": '" + key + "' must be a number, got " + shown(*v)};
        return v->d;
    }
    bool opt_bool(const char* key, bool fallback) {
        const Value* v = get(key);
        if (v == nullptr) {
            defaults_used.push_back(key);
            return fallback;
        }
        if (v->kind != Value::Bool) throw ConfigError{where_ + ": '" + key + "' must be true or false, got " + shown(*v)};
        return v->b;
    }
    bool opt_str(const char* key, std::string* out) {
        const Value* v = get(key);
        if (v == nullptr) {
            defaults_used.push_back(key);
            return false;
        }
        if (v->kind != Value::String) throw ConfigError{where_ + ": '" + key + "' must be a string, got " + shown(*v)};
        *out = v->s;
        return true;
    }
    std::vector<std::string> defaults_used;

  private:
    const Value& obj_;
    std::string where_;
};

std::string parse_qwen2(const Value& obj, const std::string& where) {
    if (obj.kind != Value::Object) throw ConfigError{where + ": not a JSON object"};
    // Multimodal checkpoints nest the text model under "text_config" (src/runtime/nvfp4/Qwen3_5MoeConfig.cpp:27-31).
    const Value* text = obj.find("text_config");
    const bool nested = text != nullptr && text->kind == Value::Object;
    Reader r(nested ? *text : obj, nested ? where + ":text_config" : where);

    const Value* archs = obj.find("architectures");
    if (archs == nullptr || archs->kind != Value::Array || archs->items.empty() || archs->items[0].kind != Value::String)
        throw ConfigError{where + ": missing 'architectures' (a list naming the model class)"};
    const std::string architecture = archs->items[0].s;

    const long long layers = r.req_int("num_hidden_layers");
    const long long hidden = r.req_int("hidden_size");
    const long long heads = r.req_int("num_attention_heads");
    const long long inter = r.req_int("intermediate_size");
    const long long vocab = r.req_int("vocab_size");
    // defaults of the reference: KV heads = heads, head size = hidden / heads (src/model/LlmConfig.hpp:145-150),
    // eps 1e-6, theta 10000 (src/model/LlmConfig.cpp:97-106, 159-161)
    long long kv_heads = heads;
    r.opt_int("num_key_value_heads", &kv_heads, 1);
    long long head_dim = 0;
    if (!r.opt_int("head_dim", &head_dim, 1)) {
        if (hidden % heads != 0)
            throw ConfigError{where + ": hidden_size " + std::to_string(hidden) + " is not a multiple of num_attention_heads " + std::to_string(heads) +
                              " and no 'head_dim' is given"};
        head_dim = hidden / heads;
    }
    const double eps = r.opt_float("rms_norm_eps", 1e-6);
    const double theta = r.opt_float("rope_theta", 10000.0);
    long long max_pos = 32768;
    r.opt_int("max_position_embeddings", &max_pos, 1);
    const bool tied = r.opt_bool("tie_word_embeddings", false);
    std::string act = "silu";
    r.opt_str("hidden_act", &act);
    std::string dtype;
    if (!r.opt_str("torch_dtype", &dtype) || dtype.empty()) {
        dtype = "bfloat16";
        r.opt_str("dtype", &dtype);
    }

    if (heads % kv_heads != 0)      // src/compute/Attention.cpp:28-31
        throw ConfigError{where + ": num_attention_heads " + std::to_string(heads) + " must be a multiple of num_key_value_heads " + std::to_string(kv_heads)};
    if (head_dim % 2 != 0)          // src/compute/Rope.cpp:20-22
        throw ConfigError{where + ": head_dim " + std::to_string(head_dim) + " must be even for rotary position encoding"};
    if (!(eps > 0.0)) throw ConfigError{where + ": rms_norm_eps must be positive, got " + num(eps)};
    if (!(theta > 0.0)) throw ConfigError{where + ": rope_theta must be positive, got " + num(theta)};
    if (act != "silu") throw ConfigError{where + ": hidden_act '" + act + "' is not supported (this architecture uses 'silu')"};
    if (dtype != "bfloat16" && dtype != "float32" && dtype != "float16")
        throw ConfigError{where + ": torch_dtype '" + dtype + "' is not one of bfloat16, float16, float32"};

    // The reference runs plain rotary for this architecture: frequency factors are applied only when a factor tensor
    // exists (src/runtime/arch/Qwen2Backend.cpp:54-71).
    if (const Value* scaling = r.get("rope_scaling"))
        throw ConfigError{where + ": rope_scaling " + shown(*scaling) + " is not supported (only plain rotary)"};

    // Sliding window.  `layer_types` is authoritative when present (src/runtime/nvfp4/Qwen3_5MoeConfig.cpp:101-106);
    // otherwise the first `max_window_layers` layers see every key and the rest see a window.  0 = the layer sees every
    // earlier key, W > 0 = the last W keys, itself included (src/compute/Attention.cpp:46-50).
    const bool use_window = r.opt_bool("use_sliding_window", false);
    long long window = 0;
    const bool has_window = r.opt_int("sliding_window", &window, 1);
    std::vector<long long> windows((size_t)layers, 0);
    if (use_window) {
        if (!has_window) throw ConfigError{where + ": use_sliding_window is true but 'sliding_window' is missing"};
        if (const Value* types = r.get("layer_types")) {
            if (types->kind != Value::Array || (long long)types->items.size() != layers)
                throw ConfigError{where + ": 'layer_types' must list " + std::to_string(layers) + " layers"};
            for (long long i = 0; i < layers; ++i) {
                const Value& t = types->items[(size_t)i];
                if (t.kind == Value::String && t.s == "full_attention") windows[(size_t)i] = 0;
                else if (t.kind == Value::String && t.s == "sliding_attention") windows[(size_t)i] = window;
                else throw ConfigError{where + ": layer_types[" + std::to_string(i) + "] = " + shown(t) + " is not a kind this architecture has"};
            }
        } else {
            // no default: a guessed boundary would silently turn a windowed checkpoint into a full-attention one
            if (!r.has("max_window_layers"))
                throw ConfigError{where + ": use_sliding_window is true but neither 'layer_types' nor 'max_window_layers' says which layers are windowed"};
            long long first_windowed = layers;
            r.opt_int("max_window_layers", &first_windowed, 0);
            for (long long i = 0; i < layers; ++i) windows[(size_t)i] = i < first_windowed ? 0 : window;
        }
    }

    std::vector<long long> eos;
    if (const Value* e = r.get("eos_token_id")) {
        bool ok = true;
        if (e->is_int()) eos.push_back(e->i);
        else if (e->kind == Value::Array) {
            for (const Value& x : e->items) {
                if (!x.is_int()) ok = false;
                else eos.push_back(x.i);
            }
        } else ok = false;
        if (!ok) throw ConfigError{where + ": 'eos_token_id' must be an integer or a list of integers"};
    }

    // plain string appends: number formatting through a stream depends on the process's C++ locale objects, which another
    // library loaded before this one may have replaced
    auto n = [](long long v) { return std::to_string(v); };
    std::string o = "{\"architecture\": " + mmjson::quote(architecture) + ", \"vocab_size\": " + n(vocab) + ", \"hidden_size\": " + n(hidden) +
                    ", \"intermediate_size\": " + n(inter) + ", \"num_hidden_layers\": " + n(layers) + ", \"num_attention_heads\": " + n(heads) +
                    ", \"num_key_value_heads\": " + n(kv_heads) + ", \"head_dim\": " + n(head_dim) + ", \"rms_norm_eps\": " + num(eps) +
                    ", \"rope_theta\": " + num(theta) + ", \"max_position_embeddings\": " + n(max_pos) + ", \"tie_word_embeddings\": " +
                    (tied ? "true" : "false") + ", \"hidden_act\": " + mmjson::quote(act) + ", \"torch_dtype\": " + mmjson::quote(dtype) +
                    ", \"layer_windows\": [";
    for (size_t i = 0; i < windows.size(); ++i) o += (i ? ", " : "") + n(windows[i]);
    o += "], \"eos_token_ids\": [";
    for (size_t i = 0; i < eos.size(); ++i) o += (i ? ", " : "") + n(eos[i]);
    o += "], \"defaults_used\": [";
    for (size_t i = 0; i < r.defaults_used.size(); ++i) o += (i ? ", " : "") + mmjson::quote(r.defaults_used[i]);
    o += "]}";
    return o;
}

thread_local std::string g_answer;

const char* answer(const char* text, size_t n, const std::string& where) {
    try {
        Value obj;
        std::string err;
        mmjson::Parser parser(text, n);
        if (!parser.parse(obj, err)) throw ConfigError{where + ": not valid JSON (" + err + ")"};
        g_answer = parse_qwen2(obj, where);
        return g_answer.c_str();
    } catch (const ConfigError& e) {
        mmh_set_error(e.message);
        return nullptr;
    }
}

}  // namespace

// The typed configuration of a Qwen2.5 dense decoder from the text of its config.json, as JSON text with every field
// present (valid until this thread's next call), or null with the reason in mmh_last_error().  `where` names the source in messages.
MMH_EXPORT const char* mmh_config_qwen2(const char* text, long long n, const char* where) {
    return answer(text, (size_t)n, where ? where : "config.json");
}

// The same from a model folder's config.json.
MMH_EXPORT const char* mmh_config_qwen2_folder(const char* model_dir) {
    const std::string dir = model_dir ? model_dir : "";
    const std::string path = dir + "/config.json";
    FILE* f = std::fopen(path.c_str(), "rb");
    if (f == nullptr) {
        mmh_set_error(dir + ": no config.json in the model folder");
        return nullptr;
    }
    std::string text;
    char buf[4096];
    size_t got;
    while ((got = std::fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, got);
    std::fclose(f);
    return answer(text.data(), text.size(), path);
}
