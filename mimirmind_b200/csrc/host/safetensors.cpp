// The safetensors container: reader for a single file or a sharded folder, and writer.
//
// Format and checks follow the reference's container code: an 8-byte little-endian header length, a JSON object
// {name: {dtype, shape, data_offsets}} with "__metadata__" skipped, offsets relative to the data region, byte length
// equal to prod(shape) * width, begin <= end, no negative dimension, no region past the file
// (src/core/safetensors/SafetensorsHeader.cpp:33-153); a folder holds either a shard index
// "model.safetensors.index.json" with a "weight_map" or a single "model.safetensors"
// (src/core/safetensors/SafetensorsModel.cpp:32-56); every mapped tensor must exist in its shard and no tensor may
// appear in two shards (:100-129).  A tensor named twice in one header is refused as well.
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "json.h"

void mmh_set_error(const std::string& msg);

namespace {

struct Record {
    std::string name, dtype;
    std::vector<long long> shape;
    long long begin = 0, end = 0;
    int shard = 0;
};

struct Shard {
    std::string path;
    int fd = -1;
    long long size = 0, data_start = 0;
    std::vector<Record> records;
};

struct Container {
    std::vector<Shard> shards;
    std::vector<Record> records;         // what the container offers, by position
    ~Container() {
        for (auto& s : shards)
            if (s.fd >= 0) ::close(s.fd);
    }
};

constexpr long long MAX_HEADER = 100LL * 1024 * 1024;

int dtype_width(const std::string& tag) {
    static const std::map<std::string, int> w = {{"F64", 8}, {"F32", 4}, {"F16", 2}, {"BF16", 2}, {"I64", 8},
                                                 {"I32", 4}, {"I16", 2}, {"I8", 1},  {"U8", 1},   {"BOOL", 1}};
    auto it = w.find(tag);
    return it == w.end() ? 0 : it->second;
}

std::string list_text(const mmjson::Value& v) {
    if (v.kind != mmjson::Value::Array) return "(not a list)";
    std::string s = "[";
    for (size_t i = 0; i < v.items.size(); ++i) {
        if (i) s += ", ";
        const auto& x = v.items[i];
        s += x.kind == mmjson::Value::Int ? std::to_string(x.i) : (x.kind == mmjson::Value::Number ? std::to_string(x.d) : "?");
    }
    return s + "]";
}

bool fail(const std::string& msg) {
    mmh_set_error(msg);
    return false;
}

// Parses the first bytes of a file into `shard` (records, data_start).  `blob` holds at least the length prefix.
bool parse_header(const unsigned char* blob, long long blob_len, long long file_size, const std::string& where, Shard& shard) {
    if (blob_len < 8) return fail(where + ": file shorter than the 8-byte length prefix");
    unsigned long long hlen = 0;
    for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | blob[i];
    if (hlen == 0 || hlen > (unsigned long long)MAX_HEADER) return fail(where + ": header length " + std::to_string(hlen) + " is not plausible");
    if (8 + (long long)hlen > file_size) return fail(where + ": header (" + std::to_string(hlen) + " bytes) runs past the end of the file");
    if (blob_len < 8 + (long long)hlen) return fail(where + ": header truncated");
    mmjson::Value root;
    std::string err;
    if (!mmjson::Parser(reinterpret_cast<const char*>(blob) + 8, (size_t)hlen).parse(root, err))
        return fail(where + ": header is not valid JSON (" + err + ")");
    if (root.kind != mmjson::Value::Object) return fail(where + ": header is not a JSON object");
    shard.data_start = 8 + (long long)hlen;
    const long long data_size = file_size - shard.data_start;
    std::map<std::string, int> seen;
    for (auto& m : root.members) {
        const std::string& name = m.first;
        if (name == "__metadata__") continue;
        if (seen.count(name)) return fail(where + ": tensor '" + name + "' appears twice in the header");
        seen[name] = 1;
        const mmjson::Value& e = m.second;
        const mmjson::Value *dt = e.find("dtype"), *sh = e.find("shape"), *of = e.find("data_offsets");
        if (e.kind != mmjson::Value::Object || !dt || !sh || !of) return fail(where + ": tensor '" + name + "' lacks dtype, shape or data_offsets");
        Record r;
        r.name = name;
        if (dt->kind != mmjson::Value::String || dtype_width(dt->s) == 0)
            return fail(where + ": tensor '" + name + "' has unknown dtype '" + (dt->kind == mmjson::Value::String ? dt->s : "?") + "'");
        r.dtype = dt->s;
        bool ok = sh->kind == mmjson::Value::Array;
        if (ok)
            for (auto& d : sh->items) ok = ok && d.is_int() && d.i >= 0;
        if (!ok) return fail(where + ": tensor '" + name + "' has an invalid shape " + list_text(*sh));
        for (auto& d : sh->items) r.shape.push_back(d.i);
        ok = of->kind == mmjson::Value::Array && of->items.size() == 2;
        if (ok)
            for (auto& o : of->items) ok = ok && o.is_int() && o.i >= 0;
        if (!ok) return fail(where + ": tensor '" + name + "' has invalid data_offsets " + list_text(*of));
        r.begin = of->items[0].i;
        r.end = of->items[1].i;
        if (r.begin > r.end) return fail(where + ": tensor '" + name + "' has begin " + std::to_string(r.begin) + " > end " + std::to_string(r.end));
        if (r.end > data_size)
            return fail(where + ": tensor '" + name + "' ends at " + std::to_string(r.end) + ", past the data region (" + std::to_string(data_size) + " bytes)");
        long long count = 1;
        for (long long d : r.shape) count *= d;
        const long long want = count * dtype_width(r.dtype);
        if (r.end - r.begin != want)
            return fail(where + ": tensor '" + name + "' holds " + std::to_string(r.end - r.begin) + " bytes but shape " + list_text(*sh) + " of " + r.dtype +
                        " needs " + std::to_string(want));
        shard.records.push_back(std::move(r));
    }
    return true;
}

bool open_shard(const std::string& path, Shard& s) {
    s.path = path;
    s.fd = ::open(path.c_str(), O_RDONLY);
    if (s.fd < 0) return fail(path + ": shard named by the index does not exist");
    struct stat st;
    if (fstat(s.fd, &st) != 0) return fail(path + ": cannot stat");
    s.size = (long long)st.st_size;
    unsigned char head[8];
    if (pread(s.fd, head, 8, 0) != 8) return fail(path + ": file shorter than the 8-byte length prefix");
    unsigned long long hlen = 0;
    for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | head[i];
    if (hlen == 0 || hlen > (unsigned long long)MAX_HEADER || 8 + (long long)hlen > s.size)
        return fail(path + ": header length " + std::to_string(hlen) + " runs past the end of the file or is not plausible");
    std::vector<unsigned char> blob(8 + hlen);
    if (pread(s.fd, blob.data(), blob.size(), 0) != (ssize_t)blob.size()) return fail(path + ": header truncated");
    return parse_header(blob.data(), (long long)blob.size(), s.size, path, s);
}

bool file_exists(const std::string& p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

bool read_all(const std::string& path, std::string& out) {
    const int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) return false;
    char buf[65536];
    ssize_t n;
    while ((n = ::read(fd, buf, sizeof(buf))) > 0) out.append(buf, (size_t)n);
    ::close(fd);
    return n == 0;
}

bool open_folder(const std::string& dir, Container& c) {
    const std::string index = dir + "/model.safetensors.index.json", single = dir + "/model.safetensors";
    if (file_exists(index)) {
        std::string text;
        if (!read_all(index, text)) return fail(index + ": cannot read");
        mmjson::Value root;
        std::string err;
        if (!mmjson::Parser(text.data(), text.size()).parse(root, err)) return fail(index + ": not valid JSON (" + err + ")");
        const mmjson::Value* wm = root.kind == mmjson::Value::Object ? root.find("weight_map") : nullptr;
        if (!wm || wm->kind != mmjson::Value::Object || wm->members.empty()) return fail(index + ": no 'weight_map' object");
        std::map<std::string, int> shard_of_file;
        for (auto& m : wm->members) {
            if (m.second.kind != mmjson::Value::String) return fail(index + ": weight_map['" + m.first + "'] is not a file name");
            const std::string path = dir + "/" + m.second.s;
            auto it = shard_of_file.find(path);
            if (it == shard_of_file.end()) {
                if (!file_exists(path)) return fail(path + ": shard named by the index does not exist");
                c.shards.emplace_back();
                if (!open_shard(path, c.shards.back())) return false;
                it = shard_of_file.emplace(path, (int)c.shards.size() - 1).first;
            }
            const Shard& sh = c.shards[it->second];
            const Record* found = nullptr;
            for (auto& r : sh.records)
                if (r.name == m.first) found = &r;
            if (!found) return fail(index + ": tensor '" + m.first + "' is mapped to " + m.second.s + " but is not in it");
            Record r = *found;
            r.shard = it->second;
            c.records.push_back(std::move(r));
        }
        // a tensor present in two shards is ambiguous even if the index picks one
        std::map<std::string, int> seen;
        for (size_t si = 0; si < c.shards.size(); ++si)
            for (auto& r : c.shards[si].records) {
                auto it = seen.find(r.name);
                if (it != seen.end()) return fail("tensor '" + r.name + "' appears in two shards: " + c.shards[it->second].path + " and " + c.shards[si].path);
                seen[r.name] = (int)si;
            }
        return true;
    }
    if (file_exists(single)) {
        c.shards.emplace_back();
        if (!open_shard(single, c.shards.back())) return false;
        c.records = c.shards.back().records;
        return true;
    }
    return fail(dir + ": neither model.safetensors.index.json nor model.safetensors found");
}

}  // namespace

#define MMH extern "C" __attribute__((visibility("default")))

// A header alone (the first bytes of a file, as a caller read them): null with a message when it is malformed.
MMH void* mmh_st_parse_header(const void* blob, long long blob_len, long long file_size, const char* where) {
    auto* c = new Container();
    c->shards.emplace_back();
    c->shards.back().path = where;
    if (!parse_header(static_cast<const unsigned char*>(blob), blob_len, file_size, where, c->shards.back())) {
        delete c;
        return nullptr;
    }
    c->records = c->shards.back().records;
    return c;
}
// A model folder: a shard index or a single file.
MMH void* mmh_st_open_folder(const char* dir) {
    auto* c = new Container();
    if (!open_folder(dir, *c)) {
        delete c;
        return nullptr;
    }
    return c;
}
MMH void mmh_st_close(void* h) { delete static_cast<Container*>(h); }
MMH int mmh_st_count(void* h) { return (int)static_cast<Container*>(h)->records.size(); }
MMH const char* mmh_st_name(void* h, int i) { return static_cast<Container*>(h)->records[i].name.c_str(); }
MMH const char* mmh_st_dtype(void* h, int i) { return static_cast<Container*>(h)->records[i].dtype.c_str(); }
MMH const char* mmh_st_shard(void* h, int i) {
    Container* c = static_cast<Container*>(h);
    return c->shards[c->records[i].shard].path.c_str();
}
// copies up to cap dimensions; returns their number
MMH int mmh_st_shape(void* h, int i, long long* out, int cap) {
    const auto& s = static_cast<Container*>(h)->records[i].shape;
    for (int k = 0; k < (int)s.size() && k < cap; ++k) out[k] = s[k];
    return (int)s.size();
}
// which: 0 begin, 1 end (byte offsets inside the data region), 2 start of the data region in the tensor's file
MMH long long mmh_st_offset(void* h, int i, int which) {
    Container* c = static_cast<Container*>(h);
    const Record& r = c->records[i];
    return which == 0 ? r.begin : (which == 1 ? r.end : c->shards[r.shard].data_start);
}
// copies the tensor's bytes to dst (nbytes must be its size)
MMH int mmh_st_read(void* h, int i, void* dst, long long nbytes) {
    Container* c = static_cast<Container*>(h);
    const Record& r = c->records[i];
    const Shard& s = c->shards[r.shard];
    if (s.fd < 0 || nbytes != r.end - r.begin) {
        mmh_set_error("tensor '" + r.name + "': wrong size or no file behind it");
        return -2;
    }
    long long done = 0;
    while (done < nbytes) {
        const ssize_t n = pread(s.fd, static_cast<char*>(dst) + done, (size_t)(nbytes - done), s.data_start + r.begin + done);
        if (n <= 0) {
            mmh_set_error(s.path + ": read failed for tensor '" + r.name + "'");
            return -2;
        }
        done += n;
    }
    return 0;
}

// What a model needs against what the container offers: n tensors by name with their shapes (flat, one after the other)
// and whether each may be absent.  0 when they match; else 1 with ONE message in mmh_last_error() that lists every missing
// tensor, every unexpected one and every wrong shape (the reference finds a missing block tensor only at first use,
// src/runtime/arch/Qwen2Backend.cpp:174-181; here the whole checkpoint is checked when it is opened).
MMH int mmh_st_check(void* h, const char* where, int n, const char** names, const int* ndims, const long long* shapes, const int* optional) {
    Container* c = static_cast<Container*>(h);
    auto listed = [](const std::vector<long long>& shape) {
        std::string out = "[";
        for (size_t i = 0; i < shape.size(); ++i) out += (i ? ", " : "") + std::to_string(shape[i]);
        return out + "]";
    };
    std::map<std::string, std::vector<long long>> want, have;
    std::map<std::string, bool> may_miss;
    size_t at = 0;
    for (int i = 0; i < n; ++i) {
        want[names[i]] = std::vector<long long>(shapes + at, shapes + at + ndims[i]);
        may_miss[names[i]] = optional != nullptr && optional[i] != 0;
        at += (size_t)ndims[i];
    }
    for (const Record& r : c->records) have[r.name] = r.shape;
    std::vector<std::string> missing, unexpected, wrong;          // std::map walks its names in sorted order
    for (auto& w : want) {
        auto it = have.find(w.first);
        if (it == have.end()) {
            if (!may_miss[w.first]) missing.push_back("    " + w.first + "  " + listed(w.second));
        } else if (it->second != w.second) {
            wrong.push_back("    " + w.first + ": file has " + listed(it->second) + ", config needs " + listed(w.second));
        }
    }
    for (auto& hv : have)
        if (want.find(hv.first) == want.end()) unexpected.push_back("    " + hv.first + "  " + listed(hv.second));
    if (missing.empty() && unexpected.empty() && wrong.empty()) return 0;
    std::string msg = std::string(where ? where : "model") + ": the checkpoint does not match the model described by config.json";
    auto section = [&](const char* title, const std::vector<std::string>& lines) {
        if (lines.empty()) return;
        msg += "\n  " + std::string(title) + " (" + std::to_string(lines.size()) + "):";
        for (auto& l : lines) msg += "\n" + l;
    };
    section("missing tensors", missing);
    section("unexpected tensors", unexpected);
    section("wrong shapes", wrong);
    mmh_set_error(msg);
    return 1;
}

// Writes one file: names in the order given (the caller sorts), shapes flat one after the other, metadata as
// alternating keys and values (may be null).  Written to a temporary name and renamed.
MMH int mmh_st_write(const char* path, int n, const char* const* names, const char* const* dtypes, const int* ndims, const long long* shapes,
                     const void* const* data, const long long* nbytes, int n_meta, const char* const* meta) {
    std::string header = "{";
    bool first = true;
    if (n_meta > 0) {
        header += "\"__metadata__\":{";
        for (int i = 0; i < n_meta; ++i) header += (i ? "," : "") + mmjson::quote(meta[2 * i]) + ":" + mmjson::quote(meta[2 * i + 1]);
        header += "}";
        first = false;
    }
    long long offset = 0;
    const long long* sp = shapes;
    for (int i = 0; i < n; ++i) {
        const int w = dtype_width(dtypes[i]);
        long long count = 1;
        std::string shape = "[";
        for (int k = 0; k < ndims[i]; ++k) {
            count *= sp[k];
            shape += (k ? "," : "") + std::to_string(sp[k]);
        }
        shape += "]";
        sp += ndims[i];
        if (w == 0 || count * w != nbytes[i]) {
            mmh_set_error(std::string("cannot store tensor '") + names[i] + "': unknown dtype or size mismatch");
            return -2;
        }
        header += std::string(first ? "" : ",") + mmjson::quote(names[i]) + ":{\"dtype\":\"" + dtypes[i] + "\",\"shape\":" + shape + ",\"data_offsets\":[" +
                  std::to_string(offset) + "," + std::to_string(offset + nbytes[i]) + "]}";
        first = false;
        offset += nbytes[i];
    }
    header += "}";
    while (header.size() % 8) header.push_back(' ');
    const std::string tmp = std::string(path) + ".tmp";
    const int fd = ::open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
    if (fd < 0) {
        mmh_set_error(tmp + ": cannot create");
        return -2;
    }
    auto put = [&](const void* p, long long len) {
        long long done = 0;
        while (done < len) {
            const ssize_t k = ::write(fd, static_cast<const char*>(p) + done, (size_t)(len - done));
            if (k <= 0) return false;
            done += k;
        }
        return true;
    };
    unsigned char prefix[8];
    unsigned long long hl = header.size();
    for (int i = 0; i < 8; ++i) prefix[i] = (unsigned char)(hl >> (8 * i));
    bool ok = put(prefix, 8) && put(header.data(), (long long)header.size());
    for (int i = 0; i < n && ok; ++i) ok = put(data[i], nbytes[i]);
    ::close(fd);
    if (!ok || ::rename(tmp.c_str(), path) != 0) {
        mmh_set_error(std::string(path) + ": write failed");
        return -2;
    }
    return 0;
}
