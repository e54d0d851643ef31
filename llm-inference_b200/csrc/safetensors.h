// Reader of .safetensors checkpoints: 8-byte little-endian header length, a JSON header (name -> dtype, shape,
// data_offsets relative to the end of the header), then the raw tensor bytes. The file is read into host memory once.
#pragma once
#include <cstdint>
#include <cstdio>
#include <map>
#include <string>
#include <vector>

#include "json_min.h"

namespace b200 {

struct SafeTensor {
    std::string dtype;               // "BF16", "F32", "I32", ...
    std::vector<long long> shape;
    const unsigned char* data = nullptr;
    size_t bytes = 0;
    size_t elems() const { size_t n = 1; for (long long d : shape) n *= (size_t)d; return n; }
};

class SafeTensorsFile {
public:
    bool open(const std::string& path, std::string& err) {
        FILE* f = fopen(path.c_str(), "rb");
        if (!f) { err = "cannot open " + path; return false; }
        fseek(f, 0, SEEK_END);
        const long long size = ftell(f);
        fseek(f, 0, SEEK_SET);
        if (size < 8) { fclose(f); err = path + ": too short"; return false; }
        buf_.resize((size_t)size);
        const size_t got = fread(buf_.data(), 1, (size_t)size, f);
        fclose(f);
        if (got != (size_t)size) { err = path + ": short read"; return false; }
        uint64_t hl = 0;
        for (int i = 7; i >= 0; --i) hl = (hl << 8) | buf_[i];
        if (hl > (uint64_t)size - 8) { err = path + ": header length beyond the file"; return false; }
        Json h;
        if (!JsonParser::parse((const char*)buf_.data() + 8, (size_t)hl, h, err)) return false;
        if (h.kind != Json::Obj) { err = path + ": header is not an object"; return false; }
        const size_t base = 8 + (size_t)hl;
        for (auto& kv : h.obj) {
            if (kv.first == "__metadata__") continue;
            SafeTensor t;
            t.dtype = kv.second.text("dtype");
            const Json* sh = kv.second.get("shape");
            const Json* off = kv.second.get("data_offsets");
            if (!sh || sh->kind != Json::Arr || !off || off->kind != Json::Arr || off->arr.size() != 2) {
                err = path + ": bad entry " + kv.first;
                return false;
            }
            for (auto& d : sh->arr) t.shape.push_back((long long)d.num);
            const size_t lo = (size_t)off->arr[0].num, hi = (size_t)off->arr[1].num;
            if (hi < lo || base + hi > buf_.size()) { err = path + ": offsets of " + kv.first + " beyond the file"; return false; }
            t.data = buf_.data() + base + lo;
            t.bytes = hi - lo;
            const size_t esz = t.dtype == "BF16" || t.dtype == "F16" ? 2 : t.dtype == "F32" || t.dtype == "I32" ? 4 : 0;
            if (esz == 0 || t.elems() * esz != t.bytes) { err = path + ": " + kv.first + " has dtype " + t.dtype + " or a size that does not fit its shape"; return false; }
            tensors_[kv.first] = t;
        }
        return true;
    }
    const SafeTensor* find(const std::string& name) const {
        auto it = tensors_.find(name);
        return it == tensors_.end() ? nullptr : &it->second;
    }
    const std::map<std::string, SafeTensor>& all() const { return tensors_; }

private:
    std::vector<unsigned char> buf_;
    std::map<std::string, SafeTensor> tensors_;
};

// element i of a checkpoint tensor as float (BF16 / F32 / F16 sources)
inline float st_value(const SafeTensor& t, size_t i) {
    if (t.dtype == "F32") { float v; memcpy(&v, t.data + 4 * i, 4); return v; }
    if (t.dtype == "BF16") {
        uint32_t u = ((uint32_t)t.data[2 * i + 1] << 24) | ((uint32_t)t.data[2 * i] << 16);
        float v; memcpy(&v, &u, 4); return v;
    }
    return 0.f;
}

}  // namespace b200
