// Weights by tensor name: a safetensors reader over a memory map, the list of tensors a model wants, and one
// error that lists everything that does not fit (missing, unexpected, wrongly shaped, wrongly typed).
// File format (parsed by hand, as the reference does in model/export_safetensors.py:24-48): 8 bytes little-endian
// header length n; n bytes of JSON {name: {dtype, shape, data_offsets}}; then the raw tensor bytes.  Sharded
// models carry model.safetensors.index.json whose weight_map names each tensor's shard (:51-60).
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <set>

#include "ops.hpp"

namespace tb {

struct TensorSpec {
    std::vector<int64_t> shape;
    std::string role = "matrix";         // matrix, embedding, norm (random mode: other std), table (integers)
    bool optional = false;
    int64_t numel() const {
        int64_t n = 1;
        for (auto d : shape) n *= d;
        return n;
    }
};

struct WantedTensors {
    std::vector<std::string> order;
    std::map<std::string, TensorSpec> specs;
    void add(const std::string& name, TensorSpec s) {
        auto it = specs.find(name);
        if (it == specs.end()) { order.push_back(name); specs[name] = std::move(s); return; }
        if (it->second.shape != s.shape) throw Error("tensor '" + name + "' is declared with two shapes");
        if (it->second.optional) it->second = std::move(s);          // needed by one part: needed
    }
};

// A tensor on the device, owned by the model.
struct DeviceTensor {
    DeviceBuffer buf;
    DType dt = BF16;
    std::vector<int64_t> shape;
    Mat mat() const {
        if (shape.size() == 1) return Mat(buf.p, dt, 1, shape[0]);
        return Mat(buf.p, dt, shape[0], shape.size() > 1 ? shape[1] : 1);
    }
};
typedef std::map<std::string, std::shared_ptr<DeviceTensor>> TensorMap;

class SafetensorsFile {
public:
    struct Entry { std::string dtype; std::vector<int64_t> shape; size_t begin, end; };
    std::string path;
    std::map<std::string, Entry> entries;
    std::vector<std::string> names;

    explicit SafetensorsFile(const std::string& p) : path(p) {
        fd_ = open(p.c_str(), O_RDONLY);
        if (fd_ < 0) throw Error("cannot open " + p + ": " + strerror(errno));
        struct stat st;
        fstat(fd_, &st);
        size_ = (size_t)st.st_size;
        if (size_ < 8) throw Error(fmt("%s: %zu bytes is too short for a safetensors header", p.c_str(), size_));
        map_ = (const unsigned char*)mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
        if (map_ == MAP_FAILED) { map_ = nullptr; throw Error("cannot map " + p); }
        uint64_t n = 0;
        memcpy(&n, map_, 8);
        if (8 + n > size_) throw Error(fmt("%s: header claims %llu bytes but the file has %zu", p.c_str(), (unsigned long long)n, size_));
        Json header;
        try {
            header = Json::parse(std::string((const char*)map_ + 8, (size_t)n));
        } catch (const Error& e) {
            throw Error(p + ": header is not valid JSON (" + e.what() + ")");
        }
        base_ = 8 + (size_t)n;
        for (auto& kv : header.obj) {
            if (kv.first == "__metadata__") continue;
            Entry e;
            e.dtype = kv.second.at("dtype").string("dtype");
            if (elem_size(e.dtype) == 0) throw Error(p + ": tensor '" + kv.first + "' has unsupported dtype " + e.dtype);
            int64_t numel = 1;
            for (auto& d : kv.second.at("shape").arr) { e.shape.push_back(d.integer("shape")); numel *= e.shape.back(); }
            auto& off = kv.second.at("data_offsets").arr;
            e.begin = (size_t)off.at(0).integer("data_offsets");
            e.end = (size_t)off.at(1).integer("data_offsets");
            if (e.end - e.begin != (size_t)numel * elem_size(e.dtype))
                throw Error(fmt("%s: tensor '%s' spans %zu bytes, its shape needs %zu", p.c_str(), kv.first.c_str(),
                                e.end - e.begin, (size_t)numel * elem_size(e.dtype)));
            if (base_ + e.end > size_)
                throw Error(fmt("%s: tensor '%s' ends at byte %zu, the file has %zu (truncated?)", p.c_str(), kv.first.c_str(),
                                base_ + e.end, size_));
            names.push_back(kv.first);
            entries[kv.first] = e;
        }
    }
    ~SafetensorsFile() {
        if (map_) munmap((void*)map_, size_);
        if (fd_ >= 0) close(fd_);
    }
    SafetensorsFile(const SafetensorsFile&) = delete;
    const unsigned char* data(const std::string& name) const { return map_ + base_ + entries.at(name).begin; }
    static size_t elem_size(const std::string& d) {
        if (d == "BF16" || d == "F16" || d == "I16") return 2;
        if (d == "F32" || d == "I32") return 4;
        if (d == "F64" || d == "I64") return 8;
        if (d == "I8" || d == "U8" || d == "BOOL") return 1;
        return 0;
    }
    static bool is_float(const std::string& d) { return d == "BF16" || d == "F16" || d == "F32" || d == "F64"; }

private:
    int fd_ = -1;
    size_t size_ = 0, base_ = 0;
    const unsigned char* map_ = nullptr;
};

inline bool file_exists(const std::string& p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0;
}

inline std::string read_text(const std::string& p) {
    std::ifstream f(p);
    if (!f) throw Error("cannot read " + p);
    std::stringstream ss;
    ss << f.rdbuf();
    return ss.str();
}

inline float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000) << 16;
    uint32_t exp = (h >> 10) & 0x1F, man = h & 0x3FF, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int e = -1;
            do { e++; man <<= 1; } while (!(man & 0x400));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FF) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
    else bits = sign | ((exp + 112) << 23) | (man << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

inline uint16_t float_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x7FFFFFu)) return (uint16_t)((u >> 16) | 0x40);      // NaN stays NaN
    return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

// Storage rules: bfloat16 stays bfloat16 in a bfloat16 engine; a tensor stored in 32 bits stays so; float16 has three
// bits more than bfloat16 and is widened to float32 ("widen", exact), rounded on request ("round") or reported
// ("refuse"); the float32 engine widens everything; integer tables become int32.
inline DType storage_dtype(const std::string& stored, const std::string& role, DType engine, const std::string& fp16) {
    if (role == "table") return I32;
    if (engine == F32) return F32;
    if (stored == "F32" || stored == "F64") return F32;
    if (stored == "F16" && fp16 != "round") return F32;
    return BF16;
}

struct OpenedWeights {
    std::vector<std::unique_ptr<SafetensorsFile>> files;
    std::map<std::string, SafetensorsFile*> by_name;
};

// Opens the weight files of a model folder and holds them against what the model wants; every misfit (missing,
// unexpected, wrongly shaped, wrongly typed) goes into ONE error.  Needs no GPU.
inline OpenedWeights check_tensors(const std::string& folder, const WantedTensors& wanted, DType engine, const std::string& fp16 = "widen") {
    if (fp16 != "widen" && fp16 != "round" && fp16 != "refuse") throw Error("fp16 must be widen, round or refuse, got " + fp16);
    OpenedWeights opened;
    auto& files = opened.files;
    auto& by_name = opened.by_name;
    const std::string idx = folder + "/model.safetensors.index.json", single = folder + "/model.safetensors";
    if (file_exists(idx)) {
        Json j = Json::parse(read_text(idx));
        std::map<std::string, SafetensorsFile*> shards;
        if (const Json* wm = j.find("weight_map"))
            for (auto& kv : wm->obj) {
                const std::string shard = kv.second.string("weight_map entry");
                if (!shards.count(shard)) {
                    files.emplace_back(new SafetensorsFile(folder + "/" + shard));
                    shards[shard] = files.back().get();
                }
                if (!shards[shard]->entries.count(kv.first))
                    throw Error(idx + " places '" + kv.first + "' in " + shard + ", which does not hold it");
                by_name[kv.first] = shards[shard];
            }
        for (auto& f : files)
            for (auto& n : f->names) by_name.emplace(n, f.get());
    } else if (file_exists(single)) {
        files.emplace_back(new SafetensorsFile(single));
        for (auto& n : files.back()->names) by_name[n] = files.back().get();
    } else throw Error(folder + " holds neither model.safetensors nor model.safetensors.index.json");

    std::vector<std::string> missing, unexpected, wrong_shape, wrong_kind;
    for (auto& name : wanted.order) {
        const TensorSpec& spec = wanted.specs.at(name);
        auto it = by_name.find(name);
        if (it == by_name.end()) {
            if (!spec.optional) missing.push_back(name);
            continue;
        }
        const auto& e = it->second->entries.at(name);
        if (e.shape != spec.shape) {
            auto show = [](const std::vector<int64_t>& s) {
                std::string o = "[";
                for (size_t i = 0; i < s.size(); i++) o += (i ? ", " : "") + std::to_string(s[i]);
                return o + "]";
            };
            wrong_shape.push_back(name + " is " + show(e.shape) + ", expected " + show(spec.shape));
        }
        const bool fl = SafetensorsFile::is_float(e.dtype);
        if (spec.role == "table" && fl) wrong_kind.push_back(name + " is " + e.dtype + ", expected an integer type");
        if (spec.role != "table" && !fl) wrong_kind.push_back(name + " is " + e.dtype + ", expected a floating-point type");
        if (spec.role != "table" && e.dtype == "F16" && fp16 == "refuse" && engine != F32)
            wrong_kind.push_back(name + " is float16, expected bfloat16 or float32 (float16 does not fit bfloat16 without "
                                        "rounding; load with fp16 = widen or round)");
    }
    for (auto& kv : by_name)
        if (!wanted.specs.count(kv.first)) unexpected.push_back(kv.first);
    if (!missing.empty() || !unexpected.empty() || !wrong_shape.empty() || !wrong_kind.empty()) {
        std::sort(missing.begin(), missing.end());
        std::sort(unexpected.begin(), unexpected.end());
        auto join = [](const std::vector<std::string>& v) {
            std::string o;
            for (size_t i = 0; i < v.size(); i++) o += (i ? ", " : "") + v[i];
            return o;
        };
        std::string msg = "weights in " + folder + " do not fit the model:";
        if (!missing.empty()) msg += fmt("\n  missing (%zu): ", missing.size()) + join(missing);
        if (!unexpected.empty()) msg += fmt("\n  unexpected (%zu): ", unexpected.size()) + join(unexpected);
        if (!wrong_shape.empty()) msg += fmt("\n  wrong shape (%zu): ", wrong_shape.size()) + join(wrong_shape);
        if (!wrong_kind.empty()) msg += fmt("\n  wrong dtype (%zu): ", wrong_kind.size()) + join(wrong_kind);
        throw Error(msg);
    }
    return opened;
}

// Reads the wanted tensors of a model folder onto the device.
inline TensorMap load_tensors(const std::string& folder, const WantedTensors& wanted, DType engine, const std::string& fp16 = "widen") {
    OpenedWeights opened = check_tensors(folder, wanted, engine, fp16);
    auto& by_name = opened.by_name;
    TensorMap out;
    std::vector<unsigned char> stage;
    for (auto& name : wanted.order) {
        auto it = by_name.find(name);
        if (it == by_name.end()) continue;
        const TensorSpec& spec = wanted.specs.at(name);
        const auto& e = it->second->entries.at(name);
        const unsigned char* src = it->second->data(name);
        const int64_t n = spec.numel();
        auto t = std::make_shared<DeviceTensor>();
        t->shape = spec.shape;
        t->dt = storage_dtype(e.dtype, spec.role, engine, fp16);
        t->buf.alloc((size_t)n * dtype_size(t->dt));
        const bool same = (t->dt == BF16 && e.dtype == "BF16") || (t->dt == F32 && e.dtype == "F32") || (t->dt == I32 && e.dtype == "I32");
        const void* host = src;
        if (!same) {
            stage.resize((size_t)n * dtype_size(t->dt));
            host = stage.data();
            for (int64_t i = 0; i < n; i++) {
                double v;
                if (e.dtype == "BF16") { uint32_t u = (uint32_t)((const uint16_t*)src)[i] << 16; float f; memcpy(&f, &u, 4); v = f; }
                else if (e.dtype == "F16") v = half_to_float(((const uint16_t*)src)[i]);
                else if (e.dtype == "F32") v = ((const float*)src)[i];
                else if (e.dtype == "F64") v = ((const double*)src)[i];
                else if (e.dtype == "I64") v = (double)((const int64_t*)src)[i];
                else if (e.dtype == "I32") v = ((const int32_t*)src)[i];
                else if (e.dtype == "I16") v = ((const int16_t*)src)[i];
                else if (e.dtype == "I8") v = ((const int8_t*)src)[i];
                else v = src[i];
                if (t->dt == F32) ((float*)stage.data())[i] = (float)v;
                else if (t->dt == BF16) ((uint16_t*)stage.data())[i] = float_to_bf16((float)v);
                else ((int32_t*)stage.data())[i] = (int32_t)v;
            }
        }
        if (n) cuda_ok(cudaMemcpy(t->buf.p, host, (size_t)n * dtype_size(t->dt), cudaMemcpyHostToDevice), "copying weights");
        out[name] = t;
    }
    return out;
}

// The key of a tensor in the counter-based random-weights generator: FNV-1a-64 of the name, xor the seed.
inline void name_key(uint64_t seed, const std::string& name, unsigned& k0, unsigned& k1) {
    uint64_t h = 0xCBF29CE484222325ull;
    for (unsigned char c : name) h = (h ^ c) * 0x100000001B3ull;
    h ^= seed;
    k0 = (unsigned)(h & 0xFFFFFFFFu);
    k1 = (unsigned)(h >> 32);
}

// Random-weights mode on the device: element i of tensor `name` depends on (seed, name, i) only (csrc/random_init.cu),
// the same values a folder written for that seed holds.
inline TensorMap random_tensors(const WantedTensors& wanted, uint64_t seed, float std_, float norm_std, DType engine, Ops& ops) {
    TensorMap out;
    for (auto& name : wanted.order) {
        const TensorSpec& spec = wanted.specs.at(name);
        if (spec.optional) continue;
        auto t = std::make_shared<DeviceTensor>();
        t->shape = spec.shape;
        const int64_t n = spec.numel();
        if (spec.role == "table") {
            t->dt = I32;
            t->buf.alloc((size_t)n * 4);
            cuda_ok(cudaMemsetAsync(t->buf.p, 0, (size_t)n * 4, ops.stream), "zeroing a table");
        } else {
            t->dt = engine;
            t->buf.alloc((size_t)n * dtype_size(engine));
            unsigned k0, k1;
            name_key(seed, name, k0, k1);
            ops.random_normal(t->buf.p, engine, n, k0, k1, spec.role == "norm" ? norm_std : std_);
        }
        out[name] = t;
    }
    return out;
}

}  // namespace tb
