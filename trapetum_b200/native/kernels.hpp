// The kernel libraries (one shared library per .cu file of csrc/, built by csrc/build.py) loaded with dlopen,
// and their C entry points as typed function pointers.  A manifest beside the libraries maps each library's
// name to its file (the file names carry a hash of the source).  Nothing is compiled from here: a missing
// library is an error that says how to build it.
#pragma once
#include <dlfcn.h>

#include <fstream>
#include <mutex>
#include <sstream>

#include "../csrc/decode_args.h"
#include "base.hpp"

namespace tb {

struct RopeKvArgs {                      // mirrors csrc/rope_kv.cu
    void* qkv; long long row_stride;
    int q_off, k_off, v_off;
    int n_heads, n_kv_heads, head_dim, rotary_dim;
    const float* inv_freq;
    const int* positions;
    const int* token_seq;
    const int* len_after;
    void* k_pool; void* v_pool;
    const int* page_table; int pt_stride;
    int page_rows; int ring_rows;
    const float* partial; int n_splits; long long split_stride, partial_row_stride;
};

struct SampleArgs {                      // mirrors csrc/sampling.cu
    float* logits; long long row_stride; int vocab;
    const float* temperature;
    const float* top_p;
    const float* penalty;
    const float* draw;
    const int* recent; int n_recent;
    int* out;
};

struct KernelLib {
    std::string name;
    void* handle = nullptr;
    const char* (*error)() = nullptr;
    template <typename F> F sym(const char* s) const {
        void* f = dlsym(handle, s);
        if (!f) throw Error(fmt("kernel library '%s' has no symbol %s", name.c_str(), s));
        return reinterpret_cast<F>(f);
    }
};

class Kernels {
public:
    static Kernels& get() {
        static Kernels k;
        return k;
    }
    // Where the libraries and their manifest.json lie.  Default: $TRAPETUM_KERNEL_DIR, else ../csrc/_build
    // relative to this library's own file.
    void set_dir(const std::string& d) {
        std::lock_guard<std::mutex> g(mu_);
        dir_ = d;
        manifest_ = Json();
    }
    const KernelLib& lib(const std::string& name) {
        std::lock_guard<std::mutex> g(mu_);
        auto it = libs_.find(name);
        if (it != libs_.end()) return it->second;
        load_manifest();
        const Json* f = manifest_.find(name);
        if (!f)
            throw Error("kernel library '" + name + "' is not in " + dir_ + "/manifest.json; build the kernels first "
                        "(python -c 'import __graft_entry__ as g; g.build()', or python -m trapetum_b200.csrc.build)");
        const std::string path = dir_ + "/" + f->string("manifest entry");
        KernelLib l;
        l.name = name;
        l.handle = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
        if (!l.handle) throw Error("cannot load " + path + ": " + dlerror());
        l.error = l.sym<const char* (*)()>("tb_error");
        return libs_.emplace(name, l).first->second;
    }
    bool has(const std::string& name) {
        std::lock_guard<std::mutex> g(mu_);
        load_manifest();
        return manifest_.find(name) != nullptr;
    }
    std::vector<std::string> loaded() {
        std::lock_guard<std::mutex> g(mu_);
        std::vector<std::string> v;
        for (auto& kv : libs_) v.push_back(kv.first);
        return v;
    }
    // Throws if a launcher's status says "refused" (< 0: the library's message) or "CUDA error" (> 0).
    static void check(const KernelLib& l, int status, const char* what) {
        if (status == 0) return;
        if (status < 0) throw Error(std::string(what) + ": " + l.error());
        throw Error(fmt("%s: CUDA error %d at launch (%s)", what, status, cudaGetErrorString((cudaError_t)status)));
    }
    long long launches = 0;              // kernels launched through this table (graph replays add their kernels)

private:
    void load_manifest() {
        if (!manifest_.is_null()) return;
        if (dir_.empty()) {
            const char* env = getenv("TRAPETUM_KERNEL_DIR");
            if (env && *env) dir_ = env;
            else {
                Dl_info info;
                if (dladdr((void*)&Kernels::get, &info) && info.dli_fname) {
                    std::string self = info.dli_fname;
                    const size_t slash = self.rfind('/');
                    dir_ = (slash == std::string::npos ? std::string(".") : self.substr(0, slash));
                } else dir_ = ".";
            }
        }
        std::ifstream f(dir_ + "/manifest.json");
        if (!f) throw Error("no kernel manifest at " + dir_ + "/manifest.json; build the kernels first "
                            "(python -c 'import __graft_entry__ as g; g.build()')");
        std::stringstream ss;
        ss << f.rdbuf();
        manifest_ = Json::parse(ss.str());
    }
    std::mutex mu_;
    std::string dir_;
    Json manifest_;
    std::map<std::string, KernelLib> libs_;
};

}  // namespace tb
