// gemma_run <model_dir> <prompt.bin> [<prompt.bin> ...] [options]
// gemma_run --random-weights <config.json> --seed S <prompt.bin> [...] [options]
//
// The command line over the C interface, in the manner of the reference's `gemma_run <model.cbk> <prompt.bin>`
// (runtime/src/bin/gemma_run.rs:2-18): positional model and prompt, the prompt a file of little-endian int32 token
// ids as its exporter writes it (model/export_gemma.py:77-78), greedy continuation of 24 tokens by default, and the
// same three lines of output (load time and prompt, continuation ids, ms/token and tok/s).  Several prompt files run
// as one batch.  The sampling options carry the names of the reference server's request fields
// (runtime/src/bin/serve.rs:1284-1292).
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "trapetum_b200.h"

static double now() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

static int usage(const char* msg) {
    fprintf(stderr, "gemma_run: %s\nusage: gemma_run <model_dir> <prompt.bin> [...] [--prompt_ids a,b,c] [--max_tokens N] "
                    "[--temperature T] [--top_p P] [--repetition_penalty R] [--seed S] [--stop_id I]... [--dtype bfloat16|float32] "
                    "[--max_batch B] [--random-weights config.json [--std S] [--norm_std S]] [--kernels DIR]\n", msg);
    return 2;
}

int main(int argc, char** argv) {
    std::vector<std::string> pos, prompt_ids;
    std::vector<int> stops;
    bool have_stops = false;
    std::string dtype = "bfloat16", random_cfg, kernels;
    tb_sampling sp = {0.f, 0.95f, 1.0f, 24, 0ull};
    int max_batch = 64, device = 0;
    float std_ = 0.02f, norm_std = 0.1f;
    for (int i = 1; i < argc; i++) {
        std::string a = argv[i];
        for (auto& c : a) if (c == '-' && &c - a.data() >= 2) c = '_';
        auto val = [&](const char* name) -> const char* {
            if (i + 1 >= argc) { usage((std::string(name) + " needs a value").c_str()); exit(2); }
            return argv[++i];
        };
        if (a == "--max_tokens") sp.max_tokens = atoi(val("--max_tokens"));
        else if (a == "--temperature") sp.temperature = (float)atof(val("--temperature"));
        else if (a == "--top_p") sp.top_p = (float)atof(val("--top_p"));
        else if (a == "--repetition_penalty") sp.repetition_penalty = (float)atof(val("--repetition_penalty"));
        else if (a == "--seed") sp.seed = strtoull(val("--seed"), nullptr, 10);
        else if (a == "--stop_id") { stops.push_back(atoi(val("--stop_id"))); have_stops = true; }
        else if (a == "--dtype") dtype = val("--dtype");
        else if (a == "--device") device = atoi(val("--device"));
        else if (a == "--max_batch") max_batch = atoi(val("--max_batch"));
        else if (a == "--random_weights") random_cfg = val("--random-weights");
        else if (a == "--std") std_ = (float)atof(val("--std"));
        else if (a == "--norm_std") norm_std = (float)atof(val("--norm_std"));
        else if (a == "--prompt_ids") prompt_ids.push_back(val("--prompt_ids"));
        else if (a == "--kernels") kernels = val("--kernels");
        else if (a.size() > 2 && a[0] == '-' && a[1] == '-') return usage(("unknown option " + a).c_str());
        else pos.push_back(argv[i]);
    }
    if (!kernels.empty()) tb_set_kernel_dir(kernels.c_str());
    std::string model_dir;
    if (random_cfg.empty()) {
        if (pos.empty()) return usage("the model folder is missing");
        model_dir = pos.front();
        pos.erase(pos.begin());
    }
    std::vector<std::vector<int>> prompts;
    for (auto& p : pos) {
        std::ifstream f(p, std::ios::binary);
        if (!f) return usage(("cannot read prompt file " + p).c_str());
        std::vector<char> bytes((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
        std::vector<int> ids(bytes.size() / 4);
        memcpy(ids.data(), bytes.data(), ids.size() * 4);
        prompts.push_back(ids);
    }
    for (auto& s : prompt_ids) {
        std::vector<int> ids;
        std::stringstream ss(s);
        std::string tok;
        while (std::getline(ss, tok, ',')) if (!tok.empty()) ids.push_back(atoi(tok.c_str()));
        prompts.push_back(ids);
    }
    if (prompts.empty()) return usage("no prompt: give a prompt.bin file or --prompt_ids");

    const double t0 = now();
    tb_model* model;
    if (!random_cfg.empty()) {
        std::ifstream f(random_cfg);
        if (!f) return usage(("cannot read " + random_cfg).c_str());
        std::stringstream ss;
        ss << f.rdbuf();
        model = tb_model_random(ss.str().c_str(), sp.seed, std_, norm_std, dtype.c_str(), device);
    } else model = tb_model_load(model_dir.c_str(), nullptr, dtype.c_str(), device, nullptr);
    if (!model) { fprintf(stderr, "gemma_run: %s\n", tb_last_error()); return 1; }
    printf("loaded in %.1fs vocab=%d", now() - t0, tb_model_vocab(model));
    std::vector<int> flat, lens;
    long long need = 0;
    for (auto& p : prompts) {
        printf(" prompt=%zu tokens [", p.size());
        for (size_t i = 0; i < p.size(); i++) printf("%s%d", i ? ", " : "", p[i]);
        printf("]");
        flat.insert(flat.end(), p.begin(), p.end());
        lens.push_back((int)p.size());
        need += ((long long)p.size() + sp.max_tokens + 63) / 64 * 64;
    }
    printf("\n");
    fflush(stdout);
    tb_engine* engine = tb_engine_new(model, need, max_batch, 1);
    if (!engine) { fprintf(stderr, "gemma_run: %s\n", tb_last_error()); return 1; }
    const int cap = sp.max_tokens > 0 ? sp.max_tokens : 1;
    std::vector<int> out((size_t)prompts.size() * cap), out_lens(prompts.size());
    const double t1 = now();
    const int rc = tb_generate(engine, flat.data(), lens.data(), (int)prompts.size(), &sp, have_stops ? stops.data() : nullptr,
                               have_stops ? (int)stops.size() : -1, max_batch, nullptr, nullptr, out.data(), out_lens.data(), cap);
    if (rc != TB_OK) { fprintf(stderr, "gemma_run: %s\n", tb_last_error()); return 1; }
    tb_engine_synchronize(engine);
    const double dt = now() - t1;
    int total = 0, longest = 1;
    for (size_t i = 0; i < prompts.size(); i++) {
        printf("continuation ids: [");
        for (int k = 0; k < out_lens[i]; k++) printf("%s%d", k ? ", " : "", out[i * cap + k]);
        printf("]\n");
        total += out_lens[i];
        if (out_lens[i] > longest) longest = out_lens[i];
    }
    printf("decode: %.1f ms/token (%.1f tok/s), trapetum_b200 %s (native host)\n", dt * 1e3 / longest, (total ? total : 1) / dt,
           dtype.c_str());
    tb_engine_free(engine);
    tb_model_free(model);
    return 0;
}
