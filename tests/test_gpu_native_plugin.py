"""Parts from outside the library on the native host: CUDA files of the test's own (a mixer: a running mean with a
state of its own per sequence; a feed-forward that routes each token to one of several experts) are compiled here,
registered through the plugin interface (native/plugin.h) under kind names, and models whose specs name those kinds
are built, given weights, and stepped (prompts of unequal lengths, then token by token, slots used again) by the
library's native engine, cache and generation code, none of which was changed for them.  The Python host's
counterparts are in test_gpu_parts.py."""
import ctypes
import os
import subprocess
from dataclasses import dataclass

import numpy as np
import pytest
import torch

from conftest import make_prompts, rel_l2
from test_gpu_parts import _toy_plain

pytestmark = pytest.mark.gpu

PLUGIN_CU = r"""
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "plugin.h"

// y_t = W * mean(x_0 .. x_t); the state of a sequence is the running sum and the count: [hidden + 1] floats.
struct RunningMean {
    int hidden, dtype;
    char weight_name[192];
    const void* w;
    int w_dtype;
};

__device__ float rd(const void* p, int dtype, size_t i) {
    return dtype == TB_DTYPE_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}

__global__ void running_mean_kernel(const void* x, int x_dtype, const void* w, int w_dtype, float* out, int hidden,
                                    const int* seq_start, const int* slot_ids, char* state, long long state_bytes) {
    extern __shared__ float mean[];
    const int b = blockIdx.x;
    float* st = (float*)(state + (size_t)slot_ids[b] * state_bytes);
    for (int t = seq_start[b]; t < seq_start[b + 1]; t++) {
        __syncthreads();
        const float count = st[hidden] + 1.f;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float s = st[i] + rd(x, x_dtype, (size_t)t * hidden + i);
            st[i] = s;
            mean[i] = s / count;
        }
        __syncthreads();
        if (threadIdx.x == 0) st[hidden] = count;
        for (int o = threadIdx.x; o < hidden; o += blockDim.x) {
            float acc = 0.f;
            for (int i = 0; i < hidden; i++) acc += rd(w, w_dtype, (size_t)o * hidden + i) * mean[i];
            out[(size_t)t * hidden + o] = acc;
        }
    }
}

static void* create(const char* params, const char* prefix, int dtype, const char** error) {
    const char* h = strstr(params, "\"hidden_size\":");
    const char* wn = strstr(params, "\"weight\":\"");
    if (!h || !wn) { *error = "running mean: needs hidden_size and weight"; return nullptr; }
    RunningMean* m = (RunningMean*)calloc(1, sizeof(RunningMean));
    m->hidden = atoi(h + strlen("\"hidden_size\":"));
    m->dtype = dtype;
    wn += strlen("\"weight\":\"");
    snprintf(m->weight_name, sizeof m->weight_name, "%s%.*s", prefix, (int)(strchr(wn, '"') - wn), wn);
    return m;
}
static void destroy(void* self) { free(self); }
static int tensor_count(void*) { return 1; }
static int tensor_decl(void* self, int, tb_tensor_decl* d) {
    RunningMean* m = (RunningMean*)self;
    snprintf(d->name, sizeof d->name, "%s", m->weight_name);
    d->shape[0] = d->shape[1] = m->hidden; d->ndim = 2;
    snprintf(d->role, sizeof d->role, "matrix");
    return 0;
}
static int bind(void* self, const char*, const void* data, int dtype, const char**) {
    ((RunningMean*)self)->w = data; ((RunningMean*)self)->w_dtype = dtype;
    return 0;
}
static int cache_need(void* self, tb_cache_need* n) {
    n->kind = TB_NEED_STATE;
    n->state_bytes = (((RunningMean*)self)->hidden + 1) * 4;
    return 0;
}
static int forward(void* self, const tb_part_ctx* c, const void* x, int x_dtype, long long rows, long long cols, float* out,
                   const char** error) {
    RunningMean* m = (RunningMean*)self;
    if (cols != m->hidden || !c->state) { *error = "running mean: wrong width, or no state area"; return 1; }
    if (c->dry) return 0;
    running_mean_kernel<<<c->batch, 128, m->hidden * sizeof(float), (cudaStream_t)c->stream>>>(
        x, x_dtype, m->w, m->w_dtype, out, m->hidden, c->seq_start, c->slot_ids, (char*)c->state, c->state_bytes);
    return cudaGetLastError() != cudaSuccess;
}
static const tb_mixer_plugin plugin = {create, destroy, tensor_count, tensor_decl, bind, cache_need, forward, 1};
extern "C" const tb_mixer_plugin* running_mean_plugin() { return &plugin; }
"""


ROUTED_CU = r"""
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "plugin.h"

// Each token goes to the expert whose router row gives the largest product (the lowest index on a tie):
// y = W2[e] relu(W1[e] x).  Router logits and everything else in 32-bit.
struct Routed {
    int hidden, inter, experts;
    char prefix[160];
    const void* router; const void* w1; const void* w2;
    int dt_router, dt_w1, dt_w2;
};

__device__ float rdv(const void* p, int dtype, size_t i) {
    return dtype == TB_DTYPE_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}

__global__ void routed_kernel(const void* x, int x_dtype, Routed m, float* out) {
    extern __shared__ float sh[];                  // [hidden] the token, [inter] the expert's inner values, [experts] logits
    float* xs = sh; float* mid = sh + m.hidden; float* logit = mid + m.inter;
    const size_t t = blockIdx.x;
    for (int i = threadIdx.x; i < m.hidden; i += blockDim.x) xs[i] = rdv(x, x_dtype, t * m.hidden + i);
    __syncthreads();
    for (int e = threadIdx.x; e < m.experts; e += blockDim.x) {
        float acc = 0.f;
        for (int i = 0; i < m.hidden; i++) acc += rdv(m.router, m.dt_router, (size_t)e * m.hidden + i) * xs[i];
        logit[e] = acc;
    }
    __syncthreads();
    int best = 0;
    for (int e = 1; e < m.experts; e++) if (logit[e] > logit[best]) best = e;
    for (int j = threadIdx.x; j < m.inter; j += blockDim.x) {
        float acc = 0.f;
        for (int i = 0; i < m.hidden; i++) acc += rdv(m.w1, m.dt_w1, ((size_t)best * m.inter + j) * m.hidden + i) * xs[i];
        mid[j] = fmaxf(acc, 0.f);
    }
    __syncthreads();
    for (int o = threadIdx.x; o < m.hidden; o += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < m.inter; j++) acc += rdv(m.w2, m.dt_w2, ((size_t)best * m.hidden + o) * m.inter + j) * mid[j];
        out[t * m.hidden + o] = acc;
    }
}

static int param(const char* params, const char* key) {
    char pat[64];
    snprintf(pat, sizeof pat, "\"%s\":", key);
    const char* at = strstr(params, pat);
    return at ? atoi(at + strlen(pat)) : -1;
}
static void* create(const char* params, const char* prefix, int, const char** error) {
    Routed* m = (Routed*)calloc(1, sizeof(Routed));
    m->hidden = param(params, "hidden_size"); m->inter = param(params, "intermediate_size"); m->experts = param(params, "experts");
    if (m->hidden <= 0 || m->inter <= 0 || m->experts <= 0) { free(m); *error = "routed: needs hidden_size, intermediate_size, experts"; return nullptr; }
    snprintf(m->prefix, sizeof m->prefix, "%s", prefix);
    return m;
}
static void destroy(void* self) { free(self); }
static int tensor_count(void*) { return 3; }
static int tensor_decl(void* self, int i, tb_tensor_decl* d) {
    Routed* m = (Routed*)self;
    const char* names[3] = {"router.weight", "w1.weight", "w2.weight"};
    snprintf(d->name, sizeof d->name, "%s%s", m->prefix, names[i]);
    snprintf(d->role, sizeof d->role, "matrix");
    if (i == 0) { d->shape[0] = m->experts; d->shape[1] = m->hidden; d->ndim = 2; }
    if (i == 1) { d->shape[0] = m->experts; d->shape[1] = m->inter; d->shape[2] = m->hidden; d->ndim = 3; }
    if (i == 2) { d->shape[0] = m->experts; d->shape[1] = m->hidden; d->shape[2] = m->inter; d->ndim = 3; }
    return 0;
}
static int bind(void* self, const char* name, const void* data, int dtype, const char**) {
    Routed* m = (Routed*)self;
    if (strstr(name, "router.weight")) { m->router = data; m->dt_router = dtype; }
    else if (strstr(name, "w1.weight")) { m->w1 = data; m->dt_w1 = dtype; }
    else { m->w2 = data; m->dt_w2 = dtype; }
    return 0;
}
static int forward(void* self, const tb_part_ctx* c, const void* x, int x_dtype, long long rows, long long cols, float* out,
                   const char** error) {
    Routed* m = (Routed*)self;
    if (cols != m->hidden) { *error = "routed: wrong width"; return 1; }
    if (c->state || c->k || c->page_table) { *error = "routed: a feed-forward was handed a cache"; return 1; }
    if (c->dry || rows == 0) return 0;
    routed_kernel<<<(unsigned)rows, 64, (m->hidden + m->inter + m->experts) * sizeof(float), (cudaStream_t)c->stream>>>(x, x_dtype, *m, out);
    return cudaGetLastError() != cudaSuccess;
}
static const tb_mixer_plugin plugin = {create, destroy, tensor_count, tensor_decl, bind, nullptr, forward, 1};
extern "C" const tb_mixer_plugin* routed_plugin() { return &plugin; }
"""


def _compile(tmp_path_factory, name, source):
    from trapetum_b200.csrc import build
    d = tmp_path_factory.mktemp(name)
    src, out = os.path.join(d, name + ".cu"), os.path.join(d, name + ".so")
    with open(src, "w") as f:
        f.write(source)
    native_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(build.__file__))), "native")
    subprocess.run([build._nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "--shared", "-Xcompiler", "-fPIC",
                    "-I", native_dir, "-o", out, src], check=True)
    return ctypes.CDLL(out)


@pytest.fixture(scope="module")
def routed_plugin(tmp_path_factory):
    from trapetum_b200 import native
    so = _compile(tmp_path_factory, "routed", ROUTED_CU)
    so.routed_plugin.restype = ctypes.c_void_p
    assert native.lib().tb_register_feed_forward(b"test_routed_native", ctypes.c_void_p(so.routed_plugin())) == 0
    return so


@pytest.fixture(scope="module")
def plugin(tmp_path_factory):
    from trapetum_b200 import native
    so = _compile(tmp_path_factory, "running_mean", PLUGIN_CU)
    so.running_mean_plugin.restype = ctypes.c_void_p
    assert native.lib().tb_register_mixer(b"test_running_mean_native", ctypes.c_void_p(so.running_mean_plugin())) == 0
    return so


def _register_architecture():
    from trapetum_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
    from trapetum_b200.config.base import _get

    @dataclass(frozen=True)
    class Cfg:
        layers: int; hidden: int; inter: int; vocab: int; eps: float; experts: int

        @classmethod
        def from_dict(cls, d):
            return cls(_get(d, "toy_layers", int), _get(d, "toy_hidden", int), _get(d, "toy_inter", int), _get(d, "toy_vocab", int),
                       _get(d, "toy_eps", float), int(d.get("toy_experts", 0)))

    def spec(c):
        norm = lambda n: PartSpec("rmsnorm", {"size": c.hidden, "eps": c.eps, "unit_offset": False, "weight": n})
        layers = tuple(LayerSpec(
            block=PartSpec("pre_norm", {"pre_mixer_norm": norm("n1.weight"), "pre_ffn_norm": norm("n2.weight")}),
            mixer=PartSpec("test_running_mean_native", {"hidden_size": c.hidden, "weight": "mix.weight"}),
            # odd layers route their tokens to experts (a feed-forward from a plugin) when the configuration has experts
            feed_forward=(PartSpec("test_routed_native", {"hidden_size": c.hidden, "intermediate_size": c.inter, "experts": c.experts})
                          if c.experts and i % 2 else
                          PartSpec("gated_mlp", {"hidden_size": c.hidden, "intermediate_size": c.inter, "activation": "silu",
                                                 "gate": "g.weight", "up": "u.weight", "down": "d.weight"})),
            prefix=f"blocks.{i}.") for i in range(c.layers))
        return ModelSpec(architecture="TestNativeToyLM", hidden_size=c.hidden, vocab_size=c.vocab,
                         embedding=PartSpec("embedding", {"vocab_size": c.vocab, "hidden_size": c.hidden, "scale": 1.0, "weight": "emb.weight"}),
                         layers=layers, schedule=tuple(ScheduleEntry(i) for i in range(c.layers)), final_norm=norm("out_norm.weight"),
                         head=PartSpec("linear_head", {"vocab_size": c.vocab, "hidden_size": c.hidden, "softcap": None,
                                                       "weight": "head.weight", "tied_to": None}),
                         max_positions=512)
    register_architecture("TestNativeToyLM", Cfg, spec)


def _weights(cfg, seed, std, norm_std):
    """The tensors the generator makes for this model and seed, on the host, for the plain computation."""
    from trapetum_b200.weights.random_init import name_key, normal_host
    H, I, V = cfg["toy_hidden"], cfg["toy_inter"], cfg["toy_vocab"]
    shapes = {"emb.weight": (V, H), "head.weight": (V, H), "out_norm.weight": (H,)}
    E = cfg.get("toy_experts", 0)
    for i in range(cfg["toy_layers"]):
        p = f"blocks.{i}."
        shapes.update({p + "n1.weight": (H,), p + "n2.weight": (H,), p + "mix.weight": (H, H)})
        if E and i % 2:
            shapes.update({p + "router.weight": (E, H), p + "w1.weight": (E, I, H), p + "w2.weight": (E, H, I)})
        else:
            shapes.update({p + "g.weight": (I, H), p + "u.weight": (I, H), p + "d.weight": (H, I)})
    out = {}
    for name, shape in shapes.items():
        s = norm_std if ("n1." in name or "n2." in name or "out_norm" in name) else std
        out[name] = torch.from_numpy(normal_host(int(np.prod(shape)), name_key(seed, name), s).reshape(shape).copy())
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_mixer_from_a_plugin_runs_on_the_native_host(plugin, dtype):
    import trapetum_b200 as tb
    from trapetum_b200 import native
    _register_architecture()
    cfg = {"architectures": ["TestNativeToyLM"], "toy_layers": 2, "toy_hidden": 40, "toy_inter": 56, "toy_vocab": 90, "toy_eps": 1e-5}
    assert native.is_native(tb.load_config(cfg)[1])                      # the kind is known now
    model = tb.random_model(cfg, 9, 0.2, 0.3, dtype)                       # host "auto" picks the native host
    assert isinstance(model, native.Model)
    eng = tb.Engine(model, 64 * 4, max_slots=4)
    assert eng.cache.groups == []                                          # no keys or values: state only
    pw = _weights(cfg, 9, 0.2, 0.3)
    prompts = make_prompts(90, [21, 8, 13], seed=1)
    truth = [_toy_plain(cfg, pw, p) for p in prompts]
    tol = 1e-5 if dtype == "float32" else 3e-2
    for round_ in range(2):                                                # the second round reuses slots: the state must restart
        s = eng.start(3)
        cut = [10, 5, 1]
        first = eng.step(s, [p[:c] for p, c in zip(prompts, cut)], [list(range(c)) for c in cut])
        o = 0
        for r in range(3):
            assert max(rel_l2(first[o + i], truth[r][i]) for i in range(cut[r])) < tol
            o += cut[r]
        live = list(range(3))
        t = 0
        while live:
            for r in [r for r in live if cut[r] + t >= len(prompts[r])]:
                eng.release([s[r]]); live.remove(r)
            if not live:
                break
            out = eng.step([s[r] for r in live], [[prompts[r][cut[r] + t]] for r in live])
            for i, r in enumerate(live):
                assert rel_l2(out[i], truth[r][cut[r] + t]) < tol, (round_, r, t)
            t += 1
        eng.cache.check()
    assert eng.graphs_captured >= 1                                        # its decode steps ran as captured graphs
    # the generation loop, too, knows nothing of the mixer
    got = tb.generate(model, prompts, max_tokens=6, stop_ids=[])
    if dtype == "float32":
        for p, g in zip(prompts, got):
            ids = list(p)
            for tok in g:
                assert tok == int(_toy_plain(cfg, pw, ids)[-1].argmax())
                ids.append(tok)


def _routed_plain(cfg, w, ids):
    """The toy model whose odd layers route (see ROUTED_CU), whole sequence, plain torch on the CPU."""
    eps = cfg["toy_eps"]
    norm = lambda x, g: x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * g
    h = w["emb.weight"][torch.tensor(ids)]
    picks = []
    for i in range(cfg["toy_layers"]):
        p = f"blocks.{i}."
        x = norm(h, w[p + "n1.weight"])
        h = h + (torch.cumsum(x, 0) / torch.arange(1, len(ids) + 1)[:, None]) @ w[p + "mix.weight"].T
        x = norm(h, w[p + "n2.weight"])
        if i % 2:
            e = (x @ w[p + "router.weight"].T).argmax(-1)
            picks.append(e.tolist())
            h = h + torch.stack([w[p + "w2.weight"][k] @ torch.relu(w[p + "w1.weight"][k] @ row) for row, k in zip(x, e.tolist())])
        else:
            g = x @ w[p + "g.weight"].T
            h = h + ((g * torch.sigmoid(g)) * (x @ w[p + "u.weight"].T)) @ w[p + "d.weight"].T
    return norm(h, w["out_norm.weight"]) @ w["head.weight"].T, picks


def test_a_routed_feed_forward_from_a_plugin_runs_on_the_native_host(plugin, routed_plugin):
    """Both branches of the odd layers come from outside the library; prompts in one step, then token by token."""
    import trapetum_b200 as tb
    from trapetum_b200 import native
    _register_architecture()
    cfg = {"architectures": ["TestNativeToyLM"], "toy_layers": 4, "toy_hidden": 40, "toy_inter": 24, "toy_vocab": 90, "toy_eps": 1e-5,
           "toy_experts": 3}
    assert native.is_native(tb.load_config(cfg)[1])
    model = tb.random_model(cfg, 5, 0.2, 0.3, "float32")
    assert isinstance(model, native.Model)
    eng = tb.Engine(model, 64 * 4, max_slots=4)
    pw = _weights(cfg, 5, 0.2, 0.3)
    prompts = make_prompts(90, [19, 7, 12], seed=2)
    truth, picks = zip(*[_routed_plain(cfg, pw, p) for p in prompts])
    assert len({e for seq in picks for layer in seq for e in layer}) == 3       # every expert is used
    s = eng.start(3)
    cut = [9, 4, 12]
    first = eng.step(s, [p[:c] for p, c in zip(prompts, cut)], [list(range(c)) for c in cut])
    o = 0
    for r in range(3):
        assert max(rel_l2(first[o + i], truth[r][i]) for i in range(cut[r])) < 1e-5
        o += cut[r]
    for t in range(7):
        live = [r for r in range(3) if cut[r] + t < len(prompts[r])]
        out = eng.step([s[r] for r in live], [[prompts[r][cut[r] + t]] for r in live])
        for i, r in enumerate(live):
            assert rel_l2(out[i], truth[r][cut[r] + t]) < 1e-5, (r, t)
    eng.release(s)
    eng.cache.check()
    assert eng.graphs_captured >= 1
