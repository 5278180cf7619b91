"""A mixer from outside the library on the native host: a CUDA file of the test's own (a running mean with a state
of its own per sequence) is compiled here, registered through the plugin interface (native/plugin.h) under a kind
name, and a model whose spec names that kind is built, given weights, and stepped (prompts of unequal lengths,
then token by token, slots used again) by the library's native engine, cache and generation code, none of which
was changed for it.  The Python host's counterpart is in test_gpu_parts.py."""
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


@pytest.fixture(scope="module")
def plugin(tmp_path_factory):
    from trapetum_b200 import native
    from trapetum_b200.csrc import build
    d = tmp_path_factory.mktemp("plugin")
    src, out = os.path.join(d, "running_mean.cu"), os.path.join(d, "running_mean.so")
    with open(src, "w") as f:
        f.write(PLUGIN_CU)
    native_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(build.__file__))), "native")
    subprocess.run([build._nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "--shared", "-Xcompiler", "-fPIC",
                    "-I", native_dir, "-o", out, src], check=True)
    so = ctypes.CDLL(out)
    so.running_mean_plugin.restype = ctypes.c_void_p
    assert native.lib().tb_register_mixer(b"test_running_mean_native", ctypes.c_void_p(so.running_mean_plugin())) == 0
    return so


def _register_architecture():
    from trapetum_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
    from trapetum_b200.config.base import _get

    @dataclass(frozen=True)
    class Cfg:
        layers: int; hidden: int; inter: int; vocab: int; eps: float

        @classmethod
        def from_dict(cls, d):
            return cls(_get(d, "toy_layers", int), _get(d, "toy_hidden", int), _get(d, "toy_inter", int), _get(d, "toy_vocab", int),
                       _get(d, "toy_eps", float))

    def spec(c):
        norm = lambda n: PartSpec("rmsnorm", {"size": c.hidden, "eps": c.eps, "unit_offset": False, "weight": n})
        layers = tuple(LayerSpec(
            block=PartSpec("pre_norm", {"pre_mixer_norm": norm("n1.weight"), "pre_ffn_norm": norm("n2.weight")}),
            mixer=PartSpec("test_running_mean_native", {"hidden_size": c.hidden, "weight": "mix.weight"}),
            feed_forward=PartSpec("gated_mlp", {"hidden_size": c.hidden, "intermediate_size": c.inter, "activation": "silu",
                                                "gate": "g.weight", "up": "u.weight", "down": "d.weight"}),
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
    for i in range(cfg["toy_layers"]):
        p = f"blocks.{i}."
        shapes.update({p + "n1.weight": (H,), p + "n2.weight": (H,), p + "mix.weight": (H, H), p + "g.weight": (I, H),
                       p + "u.weight": (I, H), p + "d.weight": (H, I)})
    out = {}
    for name, shape in shapes.items():
        s = norm_std if len(shape) == 1 else std
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
