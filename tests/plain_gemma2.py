"""A plain, slow Gemma-2: whole sequences, no cache, no batching, one function per part.

This file is the oracle of the tests.  It shares no code with ``trapetum_b200``:
it reads the model folder with the ``safetensors`` library and computes with
ordinary torch operations on the CPU, one sequence at a time, in float32 (or
float64 when asked).  It rests on the formulas of neuralboot/trapetum's Gemma-2
path, cited per function below by the file's path in that project; the
reference's own model code is Rust over CUDA kernels and cannot be imported or
compiled on a CPU, so no numeric comparison with it exists (its exporter writes
no reference logits either, model/export_gemma.py:74-79).  Where the reference
leaves something out (the sliding window, runtime/src/lib.rs:4455) or fixes it
(the score scale, runtime/cuda/codebook_gemv.cu:250), the formula here follows
the architecture's configuration keys that the exporter reads
(model/export_gemma.py:40-46).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch


# ----------------------------------------------------------------------------
# Reading a model folder
# ----------------------------------------------------------------------------
def load_folder(folder: str, dtype=torch.float32) -> Tuple[dict, Dict[str, torch.Tensor]]:
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    w = {k: v.to(dtype) for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    return cfg, w


def layer_is_sliding(cfg: dict, i: int) -> bool:
    """Even layers slide, odd layers see everything (unless config.json lists layer_types)."""
    if cfg.get("sliding_window") is None:
        return False
    lt = cfg.get("layer_types")
    if lt is not None:
        return lt[i] == "sliding_attention"
    return i % 2 == 0


# ----------------------------------------------------------------------------
# Parts
# ----------------------------------------------------------------------------
def _same(x):
    return x


def to_bf16(x: torch.Tensor) -> torch.Tensor:
    """Round to bfloat16 and back: what a 16-bit activation buffer does to its contents."""
    return x.to(torch.bfloat16).to(x.dtype)


def embed(ids: Sequence[int], table: torch.Tensor, hidden: int) -> torch.Tensor:
    """h[t] = E[id_t] * sqrt(hidden)   (model/export_gemma.py:59-61; runtime/src/lib.rs:4554-4555)."""
    return table[torch.tensor(list(ids), dtype=torch.long)] * math.sqrt(hidden)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * (1 + w)
    (runtime/cuda/codebook_gemv.cu:192-202 with the +1 of model/export_gemma.py:25-26)."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps) * (1.0 + w)


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """x [T, heads, hd]; pairs (i, i + hd/2) rotated by pos * theta^(-2i/hd)
    (runtime/cuda/codebook_gemv.cu:219-230; table as in model/export_gemma.py:53)."""
    hd = x.shape[-1]
    inv_freq = 1.0 / (theta ** (torch.arange(0, hd, 2).float() / hd))
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]          # [T, hd/2], 32-bit as in the kernel
    cos, sin = ang.cos().to(x.dtype)[:, None, :], ang.sin().to(x.dtype)[:, None, :]
    x0, x1 = x[..., : hd // 2], x[..., hd // 2:]
    return torch.cat([x0 * cos - x1 * sin, x1 * cos + x0 * sin], dim=-1)


def visible(i: int, j: int, window: Optional[int]) -> bool:
    """Key j is visible to query i: causal, and within the last `window` tokens (the query's own included)."""
    return j <= i and (window is None or i - j < window)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, cap: Optional[float],
              window: Optional[int], rnd=_same) -> torch.Tensor:
    """q [T, nh, hd], k and v [T, nkv, hd] -> [T, nh, hd].
    s = (q.k) * scale; s = cap*tanh(s/cap); softmax with the maximum subtracted; sum of p*v
    (runtime/cuda/codebook_gemv.cu:240-270); query head h reads kv head h // (nh // nkv) (:244).
    ``rnd`` is applied to the unnormalised probabilities before they meet v: a 16-bit engine hands
    them to its tensor cores in 16 bits, while their sum stays 32-bit."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    out = torch.zeros_like(q)
    for h in range(nh):
        kh = h // (nh // nkv)
        s = (q[:, h, :] @ k[:, kh, :].T) * scale                              # [T, T]
        if cap:
            s = cap * torch.tanh(s / cap)
        mask = torch.tensor([[visible(i, j, window) for j in range(T)] for i in range(T)])
        s = s.masked_fill(~mask, float("-inf"))
        s = s - s.max(dim=-1, keepdim=True).values
        p = s.exp()
        out[:, h, :] = (rnd(p) @ v[:, kh, :]) / p.sum(dim=-1, keepdim=True)
    return out


def gelu_tanh(g: torch.Tensor) -> torch.Tensor:
    """0.5 g (1 + tanh(0.7978845608 (g + 0.044715 g^3)))   (runtime/cuda/codebook_gemv.cu:531-537)."""
    return 0.5 * g * (1.0 + torch.tanh(0.7978845608 * (g + 0.044715 * g * g * g)))


def feed_forward(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor, rnd=_same) -> torch.Tensor:
    """down(gelu_tanh(gate(x)) * up(x))   (runtime/src/lib.rs:4511-4516)."""
    return rnd(gelu_tanh(rnd(x @ wg.T)) * rnd(x @ wu.T)) @ wd.T


def attention_block(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, cfg: dict, window: Optional[int],
                    kv_from: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, rnd=_same):
    """Projections without bias, rope on q and k, attention, output projection
    (runtime/src/lib.rs:4483-4496).  Returns (output, (k_rot, v)).  ``rnd`` is applied wherever a
    16-bit engine stores an activation (identity for the oracle; see :func:`forward`)."""
    T = x.shape[0]
    nh, nkv, hd = cfg["num_attention_heads"], cfg.get("num_key_value_heads", cfg["num_attention_heads"]), cfg["head_dim"]
    pos = torch.arange(T)
    theta = float(cfg.get("rope_theta", 10000.0))
    q = rnd(rope(rnd(x @ w[prefix + "self_attn.q_proj.weight"].T).view(T, nh, hd), pos, theta))
    if kv_from is None:
        k = rnd(rope(rnd(x @ w[prefix + "self_attn.k_proj.weight"].T).view(T, nkv, hd), pos, theta))
        v = rnd(x @ w[prefix + "self_attn.v_proj.weight"].T).view(T, nkv, hd)
    else:
        k, v = kv_from
    scale = float(cfg.get("query_pre_attn_scalar", hd)) ** -0.5
    cap = cfg.get("attn_logit_softcapping") or None
    o = rnd(attention(q, k, v, scale, cap, window, rnd))
    return o.reshape(T, nh * hd) @ w[prefix + "self_attn.o_proj.weight"].T, (k, v)


def decoder_layer(h: torch.Tensor, w: Dict[str, torch.Tensor], i: int, cfg: dict, kv_from=None, rnd=_same):
    """h += post_attn_norm(attn(input_norm(h))); h += post_ff_norm(mlp(pre_ff_norm(h)))
    (runtime/src/lib.rs:4527-4540)."""
    p = f"model.layers.{i}."
    eps = float(cfg.get("rms_norm_eps", 1e-6))
    window = cfg["sliding_window"] if layer_is_sliding(cfg, i) else None
    a, kv = attention_block(rnd(rmsnorm(h, w[p + "input_layernorm.weight"], eps)), w, p, cfg, window, kv_from, rnd)
    h = h + rmsnorm(a, w[p + "post_attention_layernorm.weight"], eps)
    m = feed_forward(rnd(rmsnorm(h, w[p + "pre_feedforward_layernorm.weight"], eps)),
                     w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"], rnd)
    h = h + rmsnorm(m, w[p + "post_feedforward_layernorm.weight"], eps)
    return h, kv


def head(h: torch.Tensor, w: Dict[str, torch.Tensor], cfg: dict, rnd=_same) -> torch.Tensor:
    """logits = final_norm(h) E^T (tied, unscaled), then cap*tanh(logits/cap)
    (runtime/src/lib.rs:4557-4560; model/export_gemma.py:73)."""
    x = rnd(rmsnorm(h, w["model.norm.weight"], float(cfg.get("rms_norm_eps", 1e-6))))
    E = w.get("lm_head.weight", w["model.embed_tokens.weight"])
    logits = x @ E.T
    cap = cfg.get("final_logit_softcapping") or None
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits


def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: Sequence[int],
            schedule: Optional[List[Tuple[int, Optional[int]]]] = None, rnd=_same) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``schedule``: (layer, entry whose keys and values
    this call reads, or None) per call; by default every layer once, in order.

    ``rnd=to_bf16`` rounds every activation that a 16-bit engine stores between two kernels (normed
    inputs, q/k/v before and after rope, attention output, gate, up and their product) while the
    residual stream, all sums and the logits stay 32-bit.  Its distance from the exact run measures
    what 16-bit storage alone costs on a given model; the tests size the bfloat16 budget with it."""
    h = embed(ids, w["model.embed_tokens.weight"], cfg["hidden_size"])
    if schedule is None:
        schedule = [(i, None) for i in range(cfg["num_hidden_layers"])]
    kvs = {}
    for e, (layer, cache_of) in enumerate(schedule):
        h, kv = decoder_layer(h, w, layer, cfg, None if cache_of is None else kvs[cache_of], rnd)
        if cache_of is None:
            kvs[e] = kv
    return head(h, w, cfg, rnd)


# ----------------------------------------------------------------------------
# Choosing tokens
# ----------------------------------------------------------------------------
def greedy(logits: torch.Tensor) -> int:
    """The largest logit, the first one on a tie (runtime/src/lib.rs:1376-1380)."""
    best, arg = -float("inf"), 0
    for i, v in enumerate(logits.tolist()):
        if v > best:
            best, arg = v, i
    return arg


def repetition_penalty(logits: torch.Tensor, recent: Sequence[int], penalty: float) -> torch.Tensor:
    """Each distinct recent id once: logit > 0 ? logit / penalty : logit * penalty
    (runtime/src/bin/serve.rs:285-294)."""
    out = logits.clone()
    if penalty <= 1.0:
        return out
    for t in set(int(x) for x in recent if x >= 0):
        out[t] = out[t] / penalty if out[t] > 0 else out[t] * penalty
    return out


def nucleus(logits: torch.Tensor, temperature: float, top_p: float) -> torch.Tensor:
    """Probabilities after temperature and nucleus truncation, in float64, renormalised over the
    kept set: the smallest set of most probable tokens whose mass reaches top_p
    (runtime/src/bin/serve.rs:49-62, without its cut to the 256 largest logits)."""
    z = (logits.double() - logits.double().max()) / temperature
    p = z.exp()
    p = p / p.sum()
    if top_p >= 1.0:
        return p
    order = torch.argsort(p, descending=True, stable=True)
    cum = torch.cumsum(p[order], 0)
    keep_n = int((cum < top_p).sum().item()) + 1
    kept = torch.zeros_like(p)
    kept[order[:keep_n]] = p[order[:keep_n]]
    return kept / kept.sum()


def generate_greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], n_new: int,
                    stop_ids: Sequence[int] = ()) -> List[int]:
    """Greedy continuation by re-running the whole sequence for each new token
    (runtime/src/bin/gemma_run.rs:12-15); a stop id ends it and is not emitted
    (runtime/src/bin/serve.rs:347-350)."""
    ids = list(prompt)
    out: List[int] = []
    for _ in range(n_new):
        nxt = greedy(forward(cfg, w, ids)[-1])
        if nxt in stop_ids:
            break
        out.append(nxt)
        ids.append(nxt)
    return out
