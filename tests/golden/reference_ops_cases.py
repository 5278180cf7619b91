"""The small cases on which the reference's own CUDA operators and the plain implementation are compared.

Inputs are made here from fixed seeds (float16 values, as the reference's activations are), so that the
script that runs the reference on a GPU (make_reference_ops_golden.py) and the CPU test that checks the
plain implementation against the stored outputs use the same numbers without storing them.
"""
import torch

ATTN = [  # name, heads, kv heads, head_dim, keys, softcap (0: off); the reference scales by rsqrt(head_dim)
    ("attn_cap", 4, 2, 64, 77, 50.0),
    ("attn_nocap", 6, 1, 128, 200, 0.0),
    ("attn_sharp", 2, 2, 64, 300, 20.0),
]


def half(*shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.float16)


def inputs():
    """name -> dict of input tensors (float16 unless said otherwise) and plain numbers."""
    c = {}
    c["rmsnorm"] = {"x": half(200, seed=1, scale=3.0), "w": torch.randn(200, generator=torch.Generator().manual_seed(2)) * 0.1,
                    "eps": 1e-6}
    c["rope"] = {"x": half(3, 64, seed=3), "pos": 37, "theta": 10000.0}
    c["rope_far"] = {"x": half(2, 128, seed=4), "pos": 8000, "theta": 10000.0}
    for i, (name, nh, nkv, hd, n, cap) in enumerate(ATTN):
        # one key far back is made to stand out for head 0, so that a wrong row or a wrong cap shows
        q, k, v = half(nh, hd, seed=10 + i), half(n, nkv, hd, seed=20 + i), half(n, nkv, hd, seed=30 + i)
        k[n // 3, 0] = (q[0].float() * 0.6).to(torch.float16)
        c[name] = {"q": q, "k": k, "v": v, "cap": cap}
    c["gelu_mul"] = {"gate": torch.randn(300, generator=torch.Generator().manual_seed(5)) * 2.0,
                     "up": torch.randn(300, generator=torch.Generator().manual_seed(6))}
    c["resadd_h"] = {"h": half(100, seed=7, scale=4.0), "d": half(100, seed=8)}
    a = torch.randn(5000, generator=torch.Generator().manual_seed(9))
    a[[1234, 4321, 77]] = 9.5                       # a three-way tie at the top: the smallest index must win
    c["argmax"] = {"logits": a}
    return c
