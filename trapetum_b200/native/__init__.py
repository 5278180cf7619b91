"""The native host seen from Python: a thin ctypes binding over ``libtrapetum_b200.so``.

The library (C++, ``native/*.hpp``, C interface in ``native/trapetum_b200.h``) holds the whole path from a model
folder to tokens: the spec turned into parts, weights by name, the paged cache, the step function with its CUDA
graphs, the generation loop and sampling, all over the kernel libraries of ``csrc/``.  The reference's entry is of
the same kind: a compiled library with a C interface (runtime/include/trapetum.h:17-29, runtime/src/ffi.rs:27-124)
and a binary over it (runtime/src/bin/gemma_run.rs).  Here configuration and the registry of architectures stay in
Python, which hands the model's spec over as JSON; a model whose parts all have native classes runs without Python
in its steps.  Parts written in Python (see ``trapetum_b200.parts``) run on the Python host instead.

    from trapetum_b200 import native
    model = native.load_model("folder", "bfloat16")
    engine = native.Engine(model, max_tokens=8192)
    slots = engine.start(2)
    logits = engine.step(slots, [[5, 17, 3], [9]], want=[[2], [0]])        # a torch tensor on the device
    out = native.generate(model, [[2, 651, 6037]], max_tokens=24)
"""
from __future__ import annotations

import ctypes
import json
from ctypes import POINTER, byref, c_char_p, c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Callable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.slots import CacheError, CacheFull
from ..config.base import load_config, spec_to_json
from ..csrc import build
from ..csrc.ops import KernelError
from ..engine.step import StepError

_lib = None


class _Sampling(ctypes.Structure):
    _fields_ = [("temperature", c_float), ("top_p", c_float), ("repetition_penalty", c_float), ("max_tokens", c_int),
                ("seed", c_ulonglong)]


_ON_TOKEN = ctypes.CFUNCTYPE(c_int, c_int, c_int, c_void_p)


def lib():
    """The loaded library (built at first use, like the kernels; no fallback)."""
    global _lib
    if _lib is None:
        path = build.build_native()
        L = ctypes.CDLL(path)
        L.tb_last_error.restype = c_char_p
        L.tb_kernel_errors.restype = c_char_p
        for name in ("tb_model_load", "tb_model_random", "tb_engine_new"):
            getattr(L, name).restype = c_void_p
        for name in ("tb_cache_max_tokens", "tb_cache_length", "tb_kernel_launches", "tb_last_h2d_bytes"):
            getattr(L, name).restype = c_longlong
        L.tb_model_free.argtypes = [c_void_p]
        L.tb_engine_free.argtypes = [c_void_p]
        L.tb_model_free.restype = None
        L.tb_engine_free.restype = None
        L.tb_set_kernel_dir(build._build_dir().encode())
        _lib = L
    return _lib


# Handles whose Python objects are gone.  Freeing device memory is not allowed while some stream of the process
# captures a graph (the Python host captures with Python code running, so the collector may run in the middle of
# it): objects only put their handle here, and it is freed at the next native call that finds no capture under way.
_graveyard: list = []


def _reap() -> None:
    if not _graveyard or _lib is None:
        return
    if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
        return
    while _graveyard:
        kind, h = _graveyard.pop(0)
        (_lib.tb_engine_free if kind == "engine" else _lib.tb_model_free)(c_void_p(h))


def _raise(status: int, what: str):
    msg = lib().tb_last_error().decode()
    if status == 2:
        raise StepError(msg)
    if status == 3:
        raise CacheFull(msg)
    if "pool:" in msg or "is not held" in msg:
        raise CacheError(msg)
    raise KernelError(f"{what}: {msg}")


def _ok(status: int, what: str) -> None:
    if status != 0:
        _raise(status, what)


def _ints(values) -> "ctypes.Array":
    a = np.ascontiguousarray(values, dtype=np.int32)
    return a.ctypes.data_as(POINTER(c_int)), a


def _rope_tables(spec_json: str) -> str:
    """Put the table of inverse frequencies, as the Python host makes it, into every rope part of a spec, so that
    both hosts of a process rotate by the same bits."""
    def walk(v):
        if isinstance(v, dict):
            if v.get("kind") == "rope" and isinstance(v.get("params"), dict):
                p = v["params"]
                rd = int(p.get("rotary_dim", p["head_dim"]))
                idx = torch.arange(0, rd, 2, dtype=torch.float32)
                p["inv_freq"] = (1.0 / (torch.tensor(float(p["theta"]), dtype=torch.float32) ** (idx / rd))).tolist()
            for x in v.values():
                walk(x)
        elif isinstance(v, list):
            for x in v:
                walk(x)
    d = json.loads(spec_json)
    walk(d)
    return json.dumps(d)


class Model:
    """A model held by the native host."""

    def __init__(self, handle, spec, dtype: str, device: int):
        self._h = handle
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device("cuda", device)
        self.vocab_size = lib().tb_model_vocab(c_void_p(handle))

    def __del__(self):
        if getattr(self, "_h", None) and _graveyard is not None:         # (None while the interpreter shuts down)
            _graveyard.append(("model", self._h))
            self._h = None


def _device_index(device) -> int:
    dev = torch.device(device)
    if dev.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("trapetum_b200 computes on a CUDA device only (no CPU path); got device " + str(device))
    return dev.index or 0


def _dtype_name(dtype) -> str:
    from ..engine.model import parse_dtype
    return "float32" if parse_dtype(dtype) == torch.float32 else "bfloat16"


def _prepare(spec) -> str:
    import trapetum_b200.models  # noqa: F401  (registers the architectures)
    L = lib()
    text = _rope_tables(spec_to_json(spec))
    if not L.tb_spec_is_native(text.encode()):
        raise NotImplementedError(L.tb_last_error().decode() + "; this model runs on the Python host")
    return text


def is_native(spec) -> bool:
    """Whether every part of a spec has a native class."""
    try:
        return bool(lib().tb_spec_is_native(spec_to_json(spec).encode()))
    except Exception:
        return False


def _kernel_files(spec, dtype) -> None:
    """Build the kernel libraries the model's parts launch (the Python parts know which)."""
    from ..engine.model import Model as PyModel
    from ..engine.model import parse_dtype
    from ..parts import Runtime
    try:
        names = tuple(PyModel(spec, Runtime(parse_dtype(dtype), torch.device("cpu"))).kernel_files())
    except Exception:
        names = tuple(build.SOURCES)          # a part that only the native host knows (a plugin): build them all
    build.require(names + ("random_init", "activation", "rope_kv", "norm"))
    build.write_manifest()


def load_model(folder: str, dtype="bfloat16", device="cuda:0", fp16: str = "widen") -> Model:
    idx = _device_index(device)
    _reap()
    _, spec = load_config(folder)
    text = _prepare(spec)
    _kernel_files(spec, dtype)
    h = lib().tb_model_load(str(folder).encode(), text.encode(), _dtype_name(dtype).encode(), c_int(idx), fp16.encode())
    if not h:
        raise RuntimeError(lib().tb_last_error().decode())
    return Model(h, spec, _dtype_name(dtype), idx)


def random_model(config, seed: int = 0, std: float = 0.02, norm_std: float = 0.1, dtype="bfloat16", device="cuda:0") -> Model:
    idx = _device_index(device)
    _reap()
    _, spec = load_config(config)
    text = _prepare(spec)
    _kernel_files(spec, dtype)
    h = lib().tb_model_random(text.encode(), c_ulonglong(int(seed) & (2 ** 64 - 1)), c_float(std), c_float(norm_std),
                              _dtype_name(dtype).encode(), c_int(idx))
    if not h:
        raise RuntimeError(lib().tb_last_error().decode())
    return Model(h, spec, _dtype_name(dtype), idx)


class _DeviceArray:
    """A window onto device memory that the native host owns, for ``torch.as_tensor``."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 3,
                                         "strides": None}


def _tensor(ptr: int, shape, dtype: torch.dtype, device) -> torch.Tensor:
    if dtype == torch.bfloat16:
        return torch.as_tensor(_DeviceArray(ptr, shape, "<u2"), device=device).view(torch.int16).view(torch.bfloat16)
    typestr = {torch.float32: "<f4", torch.int32: "<i4"}[dtype]
    return torch.as_tensor(_DeviceArray(ptr, shape, typestr), device=device)


class _Group:
    def __init__(self, k, v, ring_rows, lines):
        self.k, self.v, self.ring_rows, self.lines = k, v, ring_rows, lines


class _CacheView:
    """What tests and tools look at in the native cache: the pools as tensors, lengths, pages, invariants."""

    def __init__(self, engine: "Engine"):
        self._e = engine
        L, h = lib(), c_void_p(engine._h)
        self.max_slots = L.tb_cache_max_slots(h)
        self.max_tokens = int(L.tb_cache_max_tokens(h))
        self.groups: List[_Group] = []
        for gi in range(L.tb_cache_groups(h)):
            k, v = c_void_p(), c_void_p()
            lines, pages, nkv, hd, ring, code = (c_int() for _ in range(6))
            _ok(L.tb_cache_group_info(h, gi, byref(k), byref(v), byref(lines), byref(pages), byref(nkv), byref(hd), byref(ring),
                                      byref(code)), "cache")
            dt = torch.float32 if code.value == 0 else torch.bfloat16
            shape = (lines.value, pages.value, nkv.value, 64, hd.value)
            self.groups.append(_Group(_tensor(k.value, shape, dt, engine.device), _tensor(v.value, shape, dt, engine.device),
                                      ring.value, lines.value))

    def length(self, slot: int) -> int:
        n = int(lib().tb_cache_length(c_void_p(self._e._h), c_int(slot)))
        if n < 0:
            raise CacheError(f"slot {slot} is not held by any sequence")
        return n

    def pages(self, slot: int, group: int) -> List[int]:
        buf = (c_int * 4096)()
        n = lib().tb_cache_pages(c_void_p(self._e._h), c_int(slot), c_int(group), buf, c_int(4096))
        if n < 0:
            raise CacheError(lib().tb_last_error().decode())
        return list(buf[:n])

    def live_slots(self) -> List[int]:
        buf = (c_int * 4096)()
        n = lib().tb_cache_live(c_void_p(self._e._h), buf, c_int(4096))
        return list(buf[:n])

    def check(self) -> None:
        if lib().tb_cache_check(c_void_p(self._e._h)) != 0:
            raise CacheError(lib().tb_last_error().decode())

    def grow(self, growth) -> None:
        slots, ka = _ints(list(growth.keys()))
        g, kb = _ints(list(growth.values()))
        _ok(lib().tb_cache_grow(c_void_p(self._e._h), slots, g, c_int(len(growth))), "cache")


class Engine:
    """The native engine: a model, its cache, the step function."""

    def __init__(self, model: Model, max_tokens: int, max_slots: Optional[int] = None, use_graphs: bool = True):
        _reap()
        self.model = model
        self.device = model.device
        self.vocab_size = model.vocab_size
        h = lib().tb_engine_new(c_void_p(model._h), c_longlong(int(max_tokens)), c_int(max_slots or 0), c_int(1 if use_graphs else 0))
        if not h:
            raise RuntimeError(lib().tb_last_error().decode())
        self._h = h
        self.cache = _CacheView(self)

    def __del__(self):
        if getattr(self, "_h", None):
            if _graveyard is not None:                        # (None while the interpreter shuts down)
                _graveyard.insert(0, ("engine", self._h))      # engines go before their models
            self._h = None

    def _on_torch_stream(self) -> None:
        from ..csrc.ops import _stream
        lib().tb_engine_set_stream(c_void_p(self._h), _stream())

    def start(self, n: int) -> List[int]:
        self._on_torch_stream()
        out = (c_int * max(1, n))()
        _ok(lib().tb_start(c_void_p(self._h), c_int(n), out), "start")
        return list(out[:n])

    def release(self, slots: Sequence[int]) -> None:
        p, keep = _ints(list(slots))
        _ok(lib().tb_release(c_void_p(self._h), p, c_int(len(slots))), "release")

    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]], want: Optional[Sequence[Sequence[int]]] = None,
             borrow: bool = False, greedy: bool = False) -> Optional[torch.Tensor]:
        """As :meth:`trapetum_b200.engine.Engine.step`: float32 logits [wanted, vocab] on the device (or, with
        ``greedy``, int32 ids), None if nothing is wanted.  ``borrow=True``: the result may alias memory that the
        next step overwrites."""
        self._on_torch_stream()
        if len(tokens) != len(slots):
            raise StepError(f"{len(slots)} slots but {len(tokens)} token lists")
        sl, k0 = _ints(list(slots))
        flat, k1 = _ints([int(t) for seq in tokens for t in seq])
        n_new, k2 = _ints([len(seq) for seq in tokens])
        if want is not None:
            if len(want) != len(slots):
                raise StepError(f"{len(slots)} sequences but {len(want)} 'want' lists")
            w, k3 = _ints([int(j) for seq in want for j in seq])
            nw, k4 = _ints([len(seq) for seq in want])
        else:
            w, nw = None, None
        logits, ids, rows = c_void_p(), c_void_p(), c_int()
        _ok(lib().tb_step(c_void_p(self._h), sl, c_int(len(slots)), flat, n_new, w, nw, c_int(1 if greedy else 0), byref(logits),
                          byref(ids), byref(rows)), "step")
        if rows.value == 0:
            return None
        if greedy:
            t = _tensor(ids.value, (rows.value,), torch.int32, self.device)
        else:
            t = _tensor(logits.value, (rows.value, self.vocab_size), torch.float32, self.device)
        return t if borrow else t.clone()

    def step_tokens(self, slots: Sequence[int], tokens: Sequence[Sequence[int]]) -> List[int]:
        """One step of a generation loop: host token lists in, each sequence's greedy next token out (host ints)."""
        self._on_torch_stream()
        if len(tokens) != len(slots):
            raise StepError(f"{len(slots)} slots but {len(tokens)} token lists")
        n = len(slots)
        sl, k0 = _ints(list(slots))
        flat, k1 = _ints([int(t) for seq in tokens for t in seq])
        n_new, k2 = _ints([len(seq) for seq in tokens])
        out = (c_int * max(1, n))()
        _ok(lib().tb_step_tokens(c_void_p(self._h), sl, c_int(n), flat, n_new, out), "step")
        return list(out[:n])

    def check_kernels(self) -> None:
        err = lib().tb_kernel_errors(c_void_p(self._h)).decode()
        if err:
            raise KernelError(f"a kernel gave up waiting and its results are not valid: {err}")

    @property
    def graphs_captured(self) -> int:
        return lib().tb_graphs_captured(c_void_p(self._h))

    @property
    def last_h2d_bytes(self) -> int:
        return int(lib().tb_last_h2d_bytes(c_void_p(self._h)))


def set_decode_partition(mode: Optional[str]) -> Optional[str]:
    """As ``csrc.ops.set_decode_partition``, for the native host: "split", "stream" or None (chosen per launch)."""
    codes = {None: 0, "split": 1, "stream": 2}
    if mode not in codes:
        raise ValueError(f"decode partition {mode!r}: None, 'split' or 'stream'")
    was = int(lib().tb_set_decode_partition(ctypes.c_int(codes[mode])))
    return {0: None, 1: "split", 2: "stream"}[was]


def launches() -> int:
    """Kernels launched by the native host in this process (graph replays count their kernels)."""
    return int(lib().tb_kernel_launches())


def generate(model_or_engine, prompts: Sequence[Sequence[int]], max_tokens: int = 256, temperature: float = 0.0,
             top_p: float = 0.95, repetition_penalty: float = 1.0, seed: int = 0, stop_ids: Optional[Sequence[int]] = None,
             max_batch: int = 64, cache_tokens: Optional[int] = None,
             on_token: Optional[Callable[[int, int], None]] = None) -> List[List[int]]:
    """As :func:`trapetum_b200.generate`, with the whole loop (batches, steps, sampling, stop decisions) in the
    native host; ``on_token(request, id)`` is called from inside it for each emitted token, like the reference's
    streaming callback (runtime/include/trapetum.h:20-27)."""
    from ..cache import pages_for
    prompts = [list(map(int, p)) for p in prompts]
    if isinstance(model_or_engine, Engine):
        engine = model_or_engine
    else:
        model = model_or_engine
        if cache_tokens is None:
            by_need = sorted((pages_for(min(len(p) + max_tokens, model.spec.max_positions)) for p in prompts), reverse=True)
            cache_tokens = max(1, sum(by_need[:max_batch])) * 64
        engine = Engine(model, cache_tokens, max_slots=max_batch)
    if not prompts or max_tokens == 0:
        return [[] for _ in prompts]
    engine._on_torch_stream()
    params = _Sampling(temperature, top_p, repetition_penalty, max_tokens, int(seed) & (2 ** 64 - 1))
    flat, k0 = _ints([t for p in prompts for t in p])
    lens, k1 = _ints([len(p) for p in prompts])
    if stop_ids is None:
        stops, n_stop, k2 = None, -1, None
    else:
        stops, k2 = _ints(list(stop_ids) or [0])
        n_stop = len(stop_ids)
    failure = []

    def trampoline(request, token, _user):
        try:
            on_token(request, token)
            return 0
        except BaseException as e:          # an exception must not cross the C frames: stop the loop, raise after it
            failure.append(e)
            return 1
    cb = _ON_TOKEN(trampoline) if on_token is not None else ctypes.cast(None, _ON_TOKEN)
    cap = max(1, max_tokens)
    out = np.zeros((len(prompts), cap), dtype=np.int32)
    out_lens = np.zeros(len(prompts), dtype=np.int32)
    status = lib().tb_generate(c_void_p(engine._h), flat, lens, c_int(len(prompts)), byref(params), stops, c_int(n_stop),
                               c_int(max_batch), cb, None, out.ctypes.data_as(POINTER(c_int)),
                               out_lens.ctypes.data_as(POINTER(c_int)), c_int(cap))
    if failure:
        raise failure[0]
    if status not in (0, 4):
        _raise(status, "generate")
    return [out[i, :out_lens[i]].tolist() for i in range(len(prompts))]
