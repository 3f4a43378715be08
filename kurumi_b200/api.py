"""ctypes binding of the kurumi C ABI (include/kurumi.h, include/kurumi_cuda.h).

The classes mirror the reference's Rust surface so tests read like the reference's own:
``Graph`` has the builder methods of kurumi_core/src/graph/ops/** (same names, same argument
order, an ``Error`` on a failed build instead of ``Err``), ``Backend.eval(g, node)`` /
``eval_with`` / ``eval_many_with`` are the trait methods of kurumi_core/src/backend.rs:14-31.

``Library(path)`` binds any shared library that exports the ABI, so the same Python code drives
the CUDA library and, in the tests, the CPU oracle.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Iterable, Sequence

import numpy as np

KU_ERR = 0xFFFFFFFF
KU_CPU, KU_METAL, KU_CUDA = 0, 1, 2

DTYPES = ["BOOL", "U8", "U16", "U32", "U64", "I8", "I16", "I32", "I64", "F8E4M3", "F8E5M2", "F16", "BF16", "F32",
          "F64", "C64", "C128"]
(BOOL, U8, U16, U32, U64, I8, I16, I32, I64, F8E4M3, F8E5M2, F16, BF16, F32, F64, C64, C128) = range(17)
WIDTH = [1, 1, 2, 4, 8, 1, 2, 4, 8, 1, 1, 2, 2, 4, 8, 8, 16]


def dtype_width(dtype: int) -> int:
    """Bytes per element of a KuDType index."""
    return WIDTH[dtype]

# numpy carrier per dtype: narrow floats travel as their raw bit patterns
_NP = {BOOL: np.uint8, U8: np.uint8, U16: np.uint16, U32: np.uint32, U64: np.uint64, I8: np.int8, I16: np.int16,
       I32: np.int32, I64: np.int64, F8E4M3: np.uint8, F8E5M2: np.uint8, F16: np.float16, BF16: np.uint16,
       F32: np.float32, F64: np.float64}


class Error(RuntimeError):
    pass


def _sz(seq: Iterable[int]):
    seq = list(seq)
    return (C.c_size_t * max(len(seq), 1))(*seq), len(seq)


class Library:
    """One loaded shared library exporting the kurumi C ABI."""

    def __init__(self, path: str):
        if not os.path.exists(path):
            raise Error(f"{path} is missing: build it first (python -c 'import __graft_entry__ as g; g.build()')")
        self.path = path
        self.lib = C.CDLL(path)
        L = self.lib
        L.ku_last_error.restype = C.c_char_p
        for name in ("ku_graph_new", "ku_backend_new", "ku_eval", "ku_eval_with", "ku_feeds_new", "ku_tensor_f32",
                     "ku_tensor_new"):
            getattr(L, name).restype = C.c_void_p
        for name in ("ku_tensor_rank", "ku_tensor_len", "ku_tensor_nbytes", "ku_node_rank", "ku_node_count", "ku_dump"):
            getattr(L, name).restype = C.c_size_t
        for name in ("ku_node_dtype", "ku_tensor_dtype"):
            getattr(L, name).restype = C.c_uint32
        L.ku_tensor_data_f32.restype = C.c_ssize_t
        L.ku_eval_many.restype = C.c_int32
        self._node_fns = {}

    def last_error(self) -> str:
        e = self.lib.ku_last_error()
        return e.decode() if e else ""

    def node_fn(self, name: str):
        f = self._node_fns.get(name)
        if f is None:
            f = getattr(self.lib, name)
            f.restype = C.c_uint32
            self._node_fns[name] = f
        return f

    def has(self, name: str) -> bool:
        return hasattr(self.lib, name)


class Tensor:
    """Host tensor handle (the reference's TensorVal)."""

    def __init__(self, lib: Library, handle: int):
        if not handle:
            raise Error(lib.last_error() or "null tensor")
        self.lib, self.h = lib, C.c_void_p(handle)

    @staticmethod
    def from_numpy(lib: Library, arr: np.ndarray, dtype: int | None = None) -> "Tensor":
        if dtype is None:
            dtype = {np.dtype(np.float32): F32, np.dtype(np.float64): F64, np.dtype(np.int32): I32,
                     np.dtype(np.int64): I64, np.dtype(np.uint8): U8, np.dtype(np.bool_): BOOL,
                     np.dtype(np.float16): F16, np.dtype(np.int8): I8, np.dtype(np.int16): I16,
                     np.dtype(np.uint16): U16, np.dtype(np.uint32): U32, np.dtype(np.uint64): U64}[arr.dtype]
        a = np.ascontiguousarray(arr).reshape(np.shape(arr))   # ascontiguousarray promotes 0-d to 1-d
        shape, rank = _sz(a.shape)
        h = lib.lib.ku_tensor_new(C.c_uint32(dtype), a.ctypes.data_as(C.c_void_p), C.c_size_t(a.nbytes), shape,
                                  C.c_size_t(rank))
        return Tensor(lib, h)

    @property
    def dtype(self) -> int:
        return int(self.lib.lib.ku_tensor_dtype(self.h))

    @property
    def shape(self) -> tuple:
        r = self.lib.lib.ku_tensor_rank(self.h)
        out = (C.c_size_t * max(r, 1))()
        self.lib.lib.ku_tensor_shape(self.h, out)
        return tuple(out[i] for i in range(r))

    @property
    def nbytes(self) -> int:
        return int(self.lib.lib.ku_tensor_nbytes(self.h))

    def copy_into(self, ptr: int):
        """ku_tensor_bytes into a caller-owned buffer of at least nbytes."""
        self.lib.lib.ku_tensor_bytes(self.h, C.c_void_p(ptr))

    def free(self):
        """Give the storage back now instead of at garbage collection."""
        if self.h:
            self.lib.lib.ku_tensor_free(self.h)
            self.h = None

    def numpy(self) -> np.ndarray:
        """Values as numpy; bf16 / fp8 come back as raw bit patterns (uint16 / uint8)."""
        n = self.lib.lib.ku_tensor_nbytes(self.h)
        buf = np.empty(n, dtype=np.uint8)
        if n:
            self.lib.lib.ku_tensor_bytes(self.h, buf.ctypes.data_as(C.c_void_p))
        return buf.view(_NP[self.dtype]).reshape(self.shape)

    def __del__(self):
        try:
            if self.h:
                self.lib.lib.ku_tensor_free(self.h)
        except Exception:
            pass


class Feeds:
    def __init__(self, lib: Library):
        self.lib, self.h = lib, C.c_void_p(lib.lib.ku_feeds_new())
        self._keep = []

    def set(self, node: int, value, dtype: int | None = None):
        t = value if isinstance(value, Tensor) else Tensor.from_numpy(self.lib, value, dtype)
        self._keep.append(t)
        self.lib.lib.ku_feeds_set(self.h, C.c_uint32(node), t.h)
        return self

    def __del__(self):
        try:
            self.lib.lib.ku_feeds_free(self.h)
        except Exception:
            pass


class Graph:
    """Graph builder: every method returns a node id or raises Error with ku_last_error()."""

    def __init__(self, lib: Library, handle=None):
        self.lib, self.h = lib, C.c_void_p(handle if handle is not None else lib.lib.ku_graph_new())

    def __del__(self):
        try:
            self.lib.lib.ku_graph_free(self.h)
        except Exception:
            pass

    def serialize(self, outputs: Sequence[int], inputs: Sequence[tuple] = (), reachable: bool = False) -> bytes:
        """The graph as a KGPH v2 blob; `inputs` are (node, role, name) with role 0 = weight, 1 = runtime feed."""
        fn = self.lib.lib.ku_graph_serialize_reachable if reachable else self.lib.lib.ku_graph_serialize
        fn.restype = C.c_size_t
        outs = (C.c_uint32 * max(len(outputs), 1))(*outputs)
        nodes = (C.c_uint32 * max(len(inputs), 1))(*[i[0] for i in inputs])
        roles = (C.c_uint8 * max(len(inputs), 1))(*[i[1] for i in inputs])
        names = (C.c_char_p * max(len(inputs), 1))(*[i[2].encode() for i in inputs])
        args = (self.h, outs, C.c_size_t(len(outputs)), nodes, roles, names, C.c_size_t(len(inputs)))
        n = fn(*args, None, C.c_size_t(0))
        if n == 0:
            raise Error(self.lib.last_error())
        buf = (C.c_uint8 * n)()
        fn(*args, buf, C.c_size_t(n))
        return bytes(buf)

    def serialize_multi(self, entries: Sequence[tuple]) -> bytes:
        """Several named entries (name, outputs, inputs) over one arena, pruned to the union of their cones."""
        fn = self.lib.lib.ku_graph_serialize_multi
        fn.restype = C.c_size_t
        names = (C.c_char_p * len(entries))(*[e[0].encode() for e in entries])
        outs = [o for e in entries for o in e[1]]
        ins = [i for e in entries for i in e[2]]
        oc = (C.c_uint32 * len(entries))(*[len(e[1]) for e in entries])
        ic = (C.c_uint32 * len(entries))(*[len(e[2]) for e in entries])
        oa = (C.c_uint32 * max(len(outs), 1))(*outs)
        na = (C.c_uint32 * max(len(ins), 1))(*[i[0] for i in ins])
        ra = (C.c_uint8 * max(len(ins), 1))(*[i[1] for i in ins])
        sa = (C.c_char_p * max(len(ins), 1))(*[i[2].encode() for i in ins])
        args = (self.h, C.c_size_t(len(entries)), names, oc, oa, ic, na, ra, sa)
        n = fn(*args, None, C.c_size_t(0))
        if n == 0:
            raise Error(self.lib.last_error())
        buf = (C.c_uint8 * n)()
        fn(*args, buf, C.c_size_t(n))
        return bytes(buf)

    def _n(self, name: str, *args) -> int:
        r = self.lib.node_fn(name)(self.h, *args)
        if r == KU_ERR:
            raise Error(self.lib.last_error())
        return r

    # leaves
    def input(self, shape: Sequence[int], dtype: int) -> int:
        s, r = _sz(shape)
        return self._n("ku_input", s, C.c_size_t(r), C.c_uint32(dtype))

    def constant(self, arr: np.ndarray, dtype: int | None = None) -> int:
        a = np.ascontiguousarray(arr).reshape(np.shape(arr))
        if dtype is None:
            dtype = Tensor.from_numpy(self.lib, np.zeros(1, a.dtype)).dtype
        s, r = _sz(a.shape)
        return self._n("ku_constant", C.c_uint32(dtype), a.ctypes.data_as(C.c_void_p), C.c_size_t(a.nbytes), s, C.c_size_t(r))

    def gather(self, x: int, idx: int, axis: int) -> int:
        return self._n("ku_gather", C.c_uint32(x), C.c_uint32(idx), C.c_size_t(axis))

    def gather_along(self, x: int, idx: int, axis: int) -> int:
        return self._n("ku_gather_along", C.c_uint32(x), C.c_uint32(idx), C.c_size_t(axis))

    def scatter(self, operand: int, idx: int, updates: int, axis: int, combine: int = 0) -> int:
        return self._n("ku_scatter", C.c_uint32(operand), C.c_uint32(idx), C.c_uint32(updates), C.c_size_t(axis), C.c_uint32(combine))

    def scatter_along(self, operand: int, idx: int, updates: int, axis: int, combine: int = 0) -> int:
        return self._n("ku_scatter_along", C.c_uint32(operand), C.c_uint32(idx), C.c_uint32(updates), C.c_size_t(axis), C.c_uint32(combine))

    def argsort(self, x: int, axis: int, descending: bool = False) -> int:
        return self._n("ku_argsort", C.c_uint32(x), C.c_size_t(axis), C.c_uint32(1 if descending else 0))

    def sort(self, x: int, axis: int, descending: bool = False) -> int:
        return self._n("ku_sort", C.c_uint32(x), C.c_size_t(axis), C.c_uint32(1 if descending else 0))

    def argmax(self, x: int, axis: int) -> int:
        return self._n("ku_argmax", C.c_uint32(x), C.c_size_t(axis))

    def argmin(self, x: int, axis: int) -> int:
        return self._n("ku_argmin", C.c_uint32(x), C.c_size_t(axis))

    def quant_matmul(self, act: int, qweight: int, scales: int, mins: int | None, bits: int, group_size: int) -> int:
        """act [M, K] x dequant(qweight [N, K*bits/8] U8, scales / mins [N, K/group_size] F16)^T -> [M, N]; mins None = symmetric."""
        return self._n("ku_quant_matmul", C.c_uint32(act), C.c_uint32(qweight), C.c_uint32(scales), C.c_uint32(KU_ERR if mins is None else mins),
                       C.c_uint8(bits), C.c_size_t(group_size))

    def scalar(self, like: int, v: float) -> int:
        return self._n("ku_scalar", C.c_uint32(like), C.c_float(v))

    def iota(self, shape, axis: int, dtype: int) -> int:
        s, r = _sz(shape)
        return self._n("ku_iota", s, C.c_size_t(r), C.c_size_t(axis), C.c_uint32(dtype))

    def rand_uniform(self, shape, seed: int) -> int:
        s, r = _sz(shape)
        return self._n("ku_rand_uniform", s, C.c_size_t(r), C.c_uint64(seed))

    def rand_uniform_keyed(self, shape, seed_node: int) -> int:
        s, r = _sz(shape)
        return self._n("ku_rand_uniform_keyed", s, C.c_size_t(r), C.c_uint32(seed_node))

    def randn(self, shape, seed: int) -> int:
        s, r = _sz(shape)
        return self._n("ku_randn", s, C.c_size_t(r), C.c_uint64(seed))

    def rand_range(self, shape, seed: int, lo: float, hi: float) -> int:
        s, r = _sz(shape)
        return self._n("ku_rand_range", s, C.c_size_t(r), C.c_uint64(seed), C.c_float(lo), C.c_float(hi))

    def cast(self, x: int, dtype: int) -> int:
        return self._n("ku_cast", C.c_uint32(x), C.c_uint32(dtype))

    def bitcast(self, x: int, dtype: int) -> int:
        return self._n("ku_bitcast", C.c_uint32(x), C.c_uint32(dtype))

    # axis ops
    def sum(self, x, axis): return self._n("ku_sum", C.c_uint32(x), C.c_size_t(axis))
    def prod(self, x, axis): return self._n("ku_prod", C.c_uint32(x), C.c_size_t(axis))
    def mean(self, x, axis): return self._n("ku_mean", C.c_uint32(x), C.c_size_t(axis))
    def reduce_max(self, x, axis): return self._n("ku_reduce_max", C.c_uint32(x), C.c_size_t(axis))
    def reduce_min(self, x, axis): return self._n("ku_reduce_min", C.c_uint32(x), C.c_size_t(axis))
    def softmax(self, x, axis): return self._n("ku_softmax", C.c_uint32(x), C.c_size_t(axis))
    def rmsnorm(self, x, axis, eps): return self._n("ku_rmsnorm", C.c_uint32(x), C.c_size_t(axis), C.c_float(eps))
    def clamp_min(self, x, v): return self._n("ku_clamp_min", C.c_uint32(x), C.c_float(v))

    # contraction
    def matmul(self, a, b): return self._n("ku_matmul", C.c_uint32(a), C.c_uint32(b))

    def dot_general(self, a, b, lc, rc, lb=(), rb=()):
        lc_, nlc = _sz(lc); rc_, nrc = _sz(rc); lb_, nlb = _sz(lb); rb_, nrb = _sz(rb)
        return self._n("ku_dot_general", C.c_uint32(a), C.c_uint32(b), lc_, C.c_size_t(nlc), rc_, C.c_size_t(nrc), lb_,
                       C.c_size_t(nlb), rb_, C.c_size_t(nrb))

    def where(self, c, a, b): return self._n("ku_where", C.c_uint32(c), C.c_uint32(a), C.c_uint32(b))
    select = where

    def sdpa(self, q, k, v, causal: bool):
        return self._n("ku_sdpa", C.c_uint32(q), C.c_uint32(k), C.c_uint32(v), C.c_uint32(1 if causal else 0))

    def sdpa_fused(self, q, k, v, causal: bool):
        return self._n("ku_sdpa_fused", C.c_uint32(q), C.c_uint32(k), C.c_uint32(v), C.c_uint32(1 if causal else 0))

    def sdpa_decomposed(self, q, k, v, causal: bool):
        return self._n("ku_sdpa_decomposed", C.c_uint32(q), C.c_uint32(k), C.c_uint32(v), C.c_uint32(1 if causal else 0))

    # movement
    def reshape(self, x, shape):
        s, r = _sz(shape); return self._n("ku_reshape", C.c_uint32(x), s, C.c_size_t(r))

    def expand(self, x, shape):
        s, r = _sz(shape); return self._n("ku_expand", C.c_uint32(x), s, C.c_size_t(r))

    def permute(self, x, perm):
        s, r = _sz(perm); return self._n("ku_permute", C.c_uint32(x), s, C.c_size_t(r))

    def transpose(self, x, i, j): return self._n("ku_transpose", C.c_uint32(x), C.c_size_t(i), C.c_size_t(j))

    def flip(self, x, axes):
        s, r = _sz(axes); return self._n("ku_flip", C.c_uint32(x), s, C.c_size_t(r))

    def slice(self, x, ranges):
        flat = [v for r in ranges for v in r]; s, _ = _sz(flat)
        return self._n("ku_slice", C.c_uint32(x), s, C.c_size_t(len(ranges)))

    def slice_step(self, x, ranges):
        flat = [v for r in ranges for v in r]; s, _ = _sz(flat)
        return self._n("ku_slice_step", C.c_uint32(x), s, C.c_size_t(len(ranges)))

    def pad(self, x, pads):
        flat = [v for r in pads for v in r]; s, _ = _sz(flat)
        return self._n("ku_pad", C.c_uint32(x), s, C.c_size_t(len(pads)))

    def broadcast_to(self, x, shape):
        s, r = _sz(shape); return self._n("ku_broadcast_to", C.c_uint32(x), s, C.c_size_t(r))

    # passes / inspection
    def amp(self, root): return self._n("ku_amp", C.c_uint32(root))

    def amp_to(self, root, dtype):
        name = "ku_cuda_amp_to" if self.lib.has("ku_cuda_amp_to") else "ko_amp_to"
        return self._n(name, C.c_uint32(root), C.c_uint32(dtype))

    def shape(self, node) -> tuple:
        r = self.lib.lib.ku_node_rank(self.h, C.c_uint32(node))
        if r == C.c_size_t(-1).value:
            raise Error(self.lib.last_error())
        out = (C.c_size_t * max(r, 1))()
        self.lib.lib.ku_node_shape(self.h, C.c_uint32(node), out)
        return tuple(out[i] for i in range(r))

    def dtype(self, node) -> int:
        d = self.lib.lib.ku_node_dtype(self.h, C.c_uint32(node))
        if d == KU_ERR:
            raise Error(self.lib.last_error())
        return d

    def node_count(self, root) -> int:
        return self.lib.lib.ku_node_count(self.h, C.c_uint32(root))

    def dump(self, root) -> str:
        n = self.lib.lib.ku_dump(self.h, C.c_uint32(root), None, C.c_size_t(0))
        buf = (C.c_uint8 * max(n, 1))()
        self.lib.lib.ku_dump(self.h, C.c_uint32(root), buf, C.c_size_t(n))
        return bytes(buf[:n]).decode()


def _bin(name):
    def f(self, a, b): return self._n("ku_" + name, C.c_uint32(a), C.c_uint32(b))
    return f


def _un(name):
    def f(self, x): return self._n("ku_" + name, C.c_uint32(x))
    return f


for _m in ("add", "sub", "mul", "div", "max", "min", "idiv", "and", "or", "xor", "shl", "shr", "lt", "eq", "le", "gt",
           "ge", "ne"):
    setattr(Graph, {"and": "and_", "or": "or_"}.get(_m, _m), _bin(_m))
Graph.cmp_lt, Graph.cmp_eq = Graph.lt, Graph.eq
for _m in ("neg", "recip", "sqrt", "square", "abs", "floor", "exp", "exp2", "ln", "log2", "sin", "cos", "relu", "gelu",
           "silu", "sigmoid", "tanh", "logical_not", "detach"):
    setattr(Graph, _m, _un(_m))


class Backend:
    """Evaluation seam (kurumi_core/src/backend.rs:14-31) over ku_backend_new / ku_eval*."""

    def __init__(self, lib: Library, kind: int):
        self.lib = lib
        h = lib.lib.ku_backend_new(C.c_uint32(kind))
        if not h:
            raise Error(lib.last_error() or f"backend kind {kind} unavailable")
        self.h = C.c_void_p(h)

    def __del__(self):
        try:
            self.lib.lib.ku_backend_free(self.h)
        except Exception:
            pass

    def eval(self, g: Graph, node: int) -> Tensor:
        return Tensor(self.lib, self.lib.lib.ku_eval(g.h, C.c_uint32(node), self.h))

    def eval_with(self, g: Graph, node: int, feeds: Feeds) -> Tensor:
        return Tensor(self.lib, self.lib.lib.ku_eval_with(g.h, C.c_uint32(node), self.h, feeds.h))

    def eval_many_with(self, g: Graph, nodes: Sequence[int], feeds: Feeds | None = None) -> list:
        feeds = feeds or Feeds(self.lib)
        ids = (C.c_uint32 * max(len(nodes), 1))(*nodes)
        out = (C.c_void_p * max(len(nodes), 1))()
        rc = self.lib.lib.ku_eval_many(g.h, ids, C.c_size_t(len(nodes)), self.h, feeds.h, out)
        if rc != 0:
            raise Error(self.lib.last_error())
        return [Tensor(self.lib, out[i]) for i in range(len(nodes))]


# ---- helpers for the narrow float formats (numpy has no bf16 / fp8) -------------------------------
def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (NaN kept quiet)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        r = np.where(nan, ((u >> 16) | 0x40).astype(np.uint16), r)
    return r


def e4m3_to_f32(bits: np.ndarray) -> np.ndarray:
    b = bits.astype(np.uint32)
    e, m, s = (b >> 3) & 0xF, b & 7, (b >> 7) & 1
    v = np.where(e == 0, m.astype(np.float64) * 2.0 ** -9, (8 + m).astype(np.float64) * np.exp2(e.astype(np.float64) - 10))
    v = np.where((b & 0x7F) == 0x7F, np.nan, v)
    return np.where(s == 1, -v, v).astype(np.float32)


# ---- device-resident surface of include/kurumi_cuda.h -------------------------------------------
class DevTensor:
    def __init__(self, backend: "CudaBackend", handle):
        if not handle:
            raise Error(backend.lib.last_error() or "null device tensor")
        self.backend, self.h = backend, C.c_void_p(handle)

    @property
    def nbytes(self) -> int:
        return self.backend.lib.lib.ku_cuda_dev_nbytes(self.h)

    @property
    def ptr(self) -> int:
        return self.backend.lib.lib.ku_cuda_dev_ptr(self.h) or 0

    @property
    def dtype(self) -> int:
        return int(self.backend.lib.lib.ku_cuda_dev_dtype(self.h))

    @property
    def shape(self) -> tuple:
        r = self.backend.lib.lib.ku_cuda_dev_rank(self.h)
        out = (C.c_size_t * max(r, 1))()
        self.backend.lib.lib.ku_cuda_dev_shape(self.h, out)
        return tuple(out[i] for i in range(r))

    def numpy(self) -> np.ndarray:
        buf = np.empty(self.nbytes, dtype=np.uint8)
        rc = self.backend.lib.lib.ku_cuda_download_bytes(self.backend.h, self.h, buf.ctypes.data_as(C.c_void_p), C.c_size_t(buf.nbytes))
        if rc != 0:
            raise Error(self.backend.lib.last_error())
        return buf.view(_NP[self.dtype]).reshape(self.shape)

    def download_into(self, ptr: int, cap: int):
        rc = self.backend.lib.lib.ku_cuda_download_bytes(self.backend.h, self.h, C.c_void_p(ptr), C.c_size_t(cap))
        if rc != 0:
            raise Error(self.backend.lib.last_error())

    def free(self):
        if self.h:
            self.backend.lib.lib.ku_cuda_dev_free(self.backend.h, self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class CudaBackend(Backend):
    """ku_cuda_backend_new(device) plus the device-resident calls."""

    def __init__(self, lib: Library, device: int = 0):
        self.lib = lib
        L = lib.lib
        for name in ("ku_cuda_backend_new", "ku_cuda_upload", "ku_cuda_upload_bytes", "ku_cuda_download", "ku_cuda_dev_ptr",
                     "ku_cuda_stream", "ku_cuda_dev_feeds_new"):
            getattr(L, name).restype = C.c_void_p
        for name in ("ku_cuda_dev_nbytes", "ku_cuda_dev_rank", "ku_cuda_stats", "ku_cuda_profile_take"):
            getattr(L, name).restype = C.c_size_t
        h = L.ku_cuda_backend_new(C.c_int32(device))
        if not h:
            raise Error(lib.last_error() or "CUDA backend unavailable")
        self.h = C.c_void_p(h)

    def upload(self, arr: np.ndarray, dtype: int | None = None) -> DevTensor:
        t = Tensor.from_numpy(self.lib, arr, dtype)
        return DevTensor(self, self.lib.lib.ku_cuda_upload(self.h, t.h))

    def upload_ptr(self, ptr: int, nbytes: int, shape, dtype: int) -> DevTensor:
        s, r = _sz(shape)
        return DevTensor(self, self.lib.lib.ku_cuda_upload_bytes(self.h, C.c_uint32(dtype), C.c_void_p(ptr), C.c_size_t(nbytes), s, C.c_size_t(r)))

    def prepare_device_step(self, g: Graph, nodes, dev_feeds: dict):
        """A repeated device-resident evaluation with the argument marshalling done once: returns step() -> DevTensor of
        the first root (ku_cuda_eval_device with a kept ku_cuda_dev_feeds handle) and close(). For loops whose evaluations
        take tens of microseconds, where rebuilding the feeds handle per call would be the larger part of a step."""
        L = self.lib.lib
        ids = (C.c_uint32 * max(len(nodes), 1))(*nodes)
        out = (C.c_void_p * max(len(nodes), 1))()
        n = C.c_size_t(len(nodes))
        df = C.c_void_p(L.ku_cuda_dev_feeds_new())
        for node, t in dev_feeds.items():
            L.ku_cuda_dev_feeds_set(df, C.c_uint32(node), t.h)
        fn, gh, bh = L.ku_cuda_eval_device, g.h, self.h

        def step():
            if fn(gh, ids, n, bh, None, df, out) != 0:
                raise Error(self.lib.last_error())
            return DevTensor(self, out[0])

        def close():
            L.ku_cuda_dev_feeds_free(df)
        return step, close

    def eval_device(self, g: Graph, nodes, feeds: Feeds | None = None, dev_feeds: dict | None = None) -> list:
        ids = (C.c_uint32 * max(len(nodes), 1))(*nodes)
        out = (C.c_void_p * max(len(nodes), 1))()
        df = C.c_void_p(self.lib.lib.ku_cuda_dev_feeds_new())
        try:
            for node, t in (dev_feeds or {}).items():
                self.lib.lib.ku_cuda_dev_feeds_set(df, C.c_uint32(node), t.h)
            rc = self.lib.lib.ku_cuda_eval_device(g.h, ids, C.c_size_t(len(nodes)), self.h, feeds.h if feeds else None, df, out)
        finally:
            self.lib.lib.ku_cuda_dev_feeds_free(df)
        if rc != 0:
            raise Error(self.lib.last_error())
        return [DevTensor(self, out[i]) for i in range(len(nodes))]

    def softmax_lines(self, x: DevTensor, bias, out: DevTensor, lines: int, length: int, ld: int, entry: str = "ku_cuda_softmax_lines_f32"):
        """out[i, j] = softmax_j(x[j * ld + i] + bias[j]) on device buffers (ku_cuda_softmax_lines_f32)."""
        fn = getattr(self.lib.lib, entry)
        fn.restype = C.c_int32
        args = [C.c_void_p(x.ptr), C.c_void_p(bias.ptr if bias is not None else None), C.c_void_p(out.ptr), C.c_size_t(lines), C.c_size_t(length), C.c_size_t(ld)]
        rc = fn(self.h, *args) if entry == "ku_cuda_softmax_lines_f32" else fn(*args, C.c_void_p(self.stream))
        if rc != 0:
            raise Error(self.lib.last_error())

    def sync(self):
        if self.lib.lib.ku_cuda_sync(self.h) != 0:
            raise Error(self.lib.last_error())

    def release_graph(self, g: Graph):
        self.lib.lib.ku_cuda_release_graph(self.h, g.h)

    def comm_unique_id(self) -> bytes:
        buf = (C.c_uint8 * 128)()
        if self.lib.lib.ku_cuda_comm_unique_id(buf) != 0:
            raise Error(self.lib.last_error())
        return bytes(buf)

    def comm_init(self, uid: bytes, rank: int, world: int):
        buf = (C.c_uint8 * 128)(*uid)
        if self.lib.lib.ku_cuda_comm_init(self.h, buf, C.c_int32(rank), C.c_int32(world)) != 0:
            raise Error(self.lib.last_error())

    def comm_free(self):
        self.lib.lib.ku_cuda_comm_free(self.h)

    def all_gather_rows(self, shard: "DevTensor") -> "DevTensor":
        self.lib.lib.ku_cuda_all_gather_rows.restype = C.c_void_p
        return DevTensor(self, self.lib.lib.ku_cuda_all_gather_rows(self.h, shard.h))

    @property
    def stream(self) -> int:
        return self.lib.lib.ku_cuda_stream(self.h) or 0

    def stats(self) -> dict:
        out = (C.c_uint64 * 7)()
        self.lib.lib.ku_cuda_stats(self.h, out, C.c_size_t(7))
        keys = ["launches", "nvrtc_compiles", "nvrtc_hits", "h2d_bytes", "d2h_bytes", "pool_allocs", "pool_hits"]
        return dict(zip(keys, [int(v) for v in out]))

    def profile(self, on: bool):
        self.lib.lib.ku_cuda_profile_enable(self.h, C.c_uint32(1 if on else 0))

    def take_profile(self) -> dict:
        buf = (C.c_uint8 * 65536)()
        n = self.lib.lib.ku_cuda_profile_take(self.h, buf, C.c_size_t(65536))
        res = {}
        for line in bytes(buf[:n]).decode().splitlines():
            name, launches, ms, nbytes, flops = line.split()
            res[name] = {"launches": int(launches), "ms": float(ms), "algo_bytes": float(nbytes), "flops": float(flops)}
        return res


class Plan:
    """ku_plan_compile / ku_plan_run / ku_plan_free: compile once, replay with new feeds."""

    def __init__(self, g: Graph, node: int):
        L = g.lib.lib
        L.ku_plan_compile.restype = C.c_void_p
        L.ku_plan_run.restype = C.c_void_p
        h = L.ku_plan_compile(g.h, C.c_uint32(node))
        if not h:
            raise Error(g.lib.last_error() or "ku_plan_compile failed")
        self.g, self.h = g, C.c_void_p(h)

    def run(self, feeds: Feeds, graph: Graph | None = None) -> Tensor:
        g = graph or self.g
        return Tensor(g.lib, g.lib.lib.ku_plan_run(self.h, g.h, feeds.h))

    def __del__(self):
        try:
            self.g.lib.lib.ku_plan_free(self.h)
        except Exception:
            pass


def row_split(g: Graph, root: int, parts: int):
    """(part graph, part root, [(original input node, part input node, axis or None)]) of core/split.h; raises Error
    with the reason when the evaluation does not separate by rows."""
    L = g.lib.lib
    L.ku_graph_row_split.restype = C.c_void_p
    cap = 256
    proot, n = C.c_uint32(0), C.c_size_t(0)
    orig, part, axes = (C.c_uint32 * cap)(), (C.c_uint32 * cap)(), (C.c_int32 * cap)()
    h = L.ku_graph_row_split(g.h, C.c_uint32(root), C.c_size_t(parts), C.byref(proot), orig, part, axes, C.c_size_t(cap), C.byref(n))
    if not h:
        raise Error(g.lib.last_error())
    return Graph(g.lib, h), int(proot.value), [(int(orig[i]), int(part[i]), None if axes[i] < 0 else int(axes[i])) for i in range(min(n.value, cap))]


def compile_check(lib: Library, g: Graph, nodes) -> list:
    """NVRTC-compile every kernel the evaluation needs (no GPU). Returns the kernel families."""
    lib.lib.ku_cuda_compile_check.restype = C.c_size_t
    ids = (C.c_uint32 * max(len(nodes), 1))(*nodes)
    buf = (C.c_uint8 * 16384)()
    n = lib.lib.ku_cuda_compile_check(g.h, ids, C.c_size_t(len(nodes)), buf, C.c_size_t(16384))
    if n == C.c_size_t(-1).value:
        raise Error(lib.last_error())
    return bytes(buf[:n]).decode().split()


def quantize(lib: Library, w: np.ndarray, bits: int, group_size: int, symmetric: bool):
    """Group-wise weight quantisation (ku_quantize): returns (packed u8 [rows, cols*bits/8], scales f16 [rows, cols/group], mins or None)."""
    w = np.ascontiguousarray(w, np.float32)
    rows, cols = w.shape
    if bits not in (2, 4, 8) or group_size <= 0 or cols % group_size:
        raise Error("quantize: bits must be 2, 4 or 8 and cols a multiple of group_size")
    packed = np.zeros((rows, cols * bits // 8), np.uint8)
    scales = np.zeros((rows, cols // group_size), np.float16)
    mins = None if symmetric else np.zeros((rows, cols // group_size), np.float16)
    lib.lib.ku_quantize.restype = None
    lib.lib.ku_quantize(w.ctypes.data_as(C.c_void_p), C.c_size_t(rows), C.c_size_t(cols), C.c_uint8(bits), C.c_size_t(group_size), C.c_uint32(1 if symmetric else 0),
                        packed.ctypes.data_as(C.c_void_p), scales.ctypes.data_as(C.c_void_p), None if mins is None else mins.ctypes.data_as(C.c_void_p))
    return packed, scales, mins


def deserialize(lib: Library, blob: bytes):
    """Rebuild a KGPH v2 blob: (Graph, [(entry name, outputs, [(node, role, name), ...]), ...]). Raises Error when malformed."""
    L = lib.lib
    L.ku_graph_deserialize.restype = C.c_void_p
    L.ku_runnable_take_graph.restype = C.c_void_p
    for name in ("ku_runnable_entry_count", "ku_runnable_entry_name", "ku_runnable_entry_output_count", "ku_runnable_entry_input_count",
                 "ku_runnable_entry_input_name"):
        getattr(L, name).restype = C.c_size_t
    for name in ("ku_runnable_entry_output", "ku_runnable_entry_input_node", "ku_runnable_entry_input_role"):
        getattr(L, name).restype = C.c_uint32
    buf = (C.c_uint8 * max(len(blob), 1)).from_buffer_copy(blob if blob else b"\0")
    h = L.ku_graph_deserialize(buf, C.c_size_t(len(blob)))
    if not h:
        raise Error(lib.last_error())
    h = C.c_void_p(h)
    try:
        def text(fn, *idx):
            n = fn(h, *idx, None, C.c_size_t(0))
            b = (C.c_uint8 * max(n, 1))()
            fn(h, *idx, b, C.c_size_t(n))
            return bytes(b[:n]).decode()
        entries = []
        for e in range(L.ku_runnable_entry_count(h)):
            ce = C.c_size_t(e)
            outs = [L.ku_runnable_entry_output(h, ce, C.c_size_t(j)) for j in range(L.ku_runnable_entry_output_count(h, ce))]
            ins = [(L.ku_runnable_entry_input_node(h, ce, C.c_size_t(j)), L.ku_runnable_entry_input_role(h, ce, C.c_size_t(j)),
                    text(L.ku_runnable_entry_input_name, ce, C.c_size_t(j))) for j in range(L.ku_runnable_entry_input_count(h, ce))]
            entries.append((text(L.ku_runnable_entry_name, ce), outs, ins))
        g = L.ku_runnable_take_graph(h)
        if not g:
            raise Error(lib.last_error())
        return Graph(lib, g), entries
    finally:
        L.ku_runnable_free(h)


def load_cuda_library() -> Library:
    from . import build
    return Library(build.LIB)
