"""The five benchmark graphs, recorded with the reference's own builders.

Each function takes a graph builder (kurumi_b200.api.Graph, of either library) and sizes, and
returns (root node, {input node: (shape, dtype, generator)}) where the generator is a graph whose
evaluation yields the seeded synthetic input: kurumi's own RNG decomposition
(kurumi_core/src/graph/ops/core/random.rs:28-49 over threefry2x32, kurumi_core/src/rng.rs:10-31),
so host and device agree bit for bit on integer work. Independent tensors of one config draw their
sub-seeds from Key::new(seed).split_n(k) (kurumi_core/src/rng.rs:51-53).
"""
from __future__ import annotations

import math

import numpy as np

from . import api


def _threefry(key: int, ctr: int) -> int:
    rot = [13, 15, 26, 6, 17, 29, 16, 24]
    M = 0xFFFFFFFF
    k0, k1 = key & M, (key >> 32) & M
    ks = [k0, k1, 0x1BD11BDA ^ k0 ^ k1]
    x0, x1 = ((ctr & M) + ks[0]) & M, (((ctr >> 32) & M) + ks[1]) & M
    for r in range(20):
        x0 = (x0 + x1) & M
        s = rot[r % 8]
        x1 = ((x1 << s) | (x1 >> (32 - s))) & M
        x1 ^= x0
        if r % 4 == 3:
            inj = r // 4 + 1
            x0 = (x0 + ks[inj % 3]) & M
            x1 = (x1 + ks[(inj + 1) % 3] + inj) & M
    return x0 | (x1 << 32)


def split_n(seed: int, n: int) -> list:
    return [_threefry(seed, i) for i in range(n)]


def fused_reduce(g: api.Graph, rows=4096, cols=4096):
    """Config 1: out = sum over the last axis of relu(x*y + 0.5*x), f32."""
    x, y = g.input([rows, cols], api.F32), g.input([rows, cols], api.F32)
    s = g.scalar(x, 0.5)
    out = g.sum(g.relu(g.add(g.mul(x, y), g.mul(s, x))), 1)
    k = split_n(0, 2)
    gens = {x: lambda h, k=k: h.rand_range([rows, cols], k[0], -1.0, 1.0), y: lambda h, k=k: h.rand_range([rows, cols], k[1], -1.0, 1.0)}
    return out, gens


def transposed_softmax(g: api.Graph, n=8192, lines=None):
    """Config 2: softmax over axis 0 of L (rows of L^T) after adding a broadcast bias, f32. `lines` (default n)
    is the number of columns of L, i.e. of softmax lines: a column slab of the square problem."""
    lines = n if lines is None else lines
    L, bias = g.input([n, lines], api.F32), g.input([n], api.F32)
    lt = g.permute(L, [1, 0])
    out = g.softmax(g.add(lt, g.broadcast_to(bias, [lines, n])), 1)
    k = split_n(1, 2)

    def gen_l(h):
        z = h.randn([n, lines], k[0])
        return h.mul(z, h.scalar(z, 2.0))
    gens = {L: gen_l, bias: lambda h: h.rand_range([n], k[1], -1.0, 1.0)}
    return out, gens


def gemm_bias_gelu(g: api.Graph, m=8192, n=8192, kdim=8192):
    """Config 3: out = gelu(A @ B + bias), bf16 operands, f32 accumulation, bf16 output."""
    A, B, bias = g.input([m, kdim], api.BF16), g.input([kdim, n], api.BF16), g.input([n], api.BF16)
    out = g.gelu(g.add(g.matmul(A, B), g.broadcast_to(bias, [m, n])))
    k = split_n(2, 3)
    std = 1.0 / math.sqrt(kdim)

    def gen_mat(shape, seed):
        def f(h):
            z = h.randn(shape, seed)
            return h.cast(h.mul(z, h.scalar(z, std)), api.BF16)
        return f
    gens = {A: gen_mat([m, kdim], k[0]), B: gen_mat([kdim, n], k[1]), bias: lambda h: h.cast(h.rand_range([n], k[2], -0.1, 0.1), api.BF16)}
    return out, gens


def causal_attention(g: api.Graph, batch=8, heads=32, seq=4096, dh=128, fused=None):
    """Config 4: causal multi-head attention, bf16. `fused` forces the primitive / the decomposition."""
    shape = [batch, heads, seq, dh]
    q, kk, v = (g.input(shape, api.BF16) for _ in range(3))
    if fused is None:
        out = g.sdpa(q, kk, v, True)
    elif fused:
        out = g.sdpa_fused(q, kk, v, True)
    else:
        out = g.sdpa_decomposed(q, kk, v, True)
    k = split_n(3, 3)
    gens = {n: (lambda h, s=s: h.cast(h.randn(shape, s), api.BF16)) for n, s in zip((q, kk, v), k)}
    return out, gens


def fp8_weight_gemm(g: api.Graph, m=16384, kdim=8192, n=28672, amp=True):
    """Config 5: out = silu((X @ dequant(W)) * scale) with fp8 e4m3 weights and per-output-channel
    f32 scales, bf16 output. With `amp` the mixed-precision pass quantises X to e4m3 as well, so the
    contraction runs fp8 x fp8 with f32 accumulation."""
    X, Wq, scales = g.input([m, kdim], api.BF16), g.input([kdim, n], api.F8E4M3), g.input([n], api.F32)
    wd = g.cast(Wq, api.BF16)
    acc = g.matmul(X, wd)
    z = g.mul(g.cast(acc, api.F32), g.broadcast_to(scales, [m, n]))
    out = g.cast(g.silu(z), api.BF16)
    if amp:
        out = g.amp_to(out, api.F8E4M3)
    k = split_n(4, 2)

    def gen_wf(h):
        z = h.randn([kdim, n], k[1])
        return h.mul(z, h.scalar(z, 0.02))

    def gen_scales(h):
        wf = gen_wf(h)
        mx = h.reduce_max(h.abs(wf), 0)
        return h.mul(mx, h.scalar(mx, 1.0 / 448.0))

    def gen_wq(h):
        wf = gen_wf(h)
        sc = gen_scales(h)
        return h.cast(h.div(wf, h.broadcast_to(sc, [kdim, n])), api.F8E4M3)
    gens = {X: lambda h: h.cast(h.randn([m, kdim], k[0]), api.BF16), Wq: gen_wq, scales: gen_scales}
    return out, gens


def quant_gemv(g: api.Graph, m=1, n=28672, kdim=8192, bits=4, group=128):
    """Decode step of a weight-only quantised projection (Op::QuantMatmul): m activation rows in bf16 against
    [n, kdim] weights packed `bits` wide with f16 scale and minimum per `group` columns."""
    kb, ng = kdim * bits // 8, kdim // group
    act, qw = g.input([m, kdim], api.BF16), g.input([n, kb], api.U8)
    sc, mn = g.input([n, ng], api.F16), g.input([n, ng], api.F16)
    out = g.quant_matmul(act, qw, sc, mn, bits, group)
    k = split_n(5, 4)
    gens = {act: lambda h: h.cast(h.randn([m, kdim], k[0]), api.BF16),
            qw: lambda h: h.cast(h.rand_range([n, kb], k[1], 0.0, 256.0), api.U8),        # every byte value, i.e. every pair of fields
            sc: lambda h: h.cast(h.rand_range([n, ng], k[2], 0.004, 0.012), api.F16),
            mn: lambda h: h.cast(h.rand_range([n, ng], k[3], -0.09, -0.03), api.F16)}
    return out, gens
