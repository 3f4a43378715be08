"""A graph that arrives as a KGPH v2 blob runs on the device like one recorded through the builders."""
import os

import numpy as np
import pytest

from kurumi_b200 import api, configs
from tests import util

pytestmark = pytest.mark.gpu

GOLDEN = bytes.fromhex(open(os.path.join(os.path.dirname(__file__), "golden", "graph_v2.kgph.hex")).read().strip())


def test_golden_blob_on_the_device(cuda_lib, gpu):
    g, entries = api.deserialize(cuda_lib, GOLDEN)
    np.testing.assert_array_equal(gpu.eval(g, entries[0][1][0]).numpy(), np.array([12.0, 21.0], np.float32))


def test_transposed_softmax_from_a_blob(oracle_lib, cuda_lib, cpu64, gpu):
    go = api.Graph(oracle_lib)
    root, gens = configs.transposed_softmax(go, n=1024)
    blob = go.serialize([root], [(n, 1, f"in{i}") for i, n in enumerate(gens)], reachable=True)
    gc, entries = api.deserialize(cuda_lib, blob)
    (_, outs, ins) = entries[0]
    fo, fc = api.Feeds(oracle_lib), api.Feeds(cuda_lib)
    cpu32 = api.Backend(oracle_lib, 0)
    for (node, _, _), (onode, mk) in zip(ins, gens.items()):
        h = api.Graph(oracle_lib)
        t = cpu32.eval(h, mk(h))
        fo.set(onode, t.numpy(), t.dtype)
        fc.set(node, t.numpy(), t.dtype)
    got = gpu.eval_with(gc, outs[0], fc).numpy()
    want = cpu64.eval_with(go, root, fo).numpy()
    util.assert_close(want, got, 1e-5, 1e-12, "softmax from a blob")


def gemm_bias_gelu_backward(g, m, n, k):
    """The reverse-mode graph of configuration 3, out = gelu(A @ B + bias), for a cotangent dOut, written out with the
    builders as the reference's autograd (kurumi_core/src/grad/**) emits it: primitives only, the two backward
    contractions are transposed dot_generals (kurumi_metal/src/backend/eval/matmul.rs:81-147 lists the layouts).
    gelu(z) = 0.5 z (1 + tanh(u)), u = c (z + a z^3); d/dz = 0.5 (1 + t) + 0.5 z (1 - t^2) c (1 + 3 a z^2)."""
    A, B, bias, dout = g.input([m, k], api.BF16), g.input([k, n], api.BF16), g.input([n], api.BF16), g.input([m, n], api.BF16)
    z = g.add(g.matmul(A, B), g.broadcast_to(bias, [m, n]))
    c, a = 0.7978845608028654, 0.044715
    z2 = g.mul(z, z)
    t = g.tanh(g.mul(g.scalar(z, c), g.add(z, g.mul(g.scalar(z, a), g.mul(z2, z)))))
    one = g.scalar(z, 1.0)
    left = g.mul(g.scalar(z, 0.5), g.add(one, t))
    sech2 = g.add(one, g.neg(g.mul(t, t)))
    right = g.mul(g.mul(g.scalar(z, 0.5), z), g.mul(sech2, g.mul(g.scalar(z, c), g.add(one, g.mul(g.scalar(z, 3 * a), z2)))))
    dz = g.mul(dout, g.add(left, right))
    dA = g.dot_general(dz, B, [1], [1])          # [m, n] x [k, n]^T -> [m, k]
    dB = g.dot_general(A, dz, [0], [0])          # [m, k]^T x [m, n] -> [k, n]
    dbias = g.sum(dz, 0)                         # a reduction over the rows
    return (A, B, bias, dout), (dA, dB, dbias)


def test_backward_graph_of_the_gemm_configuration_from_a_blob(oracle_lib, cuda_lib, cpu, cpu64, gpu):
    m, n, k = 384, 512, 256
    go = api.Graph(oracle_lib)
    ins_o, outs_o = gemm_bias_gelu_backward(go, m, n, k)
    blob = go.serialize(list(outs_o), [(node, 1, name) for node, name in zip(ins_o, ("A", "B", "bias", "dOut"))], reachable=True)
    gc, entries = api.deserialize(cuda_lib, blob)
    (_, outs, ins) = entries[0]
    by_name = {name: node for node, _, name in ins}
    rng = np.random.default_rng(33)
    vals = {"A": rng.standard_normal((m, k)) / np.sqrt(k), "B": rng.standard_normal((k, n)), "bias": rng.uniform(-0.1, 0.1, n), "dOut": rng.standard_normal((m, n))}
    fo, fc = api.Feeds(oracle_lib), api.Feeds(cuda_lib)
    for (node_o, name) in zip(ins_o, ("A", "B", "bias", "dOut")):
        bits = api.f32_to_bf16(vals[name].astype(np.float32))
        fo.set(node_o, bits, api.BF16)
        fc.set(by_name[name], bits, api.BF16)
    fams = api.compile_check(cuda_lib, gc, outs)
    assert fams.count("gemm_tc") == 3, fams          # forward and the two transposed backward contractions on the tensor cores
    got = gpu.eval_many_with(gc, outs, fc)
    want = cpu64.eval_many_with(go, list(outs_o), fo)
    native = cpu.eval_many_with(go, list(outs_o), fo)
    for name, a, nat, b in zip(("dA", "dB", "dbias"), want, native, got):
        # the derivative of gelu is some 25 bf16 primitives, each rounded (the interpreter's semantics, which the device keeps):
        # against the bf16 interpreter the contraction band applies; the f64 run, which rounds nothing on the way, is further off
        util.assert_band(util.to_f64(nat.numpy(), api.BF16), util.to_f64(b.numpy(), api.BF16), 2e-2, 2.0 ** -7, f"backward of gemm + bias + gelu vs bf16 interpreter, {name}")
        util.assert_band(a.numpy(), util.to_f64(b.numpy(), api.BF16), 4e-2, 2.0 ** -6, f"backward of gemm + bias + gelu vs f64 run, {name}")


def attention_backward(g, b, h, s, dh):
    """The reverse-mode graph of configuration 4 for a cotangent dOut, written out as the reference's VJP of Op::Sdpa emits it
    (kurumi_core/src/grad/nn.rs:52-92): P is recomputed exactly as the forward computes it (batched dot_general, scalar
    scale, additive causal bias, softmax over the keys), then dV = P^T dOut, dP = dOut V^T,
    dS = P * (dP - rowsum(dP * P)), dQ = scale dS K, dK = scale dS^T Q. Primitives only; the bias arrives as an input."""
    shape, r = [b, h, s, dh], 4
    q, k, v, ct = (g.input(shape, api.BF16) for _ in range(4))
    bias = g.input([s, s], api.BF16)                              # 0 on and below the diagonal, -inf above
    batch = [0, 1]
    scale = 1.0 / np.sqrt(dh)
    raw = g.dot_general(q, k, [r - 1], [r - 1], batch, batch)
    scores = g.add(g.mul(raw, g.scalar(raw, scale)), g.broadcast_to(bias, [b, h, s, s]))
    p = g.softmax(scores, r - 1)
    dv = g.dot_general(p, ct, [r - 2], [r - 2], batch, batch)
    dp = g.dot_general(ct, v, [r - 1], [r - 1], batch, batch)
    rs = g.sum(g.mul(dp, p), r - 1)
    diff = g.add(dp, g.neg(g.broadcast_to(g.reshape(rs, [b, h, s, 1]), [b, h, s, s])))
    draw = g.mul(g.mul(p, diff), g.scalar(p, scale))
    dq = g.dot_general(draw, k, [r - 1], [r - 2], batch, batch)
    dk = g.dot_general(draw, q, [r - 2], [r - 2], batch, batch)
    return (q, k, v, ct, bias), (dq, dk, dv)


def test_backward_graph_of_the_attention_configuration_from_a_blob(oracle_lib, cuda_lib, cpu, cpu64, gpu):
    b, h, s, dh = 1, 2, 256, 64
    go = api.Graph(oracle_lib)
    ins_o, outs_o = attention_backward(go, b, h, s, dh)
    names = ("Q", "K", "V", "dOut", "bias")
    blob = go.serialize(list(outs_o), [(node, 1, name) for node, name in zip(ins_o, names)], reachable=True)
    gc, entries = api.deserialize(cuda_lib, blob)
    (_, outs, ins) = entries[0]
    by_name = {name: node for node, _, name in ins}
    rng = np.random.default_rng(34)
    vals = {n: rng.standard_normal((b, h, s, dh)).astype(np.float32) for n in names[:4]}
    vals["bias"] = np.where(np.arange(s)[None, :] > np.arange(s)[:, None], -np.inf, 0.0).astype(np.float32)
    fo, fc = api.Feeds(oracle_lib), api.Feeds(cuda_lib)
    for node_o, name in zip(ins_o, names):
        bits = api.f32_to_bf16(vals[name])
        fo.set(node_o, bits, api.BF16)
        fc.set(by_name[name], bits, api.BF16)
    fams = api.compile_check(cuda_lib, gc, outs)
    assert sum(f.startswith("gemm") for f in fams) >= 5, fams     # the five batched contractions run as contraction kernels
    got = gpu.eval_many_with(gc, outs, fc)
    want = cpu64.eval_many_with(go, list(outs_o), fo)
    native = cpu.eval_many_with(go, list(outs_o), fo)
    for name, a, nat, c in zip(("dQ", "dK", "dV"), want, native, got):
        assert c.shape == (b, h, s, dh)
        # every intermediate ([.., S, S] scores, probabilities, their cotangents) is rounded to bf16, on the device as in the
        # interpreter: the contraction band against the bf16 interpreter, a wider one against the f64 run that rounds nothing
        util.assert_band(util.to_f64(nat.numpy(), api.BF16), util.to_f64(c.numpy(), api.BF16), 2e-2, 2.0 ** -7, f"backward of causal attention vs bf16 interpreter, {name}")
        util.assert_band(a.numpy(), util.to_f64(c.numpy(), api.BF16), 4e-2, 2.0 ** -6, f"backward of causal attention vs f64 run, {name}")
    # causality: key t receives nothing from queries before it; the last key's dK / dV come from the last query alone
    dV = util.to_f64(got[2].numpy(), api.BF16)
    assert np.isfinite(dV).all()
