"""Row splitting of an evaluation (kurumi_b200/csrc/core/split.cc) on the CPU oracle: the parts, evaluated on the
matching input slices and stacked, are the whole evaluation bit for bit, for each of the five benchmark graphs at
reduced sizes; graphs that mix rows are refused with a reason."""
import numpy as np
import pytest

from kurumi_b200 import api, configs


def run_whole_and_parts(oracle_lib, cpu, make, kwargs, parts):
    g = api.Graph(oracle_lib)
    root, gens = make(g, **kwargs)
    vals = {}
    for node, mk in gens.items():
        h = api.Graph(oracle_lib)
        t = cpu.eval(h, mk(h))
        vals[node] = (t.numpy(), t.dtype)
    feeds = api.Feeds(oracle_lib)
    for n, (v, dt) in vals.items():
        feeds.set(n, v, dt)
    whole = cpu.eval_with(g, root, feeds).numpy()
    pg, proot, inputs = api.row_split(g, root, parts)
    assert sorted(o for o, _, _ in inputs) == sorted(vals)
    pieces = []
    for c in range(parts):
        f = api.Feeds(oracle_lib)
        for orig, part, axis in inputs:
            v, dt = vals[orig]
            if axis is not None:
                step = v.shape[axis] // parts
                v = np.ascontiguousarray(np.take(v, range(c * step, (c + 1) * step), axis=axis))
            f.set(part, v, dt)
        pieces.append(cpu.eval_with(pg, proot, f).numpy())
    return whole, np.concatenate(pieces, 0), inputs


@pytest.mark.parametrize("make,kwargs,axes", [
    (configs.fused_reduce, dict(rows=64, cols=96), [0, 0]),
    (configs.transposed_softmax, dict(n=48, lines=32), [1, None]),
    (configs.gemm_bias_gelu, dict(m=32, n=24, kdim=40), [0, None, None]),
    (configs.causal_attention, dict(batch=4, heads=2, seq=24, dh=16, fused=True), [0, 0, 0]),
    (configs.causal_attention, dict(batch=4, heads=2, seq=24, dh=16, fused=False), [0, 0, 0]),
    (configs.fp8_weight_gemm, dict(m=16, kdim=32, n=24, amp=True), [0, None, None]),
])
def test_parts_stack_to_the_whole(oracle_lib, cpu, make, kwargs, axes):
    whole, stacked, inputs = run_whole_and_parts(oracle_lib, cpu, make, kwargs, 4)
    assert [a for _, _, a in inputs] == axes
    assert whole.shape == stacked.shape and whole.tobytes() == stacked.tobytes()


def test_movement_and_reductions_follow_the_axis(oracle_lib, cpu):
    rng = np.random.default_rng(0)
    g = api.Graph(oracle_lib)
    x = g.input([6, 8, 10], api.F32)            # root rows come from axis 1 of x
    w = g.input([10, 5], api.F32)
    y = g.permute(x, [1, 0, 2])                 # [8, 6, 10]
    y = g.reshape(y, [8, 60])
    y = g.reshape(y, [8, 6, 10])
    z = g.dot_general(y, w, [2], [0])           # [8, 6, 5]
    z = g.add(g.sum(z, 1), g.reduce_max(g.slice(z, [(0, 8), (1, 5), (0, 5)]), 1))   # [8, 5]
    root = g.softmax(g.flip(z, [1]), 1)
    xv, wv = rng.standard_normal((6, 8, 10)).astype(np.float32), rng.standard_normal((10, 5)).astype(np.float32)
    whole = cpu.eval_with(g, root, api.Feeds(oracle_lib).set(x, xv).set(w, wv)).numpy()
    pg, proot, inputs = api.row_split(g, root, 2)
    assert [(o, a) for o, _, a in inputs] == [(x, 1), (w, None)]
    px, pw = inputs[0][1], inputs[1][1]
    parts = [cpu.eval_with(pg, proot, api.Feeds(oracle_lib).set(px, np.ascontiguousarray(xv[:, c * 4:(c + 1) * 4]), api.F32).set(pw, wv)).numpy() for c in range(2)]
    assert np.concatenate(parts, 0).tobytes() == whole.tobytes()


@pytest.mark.parametrize("build,reason", [
    (lambda g, x: g.softmax(x, 0), "normalises along the split axis"),
    (lambda g, x: g.permute(g.reshape(x, [2, 4, 12]), [1, 0, 2]), "does not map onto one axis"),
    (lambda g, x: g.flip(x, [0]), "reverses the split axis"),
    (lambda g, x: g.slice(x, [(2, 6), (0, 12)]), "cuts the split axis"),
    (lambda g, x: (lambda y: g.add(y, g.permute(y, [1, 0])))(g.input([8, 8], api.F32)), "needed both along axis"),
    (lambda g, x: g.mul(x, g.rand_uniform([8, 12], 7)), "absolute element index"),
])
def test_graphs_that_mix_rows_are_refused(oracle_lib, build, reason):
    g = api.Graph(oracle_lib)
    x = g.input([8, 12], api.F32)
    root = build(g, x)
    with pytest.raises(api.Error, match=reason):
        api.row_split(g, root, 2)
    with pytest.raises(api.Error, match="does not divide"):
        api.row_split(g, g.neg(x), 3)
