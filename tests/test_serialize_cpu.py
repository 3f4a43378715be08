"""KGPH v2 graph blobs through the C ABI (ku_graph_serialize* / ku_graph_deserialize): the reference's
frozen golden blob (kurumi_core/src/graph/serialize/tests.rs:188-221), its rejection cases
(tests.rs:223-255), round trips of the benchmark graphs, and hostile inputs. No GPU needed: the graph
layer is shared by the CUDA library and the oracle, so both are exercised."""
import os
import struct

import numpy as np
import pytest

from kurumi_b200 import api, configs

GOLDEN = bytes.fromhex(open(os.path.join(os.path.dirname(__file__), "golden", "graph_v2.kgph.hex")).read().strip())


def golden_graph(lib):
    g = api.Graph(lib)
    x = g.constant(np.array([[1, 2, 3], [4, 5, 6]], np.float32))
    w = g.constant(np.full((2, 3), 2.0, np.float32))
    out = g.sum(g.add(x, w), 1)
    return g, out


@pytest.mark.parametrize("which", ["oracle", "cuda"])
def test_golden_blob_bytes_and_value(which, oracle_lib, cuda_lib, cpu):
    lib = oracle_lib if which == "oracle" else cuda_lib
    assert len(GOLDEN) == 175
    g, out = golden_graph(lib)
    assert g.serialize([out]) == GOLDEN                         # the v2 wire format, byte for byte
    rg, entries = api.deserialize(lib, GOLDEN)
    assert entries == [("", [3], [])]
    assert rg.serialize([3]) == GOLDEN                          # decode -> encode is the identity
    if which == "oracle":
        np.testing.assert_array_equal(cpu.eval(rg, 3).numpy(), np.array([12.0, 21.0], np.float32))


def test_rejections(oracle_lib):
    lib = oracle_lib
    for blob in (b"XXXX\x01", b"", b"KGPH", b"KGPH\x01" + GOLDEN[5:], b"KGPH\x03" + GOLDEN[5:]):
        with pytest.raises(api.Error):
            api.deserialize(lib, blob)
    fwd = b"KGPH\x02" + struct.pack("<I", 1) + bytes([7]) + struct.pack("<II", 1, 0)          # Add whose source is itself
    with pytest.raises(api.Error, match="not yet built"):
        api.deserialize(lib, fwd)
    under = b"KGPH\x02" + struct.pack("<I", 1) + bytes([0, 13]) + struct.pack("<Q", 4) + struct.pack("<f", 1.0) + struct.pack("<IQ", 1, 2)
    with pytest.raises(api.Error, match="needs 2"):
        api.deserialize(lib, under)
    no_entry = GOLDEN[:-len(struct.pack("<IIIII", 1, 0, 1, 3, 0))] + struct.pack("<I", 0)
    with pytest.raises(api.Error, match="no entries"):
        api.deserialize(lib, no_entry)
    solve = b"KGPH\x02" + struct.pack("<I", 1) + bytes([41]) + struct.pack("<I", 0) + struct.pack("<I", 0)
    with pytest.raises(api.Error, match="not a primitive"):
        api.deserialize(lib, solve)
    bad_role = GOLDEN[:-4] + struct.pack("<I", 1) + struct.pack("<I", 0) + bytes([2]) + struct.pack("<I", 0)
    with pytest.raises(api.Error, match="role"):
        api.deserialize(lib, bad_role)


def test_every_truncation_and_byte_flip_is_an_error_or_a_graph(oracle_lib):
    """Hostile blobs never crash the process: each prefix of the golden blob is refused, and each single-byte
    corruption either decodes to some graph or is refused."""
    for n in range(len(GOLDEN)):
        with pytest.raises(api.Error):
            api.deserialize(oracle_lib, GOLDEN[:n])
    rng = np.random.default_rng(7)
    for pos in range(len(GOLDEN)):
        for val in (0, 0xFF, int(rng.integers(0, 256))):
            b = bytearray(GOLDEN)
            b[pos] = val
            try:
                api.deserialize(oracle_lib, bytes(b))
            except api.Error:
                pass


@pytest.mark.parametrize("make,kw", [(configs.fused_reduce, dict(rows=8, cols=64)), (configs.transposed_softmax, dict(n=64)),
                                     (configs.gemm_bias_gelu, dict(m=16, n=32, kdim=64)), (configs.causal_attention, dict(batch=1, heads=2, seq=32, dh=64)),
                                     (configs.fp8_weight_gemm, dict(m=16, kdim=64, n=32, amp=True))])
def test_config_graphs_round_trip(make, kw, oracle_lib, cuda_lib, cpu):
    g = api.Graph(oracle_lib)
    root, gens = make(g, **kw)
    inputs = [(node, 1, f"in{i}") for i, node in enumerate(gens)]
    blob = g.serialize([root], inputs)
    rg, entries = api.deserialize(oracle_lib, blob)
    assert entries == [("", [root], inputs)]
    assert rg.serialize([root], inputs) == blob
    assert api.deserialize(cuda_lib, blob)[1] == entries      # the CUDA library reads the same blob
    # same values from the rebuilt graph
    feeds_a, feeds_b = api.Feeds(oracle_lib), api.Feeds(oracle_lib)
    for node, mk in gens.items():
        h = api.Graph(oracle_lib)
        t = cpu.eval(h, mk(h))
        feeds_a.set(node, t.numpy(), t.dtype)
        feeds_b.set(node, t.numpy(), t.dtype)
    a, b = cpu.eval_with(g, root, feeds_a), cpu.eval_with(rg, root, feeds_b)
    assert a.dtype == b.dtype and a.numpy().tobytes() == b.numpy().tobytes()


def test_reachable_and_multi(oracle_lib, cpu):
    lib = oracle_lib
    g = api.Graph(lib)
    x = g.input([4], api.F32)
    dead = g.exp2(x)                                              # not on any output's cone
    y = g.input([4], api.F32)
    s = g.add(x, g.mul(y, y))
    t = g.neg(s)
    whole = g.serialize([s], [(x, 1, "x"), (y, 0, "w.y")])
    cone = g.serialize([s], [(x, 1, "x"), (y, 0, "w.y")], reachable=True)
    assert len(cone) < len(whole)
    rg, entries = api.deserialize(lib, cone)
    (name, outs, ins) = entries[0]
    assert name == "" and len(outs) == 1 and [(r, n) for (_, r, n) in ins] == [(1, "x"), (0, "w.y")]
    f = api.Feeds(lib).set(ins[0][0], np.arange(4, dtype=np.float32)).set(ins[1][0], np.full(4, 3.0, np.float32))
    np.testing.assert_array_equal(cpu.eval_with(rg, outs[0], f).numpy(), np.arange(4, dtype=np.float32) + 9.0)
    # an input binding outside the cone is dropped, not an error
    only_y = g.serialize([g.mul(y, y)], [(x, 1, "x"), (y, 1, "y")], reachable=True)
    assert [n for (_, _, n) in api.deserialize(lib, only_y)[1][0][2]] == ["y"]
    multi = g.serialize_multi([("forward", [s], [(x, 1, "x"), (y, 1, "y")]), ("negated", [t], [(x, 1, "x"), (y, 1, "y")])])
    rg2, e2 = api.deserialize(lib, multi)
    assert [e[0] for e in e2] == ["forward", "negated"] and len(e2[1][1]) == 1
    f2 = api.Feeds(lib).set(e2[1][2][0][0], np.ones(4, np.float32)).set(e2[1][2][1][0], np.full(4, 2.0, np.float32))
    np.testing.assert_array_equal(cpu.eval_with(rg2, e2[1][1][0], f2).numpy(), np.full(4, -5.0, np.float32))
    assert dead != s
    with pytest.raises(api.Error):
        g.serialize([10 ** 6])                                    # an output that is not a node
