"""Kernel selection and runtime compilation without a GPU: the CUDA library lowers a graph, generates the kernels' source
and compiles it with NVRTC for sm_100a; nothing is launched. What runs where (the families returned) is host logic, and a
generated kernel that no longer compiles shows up here before it reaches a device."""
import pytest

from kurumi_b200 import api


def families(lib, build):
    g = api.Graph(lib)
    return api.compile_check(lib, g, [build(g)])


def test_pointwise_passes_pick_the_tiled_kernel_only_for_transposed_operands(cuda_lib):
    assert families(cuda_lib, lambda g: g.add(g.input([300, 500], api.F32), g.input([300, 500], api.F32))) == ["pointwise"]
    # a transposed operand beside a row-major one: shared-memory tiles
    assert families(cuda_lib, lambda g: g.add(g.permute(g.input([300, 500], api.F32), [1, 0]), g.input([500, 300], api.F32))) == ["pointwise_tiled"]
    # every storage width (the tile is 64 x 64 for 1- and 2-byte types), and a batch dim in front
    for dt in (api.U8, api.BF16, api.F32, api.I64):
        assert families(cuda_lib, lambda g, dt=dt: g.permute(g.input([3, 70, 90], dt), [0, 2, 1])) == ["pointwise_tiled"]
    # too short an innermost dim for a tile, and an operand that is only broadcast along it: the plain kernel
    assert families(cuda_lib, lambda g: g.permute(g.input([500, 8], api.F32), [1, 0])) == ["pointwise"]
    assert families(cuda_lib, lambda g: g.add(g.input([64, 64], api.F32), g.broadcast_to(g.reshape(g.input([64], api.F32), [64, 1]), [64, 64]))) == ["pointwise"]


def test_reductions_along_rows_columns_and_short_axes(cuda_lib):
    assert families(cuda_lib, lambda g: g.sum(g.input([4096, 4096], api.F32), 1)) == ["reduce_rows"]
    assert families(cuda_lib, lambda g: g.sum(g.input([8192, 64], api.F32), 0)) == ["reduce_split"]
    assert families(cuda_lib, lambda g: g.sum(g.input([300000, 8], api.F32), 1)) == ["reduce_fold"]


def test_index_of_the_best_along_long_and_short_axes(cuda_lib):
    assert families(cuda_lib, lambda g: g.argmax(g.input([9, 4096], api.F32), 1)) == ["arg_rows"]      # 128-bit pieces
    assert families(cuda_lib, lambda g: g.argmin(g.input([9, 3001], api.BF16), 1)) == ["arg_rows"]     # element by element
    assert families(cuda_lib, lambda g: g.argmax(g.input([9, 100], api.F32), 1)) == ["arg_fold"]
    assert families(cuda_lib, lambda g: g.argmax(g.input([4096, 9], api.I32), 0)) == ["arg_fold"]


@pytest.mark.parametrize("dt", [api.F32, api.BF16, api.I64, api.U8])
def test_sorting_in_shared_memory_and_through_scratch(cuda_lib, dt):
    # one launch while a padded line of (key, index) pairs fits a CTA's shared memory
    for n in (1, 2, 5, 300, 8192):
        assert families(cuda_lib, lambda g, n=n: g.argsort(g.input([3, n], dt), 1, False)) == ["argsort"]
    assert families(cuda_lib, lambda g: g.argsort(g.input([70, 6], dt), 0, True)) == ["argsort"]
    # 40000 -> 65536 padded: chunk sort, 1 + 2 + 3 + 4 wide steps with a local pass per stage, copy out
    assert families(cuda_lib, lambda g: g.argsort(g.input([2, 40000], dt), 1, False)) == ["argsort"] * (1 + (1 + 2 + 3 + 4) + 4 + 1)


def test_gathers_and_scatters_compile_for_every_combiner(cuda_lib):
    def gathers(g):
        x, i = g.input([1000, 64], api.F32), g.input([77], api.I32)
        return g.gather(x, i, 0)
    assert families(cuda_lib, gathers) == ["gather"]
    assert families(cuda_lib, lambda g: g.gather_along(g.input([50, 64], api.BF16), g.input([50, 9], api.I64), 1)) == ["gather_along"]
    for combine in (0, 1, 2, 3):
        fams = families(cuda_lib, lambda g, c=combine: g.scatter(g.input([1000, 24], api.F32), g.input([5003], api.I64), g.input([5003, 24], api.F32), 0, c))
        assert fams[-1] == "scatter" and set(fams) <= {"pointwise", "scatter"}
        fams = families(cuda_lib, lambda g, c=combine: g.scatter_along(g.input([24, 1000], api.I8), g.input([24, 500], api.I32), g.input([24, 500], api.I8), 1, c))
        assert fams[-1] == "scatter_along" and set(fams) <= {"pointwise", "scatter_along"}


def test_decode_step_kernels_compile_for_every_field_width_and_activation_type(cuda_lib):
    """The quantised matmul with one activation row: 16-bit activations with 2- or 4-bit fields take the tensor-core
    gemv (small and full-size: the split of a row tile over warps follows the row count), f32 activations and 8-bit
    fields the scalar kernel. Both report the family quant_gemv."""
    def step(g, act, bits, n=2048, k=1024, group=128, mins=True):
        a = g.input([1, k], act)
        qw = g.input([n, k * bits // 8], api.U8)
        sc = g.input([n, k // group], api.F16)
        mn = g.input([n, k // group], api.F16) if mins else None
        return g.quant_matmul(a, qw, sc, mn, bits, group)
    for act, bits, kw in ((api.BF16, 4, {}), (api.F16, 2, dict(n=28672, k=8192, group=256)), (api.BF16, 4, dict(n=28672, k=8192, mins=False)),
                          (api.F16, 4, dict(n=100000, k=2048)), (api.F32, 4, {}), (api.BF16, 8, {}), (api.F16, 4, dict(group=32))):
        assert families(cuda_lib, lambda g: step(g, act, bits, **kw)) == ["quant_gemv"]


def test_the_named_configurations_compile_to_their_kernels_at_full_size(cuda_lib):
    """Every configuration the benchmark times, recorded at its full size, lowers to the kernel it is measured with and
    that kernel compiles for sm_100a (tcgen05 GEMM in CTA pairs, fused attention, the group softmax, the row reduction,
    the fp8 path behind an activation quantise, the decode-step gemv); so do their row shards for 2, 4 and 8 ranks."""
    from kurumi_b200 import configs
    want = {
        configs.fused_reduce: ["reduce_rows"],
        configs.transposed_softmax: ["softmax_groups_tma"],
        configs.gemm_bias_gelu: ["gemm_tc"],
        configs.causal_attention: ["attention_tc"],
        configs.fp8_weight_gemm: ["pointwise", "gemm_tc_f8"],
        configs.quant_gemv: ["quant_gemv"],
    }
    for build, fams in want.items():
        g = api.Graph(cuda_lib)
        root, _ = build(g)
        assert api.compile_check(cuda_lib, g, [root]) == fams, build.__name__
    for parts in (2, 4, 8):
        g = api.Graph(cuda_lib)
        root, _ = configs.transposed_softmax(g, n=8192, lines=8192 // parts)
        assert api.compile_check(cuda_lib, g, [root]) == ["softmax_groups_tma"]
        g = api.Graph(cuda_lib)
        root, _ = configs.fused_reduce(g, rows=4096 // parts)
        assert api.compile_check(cuda_lib, g, [root]) == ["reduce_rows"]
