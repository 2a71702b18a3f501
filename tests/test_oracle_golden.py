"""Pins the CPU oracle against every known-answer vector the reference's own tests hold for
the hot path (catena-lang/tests/runtime.rs and tests/cases/*.rs; the vectors were read from
those files as text, the reference itself needs Rust + a GPU and cannot run here)."""
import math

import numpy as np
import pytest


def bits(x):
    return int(np.float32(x).view(np.uint32))


def f32(b):
    return np.array([b], np.uint32).view(np.float32)[0]


# tests/cases/matrix.rs:6-46
def test_matmul_2x3_3x2(orc):
    out = orc.matmul_f32([1, 2, 3, 4, 5, 6], [7, 8, 9, 10, 11, 12], 2, 2, 3)
    assert np.all(np.abs(out - np.array([58, 64, 139, 154], np.float32)) < 1e-4)


# tests/cases/matrix.rs:48-82 (identity views; exact)
def test_matmul_identity_exact(orc):
    a = np.array([1, 2, 3, 4], np.float32)
    eye = np.eye(2, dtype=np.float32).ravel()
    assert orc.matmul_f32(a, eye, 2, 2, 2).tolist() == a.tolist()
    assert orc.matmul_f32(eye, a, 2, 2, 2).tolist() == a.tolist()


def test_matmul_length_assert(orc):
    with pytest.raises(ValueError):
        orc.matmul_f32([1, 2, 3], [1, 2, 3, 4], 2, 2, 2)


# tests/runtime.rs:333-363
def test_fma_is_fused_and_mul_add_is_not(orc):
    a, c = f32(0x3F800001), f32(0x33800000)
    assert bits(orc.lib().orc_f32_fma(a, a, c)) == 0x3F800003
    assert bits(orc.lib().orc_f32_mul_add(a, a, c)) == 0x3F800002


# tests/runtime.rs:365-406
def test_sin(orc):
    for x in [0.0, 0.5, 1.0, -0.5, -1.0]:
        assert abs(orc.scalar("math.sin-approx", x) - math.sin(x)) < 1e-4
    for x in [-200.0, -100.0, -10.0, -6.0, -3.0, -1.9, -0.5, 0.0, 0.5, 3.0, 6.0, 10.0, 100.0, 200.0]:
        assert abs(orc.scalar("math.sin-approx-full", x) - float(np.sin(np.float32(x)))) < 1e-4


# tests/runtime.rs:742-782
def test_exp_exp2(orc):
    for x in [-3.0, -1.0, -0.5, 0.0, 0.5, 1.0, 3.0]:
        e = math.exp(x)
        assert abs(orc.scalar("math.exp-approx", x) - e) / max(e, 1.0) < 4e-3
        e2 = 2.0 ** x
        assert abs(orc.scalar("math.exp2-approx", x) - e2) / max(e2, 1.0) < 4e-3


# tests/runtime.rs:792-877
def test_activations(orc):
    for x in [-6.0, -1.0, 0.0, 1.0, 6.0]:
        assert abs(orc.scalar("nn.sigmoid", x) - 1 / (1 + math.exp(-x))) < 4e-3
    for x in [-3.0, -1.0, 0.0, 1.0, 3.0]:
        sg = 1 / (1 + math.exp(-x))
        assert abs(orc.scalar("nn.silu", x) - x * sg) < 2e-2
        assert abs(orc.scalar("nn.tanh", x) - math.tanh(x)) < 8e-3
        g = 0.5 * x * (1 + math.tanh(math.sqrt(2 / math.pi) * (x + 0.044715 * x ** 3)))
        assert abs(orc.scalar("nn.gelu-approx", x) - g) < 2e-2


# tests/runtime.rs:879-969
def test_sqrt_log_pow(orc):
    for x in [0.0, 0.25, 1.0, 2.0, 9.0, 100.0]:
        assert abs(orc.scalar("math.sqrt", x) - math.sqrt(x)) < 1e-4
    for x in [0.1, 0.25, 0.5, 0.75, 1.0, 1.5, 2.0, 3.0, 8.0, 10.0]:
        assert abs(orc.scalar("math.log-approx", x) - math.log(x)) < 6e-4
        assert abs(orc.scalar("math.log2-approx", x) - math.log2(x)) < 1e-3
    for b, e in [(0.25, 0.5), (0.5, 2.0), (1.0, 3.0), (1.5, -1.0), (2.0, 3.0), (3.0, 0.5), (10.0, 0.25)]:
        want = b ** e
        assert abs(orc.scalar("math.powf", b, e) - want) / max(abs(want), 1.0) < 8e-3


# tests/runtime.rs:971-1044
def test_softmax_rmsnorm(orc):
    x = np.array([1.0, 2.0, 4.0], np.float32)
    y = orc.softmax(x)
    want = np.exp(x - x.max()) / np.exp(x - x.max()).sum()
    assert np.all(np.abs(y - want) < 6e-3) and abs(y.sum() - 1) < 6e-3
    x = np.array([1.0, 2.0, 4.0, -1.0, -9.0, 13.29], np.float32)
    y = orc.rmsnorm(x)
    rms = math.sqrt(float((x.astype(np.float64) ** 2).mean()) + 1e-5)
    assert np.all(np.abs(y - x / rms) < 3e-3)
    assert abs(math.sqrt(float((y.astype(np.float64) ** 2).mean())) - 1) < 3e-3


# tests/runtime.rs:1046-1197 (exact)
def test_tensor_ops(orc):
    assert orc.broadcast_f32(3.5, 0).tolist() == []
    assert orc.broadcast_f32(3.5, 4).tolist() == [3.5] * 4
    assert orc.arange_f32(0).tolist() == []
    assert orc.arange_f32(5).tolist() == [0, 1, 2, 3, 4]
    src = [10.0, 20.0, 30.0, 40.0]
    assert orc.slice_f32(src, 0, 2).tolist() == [10, 20]
    assert orc.slice_f32(src, 1, 2).tolist() == [20, 30]
    assert orc.slice_f32(src, 2, 0).tolist() == []
    assert orc.slice_f32(src, 0, 4).tolist() == src
    with pytest.raises(IndexError):
        orc.slice_f32(src, 3, 2)
    for l, r in [([1, 2], [3, 4]), ([1], [2, 3, 4]), ([], [3, 4]), ([1, 2], []), ([], [])]:
        assert orc.concat_f32(l, r).tolist() == [float(v) for v in l + r]
    for xs, want in [([5.0], 0), ([1, 2, 4], 2), ([4, 2, 1], 0), ([1, 7, 3, 2], 1), ([1, 7, 7, 2], 1),
                     ([3, 3, 3], 0)]:
        assert orc.argmax_f32(xs) == want


# tests/cases/reducec.rs:6-90
def test_reductions(orc):
    assert orc.sum_u64([2, 3, 5, 7, 11]) == 28
    assert orc.dot_u64([2, 3, 5, 7], [11, 13, 17, 19]) == 2 * 11 + 3 * 13 + 5 * 17 + 7 * 19
    x = [1.5, -0.5, 2.0, 4.0]
    assert orc.sum_f32(x) == 7.0 and orc.mean_f32(x) == 1.75 and orc.max_f32(x) == 4.0
    assert bits(orc.sum_f32([])) == 0 and bits(orc.max_f32([])) == 0xFF800000


# numeric edge semantics restated from the formulas (stdlib/math.hex:153; stdlib/sum.hex:37)
def test_edge_semantics(orc):
    assert bits(orc.scalar("math.exp-approx", 0.0)) == 0x3F7FF8FC
    assert bits(orc.sum_f32(np.array([-0.0, -0.0], np.float32))) == 0  # +0 + -0 = +0
    assert bits(orc.scalar("math.sqrt", -4.0)) == 0


def test_threads_do_not_change_bits(orc):
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (64, 96)).astype(np.float32)
    b = rng.uniform(-1, 1, (96, 48)).astype(np.float32)
    c1 = orc.matmul_f32(a, b, 64, 48, 96, threads=1)
    c4 = orc.matmul_f32(a, b, 64, 48, 96, threads=4)
    assert np.array_equal(c1.view(np.uint32), c4.view(np.uint32))


def test_primitive_table_reference_vectors(orc):
    """The integer / bit / compare primitives of the oracle's table on the reference's own vectors."""
    p = orc.prim
    # tests/runtime.rs:170-188, 190-212, 273-290 (two-times-two, sub-basic)
    two = p("u64.add", p("u64.one"), p("u64.one"))
    assert p("u64.mul", two, two) == 4 and p("u64.sub", two, p("u64.one")) == 1
    two32 = p("u32.add", p("u32.one"), p("u32.one"))
    assert p("u32.mul", two32, two32) == 4
    # tests/runtime.rs:214-271
    assert [p(f"u64.{op}", 2, 3) for op in ("ne", "lt", "lte", "gte")] == [1, 1, 1, 0]
    # tests/runtime.rs:313-331, 333-363 (fma-basic; fused against separate bits)
    one = p("f32.one")
    assert p("f32.fma", one, one, one) == 0x40000000
    assert p("f32.fma", 0x3F800001, 0x3F800001, 0x33800000) == 0x3F800003
    assert p("f32.add", p("f32.mul", 0x3F800001, 0x3F800001), 0x33800000) == 0x3F800002
    # tests/runtime.rs:408-446 (bitcasts)
    assert p("u32.bitcast-f32", 0x3F800000) == 0x3F800000 and p("f32.bitcast-u32", one) == 0x3F800000
    # tests/runtime.rs:448-473 (shift-and-sub: (0x20 >> 3) - (1 << 3) wraps)
    assert p("u32.sub", p("u32.shr", 0x20, 3), p("u32.shl", 1, 3)) == 0xFFFFFFFC
    # tests/runtime.rs:475-530
    assert p("u32.and", 0x00FF00FF, 0x0F0F0F0F) == 0x000F000F and p("u32.or", 0x00FF00FF, 0x0F0F0F0F) == 0x0FFF0FFF
    assert p("u32.xor", 0x00FF00FF, 0x0F0F0F0F) == 0x0FF00FF0 and p("u32.not", 0x00FF00FF) == 0xFF00FF00
    # tests/runtime.rs:532-605, 607-680 (2 against 3; 1.5 against 2.5)
    assert [p(f"u32.{op}", 2, 3) for op in ("eq", "ne", "lt", "gt", "lte", "gte")] == [0, 1, 1, 0, 1, 0]
    assert [p(f"f32.{op}", 0x3FC00000, 0x40200000) for op in ("lt", "eq", "ne", "gt", "lte", "gte")] == [1, 0, 1, 0, 1, 0]
    # tests/runtime.rs:15-35 of tests/cases (bool), tests/runtime.rs:37-52
    assert p("bool.not", 0) == 1 and p("bool.and", 1, 0) == 0 and p("bool.or", 0, 1) == 1
    # conversions: exact below 2^24 (stdlib/data.hex:127-128), to nearest even above
    assert p("u64.to-f32", (1 << 24) + 1) == 0x4B800000 and p("u64.to-f32", (1 << 24) + 3) == 0x4B800002
    assert p("f32.round-to-u32", 0x40200000) == 2 and p("f32.round-to-u32", 0x40600000) == 4      # 2.5 -> 2, 3.5 -> 4
