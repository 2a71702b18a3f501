"""Parity tests proper: the CUDA path, called through the C ABI (`program_*` symbols via the
reference-shaped Runtime mirror), against the CPU oracle on the same seeded inputs.

Bar: bit-exact for integer / index results, for every elementwise program, for the f32 matmul
(any shape) and for folds of up to 65536 elements; stated tolerances elsewhere (written next to
each assert).  Vectors marked with a file:line come from the reference's own tests."""
import ctypes as C
import math

import numpy as np
import pytest

import catena_lang_b200 as cb

pytestmark = pytest.mark.gpu

MATMUL_SRC = """
(def program matmul-2x2-via-mem : x -> y = ())
(def program matmul-right-identity-2x2-via-mem : x -> y = ())
(def program matmul-left-identity-2x2-via-mem : x -> y = ())
(def program gemm-bf16-rc : x -> y = ())
(def program gemm-i8-rc : x -> y = ())
(def program attn-decode-bf16 : x -> y = ())
"""


@pytest.fixture(scope="module")
def rt():
    assert cb.lib().catena_b200_device_count() > 0, "GPU tests need a CUDA device"
    cb.check(cb.lib().catena_b200_init(0))
    return cb.Runtime.from_sources([MATMUL_SRC], cb.GpuDialect.Cuda)


def u32(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def matmul(rt, a, b, n, m, k):
    [r] = rt.exec("matmul-2x2-via-mem", [rt.mem_f32(a), rt.mem_f32(b), n, m, k, n * k, k * m, n * m])
    return r.v.to_f32_vec()


# ---------------------------------------------------------------- f32 matmul (bit-exact)
def test_matmul_reference_vectors(rt):
    # tests/cases/matrix.rs:6-82
    out = matmul(rt, [1, 2, 3, 4, 5, 6], [7, 8, 9, 10, 11, 12], 2, 2, 3)
    assert out.tolist() == [58.0, 64.0, 139.0, 154.0]
    a = [1.0, 2.0, 3.0, 4.0]
    [r] = rt.exec("matmul-right-identity-2x2-via-mem", [rt.mem_f32(a), 2, 4])
    assert r.v.to_f32_vec().tolist() == a
    [r] = rt.exec("matmul-left-identity-2x2-via-mem", [rt.mem_f32(a), 2, 4])
    assert r.v.to_f32_vec().tolist() == a


@pytest.mark.parametrize("n,m,k", [(256, 256, 256), (1, 1, 1), (37, 53, 29), (130, 70, 257), (64, 64, 1), (300, 270, 131),
                                   (513, 511, 40), (640, 1280, 96), (1000, 900, 515), (2200, 2250, 67)])
def test_matmul_bit_exact(rt, orc, n, m, k):
    """Every tile shape gives the oracle's bits: 16 x 16 tiles of one element per thread (tiny products), 16 x 32 with a 2 x 2
    register tile (small ones: 256^3, and 300 x 270 x 131 / 513 x 511 x 40 with ragged edges and a partial k slab), 64 x 64 with
    a 4 x 4 register tile, and — from 296 tiles of 128 x 128 on — an 8 x 8 register tile (the last case, ragged too).  All but
    the first work on pairs of columns with packed f32x2 arithmetic."""
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (n, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, m)).astype(np.float32)
    got = matmul(rt, a, b, n, m, k)
    want = orc.matmul_f32(a, b, n, m, k, threads=orc.max_threads())
    assert np.array_equal(u32(got), u32(want))


def test_matmul_large_tile_keeps_the_bits_of_special_values(rt, orc):
    """The 128 x 128 tile multiplies and adds PAIRS of columns with the packed f32x2 instructions (the product as a packed fma
    with -0 as addend): signed zeros, subnormal products and sums, values that overflow to infinity and infinities themselves
    come out as the oracle's separately rounded scalar chain has them."""
    n, m, k = 2200, 2250, 5
    rng = np.random.default_rng(9)
    pool = np.array([0.0, -0.0, 1.0, -1.0, 1e-30, -1e-30, 1e-20, 3e-39, -3e-39, 1e30, -1e30, 3e38, np.inf, 0.5, -2.0, 1e-45],
                    np.float32)
    a = pool[rng.integers(0, len(pool), (n, k))]
    b = pool[rng.integers(0, len(pool), (k, m))]
    got = matmul(rt, a, b, n, m, k)
    want = orc.matmul_f32(a, b, n, m, k, threads=orc.max_threads())
    assert np.array_equal(np.isnan(got), np.isnan(want))        # NaN payloads are a hardware property
    ok = ~np.isnan(want)
    assert np.array_equal(u32(got)[ok], u32(want)[ok])
    subnormal = (np.abs(want[ok]) > 0) & (np.abs(want[ok]) < np.float32(1.1754944e-38))
    assert ok.sum() > got.size // 2 and subnormal.any() and np.isinf(want[ok]).any()


def test_packed_products_round_separately_from_the_sums_behind_them():
    """What the packed f32x2 kernels rest on, measured on the device over 3.9e7 operand pairs: a product written as
    fma.rn.f32x2(a, b, -0) with a run-time -0, followed by a packed add, is the scalar __fadd_rn(c, __fmul_rn(a, b)) bit for bit.
    The count for a plain packed mul + add is reported, not asserted: with CUDA 12.9 the assembler merges the two into one fma
    (a third of the results differ); a toolchain that stops doing so would only make that count zero."""
    out = (C.c_uint64 * 3)()
    cb.check(cb.lib().catena_b200_debug_packed_f32x2_check(out))
    assert out[0] == 148 * 4 * 256 * 256 and out[1] == 0
    print(f"packed mul + add merged by the assembler in {out[2]} of {out[0]} pairs")


def test_matmul_signed_zero_and_specials(rt, orc):
    a = np.array([[-0.0, 0.0, -1.0], [np.inf, 1.0, -0.0]], np.float32)
    b = np.array([[0.0, 1.0], [-0.0, 2.0], [0.0, -3.0]], np.float32)
    got = matmul(rt, a, b, 2, 2, 3)
    want = orc.matmul_f32(a, b, 2, 2, 3)
    # NaN payload and sign are hardware properties (x86 default NaN is 0xFFC00000, the GPU's is
    # 0x7FFFFFFF); everything that is not a NaN must match bit for bit
    assert np.array_equal(np.isnan(got), np.isnan(want))
    ok = ~np.isnan(want)
    assert np.array_equal(u32(got)[ok], u32(want)[ok])


def test_matmul_length_assert_is_a_status_not_a_trap(rt):
    with pytest.raises(cb.ExecError) as e:
        rt.exec("matmul-2x2-via-mem", [rt.mem_f32([1, 2, 3]), rt.mem_f32([1, 2, 3, 4]), 2, 2, 2, 4, 4, 4])
    assert e.value.status == cb.E_ASSERT
    # the context is still usable
    assert matmul(rt, [2.0], [3.0], 1, 1, 1).tolist() == [6.0]


# ---------------------------------------------------------------- elementwise programs (bit-exact)
@pytest.mark.parametrize("name", cb.SCALAR_PROGRAMS)
def test_map_bit_exact(rt, orc, name):
    rng = np.random.default_rng(3)
    # magnitudes on both sides of 64 (and of 32, which tanh doubles): batches of eight values leave the kernels' short
    # rounding / reciprocal forms as soon as one of them is larger
    edge = np.array([64.0, -64.0, 32.0, -32.0], dtype=np.float32)
    edges = np.concatenate([edge, np.nextafter(edge, np.float32(np.inf)), np.nextafter(edge, np.float32(-np.inf))])
    x = np.concatenate([rng.uniform(-30, 30, 1 << 20), rng.normal(0, 1, 1 << 18), rng.uniform(-200, 200, 1 << 14),
                        rng.uniform(-70, 70, 1 << 14), edges, [3e4, -3e4, 700.0, -700.0],
                        [0.0, -0.0, 1.0, -1.0, 80.0, -80.0, 1e-30, 3.5]]).astype(np.float32)
    if name in ("math.log-approx", "math.log2-approx", "math.sin-approx-full-nonneg", "math.exp-approx-nonneg"):
        x = np.abs(x) + np.float32(1e-6)
    x = x[: x.size - 3]  # odd length: exercises the scalar tail
    m = cb.upload(x)
    out = cb.CatenaMem()
    cb.check(cb.lib().catena_b200_map_f32_s(name.encode(), m, C.byref(out)))
    got = cb.download(out, np.float32)
    cb.free(m), cb.free(out)
    want = orc.map_unary(name, x, threads=orc.max_threads())
    assert np.array_equal(u32(got), u32(want))


def test_gpu_materialize_with_explicit_launch_parameters(rt, orc):
    """gpu.materialize (stdlib/gpu.hex:39-49): the buffer has catena_launch_len(params) elements, element i the kernel's
    value for thread_id = i; the geometry given does not enter the result."""
    x = np.random.default_rng(5).uniform(-8, 8, 100).astype(np.float32)
    m = cb.upload(x)
    want = orc.map_unary("nn.silu", x, threads=1)
    for grid, block in (((3, 2, 1), (5, 1, 2)), ((1, 1, 1), (60, 1, 1)), ((60, 1, 1), (1, 1, 1))):
        params = cb.LaunchParams(cb.Dim3(*grid), cb.Dim3(*block))
        assert cb.lib().catena_b200_launch_len(params) == 60
        out = cb.CatenaMem()
        cb.check(cb.lib().catena_b200_gpu_materialize_f32_s(b"nn.silu", params, m, C.byref(out)))
        assert out.len == 240 and np.array_equal(u32(cb.download(out, np.float32)), u32(want[:60]))
        cb.free(out)
    out = cb.CatenaMem()
    too_long = cb.LaunchParams(cb.Dim3(101, 1, 1), cb.Dim3(1, 1, 1))
    assert cb.lib().catena_b200_gpu_materialize_f32_s(b"nn.silu", too_long, m, C.byref(out)) == cb.E_ASSERT
    huge = cb.LaunchParams(cb.Dim3(2 ** 32 - 1, 2 ** 32 - 1, 2 ** 32 - 1), cb.Dim3(1024, 1, 1))
    assert cb.lib().catena_b200_gpu_materialize_f32_s(b"nn.silu", huge, m, C.byref(out)) == cb.E_TOO_LARGE
    empty = cb.LaunchParams(cb.Dim3(0, 1, 1), cb.Dim3(32, 1, 1))
    cb.check(cb.lib().catena_b200_gpu_materialize_f32_s(b"nn.silu", empty, m, C.byref(out)))
    assert out.len == 0 and not out.data
    cb.free(m)


# ---------------------------------------------------------------- folds
def test_fold_reference_vectors(rt):
    # tests/cases/reducec.rs:50-90
    x = [1.5, -0.5, 2.0, 4.0]
    assert rt.exec("sum-f32", [rt.mem_f32(x)])[0].v == 7.0
    assert rt.exec("mean-f32", [rt.mem_f32(x)])[0].v == 1.75
    assert rt.exec("max-f32", [rt.mem_f32(x)])[0].v == 4.0
    assert u32(rt.exec("sum-f32", [rt.mem_f32([])])[0].v) == 0
    assert u32(rt.exec("max-f32", [rt.mem_f32([])])[0].v) == 0xFF800000


@pytest.mark.parametrize("n", [1, 7, 2048, 2049, 65536])
def test_fold_bit_exact_up_to_65536(rt, orc, n):
    x = np.random.default_rng(n).normal(0, 3, n).astype(np.float32)
    assert u32(rt.exec("sum-f32", [rt.mem_f32(x)])[0].v) == u32(orc.sum_f32(x))
    assert u32(rt.exec("mean-f32", [rt.mem_f32(x)])[0].v) == u32(orc.mean_f32(x))
    assert u32(rt.exec("max-f32", [rt.mem_f32(x)])[0].v) == u32(orc.max_f32(x))


@pytest.mark.parametrize("n", [65537, 1 << 20, (1 << 22) + 12345])
def test_fold_tree_tolerance_and_determinism(rt, orc, n):
    x = np.random.default_rng(n).normal(0, 3, n).astype(np.float32)
    s1 = rt.exec("sum-f32", [rt.mem_f32(x)])[0].v
    s2 = rt.exec("sum-f32", [rt.mem_f32(x)])[0].v
    assert u32(s1) == u32(s2)                                  # bitwise identical across runs
    exact = float(np.sum(x.astype(np.float64)))
    bound = 4e-7 * float(np.sum(np.abs(x.astype(np.float64))))   # ~ log2(n) * eps * sum|x|, far below the
    assert abs(s1 - exact) <= bound                             # sequential fold's own n * eps * sum|x|
    assert abs(s1 - float(orc.sum_f32(x))) <= 64 * bound
    assert u32(rt.exec("max-f32", [rt.mem_f32(x)])[0].v) == u32(orc.max_f32(x))   # order-free: exact


def test_argmax(rt, orc):
    # tests/runtime.rs:1170-1197 (ties keep the first index)
    for xs, want in [([5.0], 0), ([1, 2, 4], 2), ([4, 2, 1], 0), ([1, 7, 3, 2], 1), ([1, 7, 7, 2], 1), ([3, 3, 3], 0)]:
        assert rt.exec("tensor.argmax-f32", [rt.mem_f32(xs)])[0].v == want
    rng = np.random.default_rng(5)
    for n in [4097, 65536, 65537, 3_000_001]:
        x = rng.integers(0, 1000, n).astype(np.float32)        # many exact ties
        assert rt.exec("tensor.argmax-f32", [rt.mem_f32(x)])[0].v == orc.argmax_f32(x)
    with pytest.raises(cb.ExecError) as e:
        rt.exec("tensor.argmax-f32", [rt.mem_f32([])])
    assert e.value.status == cb.E_ASSERT


# ---------------------------------------------------------------- softmax / rmsnorm
def test_softmax_rmsnorm_reference_vectors(rt):
    # tests/runtime.rs:971-1044
    x = np.array([1.0, 2.0, 4.0], np.float32)
    y = rt.exec("nn.softmax", [rt.mem_f32(x)])[0].v.to_f32_vec()
    want = np.exp(x - x.max()) / np.exp(x - x.max()).sum()
    assert np.all(np.abs(y - want) < 6e-3) and abs(y.sum() - 1) < 6e-3
    x = np.array([1.0, 2.0, 4.0, -1.0, -9.0, 13.29], np.float32)
    y = rt.exec("nn.rmsnorm", [rt.mem_f32(x)])[0].v.to_f32_vec()
    rms = math.sqrt(float((x.astype(np.float64) ** 2).mean()) + 1e-5)
    assert np.all(np.abs(y - x / rms) < 3e-3)


@pytest.mark.parametrize("n", [1, 3, 128, 4096, 5000, 65536])
def test_softmax_rmsnorm_bit_exact_up_to_65536(rt, orc, n):
    x = np.random.default_rng(n).normal(0, 2, n).astype(np.float32)
    y = rt.exec("nn.softmax", [rt.mem_f32(x)])[0].v.to_f32_vec()
    assert np.array_equal(u32(y), u32(orc.softmax(x)))
    y = rt.exec("nn.rmsnorm", [rt.mem_f32(x)])[0].v.to_f32_vec()
    assert np.array_equal(u32(y), u32(orc.rmsnorm(x)))


def test_softmax_signed_zero_maximum_and_nan_input(rt, orc):
    """The parallel maximum may return either zero of a +0 / -0 tie where the reference's fold keeps the first: the output
    bits are the same.  With a NaN in the input the reference's result depends on the NaN's position (out of contract for
    the bit-exact claim): the call must still return, and the library must stay usable."""
    for x in ([-0.0, 0.0, -1.0, -2.5], [0.0, -0.0, -1.0, -2.5], [-3.0, -0.0, 0.0]):
        x = np.array(x, np.float32)
        y = rt.exec("nn.softmax", [rt.mem_f32(x)])[0].v.to_f32_vec()
        assert np.array_equal(u32(y), u32(orc.softmax(x)))
    y = rt.exec("nn.softmax", [rt.mem_f32(np.array([1.0, np.nan, 2.0], np.float32))])[0].v.to_f32_vec()
    assert y.size == 3
    x = np.array([1.0, 2.0, 4.0], np.float32)
    assert np.array_equal(u32(rt.exec("nn.softmax", [rt.mem_f32(x)])[0].v.to_f32_vec()), u32(orc.softmax(x)))


def test_softmax_rmsnorm_long_rows(rt, orc):
    """Beyond 65536 elements the denominator is a fixed-shape tree sum.  It is compared with the exact
    (float64) sum of the same fp32 terms: relative 1e-6.  The reference's sequential fp32 fold is itself
    far from that sum at this length (it loses the small terms once the accumulator is large), so the
    distance to the oracle is bounded by the fold's own error, n * 2^-24 relative, not by ours."""
    n = (1 << 21) + 77
    x = np.random.default_rng(1).normal(0, 2, n).astype(np.float32)
    y = rt.exec("nn.softmax", [rt.mem_f32(x)])[0].v.to_f32_vec()
    e = orc.map_unary("math.exp-approx", x - x.max(), threads=orc.max_threads()).astype(np.float64)
    exact = e / e.sum()
    assert np.all(np.abs(y - exact) <= 1e-6 * exact)
    want = orc.softmax(x, threads=orc.max_threads())
    assert np.all(np.abs(y - want) <= (n * 2.0 ** -24) * want)
    y2 = rt.exec("nn.softmax", [rt.mem_f32(x)])[0].v.to_f32_vec()
    assert np.array_equal(u32(y), u32(y2))                     # bitwise identical across runs
    y = rt.exec("nn.rmsnorm", [rt.mem_f32(x)])[0].v.to_f32_vec()
    rms = math.sqrt(float((x.astype(np.float64) ** 2).sum()) / n + 1e-5)
    assert np.all(np.abs(y - x / rms) <= 1e-4 * np.abs(x / rms))   # sqrt~ is the reference's 6-step Newton
    want = orc.rmsnorm(x, threads=orc.max_threads())
    assert np.all(np.abs(y - want) <= (n * 2.0 ** -24) * np.abs(want))


# ---------------------------------------------------------------- tensor programs (exact)
def test_tensor_programs(rt):
    # tests/runtime.rs:1046-1168
    assert rt.exec("tensor.broadcast-f32", [3.5, 0])[0].v.to_f32_vec().tolist() == []
    assert rt.exec("tensor.broadcast-f32", [3.5, 4])[0].v.to_f32_vec().tolist() == [3.5] * 4
    assert rt.exec("tensor.arange-f32", [0])[0].v.to_f32_vec().tolist() == []
    assert rt.exec("tensor.arange-f32", [5])[0].v.to_f32_vec().tolist() == [0, 1, 2, 3, 4]
    src = [10.0, 20.0, 30.0, 40.0]
    for start, ln, want in [(0, 2, [10, 20]), (1, 2, [20, 30]), (2, 0, []), (0, 4, src)]:
        assert rt.exec("tensor.slice-f32", [rt.mem_f32(src), start, ln])[0].v.to_f32_vec().tolist() == want
    with pytest.raises(cb.ExecError) as e:
        rt.exec("tensor.slice-f32", [rt.mem_f32(src), 3, 2])
    assert e.value.status == cb.E_ASSERT
    for l, r in [([1, 2], [3, 4]), ([1], [2, 3, 4]), ([], [3, 4]), ([1, 2], []), ([], [])]:
        got = rt.exec("tensor.concat-f32", [rt.mem_f32(l), rt.mem_f32(r)])[0].v.to_f32_vec().tolist()
        assert got == [float(v) for v in l + r]


def test_tensor_programs_large(rt):
    n = 3_000_003
    got = rt.exec("tensor.arange-f32", [n])[0].v.to_f32_vec()
    assert np.array_equal(got, np.arange(n, dtype=np.uint64).astype(np.float32))
    x = np.random.default_rng(2).normal(size=n).astype(np.float32)
    got = rt.exec("tensor.slice-f32", [rt.mem_f32(x), 1001, n - 2002])[0].v.to_f32_vec()
    assert np.array_equal(u32(got), u32(x[1001:n - 1001]))
    got = rt.exec("tensor.concat-f32", [rt.mem_f32(x[:12345]), rt.mem_f32(x[12345:])])[0].v.to_f32_vec()
    assert np.array_equal(u32(got), u32(x))


# ---------------------------------------------------------------- tensor-core GEMMs
def bf16_inputs(seed, m, n, k):
    import oracle
    rng = np.random.default_rng(seed)
    a = oracle.f32_to_bf16_bits((rng.standard_normal((m, k)) / math.sqrt(k)).astype(np.float32))
    bt = oracle.f32_to_bf16_bits((rng.standard_normal((n, k)) / math.sqrt(k)).astype(np.float32))
    return a, bt


def assert_bf16_close(got_bits, want_bits, want_f32, floor, max_mismatch):
    """`got` must be the bf16 rounding of an fp32 value that differs from the oracle's fp32 value by
    accumulation order only: within one bf16 ulp of the oracle's fp32 result, plus an absolute floor for
    outputs that cancel to (nearly) zero, where one ulp of the result is smaller than fp32 rounding of
    the partial sums.  Also bounds the fraction of outputs whose bf16 bits differ at all."""
    import oracle
    got = oracle.bf16_bits_to_f32(got_bits.ravel())
    want = want_f32.ravel()
    assert np.all(np.abs(got - want) <= 2.0 ** -8 * np.abs(want) + floor)
    assert (got_bits.ravel() != want_bits.ravel()).mean() < max_mismatch


def run_gemm_bf16(rt, a, bt, m, n, k):
    [r] = rt.exec("gemm-bf16-rc", [rt.mem_bytes(a), rt.mem_bytes(bt), m, n, k])
    return r.v.to_array(np.uint16).reshape(m, n)


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 512), (256, 512, 128), (200, 264, 72), (1, 8, 8),
                                   (1024, 1024, 1024), (333, 1000, 200)])
def test_gemm_bf16_vs_oracle(rt, orc, m, n, k):
    a, bt = bf16_inputs(1, m, n, k)
    got = run_gemm_bf16(rt, a, bt, m, n, k)
    want, want_f32 = orc.gemm_bf16_rows(a, bt, n, k, 0, m, threads=orc.max_threads(), want_f32=True)
    # fp32 accumulation in tensor-core order vs the sequential fp32 fold: the two fp32 sums differ by
    # rounding only, so after rounding to bf16 they agree except where the sum sits on a rounding
    # boundary: 1 bf16 ulp apart, on well under 1 % of the outputs
    assert_bf16_close(got, want, want_f32, 1e-6, 0.01)


def test_gemm_bf16_4096_rows_determinism_and_grid_independence(rt, orc):
    m = n = k = 4096
    a, bt = bf16_inputs(1, m, n, k)
    got = run_gemm_bf16(rt, a, bt, m, n, k)
    again = run_gemm_bf16(rt, a, bt, m, n, k)
    assert np.array_equal(got, again)                         # bitwise identical across runs
    cb.lib().catena_b200_debug_set_cta_limit(37)
    try:
        small_grid = run_gemm_bf16(rt, a, bt, m, n, k)
    finally:
        cb.lib().catena_b200_debug_set_cta_limit(0)
    assert np.array_equal(got, small_grid)                    # the grid size never enters the arithmetic
    for row0 in (0, 2048 + 64, 4096 - 32):                    # oracle slabs (the full product takes minutes on a CPU)
        want, want_f32 = orc.gemm_bf16_rows(a, bt, n, k, row0, row0 + 32, threads=orc.max_threads(), want_f32=True)
        assert_bf16_close(got[row0:row0 + 32], want, want_f32, 1e-6, 0.01)
    # column-block partitioning (how the GEMM shards across GPUs) gives the same bits
    am, btm = cb.upload(a), cb.upload(bt)
    cm = cb.CatenaMem()
    cb.check(cb.lib().catena_b200_mem_alloc(m * n * 2, C.byref(cm)))
    parts = 4
    for p in range(parts):
        n0 = p * (n // parts)
        cb.check(cb.lib().catena_b200_gemm_bf16_into(am.data, btm.data + n0 * k * 2, cm.data + n0 * 2, m, n // parts, k, n))
    sharded = cb.download(cm, np.uint16).reshape(m, n)
    for x in (am, btm, cm):
        cb.free(x)
    assert np.array_equal(got, sharded)


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (256, 512, 256), (200, 264, 80), (1, 4, 16), (1024, 1024, 2048),
                                   (333, 1000, 208)])
def test_gemm_i8_bit_exact(rt, orc, m, n, k):
    rng = np.random.default_rng(4)
    a = rng.integers(-128, 128, (m, k), dtype=np.int8)
    bt = rng.integers(-128, 128, (n, k), dtype=np.int8)
    [r] = rt.exec("gemm-i8-rc", [rt.mem_bytes(a), rt.mem_bytes(bt), m, n, k])
    got = r.v.to_array(np.int32).reshape(m, n)
    want = orc.gemm_i8_rows(a, bt, n, k, 0, m, threads=orc.max_threads())
    assert np.array_equal(got, want)


@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (512, 768, 256), (200, 264, 72), (333, 1000, 200), (2048, 2304, 512),
                                   (4096, 4096, 4096)])
def test_gemm_pair_and_single_cta_kernels_agree_bitwise(rt, m, n, k):
    """Two independent implementations (tcgen05 cta_group::2 on CTA pairs with 256-row tiles and a
    6-stage ring; cta_group::1 with 128-row tiles and a 4-stage ring), different tile -> SM maps and
    different widths for the units of the last round: the output bits must not depend on any of it."""
    a, bt = bf16_inputs(7, m, n, k)
    rng = np.random.default_rng(8)
    k8 = max(16, k // 16 * 16)
    ai = rng.integers(-128, 128, (m, k8), dtype=np.int8)
    bi = rng.integers(-128, 128, (n, k8), dtype=np.int8)
    out = {}
    try:
        for pair in (1, 0):
            cb.lib().catena_b200_debug_set_gemm_pair(pair)
            out[pair] = (run_gemm_bf16(rt, a, bt, m, n, k),
                         rt.exec("gemm-i8-rc", [rt.mem_bytes(ai), rt.mem_bytes(bi), m, n, k8])[0].v.to_array(np.int32))
    finally:
        cb.lib().catena_b200_debug_set_gemm_pair(1)
    assert np.array_equal(out[0][0], out[1][0])
    assert np.array_equal(out[0][1], out[1][1])


def test_gemm_i8_extremes(rt):
    m, n, k = 128, 256, 8192
    a = np.full((m, k), -128, np.int8)
    bt = np.full((n, k), -128, np.int8)
    [r] = rt.exec("gemm-i8-rc", [rt.mem_bytes(a), rt.mem_bytes(bt), m, n, k])
    assert np.all(r.v.to_array(np.int32) == 128 * 128 * k)   # 134 217 728 < 2^31


def test_gemm_rejects_bad_shapes(rt):
    a, bt = bf16_inputs(1, 16, 16, 12)
    with pytest.raises(cb.ExecError) as e:
        rt.exec("gemm-bf16-rc", [rt.mem_bytes(a), rt.mem_bytes(bt), 16, 16, 12])    # K*2 not a multiple of 16 B
    assert e.value.status == cb.E_BAD_ARG


@pytest.mark.parametrize("n", [320, 296, 512])
def test_gemm_peer_stores_write_every_copy(rt, n):
    """The gather-fused GEMM stores each output tile to C and to the peer copies: here the "peers" are two more
    buffers of the same GPU, which must end up with the bits of the plain GEMM in their rows and nothing elsewhere.
    (Widths that end inside a 64-column line take the element-wise path for that line.)"""
    import oracle
    m, k, rows_total, row0 = 384, 256, 640, 128
    rng = np.random.default_rng(11)
    a = oracle.f32_to_bf16_bits(rng.standard_normal((m, k)).astype(np.float32) / 16)
    b = oracle.f32_to_bf16_bits(rng.standard_normal((n, k)).astype(np.float32) / 16)
    am, bm = cb.upload(a), cb.upload(b)
    cm = cb.CatenaMem(); cb.check(cb.lib().catena_b200_mem_alloc(m * n * 2, C.byref(cm)))
    cb.check(cb.lib().catena_b200_gemm_bf16_into(am.data, bm.data, cm.data, m, n, k, n))
    want = cb.download(cm, np.uint16).reshape(m, n)
    fill = np.full((rows_total, n), 0x7FC0, np.uint16)
    peers = [cb.upload(fill), cb.upload(fill)]
    ptrs = (C.c_void_p * 2)(*[p.data + row0 * n * 2 for p in peers])
    cb.check(cb.lib().catena_b200_mem_write(cm, np.zeros(m * n, np.uint16).ctypes.data_as(C.c_void_p), m * n * 2))
    cb.check(cb.lib().catena_b200_gemm_bf16_into_peers(am.data, bm.data, cm.data, m, n, k, n, ptrs, 2))
    assert np.array_equal(cb.download(cm, np.uint16).reshape(m, n), want)
    for p in peers:
        got = cb.download(p, np.uint16).reshape(rows_total, n)
        assert np.array_equal(got[row0:row0 + m], want)
        assert (got[:row0] == 0x7FC0).all() and (got[row0 + m:] == 0x7FC0).all()
    # needs the CTA-pair kernel
    assert cb.lib().catena_b200_gemm_bf16_into_peers(am.data, bm.data, cm.data, 64, n, k, n, ptrs, 2) == cb.E_UNSUPPORTED
    for x in [am, bm, cm] + peers:
        cb.free(x)


# ---------------------------------------------------------------- cached-attention decode
def attn_inputs(B, Hq, Hkv, L, D=128, seeds=(2, 3, 4)):
    import oracle
    q = oracle.f32_to_bf16_bits(np.random.default_rng(seeds[0]).standard_normal((B, Hq, D)).astype(np.float32))
    k = oracle.f32_to_bf16_bits(np.random.default_rng(seeds[1]).standard_normal((B, Hkv, L, D)).astype(np.float32))
    v = oracle.f32_to_bf16_bits(np.random.default_rng(seeds[2]).standard_normal((B, Hkv, L, D)).astype(np.float32))
    return q, k, v


def run_attn(rt, q, k, v, B, Hq, Hkv, L, D=128):
    [r] = rt.exec("attn-decode-bf16", [rt.mem_bytes(q), rt.mem_bytes(k), rt.mem_bytes(v), B, Hq, Hkv, D, L])
    return r.v.to_array(np.uint16).reshape(B, Hq, D)


def last_attn_launch():
    """(kernel, resident CTAs or clusters, launched, shared memory) of this thread's last decode launch."""
    g = (C.c_uint32 * 4)()
    cb.lib().catena_b200_debug_attn_last_launch(g)
    return list(g)


@pytest.fixture(params=["tcgen05", "mma.sync"])
def attn_kernel(request):
    """Runs a test once per decode kernel: the tcgen05 kernel (the default wherever it applies) and the
    mma.sync kernel (the fallback for long caches)."""
    cb.lib().catena_b200_debug_set_attn_tc(1 if request.param == "tcgen05" else 0)
    yield request.param
    cb.lib().catena_b200_debug_set_attn_tc(1)


@pytest.mark.parametrize("B,Hq,Hkv,L", [(2, 8, 2, 256), (1, 4, 1, 64), (3, 8, 8, 333), (2, 16, 2, 77), (1, 2, 1, 1),
                                        (2, 8, 4, 1000), (1, 32, 8, 4096), (1, 8, 2, 7168)])
def test_attn_decode_vs_oracle(rt, orc, attn_kernel, B, Hq, Hkv, L):
    q, k, v = attn_inputs(B, Hq, Hkv, L)
    got = run_attn(rt, q, k, v, B, Hq, Hkv, L)
    assert last_attn_launch()[0] == (1 if attn_kernel == "tcgen05" else 0)
    want, want_f32 = orc.attn_decode_bf16(q, k, v, B, Hq, Hkv, 128, L, np.float32(1.0 / math.sqrt(128.0)),
                                          threads=orc.max_threads(), want_f32=True)
    # same probabilities (global max, the reference's exp polynomial); only fp32 summation order
    # differs from the sequential folds, so the bf16 outputs agree to 1 ulp, nearly always exactly
    assert_bf16_close(got, want, want_f32, 4e-6, 0.02)


def test_attn_decode_long_cache_falls_back(rt, orc):
    """More than 7 score tiles per chunk do not fit the tcgen05 kernel's TMEM sets: the mma.sync kernel takes over."""
    B, Hq, Hkv, L = 1, 4, 1, 8192
    q, k, v = attn_inputs(B, Hq, Hkv, L)
    got = run_attn(rt, q, k, v, B, Hq, Hkv, L)
    assert last_attn_launch()[0] == 0
    want, want_f32 = orc.attn_decode_bf16(q, k, v, B, Hq, Hkv, 128, L, np.float32(1.0 / math.sqrt(128.0)),
                                          threads=orc.max_threads(), want_f32=True)
    assert_bf16_close(got, want, want_f32, 4e-6, 0.02)


def test_attn_decode_kernels_agree(rt):
    """Same semantics in both kernels: the outputs differ at most in the last bf16 bit of a few elements
    (the tensor cores add the 16 products of a k-step in a different order)."""
    B, Hq, Hkv, L = 4, 32, 8, 2048
    q, k, v = attn_inputs(B, Hq, Hkv, L)
    outs = []
    for tc in (1, 0):
        cb.lib().catena_b200_debug_set_attn_tc(tc)
        try:
            outs.append(run_attn(rt, q, k, v, B, Hq, Hkv, L))
        finally:
            cb.lib().catena_b200_debug_set_attn_tc(1)
    import oracle
    a, b = (oracle.bf16_bits_to_f32(x.ravel()) for x in outs)
    assert np.mean(outs[0] == outs[1]) > 0.99
    assert np.all(np.abs(a - b) <= 2.0 ** -7 * np.maximum(np.abs(a), np.abs(b)) + 4e-6)


def test_attn_decode_c3_partition_and_determinism(rt, orc, attn_kernel):
    B, Hq, Hkv, L = 32, 32, 8, 4096
    q, k, v = attn_inputs(B, Hq, Hkv, L)
    got = run_attn(rt, q, k, v, B, Hq, Hkv, L)
    full = last_attn_launch()
    again = run_attn(rt, q, k, v, B, Hq, Hkv, L)
    assert np.array_equal(got, again)
    cb.lib().catena_b200_debug_set_cta_limit(40)              # a fraction of the resident CTAs / clusters
    try:
        few_clusters = run_attn(rt, q, k, v, B, Hq, Hkv, L)
        assert last_attn_launch()[2] < full[2]
    finally:
        cb.lib().catena_b200_debug_set_cta_limit(0)
    assert np.array_equal(got, few_clusters)                  # the grid never enters the arithmetic
    units = list(range(0, B * Hq, 97))[:12]                   # oracle on a sample of (batch, head) rows
    for u in units:
        want, want_f32 = orc.attn_decode_bf16(q, k, v, B, Hq, Hkv, 128, L, np.float32(1.0 / math.sqrt(128.0)),
                                              unit0=u, unit1=u + 1, want_f32=True)
        assert_bf16_close(got.reshape(-1, 128)[u], want.reshape(-1, 128)[u], want_f32.reshape(-1, 128)[u], 4e-6, 0.05)
    # sharding by (batch, kv-head) ranges, as across GPUs, gives the same bits
    qm, km, vm = cb.upload(q), cb.upload(k), cb.upload(v)
    om = cb.CatenaMem()
    cb.check(cb.lib().catena_b200_mem_alloc(B * Hq * 128 * 2, C.byref(om)))
    total = B * Hkv
    for lo, hi in [(0, 100), (100, 101), (101, total)]:
        cb.check(cb.lib().catena_b200_attn_decode_bf16_into(qm.data, km.data, vm.data, om.data, B, Hq, Hkv, 128, L, lo, hi))
    sharded = cb.download(om, np.uint16).reshape(B, Hq, 128)
    for x in (qm, km, vm, om):
        cb.free(x)
    assert np.array_equal(got, sharded)


def test_attn_peer_stores_write_every_copy(rt):
    """The gather-fused decode stores every unit's outputs to O and to the peer copies of O: here the "peers" are two more
    buffers of the same GPU.  Two launches over disjoint unit ranges must leave the plain launch's bits in all three
    buffers, and nothing outside the launched ranges."""
    B, Hq, Hkv, L = 4, 8, 2, 900
    q, k, v = attn_inputs(B, Hq, Hkv, L)
    want = run_attn(rt, q, k, v, B, Hq, Hkv, L)
    G = Hq // Hkv
    qm, km, vm = cb.upload(q), cb.upload(k), cb.upload(v)
    fill = np.full((B * Hkv, G * 128), 0x7FC0, np.uint16)
    outs = [cb.upload(fill) for _ in range(3)]
    ptrs = (C.c_void_p * 2)(outs[1].data, outs[2].data)
    L_ = cb.lib()
    for lo, hi in ((0, 3), (5, 8)):                            # units 3 and 4 are left out
        cb.check(L_.catena_b200_attn_decode_bf16_into_peers(qm.data, km.data, vm.data, outs[0].data, B, Hq, Hkv, 128, L, lo, hi, ptrs, 2))
    w = want.reshape(B * Hkv, G * 128)
    for o in outs:
        got = cb.download(o, np.uint16).reshape(B * Hkv, G * 128)
        assert np.array_equal(got[:3], w[:3]) and np.array_equal(got[5:], w[5:])
        assert (got[3:5] == 0x7FC0).all()
    # the mma.sync kernel has no peer stores
    cb.lib().catena_b200_debug_set_attn_tc(0)
    try:
        assert L_.catena_b200_attn_decode_bf16_into_peers(qm.data, km.data, vm.data, outs[0].data, B, Hq, Hkv, 128, L, 0, 8, ptrs, 2) == cb.E_UNSUPPORTED
    finally:
        cb.lib().catena_b200_debug_set_attn_tc(1)
    for x in [qm, km, vm] + outs:
        cb.free(x)


def test_attn_rejects_unsupported(rt):
    q, k, v = attn_inputs(1, 4, 1, 16)
    with pytest.raises(cb.ExecError) as e:
        rt.exec("attn-decode-bf16", [rt.mem_bytes(q), rt.mem_bytes(k), rt.mem_bytes(v), 1, 4, 1, 64, 32])
    assert e.value.status in (cb.E_UNSUPPORTED, cb.E_ASSERT)
