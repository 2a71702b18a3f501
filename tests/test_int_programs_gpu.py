"""The u64 buffer programs of the reference's tests on the GPU, registered from their LOWERED modules with
`Runtime.from_modules` (the selector maps them to the u64 fold kernels and the buffer-head copy) and called through
`Runtime.exec`, against the reference's vectors and the CPU oracle.  Arithmetic is modulo 2^64, so every length is
bit-exact."""
import numpy as np
import pytest

import catena_lang_b200 as cb

import lowered_fixtures as fx

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    cb.check(cb.lib().catena_b200_init(0))
    return cb.Runtime.from_modules(fx.reducec_programs() + fx.array_head_program() + fx.all_host_modules())


def test_selector_picks_the_u64_kernels(rt):
    assert rt.signatures["sum-u64"][0] == "program_sum_u64"
    assert rt.signatures["dot-u64"][0] == "program_dot_u64"
    assert rt.signatures["array-head-u64"][0] == "program_array_head_u64"
    assert "sum-u64-at" not in rt.signatures               # a `buf` pointer on its boundary: internal (signature.rs:63-72)


def test_reference_vectors(rt):
    # tests/cases/reducec.rs:6-20, 36-48; tests/runtime.rs:713-740
    [r] = rt.exec("sum-u64", [rt.mem_u64([2, 3, 5, 7, 11])])
    assert r.kind is cb.ValueKind.U64 and r.v == 28
    [r] = rt.exec("dot-u64", [rt.mem_u64([2, 3, 5, 7]), rt.mem_u64([11, 13, 17, 19])])
    assert r.v == 2 * 11 + 3 * 13 + 5 * 17 + 7 * 19
    values = [0x123456789ABCDEF0, 7, 11]
    [r] = rt.exec("array-head-u64", [rt.mem_u64(values)])
    assert r.v == values[0]
    # scalar modules registered next to them still run on the host
    assert rt.exec("shift-and-sub", [])[0].v == 0xFFFFFFFC


def test_asserts_are_statuses(rt):
    with pytest.raises(cb.ExecError) as e:
        rt.exec("dot-u64", [rt.mem_u64([1, 2]), rt.mem_u64([1, 2, 3])])        # mem.cast.u64.same-length
    assert e.value.status == cb.E_ASSERT
    with pytest.raises(cb.ExecError) as e:
        rt.exec("array-head-u64", [rt.mem_u64([])])                              # u64.assert-nz
    assert e.value.status == cb.E_ASSERT
    assert rt.exec("sum-u64", [rt.mem_u64([])])[0].v == 0                        # an empty fold is its zero element


@pytest.mark.parametrize("n", [1, 2, 3, 255, 256, 4097, 1 << 20, (1 << 24) + 12345])
def test_u64_folds_bit_exact_for_every_length(rt, orc, n):
    rng = np.random.default_rng(n)
    x = rng.integers(0, 2 ** 64, n, dtype=np.uint64)                            # sums and products wrap many times
    y = rng.integers(0, 2 ** 64, n, dtype=np.uint64)
    assert rt.exec("sum-u64", [rt.mem_u64(x)])[0].v == orc.sum_u64(x)
    assert rt.exec("dot-u64", [rt.mem_u64(x), rt.mem_u64(y)])[0].v == orc.dot_u64(x, y)
    assert rt.exec("array-head-u64", [rt.mem_u64(x)])[0].v == int(x[0])


def test_unaligned_buffer_takes_the_scalar_path(orc):
    """A buffer that starts 8 bytes into an allocation is not 16-byte aligned: the kernel falls back to 8-byte loads."""
    import ctypes as C
    x = np.random.default_rng(9).integers(0, 2 ** 64, 100001, dtype=np.uint64)
    m = cb.upload(x)
    out = C.c_uint64(0)
    part = cb.CatenaMem(m.data + 8, m.len - 8)
    cb.check(cb.lib().program_sum_u64_s(part, C.byref(out)))
    assert out.value == orc.sum_u64(x[1:])
    cb.check(cb.lib().program_dot_u64_s(part, part, C.byref(out)))
    assert out.value == orc.dot_u64(x[1:], x[1:])
    cb.free(m)
