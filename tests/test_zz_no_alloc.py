"""catena_b200_sum_f32_noalloc: the sum for callers that must not let the library allocate (a host
that gave all of HBM to its own arena at start-up, or a loop that cannot afford the device-wide
synchronisation of a cudaMalloc).  Its reduction partials sit in a fixed array inside the library, so
the call takes only caller-owned device pointers.  Checked against program_sum_f32, which it must
match bit for bit (same tree), on two calls in a row — the second call finds the array holding the
first call's partials.  Collected last so a run that stops at the first failure has already run
every other test."""
import ctypes as C

import numpy as np
import pytest

import catena_lang_b200 as cb

pytestmark = pytest.mark.gpu


def bits(x):
    return int(np.float32(x).view(np.uint32))


def test_sum_noalloc_matches_program_sum_twice():
    L = cb.lib()
    assert L.catena_b200_device_count() > 0
    cb.check(L.catena_b200_init(0))
    rng = np.random.default_rng(11)
    # buffers are allocated up front by the caller; the entry point itself allocates nothing
    cases = [rng.normal(0, 3, (1 << 22) + 4321).astype(np.float32),     # tree path, ragged tail
             rng.normal(1, 2, 70000).astype(np.float32),                  # smallest tree sizes
             rng.normal(0, 1, 5000).astype(np.float32)]                   # sequential path, no scratch
    out = cb.CatenaMem()
    cb.check(L.catena_b200_mem_alloc(4, C.byref(out)))
    for x in cases:
        m = cb.upload(x)
        want = C.c_float()
        cb.check(L.program_sum_f32_s(m, C.byref(want)))
        for _ in range(2):
            cb.check(L.catena_b200_sum_f32_noalloc(m.data, x.size, out.data))
            got = cb.download(out, np.float32)[0]
            assert bits(got) == bits(want.value)
        cb.free(m)
    # a different, shorter input right after a long one: stale partials must not leak into the result
    a = rng.normal(0, 3, 1 << 21).astype(np.float32)
    b = rng.normal(5, 1, 100000).astype(np.float32)
    ma, mb = cb.upload(a), cb.upload(b)
    wa, wb = C.c_float(), C.c_float()
    cb.check(L.program_sum_f32_s(ma, C.byref(wa)))
    cb.check(L.program_sum_f32_s(mb, C.byref(wb)))
    cb.check(L.catena_b200_sum_f32_noalloc(ma.data, a.size, out.data))
    assert bits(cb.download(out, np.float32)[0]) == bits(wa.value)
    cb.check(L.catena_b200_sum_f32_noalloc(mb.data, b.size, out.data))
    assert bits(cb.download(out, np.float32)[0]) == bits(wb.value)
    # empty input: the fold's zero element
    cb.check(L.catena_b200_sum_f32_noalloc(None, 0, out.data))
    assert bits(cb.download(out, np.float32)[0]) == 0
    for mem in (ma, mb, out):
        cb.free(mem)


def test_sum_noalloc_rejects_oversize_and_null():
    L = cb.lib()
    cb.check(L.catena_b200_init(0))
    out = cb.CatenaMem()
    cb.check(L.catena_b200_mem_alloc(4, C.byref(out)))
    # beyond the fixed array's reach: refused before anything is launched (the pointer is never read)
    assert L.catena_b200_sum_f32_noalloc(out.data, (1 << 30) + 1, out.data) == cb.E_TOO_LARGE
    assert L.catena_b200_sum_f32_noalloc(out.data, 16, None) == cb.E_BAD_ARG
    cb.free(out)
