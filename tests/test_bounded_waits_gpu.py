"""The give-up path of the bounded device-side waits, and the allocator under two host threads.

A wait that runs out is not a fault: the waiting role records an error code, the kernel lets its copies land, frees its
tensor memory and returns, and the host reports CATENA_E_TIMEOUT (the reference's generated code would trap,
catena-lang/src/codegen/prelude.rs:38-55).  The tests shorten the limit to a few milliseconds, make one hand-over
never happen (a test hook: producers that stop early, a chunk maximum that is never published), check the status, and
then check that the same library instance still computes the right bits.
"""
import ctypes as C
import math
import threading

import numpy as np
import pytest

import catena_lang_b200 as cb

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def device():
    cb.check(cb.lib().catena_b200_init(0))


@pytest.fixture
def short_waits():
    L = cb.lib()
    L.catena_b200_debug_set_wait_limit_ns(3_000_000)          # 3 ms instead of one second
    yield L
    L.catena_b200_debug_set_wait_limit_ns(0)
    L.catena_b200_debug_stall_next(1, 0)
    L.catena_b200_debug_stall_next(2, 0)
    L.catena_b200_set_blocking(1)
    L.catena_b200_clear_status()


def alloc(nbytes):
    m = cb.CatenaMem()
    cb.check(cb.lib().catena_b200_mem_alloc(nbytes, C.byref(m)))
    return m


def bf16(rng, shape, std=1.0):
    import oracle
    return oracle.f32_to_bf16_bits((rng.standard_normal(shape) * std).astype(np.float32)).reshape(shape)


def test_gemm_wait_runs_out_then_the_library_recovers(short_waits):
    L = short_waits
    m, n, k = 512, 512, 512                                   # four CTA pairs, eight k-blocks each
    rng = np.random.default_rng(21)
    a, b = bf16(rng, (m, k), 1 / math.sqrt(k)), bf16(rng, (n, k), 1 / math.sqrt(k))
    am, bm, cm = cb.upload(a), cb.upload(b), alloc(m * n * 2)
    try:
        cb.check(L.catena_b200_gemm_bf16_into(am.data, bm.data, cm.data, m, n, k, n))
        want = cb.download(cm, np.uint16)
        # blocking mode: the entry point itself reports the expiry
        L.catena_b200_debug_stall_next(1, 4)                  # the producers stop before k-block 3 of their first tile
        assert L.catena_b200_gemm_bf16_into(am.data, bm.data, cm.data, m, n, k, n) == cb.E_TIMEOUT
        assert L.catena_b200_last_status() == cb.E_TIMEOUT
        L.catena_b200_clear_status()
        cb.check(L.catena_b200_gemm_bf16_into(am.data, bm.data, cm.data, m, n, k, n))     # the stall was one-shot
        assert np.array_equal(cb.download(cm, np.uint16), want)
        # non-blocking mode: the launch returns at once, the expiry is read afterwards
        L.catena_b200_set_blocking(0)
        L.catena_b200_debug_stall_next(1, 1)                  # not even the first k-block arrives
        cb.check(L.catena_b200_gemm_bf16_into(am.data, bm.data, cm.data, m, n, k, n))
        assert L.catena_b200_check_device_errors() == cb.E_TIMEOUT
        assert L.catena_b200_check_device_errors() == cb.OK  # reported once, then cleared
        L.catena_b200_set_blocking(1)
        L.catena_b200_clear_status()
        cb.check(L.catena_b200_gemm_bf16_into(am.data, bm.data, cm.data, m, n, k, n))
        assert np.array_equal(cb.download(cm, np.uint16), want)
    finally:
        for x in (am, bm, cm):
            cb.free(x)


def test_attention_poll_runs_out_then_the_library_recovers(short_waits):
    L = short_waits
    B, Hq, Hkv, Lk = 4, 8, 2, 1024                            # 8 units, 64 chunk items
    rng = np.random.default_rng(22)
    q, k, v = bf16(rng, (B, Hq, 128)), bf16(rng, (B, Hkv, Lk, 128)), bf16(rng, (B, Hkv, Lk, 128))
    qm, km, vm, om = cb.upload(q), cb.upload(k), cb.upload(v), alloc(B * Hq * 128 * 2)
    args = (qm.data, km.data, vm.data, om.data, B, Hq, Hkv, 128, Lk, 0, B * Hkv)
    try:
        cb.check(L.catena_b200_attn_decode_bf16_into(*args))
        want = cb.download(om, np.uint16)
        L.catena_b200_debug_stall_next(2, 1)                  # item 0 never publishes its chunk maxima
        assert L.catena_b200_attn_decode_bf16_into(*args) == cb.E_TIMEOUT
        L.catena_b200_clear_status()
        cb.check(L.catena_b200_attn_decode_bf16_into(*args))  # exchange area and tickets were reset
        assert np.array_equal(cb.download(om, np.uint16), want)
        cb.check(L.catena_b200_attn_decode_bf16_into(*args))
        assert np.array_equal(cb.download(om, np.uint16), want)
    finally:
        for x in (qm, km, vm, om):
            cb.free(x)


def test_two_host_threads_two_streams_share_the_pool():
    """Two host threads drive one device on their own streams in non-blocking mode and allocate, use and free blocks of
    the same size classes in a tight loop.  A block freed by one thread while its kernels are still queued may be handed
    to the other thread at once; the pool orders that reuse after the freeing stream's work, so every result equals the
    single-threaded one."""
    import torch
    L = cb.lib()
    rng = np.random.default_rng(23)
    n = 1 << 20
    xs = [rng.normal(0, 2, n).astype(np.float32) for _ in range(2)]
    m, nn, k = 384, 512, 256
    ab = [(bf16(rng, (m, k), 1 / 16), bf16(rng, (nn, k), 1 / 16)) for _ in range(2)]
    B, Hq, Hkv, Lk = 2, 8, 2, 512
    qkv = [(bf16(rng, (B, Hq, 128)), bf16(rng, (B, Hkv, Lk, 128)), bf16(rng, (B, Hkv, Lk, 128))) for _ in range(2)]

    def work(idx, rounds, out):
        """softmax (pool scratch for its folds), a GEMM and an attention launch into freshly allocated outputs."""
        x, (a, b), (q, kk, v) = xs[idx], ab[idx], qkv[idx]
        res = []
        ins = [cb.upload(t) for t in (x, a, b, q, kk, v)]
        for _ in range(rounds):
            y, c, o = alloc(n * 4), alloc(m * nn * 2), alloc(B * Hq * 128 * 2)
            cb.check(L.catena_b200_softmax_f32_into(ins[0].data, y.data, n))
            cb.check(L.catena_b200_gemm_bf16_into(ins[1].data, ins[2].data, c.data, m, nn, k, nn))
            cb.check(L.catena_b200_attn_decode_bf16_into(ins[3].data, ins[4].data, ins[5].data, o.data, B, Hq, Hkv, 128, Lk, 0, B * Hkv))
            got = (cb.download(y, np.uint32), cb.download(c, np.uint16), cb.download(o, np.uint16))   # download synchronises
            for t in (y, c, o):
                cb.free(t)
            res.append(got)
        for t in ins:
            cb.free(t)
        out[idx] = res

    single = {}
    for idx in range(2):
        work(idx, 1, single)

    results, errors = {}, []

    def thread_main(idx):
        try:
            cb.check(L.catena_b200_init(0))
            stream = torch.cuda.Stream(device=torch.device("cuda", 0))
            L.catena_b200_set_stream(C.c_void_p(stream.cuda_stream))
            L.catena_b200_set_blocking(0)
            work(idx, 12, results)
            cb.check(L.catena_b200_check_device_errors())
            cb.check(L.catena_b200_sync())
            L.catena_b200_set_blocking(1)
            L.catena_b200_set_stream(None)
        except Exception as exc:                               # noqa: BLE001 - reported by the main thread
            errors.append(exc)

    threads = [threading.Thread(target=thread_main, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for idx in range(2):
        for got in results[idx]:
            for g, w in zip(got, single[idx][0]):
                assert np.array_equal(g, w)
