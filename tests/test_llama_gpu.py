"""Llama-style block (rmsnorm, projections, rotary + cache append, causal / cached attention, SwiGLU,
residuals) against the CPU oracle: operator by operator, then the whole block for a prefill and decode steps.
The reference has no counterpart (parity unpinned); the oracle composes reference programs."""
import ctypes as C
import math

import numpy as np
import pytest

import catena_lang_b200 as cb

pytestmark = pytest.mark.gpu
SCALE = np.float32(1.0 / math.sqrt(128.0))


@pytest.fixture(scope="module")
def orc():
    import oracle
    oracle.build()
    return oracle


@pytest.fixture(scope="module", autouse=True)
def device():
    cb.check(cb.lib().catena_b200_init(0))


def bits(rng, shape, std=1.0):
    import oracle
    return oracle.f32_to_bf16_bits((rng.standard_normal(shape) * std).astype(np.float32)).reshape(shape)


def close(got_bits, want_bits, rel=2.0 ** -7, floor=1e-5, frac_exact=0.0):
    """bf16 outputs compared as f32 values: within `rel` of the oracle's value plus a floor; at least
    `frac_exact` of them bit-identical."""
    import oracle
    g, w = oracle.bf16_bits_to_f32(np.asarray(got_bits).ravel()), oracle.bf16_bits_to_f32(np.asarray(want_bits).ravel())
    assert np.all(np.isfinite(g))
    err = np.abs(g - w)
    bad = err > rel * np.abs(w) + floor
    assert not bad.any(), f"{bad.sum()} of {bad.size} beyond tolerance, worst {err.max():.3e}"
    assert np.mean(np.asarray(got_bits).ravel() == np.asarray(want_bits).ravel()) >= frac_exact


def dev(a):
    return cb.upload(np.ascontiguousarray(a))


def alloc(nbytes):
    m = cb.CatenaMem()
    cb.check(cb.lib().catena_b200_mem_alloc(nbytes, C.byref(m)))
    return m


def test_embed_and_bad_id(orc):
    rng = np.random.default_rng(0)
    table = bits(rng, (50, 64))
    ids = np.array([3, 49, 0, 7, 7], np.int32)
    tm, im, om = dev(table), dev(ids), alloc(5 * 64 * 2)
    cb.check(cb.lib().catena_b200_embed_bf16_into(tm.data, im.data, om.data, 5, 64, 50))
    assert np.array_equal(cb.download(om, np.uint16).reshape(5, 64), orc.embed_bf16(table, ids))
    bad = dev(np.array([1, 50], np.int32))
    assert cb.lib().catena_b200_embed_bf16_into(tm.data, bad.data, om.data, 2, 64, 50) == cb.E_ASSERT
    for m in (tm, im, om, bad):
        cb.free(m)


@pytest.mark.parametrize("rows,hidden", [(3, 256), (5, 2048), (2, 4096 + 64), (200, 256), (1500, 2048)])
def test_rmsnorm_rows(orc, rows, hidden):
    x = bits(np.random.default_rng(1), (rows, hidden), 3.0)
    xm, ym = dev(x), alloc(x.nbytes)
    cb.check(cb.lib().catena_b200_rmsnorm_rows_bf16_into(xm.data, ym.data, rows, hidden))
    # the sum of squares is a fixed tree here and a sequential fold in the oracle: the quotient moves by an ulp at most
    close(cb.download(ym, np.uint16), orc.rmsnorm_rows_bf16(x, threads=4), rel=2.0 ** -7, frac_exact=0.98)
    cb.free(xm), cb.free(ym)


def test_prefill_reciprocal_sequence_is_the_ieee_reciprocal_for_every_float_of_its_range():
    """The tcgen05 prefill kernel replaces __frcp_rn by a rcp.approx + two FMA steps for arguments in [0.5, 2^100);
    the device compares the two for all ~8.6e8 floats of that range."""
    out = (C.c_uint64 * 2)()
    cb.check(cb.lib().catena_b200_debug_rcp_check(out))
    assert out[0] == 0x71800000 - 0x3F000000 and out[1] == 0


@pytest.mark.parametrize("B,S,hq,hkv", [(2, 5, 4, 2), (1, 3, 2, 1)])      # angles from a table / evaluated in place
def test_rope_append(orc, B, S, hq, hkv):
    cap, pos0 = 16, 3
    rng = np.random.default_rng(2)
    qkv = bits(rng, (B * S, (hq + 2 * hkv) * 128))
    kc = bits(rng, (B, hkv, cap, 128)); vc = bits(rng, (B, hkv, cap, 128))
    kc_o, vc_o = kc.copy(), vc.copy()
    q_o = orc.rope_append_bf16(qkv, kc_o, vc_o, S, pos0, hq, hkv, 10000.0)
    qm, km, vm, xm = alloc(B * S * hq * 128 * 2), dev(kc), dev(vc), dev(qkv)
    cb.check(cb.lib().catena_b200_rope_append_bf16_into(xm.data, qm.data, km.data, vm.data, B * S, S, pos0, hq, hkv, cap, 10000.0))
    # identical operations in identical order: bit-exact
    assert np.array_equal(cb.download(qm, np.uint16).reshape(q_o.shape), q_o)
    assert np.array_equal(cb.download(km, np.uint16).reshape(kc.shape), kc_o)
    assert np.array_equal(cb.download(vm, np.uint16).reshape(vc.shape), vc_o)
    assert cb.lib().catena_b200_rope_append_bf16_into(xm.data, qm.data, km.data, vm.data, B * S, S, cap - 2, hq, hkv, cap, 10000.0) == cb.E_BAD_ARG
    for m in (qm, km, vm, xm):
        cb.free(m)


@pytest.fixture(params=["tcgen05", "mma.sync"])
def prefill_kernel(request):
    """Runs a test once per prefill-attention kernel."""
    cb.lib().catena_b200_debug_set_prefill_tc(1 if request.param == "tcgen05" else 0)
    yield request.param
    cb.lib().catena_b200_debug_set_prefill_tc(1)


@pytest.mark.parametrize("B,S,hq,hkv", [(1, 64, 2, 2), (2, 100, 4, 2), (1, 200, 8, 1), (1, 1, 1, 1), (1, 384, 2, 1)])
def test_attn_prefill(orc, prefill_kernel, B, S, hq, hkv):
    cap = S + 7
    rng = np.random.default_rng(3)
    q = bits(rng, (B * S, hq, 128)); kc = bits(rng, (B, hkv, cap, 128)); vc = bits(rng, (B, hkv, cap, 128))
    want, want_f32 = orc.attn_cached_bf16(q, kc, vc, B, S, 0, hq, hkv, SCALE, threads=orc.max_threads(), want_f32=True)
    qm, km, vm, om = dev(q), dev(kc), dev(vc), alloc(B * S * hq * 128 * 2)
    cb.check(cb.lib().catena_b200_attn_prefill_bf16_into(qm.data, km.data, vm.data, om.data, B, S, hq, hkv, cap))
    got = cb.download(om, np.uint16)
    close(got, want, rel=2.0 ** -7, floor=4e-6, frac_exact=0.97)
    cb.check(cb.lib().catena_b200_attn_prefill_bf16_into(qm.data, km.data, vm.data, om.data, B, S, hq, hkv, cap))
    assert np.array_equal(got, cb.download(om, np.uint16))                 # run-to-run determinism
    for m in (qm, km, vm, om):
        cb.free(m)


def test_attn_prefill_kernels_agree_long(orc):
    """Nine key tiles per query tile (the ring wraps, both consumer groups take several tiles): the tcgen05 kernel and
    the mma.sync kernel agree within one bf16 ulp, nearly everywhere exactly, and a sample of rows matches the oracle."""
    B, S, hq, hkv = 2, 1100, 4, 2
    cap = S
    rng = np.random.default_rng(12)
    q = bits(rng, (B * S, hq, 128)); kc = bits(rng, (B, hkv, cap, 128)); vc = bits(rng, (B, hkv, cap, 128))
    qm, km, vm, om = dev(q), dev(kc), dev(vc), alloc(B * S * hq * 128 * 2)
    outs = []
    for tc in (1, 0):
        cb.lib().catena_b200_debug_set_prefill_tc(tc)
        try:
            cb.check(cb.lib().catena_b200_attn_prefill_bf16_into(qm.data, km.data, vm.data, om.data, B, S, hq, hkv, cap))
        finally:
            cb.lib().catena_b200_debug_set_prefill_tc(1)
        outs.append(cb.download(om, np.uint16).reshape(B * S, hq * 128))
    close(outs[0], outs[1], rel=2.0 ** -7, floor=4e-6, frac_exact=0.97)
    rows = [0, 127, 128, 700, S - 1, S + 5, 2 * S - 1]                    # tokens across tile boundaries of both sequences
    want = orc.attn_cached_bf16(q, kc, vc, B, S, 0, hq, hkv, SCALE, threads=orc.max_threads())
    close(outs[0][rows], want[rows], rel=2.0 ** -7, floor=4e-6, frac_exact=0.95)
    for m in (qm, km, vm, om):
        cb.free(m)


@pytest.mark.parametrize("B,hq,hkv,L,cap", [(2, 4, 2, 37, 64), (4, 16, 16, 300, 512), (1, 8, 2, 129, 129)])
def test_attn_decode_with_capacity(orc, B, hq, hkv, L, cap):
    """Cached attention on caches that own `cap` rows per unit of which `L` are visible; the rest is never read."""
    rng = np.random.default_rng(4)
    q = bits(rng, (B, hq, 128)); kc = bits(rng, (B, hkv, cap, 128)); vc = bits(rng, (B, hkv, cap, 128))
    kc[:, :, L:, :] = 0x7FC0                                               # NaN beyond the visible length
    vc[:, :, L:, :] = 0x7FC0
    want = orc.attn_cached_bf16(q, kc, vc, B, 1, L - 1, hq, hkv, SCALE, threads=orc.max_threads())
    qm, km, vm, om = dev(q), dev(kc), dev(vc), alloc(B * hq * 128 * 2)
    for tc in (1, 0):
        cb.lib().catena_b200_debug_set_attn_tc(tc)
        try:
            cb.check(cb.lib().catena_b200_attn_decode_bf16_cache_into(qm.data, km.data, vm.data, om.data, B, hq, hkv, 128, L, cap))
        finally:
            cb.lib().catena_b200_debug_set_attn_tc(1)
        close(cb.download(om, np.uint16), want, rel=2.0 ** -7, floor=4e-6, frac_exact=0.97)
    for m in (qm, km, vm, om):
        cb.free(m)


def test_swiglu_and_add(orc):
    rng = np.random.default_rng(5)
    gu = bits(rng, (7, 2 * 264), 2.0)
    # gates beyond +-64 leave the kernel's short reciprocal / rounding forms for the general routine; specials too
    gu[1, :264] = bits(rng, (264,), 60.0)
    gu[2, :16] = np.array([0x42800000, 0xC2800000, 0x42810000, 0xC2810000, 0x7F800000, 0xC3000000, 0x43000000, 0x00000000,
                           0x80000000, 0x47000000, 0xC7000000, 0x7F7F0000, 0xFF7F0000, 0x00010000, 0x42B40000, 0xC2B40000],
                          dtype=np.uint32) >> 16
    gm, am = dev(gu), alloc(7 * 264 * 2)
    cb.check(cb.lib().catena_b200_swiglu_bf16_into(gm.data, am.data, 7, 264))
    assert np.array_equal(cb.download(am, np.uint16).reshape(7, 264), orc.swiglu_bf16(gu))   # bit-exact
    x, y = bits(rng, (1000 * 8,)), bits(rng, (1000 * 8,))
    xm, ym = dev(x), dev(y)
    cb.check(cb.lib().catena_b200_add_bf16_into(xm.data, ym.data, xm.data, x.size))
    assert np.array_equal(cb.download(xm, np.uint16), orc.add_bf16(x, y))
    for m in (gm, am, xm, ym):
        cb.free(m)


@pytest.mark.parametrize("m,n,k,res", [(1, 40, 256, False), (4, 300, 2048, True), (8, 64, 8192, True), (16, 256, 512, True)])
def test_linear(orc, m, n, k, res):
    rng = np.random.default_rng(6)
    x, w = bits(rng, (m, k)), bits(rng, (n, k), 1.0 / math.sqrt(k))
    r = bits(rng, (m, n)) if res else None
    want = orc.linear_bf16(x, w, r, threads=orc.max_threads())
    xm, wm, ym = dev(x), dev(w), alloc(m * n * 2)
    rm = dev(r) if res else None
    cb.check(cb.lib().catena_b200_linear_bf16_into(xm.data, wm.data, rm.data if res else None, ym.data, m, n, k))
    got = cb.download(ym, np.uint16)
    # with a residual, a one-ulp difference of the rounded product survives the addition whatever the size of the sum
    close(got, want, rel=2.0 ** -7, floor=3e-2 if res else 2e-5, frac_exact=0.9)
    cb.check(cb.lib().catena_b200_linear_bf16_into(xm.data, wm.data, rm.data if res else None, ym.data, m, n, k))
    assert np.array_equal(got, cb.download(ym, np.uint16))
    for mm in (xm, wm, ym) + ((rm,) if res else ()):
        cb.free(mm)


@pytest.mark.parametrize("m,n,k", [(300, 512, 256), (700, 1000, 512), (129, 40, 64)])
def test_linear_residual_in_the_gemm_epilogue_equals_gemm_then_add(orc, m, n, k):
    """More than 128 rows: the tcgen05 GEMM adds the residual in its epilogue.  Same two roundings as the product
    followed by the add kernel, so the results are equal bit for bit; the output may be the residual buffer itself."""
    rng = np.random.default_rng(8)
    x, w, r = bits(rng, (m, k)), bits(rng, (n, k), 1.0 / math.sqrt(k)), bits(rng, (m, n))
    xm, wm, rm, ym, y2 = dev(x), dev(w), dev(r), alloc(m * n * 2), alloc(m * n * 2)
    cb.check(cb.lib().catena_b200_linear_bf16_into(xm.data, wm.data, rm.data, ym.data, m, n, k))
    cb.check(cb.lib().catena_b200_linear_bf16_into(xm.data, wm.data, None, y2.data, m, n, k))
    cb.check(cb.lib().catena_b200_add_bf16_into(y2.data, rm.data, y2.data, m * n))
    got = cb.download(ym, np.uint16)
    assert np.array_equal(got, cb.download(y2, np.uint16))
    close(got, orc.linear_bf16(x, w, r, threads=orc.max_threads()), rel=2.0 ** -7, floor=3e-2, frac_exact=0.9)
    cb.check(cb.lib().catena_b200_linear_bf16_into(xm.data, wm.data, rm.data, rm.data, m, n, k))   # in place
    assert np.array_equal(got, cb.download(rm, np.uint16))
    for mm in (xm, wm, rm, ym, y2):
        cb.free(mm)


@pytest.mark.parametrize("m,ffn,k", [(4, 264, 512), (16, 512, 2048), (20, 256, 512), (300, 256, 512), (700, 384, 256), (129, 200, 64)])
def test_linear_swiglu_equals_two_steps(orc, m, ffn, k):
    """The fused gate/up projection + SwiGLU (one launch for m <= 16: skinny kernel; for m > 128 and ffn % 128 == 0: the
    tcgen05 GEMM with the activation in its epilogue) gives the bits of the two separate operators."""
    rng = np.random.default_rng(8)
    x, w = bits(rng, (m, k)), bits(rng, (2 * ffn, k), 1.0 / math.sqrt(k))
    xm, wm, gm, am, bm = dev(x), dev(w), alloc(m * 2 * ffn * 2), alloc(m * ffn * 2), alloc(m * ffn * 2)
    cb.check(cb.lib().catena_b200_linear_bf16_into(xm.data, wm.data, None, gm.data, m, 2 * ffn, k))
    cb.check(cb.lib().catena_b200_swiglu_bf16_into(gm.data, am.data, m, ffn))
    cb.check(cb.lib().catena_b200_linear_swiglu_bf16_into(xm.data, wm.data, gm.data, bm.data, m, ffn, k))
    two, fused = cb.download(am, np.uint16), cb.download(bm, np.uint16)
    assert np.array_equal(two, fused)
    close(fused, orc.swiglu_bf16(orc.linear_bf16(x, w, threads=orc.max_threads())), rel=2.0 ** -6, floor=2e-3)
    for mm in (xm, wm, gm, am, bm):
        cb.free(mm)


def make_block(rng, hidden, n_heads, n_kv_heads, ffn, vocab):
    return {"embedding": bits(rng, (vocab, hidden)),
            "w_qkv": bits(rng, ((n_heads + 2 * n_kv_heads) * 128, hidden), 1.0 / math.sqrt(hidden)),
            "w_o": bits(rng, (hidden, n_heads * 128), 1.0 / math.sqrt(n_heads * 128)),
            "w_gate_up": bits(rng, (2 * ffn, hidden), 1.0 / math.sqrt(hidden)),
            "w_down": bits(rng, (hidden, ffn), 1.0 / math.sqrt(ffn))}


@pytest.mark.parametrize("n_heads,n_kv_heads", [(2, 2), (4, 2)])
def test_block_prefill_then_decode(orc, n_heads, n_kv_heads):
    hidden, ffn, vocab, max_len, B, S = 256, 512, 300, 160, 2, 100
    rng = np.random.default_rng(7)
    weights = make_block(rng, hidden, n_heads, n_kv_heads, ffn, vocab)
    cfg = dict(hidden=hidden, n_heads=n_heads, n_kv_heads=n_kv_heads, ffn=ffn, max_len=max_len, rope_base=10000.0)
    blk = cb.LlamaBlock(hidden, n_heads, n_kv_heads, ffn, vocab, max_len, weights, B)
    kc = np.zeros((B, n_kv_heads, max_len, 128), np.uint16); vc = np.zeros_like(kc)
    ids = rng.integers(0, vocab, B * S).astype(np.int32)
    try:
        got = blk.prefill(ids, S)
        want = orc.llama_block(cfg, weights, ids, B, S, 0, kc, vc, threads=orc.max_threads())
        # A chain of nine rounded stages against the sequential-fold oracle.  The output is the residual stream (values up
        # to about 5, bf16 ulp 2^-6 .. 2^-5 there) plus a small addend, so its error is an ulp of the OUTPUT plus what an
        # ulp of the residual leaves behind where the two nearly cancel: measured worst |got - want| - 2^-7 |want| over
        # prefill and decode steps 1.53e-2 (one ulp of a residual in [2, 4)); the floor is twice that.  The operator
        # tests above (one ulp each) and the fused-equals-separate bit tests carry the weight; this one guards the wiring.
        close(got, want, rel=2.0 ** -7, floor=3.1e-2)
        gk, gv = blk.caches()
        close(gk[:, :, :S], kc[:, :, :S], rel=2.0 ** -6, floor=1e-2)
        close(gv[:, :, :S], vc[:, :, :S], rel=2.0 ** -6, floor=1e-2)
        for step in range(3):
            nxt = rng.integers(0, vocab, B).astype(np.int32)
            # the oracle continues from the GPU's own caches so that one step is compared, not the accumulated drift
            kc, vc = blk.caches()
            want = orc.llama_block(cfg, weights, nxt, B, 1, S + step, kc, vc, threads=orc.max_threads())
            got = blk.decode(nxt)
            close(got, want, rel=2.0 ** -7, floor=3.1e-2)
        assert blk.pos == S + 3
    finally:
        blk.close()


def test_block_prefill_fused_epilogues_equal_separate_kernels():
    """With the CTA-pair GEMM the prefill rotates q / k and appends k / v in the q/k/v projection's epilogue and adds the
    residuals in the o / down projections' epilogues; on the single-CTA GEMM it runs the projection, the rotary kernel
    and the add kernel one after the other.  Same roundings in the same places: outputs and caches agree bit for bit."""
    hidden, n_heads, n_kv_heads, ffn, vocab, max_len, B, S = 256, 3, 1, 512, 300, 200, 2, 150     # three tiles of q/k/v columns, odd head count
    rng = np.random.default_rng(9)
    weights = make_block(rng, hidden, n_heads, n_kv_heads, ffn, vocab)
    ids = rng.integers(0, vocab, B * S).astype(np.int32)
    results = []
    for pair in (1, 0):
        cb.lib().catena_b200_debug_set_gemm_pair(pair)
        blk = cb.LlamaBlock(hidden, n_heads, n_kv_heads, ffn, vocab, max_len, weights, B)
        try:
            out = blk.prefill(ids, S)
            gk, gv = blk.caches()
            results.append((out.copy(), gk[:, :, :S].copy(), gv[:, :, :S].copy()))
        finally:
            blk.close()
            cb.lib().catena_b200_debug_set_gemm_pair(1)
    for a, b in zip(*results):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("hidden,n_heads,n_kv_heads,ffn,B", [(256, 2, 1, 512, 2), (2048, 16, 16, 8192, 4), (272, 3, 3, 1040, 16),
                                                             (512, 4, 2, 304, 1), (1024, 8, 8, 2048, 7)])
def test_decode_step_fused_kernels_equal_separate_launches(hidden, n_heads, n_kv_heads, ffn, B):
    """A decode step can run on other kernels than the default ones: with the rotation and the cache append in the epilogue
    of the q/k/v projection (mode 4) or as launches of their own (mode 0); and as three launches — one persistent kernel
    before the attention (embedding, norm, q/k/v projection, rotation, cache append) and one after it (o projection, norm,
    gate/up + SwiGLU, down projection), with grid barriers between their phases (mode 3, or 5 with the first half chained).
    The arithmetic is the same everywhere (same k split over the warps, same summation trees, same roundings), so outputs
    and caches are equal bit for bit over several steps — including shapes with fewer row groups than CTAs, partial k
    batches and 16 rows."""
    vocab, max_len, S = 300, 48, 20
    rng = np.random.default_rng(13)
    weights = make_block(rng, hidden, n_heads, n_kv_heads, ffn, vocab)
    ids = rng.integers(0, vocab, B * S).astype(np.int32)
    steps = [rng.integers(0, vocab, B).astype(np.int32) for _ in range(3)]
    results = []
    for mode in (0, 4, 3, 5):
        cb.lib().catena_b200_debug_set_decode_fused(mode)
        blk = cb.LlamaBlock(hidden, n_heads, n_kv_heads, ffn, vocab, max_len, weights, B)
        try:
            blk.prefill(ids, S, download=False)
            outs = [blk.decode(t).copy() for t in steps]
            results.append(outs + list(blk.caches()))
        finally:
            blk.close()
            cb.lib().catena_b200_debug_set_decode_fused(-1)         # back to the default
    for other in results[1:]:
        for a, b in zip(results[0], other):
            assert np.array_equal(a, b)


def test_block_argument_errors():
    """Bad arguments come back as statuses before anything is launched (the generated code of the reference would
    have trapped on the device)."""
    hidden, heads, kv_heads, ffn, vocab, max_len, B = 256, 2, 1, 512, 50, 8, 1
    rng = np.random.default_rng(10)
    blk = cb.LlamaBlock(hidden, heads, kv_heads, ffn, vocab, max_len, make_block(rng, hidden, heads, kv_heads, ffn, vocab), B)
    L = cb.lib()
    try:
        ids = dev(np.zeros(max_len + 1, np.int32))
        out = alloc((max_len + 1) * hidden * 2)
        need = L.catena_b200_llama_workspace_bytes(C.byref(blk.struct), max_len + 1)
        ws = alloc(need)
        args = (blk.k_cache.data, blk.v_cache.data, out.data, ws.data)
        assert L.catena_b200_llama_prefill(C.byref(blk.struct), ids.data, B, max_len + 1, *args, need) == cb.E_BAD_ARG      # beyond max_len
        assert L.catena_b200_llama_prefill(C.byref(blk.struct), ids.data, B, 4, *args, 16) == cb.E_BAD_ARG                 # workspace too small
        assert L.catena_b200_llama_prefill(C.byref(blk.struct), None, B, 4, *args, need) == cb.E_BAD_ARG                    # null ids
        assert L.catena_b200_llama_decode(C.byref(blk.struct), ids.data, B, max_len, *args, need) == cb.E_BAD_ARG          # position == capacity
        assert L.catena_b200_llama_prefill(None, ids.data, B, 4, *args, need) == cb.E_BAD_ARG
        bad = cb.LlamaBlockStruct(hidden, 3, 2, ffn, vocab, max_len, *[blk._mems[n].data for n in ("embedding", "w_qkv", "w_o", "w_gate_up", "w_down")], 10000.0)
        assert L.catena_b200_llama_workspace_bytes(C.byref(bad), 4) == 0                                                  # 3 heads over 2 kv heads
        assert L.catena_b200_llama_prefill(C.byref(bad), ids.data, B, 4, *args, need) == cb.E_UNSUPPORTED
        # an id outside the vocabulary is an assertion status, and the library stays usable afterwards
        bad_ids = dev(np.array([vocab], np.int32))
        assert L.catena_b200_llama_decode(C.byref(blk.struct), bad_ids.data, B, 0, *args, need) == cb.E_ASSERT
        assert L.catena_b200_llama_decode(C.byref(blk.struct), ids.data, B, 0, *args, need) == cb.OK
        # the last row of the cache can still be written
        assert L.catena_b200_llama_prefill(C.byref(blk.struct), ids.data, B, max_len, *args, need) == cb.OK
        for m in (ids, out, ws, bad_ids):
            cb.free(m)
    finally:
        blk.close()
