"""Parity at the CONFIGURED sizes of the two largest workloads, through the C ABI, against the CPU oracle.

* int8 and bf16 GEMM 16384 x 16384 x 8192: the CPU needs hours for the whole product, so three 32-row slabs are
  compared — the first rows, a slab that straddles a 256-row tile boundary in the upper half (where a 32-bit byte
  offset into C would already have wrapped), and the last rows.  int8 bit for bit; bf16 within one bf16 ulp of the
  oracle's fp32 fold.
* the Llama-style block at hidden 2048, 16 x 128 heads, FFN 8192, prefill of 4 x 2048 tokens: sampled tokens
  (positions 0, 127, 128 and 2047 of two sequences — first row, both sides of a query-tile boundary, last row) are
  recomputed by the oracle from the q/k/v projection of their whole sequence, then two decode steps at positions
  2048 and 2049 for all four sequences, the oracle continuing from the GPU's own caches.
"""
import ctypes as C
import math

import numpy as np
import pytest

import catena_lang_b200 as cb

pytestmark = pytest.mark.gpu

M5 = N5 = 16384
K5 = 8192
SLABS = (0, 8192 + 256 - 16, M5 - 32)          # first rows, across the tile boundary at row 8448, last rows


@pytest.fixture(scope="module", autouse=True)
def device():
    cb.check(cb.lib().catena_b200_init(0))


def alloc(nbytes):
    m = cb.CatenaMem()
    cb.check(cb.lib().catena_b200_mem_alloc(nbytes, C.byref(m)))
    return m


def rows_of(mem, row0, rows, row_bytes, dtype):
    """Downloads rows [row0, row0 + rows) of a row-major device matrix."""
    part = cb.CatenaMem(mem.data + row0 * row_bytes, rows * row_bytes)
    return cb.download(part, dtype)


def test_gemm_i8_16384x16384x8192_slabs_bit_exact(orc):
    rng = np.random.default_rng(4)
    a = rng.integers(-128, 128, (M5, K5), dtype=np.int8)
    bt = rng.integers(-128, 128, (N5, K5), dtype=np.int8)
    am, bm, cm = cb.upload(a), cb.upload(bt), alloc(M5 * N5 * 4)
    try:
        cb.check(cb.lib().catena_b200_gemm_i8_into(am.data, bm.data, cm.data, M5, N5, K5, N5))
        for row0 in SLABS:
            got = rows_of(cm, row0, 32, N5 * 4, np.int32).reshape(32, N5)
            want = orc.gemm_i8_rows(a, bt, N5, K5, row0, row0 + 32, threads=orc.max_threads())
            assert np.array_equal(got, want), f"rows {row0}..{row0 + 31}"
    finally:
        for m in (am, bm, cm):
            cb.free(m)


def test_gemm_bf16_16384x16384x8192_slabs_within_one_ulp(orc):
    rng = np.random.default_rng(4)
    scale = np.float32(1.0 / math.sqrt(K5))
    a = orc.f32_to_bf16_bits(rng.standard_normal((M5, K5), dtype=np.float32) * scale).reshape(M5, K5)
    bt = orc.f32_to_bf16_bits(rng.standard_normal((N5, K5), dtype=np.float32) * scale).reshape(N5, K5)
    am, bm, cm = cb.upload(a), cb.upload(bt), alloc(M5 * N5 * 2)
    try:
        cb.check(cb.lib().catena_b200_gemm_bf16_into(am.data, bm.data, cm.data, M5, N5, K5, N5))
        for row0 in SLABS:
            got = rows_of(cm, row0, 32, N5 * 2, np.uint16)
            want, want_f32 = orc.gemm_bf16_rows(a, bt, N5, K5, row0, row0 + 32, threads=orc.max_threads(), want_f32=True)
            g, w = orc.bf16_bits_to_f32(got), want_f32.ravel()
            # the bf16 rounding of an fp32 sum that differs from the oracle's sequential fold by order only
            assert np.all(np.abs(g - w) <= 2.0 ** -8 * np.abs(w) + 1e-6), f"rows {row0}..{row0 + 31}"
            assert (got != want.ravel()).mean() < 0.01
    finally:
        for m in (am, bm, cm):
            cb.free(m)


# ---------------------------------------------------------------- Llama-style block at its configured size
HID, HEADS, KVH, FFN, VOCAB, BATCH, SEQ = 2048, 16, 16, 8192, 32000, 4, 2048
MAX_LEN = SEQ + 128
SCALE = np.float32(1.0 / math.sqrt(128.0))
# Bound on an output: one bf16 ulp of the value plus a floor for what an ulp of the residual stream (values up to ~4, ulp
# 2^-6 there) leaves behind where residual and addend nearly cancel.  Measured on a B200 against the sequential-fold
# oracle at this size, worst |got - want| - 2^-7 |want| over the sampled prefill tokens and the two decode steps:
# 1.24e-2; the floor is twice that.  (Worst absolute error 1.56e-2 = one ulp of a value in [2, 4).)
BLOCK_REL, BLOCK_FLOOR = 2.0 ** -7, 2.5e-2
# Cache entries: one ulp of the value plus a floor, because the normalised rows that enter the projection already differ
# by an ulp in a few elements (tree sum of squares here, sequential fold there).  Measured worst excess over one ulp:
# values 2.05e-3, rotated keys 9.6e-4 over 2^-6 of the pair's norm; the floors are twice that.
VALUE_FLOOR, KEY_FLOOR = 4.1e-3, 2.0e-3


def block_weights(orc):
    rng = np.random.default_rng(5)

    def w(rows, cols):
        return orc.f32_to_bf16_bits(rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(0.02)).reshape(rows, cols)
    return {"embedding": w(VOCAB, HID), "w_qkv": w((HEADS + 2 * KVH) * 128, HID), "w_o": w(HID, HEADS * 128),
            "w_gate_up": w(2 * FFN, HID), "w_down": w(HID, FFN)}


def oracle_tail(orc, weights, x_rows, att_rows):
    """The block after attention for a few tokens: o projection + residual, norm, gate/up, SwiGLU, down + residual."""
    t = orc.max_threads()
    x2 = orc.linear_bf16(att_rows, weights["w_o"], x_rows, threads=t)
    gu = orc.linear_bf16(orc.rmsnorm_rows_bf16(x2), weights["w_gate_up"], threads=t)
    return orc.linear_bf16(orc.swiglu_bf16(gu), weights["w_down"], x2, threads=t)


def worst(orc, got_bits, want_bits):
    g, w = orc.bf16_bits_to_f32(np.asarray(got_bits).ravel()), orc.bf16_bits_to_f32(np.asarray(want_bits).ravel())
    assert np.all(np.isfinite(g))
    err = np.abs(g - w)
    return float(err.max()), bool(np.all(err <= BLOCK_REL * np.abs(w) + BLOCK_FLOOR))


def test_llama_block_configured_size_sampled_tokens(orc):
    weights = block_weights(orc)
    rng = np.random.default_rng(6)
    ids = rng.integers(0, VOCAB, BATCH * SEQ).astype(np.int32)
    blk = cb.LlamaBlock(HID, HEADS, KVH, FFN, VOCAB, MAX_LEN, weights, BATCH)
    t = orc.max_threads()
    try:
        got = blk.prefill(ids, SEQ)
        gk, gv = blk.caches()
        for seq_i in (0, BATCH - 1):
            # the whole sequence's q/k/v projection (its keys and values feed every later token), rotated and appended
            x = orc.embed_bf16(weights["embedding"], ids[seq_i * SEQ:(seq_i + 1) * SEQ])
            qkv = orc.linear_bf16(orc.rmsnorm_rows_bf16(x, threads=t), weights["w_qkv"], threads=t)
            kc = np.zeros((1, KVH, MAX_LEN, 128), np.uint16)
            vc = np.zeros_like(kc)
            q = orc.rope_append_bf16(qkv, kc, vc, SEQ, 0, HEADS, KVH, 10000.0)
            # The GPU's caches against the oracle's: values are stored as projected, keys after the rotation
            # (r1, r2) = (x1 c - x2 s, x2 c + x1 s), which spreads an ulp of either input over both outputs, so the
            # bound for a rotated pair is relative to its norm.
            gv_f = orc.bf16_bits_to_f32(gv[seq_i, :, :SEQ].ravel())
            ov_f = orc.bf16_bits_to_f32(vc[0, :, :SEQ].ravel())
            assert np.all(np.abs(gv_f - ov_f) <= 2.0 ** -7 * np.abs(ov_f) + VALUE_FLOOR)
            gk_f = orc.bf16_bits_to_f32(gk[seq_i, :, :SEQ].ravel()).reshape(-1, 2, 64)
            ok_f = orc.bf16_bits_to_f32(kc[0, :, :SEQ].ravel()).reshape(-1, 2, 64)
            norm = np.sqrt((ok_f.astype(np.float64) ** 2).sum(axis=1, keepdims=True))
            assert np.all(np.abs(gk_f - ok_f) <= 2.0 ** -6 * norm + KEY_FLOOR)
            for g_c, o_c in ((gk, kc), (gv, vc)):
                assert np.mean(g_c[seq_i, :, :SEQ] == o_c[0, :, :SEQ]) > 0.98
            pos = [0, 127, 128, SEQ - 1]
            att = np.concatenate([orc.attn_cached_bf16(q[p:p + 1], kc, vc, 1, 1, p, HEADS, KVH, SCALE, threads=t) for p in pos])
            want = oracle_tail(orc, weights, x[pos], att)
            err, ok = worst(orc, got[[seq_i * SEQ + p for p in pos]], want)
            assert ok, f"sequence {seq_i}: worst error {err:.3e}"
        cfg = dict(hidden=HID, n_heads=HEADS, n_kv_heads=KVH, ffn=FFN, max_len=MAX_LEN, rope_base=10000.0)
        for step in range(2):
            nxt = rng.integers(0, VOCAB, BATCH).astype(np.int32)
            kc, vc = blk.caches()                      # one step is compared, not the accumulated drift
            want = orc.llama_block(cfg, weights, nxt, BATCH, 1, SEQ + step, kc, vc, threads=t)
            err, ok = worst(orc, blk.decode(nxt), want)
            assert ok, f"decode step at position {SEQ + step}: worst error {err:.3e}"
        assert blk.pos == SEQ + 2
    finally:
        blk.close()
