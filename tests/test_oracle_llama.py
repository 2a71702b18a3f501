"""CPU checks of the oracle's Llama-block restatement (no GPU): each composed operator against an independent
numpy float64 evaluation of its definition, within the accuracy of the reference's approximations."""
import math

import numpy as np
import pytest

import oracle


@pytest.fixture(scope="module", autouse=True)
def built():
    oracle.build()


def bits(rng, shape, std=1.0):
    return oracle.f32_to_bf16_bits((rng.standard_normal(shape) * std).astype(np.float32)).reshape(shape)


def val(b):
    return oracle.bf16_bits_to_f32(np.asarray(b).ravel()).astype(np.float64).reshape(np.asarray(b).shape)


def test_rmsnorm_rows_unit_rms():
    x = bits(np.random.default_rng(0), (4, 512), 2.5)
    y = val(oracle.rmsnorm_rows_bf16(x))
    want = val(x) / np.sqrt((val(x) ** 2).mean(axis=1, keepdims=True) + 1e-5)
    assert np.allclose(y, want, rtol=2.0 ** -7, atol=1e-6)          # bf16 output rounding dominates
    assert np.allclose(np.sqrt((y ** 2).mean(axis=1)), 1.0, atol=5e-3)


def test_rope_rotates_pairs_and_appends():
    B, S, hq, hkv, cap, pos0 = 1, 3, 2, 1, 8, 2
    rng = np.random.default_rng(1)
    qkv = bits(rng, (B * S, (hq + 2 * hkv) * 128))
    kc = np.zeros((B, hkv, cap, 128), np.uint16); vc = np.zeros_like(kc)
    q = oracle.rope_append_bf16(qkv, kc, vc, S, pos0, hq, hkv, 10000.0)
    x = val(qkv).reshape(B * S, hq + 2 * hkv, 128)
    inv = 10000.0 ** (-2.0 * np.arange(64) / 128.0)
    for t in range(S):
        ang = (pos0 + t) * inv
        for h in range(hq + hkv):
            want = np.concatenate([x[t, h, :64] * np.cos(ang) - x[t, h, 64:] * np.sin(ang),
                                   x[t, h, 64:] * np.cos(ang) + x[t, h, :64] * np.sin(ang)])
            got = val(q[t, h]) if h < hq else val(kc[0, h - hq, pos0 + t])
            # math.powf / sin-approx-full are low-order approximations: a few 1e-3 of absolute error on |x| ~ 1
            assert np.allclose(got, want, atol=3e-2), (t, h, np.abs(got - want).max())
        assert np.array_equal(vc[0, 0, pos0 + t], qkv[t].reshape(-1, 128)[hq + hkv])
    assert not kc[0, 0, :pos0].any() and not kc[0, 0, pos0 + S:].any()      # only the addressed rows are written


def test_attn_cached_matches_softmax_definition():
    B, S, hq, hkv, cap = 1, 5, 2, 1, 6
    rng = np.random.default_rng(2)
    q = bits(rng, (B * S, hq, 128)); kc = bits(rng, (B, hkv, cap, 128)); vc = bits(rng, (B, hkv, cap, 128))
    out = val(oracle.attn_cached_bf16(q, kc, vc, B, S, 0, hq, hkv, np.float32(1 / math.sqrt(128)))).reshape(S, hq, 128)
    for s in range(S):
        for h in range(hq):
            sc = val(kc[0, 0, :s + 1]) @ val(q[s, h]) / math.sqrt(128)
            w = np.exp(sc - sc.max()); w /= w.sum()
            assert np.allclose(out[s, h], w @ val(vc[0, 0, :s + 1]), atol=2e-2)   # exp~ is a 4e-3 approximation
    assert np.allclose(out[0, 0], val(vc[0, 0, 0]), atol=1e-2)                    # one visible key: the value itself


def test_swiglu_add_linear():
    rng = np.random.default_rng(3)
    gu = bits(rng, (3, 2 * 40))
    g, u = val(gu)[:, :40], val(gu)[:, 40:]
    assert np.allclose(val(oracle.swiglu_bf16(gu)), g / (1 + np.exp(-g)) * u, rtol=3e-2, atol=1e-2)
    x, y = bits(rng, (64,)), bits(rng, (64,))
    assert np.array_equal(oracle.add_bf16(x, y), oracle.f32_to_bf16_bits((val(x) + val(y)).astype(np.float32)))
    a, w, r = bits(rng, (3, 96)), bits(rng, (5, 96), 0.1), bits(rng, (3, 5))
    want = val(oracle.f32_to_bf16_bits((val(a) @ val(w).T).astype(np.float32)).reshape(3, 5)) + val(r)
    assert np.allclose(val(oracle.linear_bf16(a, w, r)), want, rtol=2.0 ** -6, atol=2e-2)


def test_block_decode_equals_prefill_last_token():
    """Prefill of S+1 tokens and prefill of S tokens followed by one decode step are the same computation
    in the oracle (same folds, same order): bit-identical outputs for the last token and identical caches."""
    hidden, hq, hkv, ffn, vocab, cap, B, S = 64, 2, 1, 96, 50, 12, 2, 6
    rng = np.random.default_rng(4)
    w = {"embedding": bits(rng, (vocab, hidden)), "w_qkv": bits(rng, ((hq + 2 * hkv) * 128, hidden), 0.1),
         "w_o": bits(rng, (hidden, hq * 128), 0.06), "w_gate_up": bits(rng, (2 * ffn, hidden), 0.1), "w_down": bits(rng, (hidden, ffn), 0.1)}
    cfg = dict(hidden=hidden, n_heads=hq, n_kv_heads=hkv, ffn=ffn, max_len=cap, rope_base=10000.0)
    ids = rng.integers(0, vocab, (B, S + 1)).astype(np.int32)
    k1 = np.zeros((B, hkv, cap, 128), np.uint16); v1 = np.zeros_like(k1)
    full = oracle.llama_block(cfg, w, ids.ravel(), B, S + 1, 0, k1, v1).reshape(B, S + 1, hidden)
    k2 = np.zeros_like(k1); v2 = np.zeros_like(k1)
    oracle.llama_block(cfg, w, ids[:, :S].ravel(), B, S, 0, k2, v2)
    step = oracle.llama_block(cfg, w, ids[:, S].ravel(), B, 1, S, k2, v2)
    assert np.array_equal(step, full[:, S])
    assert np.array_equal(k1, k2) and np.array_equal(v1, v2)
