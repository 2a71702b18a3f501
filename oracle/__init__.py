"""ctypes binding of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Only tests/, the smoke check and bench.py's CPU-baseline legs may import this module; the
shipped package never does.  The oracle restates catena-lang's generated code on the host
(see catena_oracle.cpp for the per-function reference citations).
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libcatena_oracle.so")

UNARY_OPS = ["math.sin-approx", "math.cos-approx", "math.sin-approx-full-nonneg",
             "math.sin-approx-full", "math.log-approx", "math.exp-approx-nonneg",
             "math.exp-approx", "math.exp2-approx", "math.log2-approx", None, "math.sqrt",
             "nn.sigmoid", "nn.silu", "nn.tanh", "nn.gelu-approx"]


def build(force=False):
    src = os.path.join(_HERE, "catena_oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libcatena_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = C.CDLL(_SO)
        f32, u64, i32, vp = C.c_float, C.c_uint64, C.c_int, C.c_void_p
        for name in ["sin_approx", "cos_approx", "sin_approx_full_nonneg", "sin_approx_full",
                     "log_approx", "exp_approx_nonneg", "exp_approx", "exp2_approx",
                     "log2_approx", "sqrt"]:
            fn = getattr(L, "orc_math_" + name)
            fn.restype, fn.argtypes = f32, [f32]
        for name in ["sigmoid", "silu", "tanh", "gelu_approx"]:
            fn = getattr(L, "orc_nn_" + name)
            fn.restype, fn.argtypes = f32, [f32]
        L.orc_math_powf.restype, L.orc_math_powf.argtypes = f32, [f32, f32]
        L.orc_f32_fma.restype, L.orc_f32_fma.argtypes = f32, [f32, f32, f32]
        L.orc_f32_mul_add.restype, L.orc_f32_mul_add.argtypes = f32, [f32, f32, f32]
        L.orc_map_unary.restype, L.orc_map_unary.argtypes = None, [i32, vp, vp, u64, i32]
        L.orc_sum_f32.restype, L.orc_sum_f32.argtypes = f32, [vp, u64]
        L.orc_mean_f32.restype, L.orc_mean_f32.argtypes = f32, [vp, u64]
        L.orc_max_f32.restype, L.orc_max_f32.argtypes = f32, [vp, u64]
        L.orc_sum_u64.restype, L.orc_sum_u64.argtypes = u64, [vp, u64]
        L.orc_dot_u64.restype, L.orc_dot_u64.argtypes = u64, [vp, vp, u64]
        L.orc_tensor_argmax_f32.restype, L.orc_tensor_argmax_f32.argtypes = u64, [vp, u64]
        L.orc_nn_softmax.restype, L.orc_nn_softmax.argtypes = None, [vp, vp, u64, i32]
        L.orc_nn_rmsnorm.restype, L.orc_nn_rmsnorm.argtypes = None, [vp, vp, u64, i32]
        L.orc_tensor_broadcast_f32.restype, L.orc_tensor_broadcast_f32.argtypes = None, [f32, u64, vp]
        L.orc_tensor_arange_f32.restype, L.orc_tensor_arange_f32.argtypes = None, [u64, vp]
        L.orc_tensor_slice_f32.restype, L.orc_tensor_slice_f32.argtypes = i32, [vp, u64, u64, u64, vp]
        L.orc_tensor_concat_f32.restype, L.orc_tensor_concat_f32.argtypes = None, [vp, u64, vp, u64, vp]
        L.orc_matmul_f32.restype = i32
        L.orc_matmul_f32.argtypes = [vp, u64, vp, u64, u64, u64, u64, u64, u64, u64, vp, i32]
        L.orc_matmul_f32_rows.restype = None
        L.orc_matmul_f32_rows.argtypes = [vp, vp, u64, u64, u64, u64, vp, i32]
        L.orc_gemm_bf16_rows.restype = None
        L.orc_gemm_bf16_rows.argtypes = [vp, vp, u64, u64, u64, u64, vp, vp, i32]
        L.orc_gemm_i8_rows.restype = None
        L.orc_gemm_i8_rows.argtypes = [vp, vp, u64, u64, u64, u64, vp, i32]
        L.orc_attn_decode_bf16.restype = None
        L.orc_attn_decode_bf16.argtypes = [vp, vp, vp, u64, u64, u64, u64, u64, f32, u64, u64, vp, vp, i32]
        L.orc_embed_bf16.restype, L.orc_embed_bf16.argtypes = None, [vp, vp, vp, u64, u64]
        L.orc_rmsnorm_rows_bf16.restype, L.orc_rmsnorm_rows_bf16.argtypes = None, [vp, vp, u64, u64, i32]
        L.orc_rope_append_bf16.restype = None
        L.orc_rope_append_bf16.argtypes = [vp, vp, vp, vp, u64, u64, u64, u64, u64, u64, f32]
        L.orc_attn_cached_bf16.restype = None
        L.orc_attn_cached_bf16.argtypes = [vp, vp, vp, vp, vp, u64, u64, u64, u64, u64, u64, f32, i32]
        L.orc_swiglu_bf16.restype, L.orc_swiglu_bf16.argtypes = None, [vp, vp, u64, u64]
        L.orc_add_bf16.restype, L.orc_add_bf16.argtypes = None, [vp, vp, vp, u64]
        L.orc_linear_bf16.restype, L.orc_linear_bf16.argtypes = None, [vp, vp, vp, vp, u64, u64, u64, i32]
        L.orc_llama_block.restype = None
        L.orc_llama_block.argtypes = [u64, u64, u64, u64, u64, f32, vp, vp, vp, vp, vp, vp, u64, u64, u64, vp, vp, vp, i32]
        L.orc_max_threads.restype = i32
        L.orc_prim.restype, L.orc_prim.argtypes = u64, [C.c_char_p, u64, u64, u64, C.POINTER(i32)]
        L.orc_f32_to_bf16.restype, L.orc_f32_to_bf16.argtypes = C.c_uint16, [f32]
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def max_threads():
    return int(lib().orc_max_threads())


def scalar(name, *args):
    """Evaluate a scalar stdlib program, e.g. scalar('math.exp-approx', 0.5)."""
    sym = "orc_" + name.replace(".", "_").replace("-", "_")
    return float(getattr(lib(), sym)(*[C.c_float(a) for a in args]))


def map_unary(name, x, threads=1):
    x = _f32(x)
    y = np.empty_like(x)
    lib().orc_map_unary(UNARY_OPS.index(name), _p(x), _p(y), x.size, threads)
    return y


def sum_f32(x):
    x = _f32(x); return np.float32(lib().orc_sum_f32(_p(x), x.size))


def mean_f32(x):
    x = _f32(x); return np.float32(lib().orc_mean_f32(_p(x), x.size))


def max_f32(x):
    x = _f32(x); return np.float32(lib().orc_max_f32(_p(x), x.size))


def sum_u64(x):
    x = np.ascontiguousarray(x, dtype=np.uint64); return int(lib().orc_sum_u64(_p(x), x.size))


def dot_u64(x, y):
    x = np.ascontiguousarray(x, dtype=np.uint64); y = np.ascontiguousarray(y, dtype=np.uint64)
    return int(lib().orc_dot_u64(_p(x), _p(y), x.size))


def argmax_f32(x):
    x = _f32(x); return int(lib().orc_tensor_argmax_f32(_p(x), x.size))


def softmax(x, threads=1):
    x = _f32(x); y = np.empty_like(x); lib().orc_nn_softmax(_p(x), _p(y), x.size, threads); return y


def rmsnorm(x, threads=1):
    x = _f32(x); y = np.empty_like(x); lib().orc_nn_rmsnorm(_p(x), _p(y), x.size, threads); return y


def broadcast_f32(v, n):
    y = np.empty(n, np.float32); lib().orc_tensor_broadcast_f32(C.c_float(v), n, _p(y)); return y


def arange_f32(n):
    y = np.empty(n, np.float32); lib().orc_tensor_arange_f32(n, _p(y)); return y


def slice_f32(x, start, length):
    x = _f32(x); y = np.empty(length, np.float32)
    rc = lib().orc_tensor_slice_f32(_p(x), x.size, start, length, _p(y))
    if rc:
        raise IndexError("tensor.slice-f32: bounds assert (the reference traps here)")
    return y


def concat_f32(l, r):
    l = _f32(l); r = _f32(r); y = np.empty(l.size + r.size, np.float32)
    lib().orc_tensor_concat_f32(_p(l), l.size, _p(r), r.size, _p(y)); return y


def matmul_f32(a, b, n, m, k, threads=1):
    a = _f32(a).ravel(); b = _f32(b).ravel(); out = np.empty(n * m, np.float32)
    rc = lib().orc_matmul_f32(_p(a), a.size, _p(b), b.size, n, m, k, n * k, k * m, n * m, _p(out), threads)
    if rc:
        raise ValueError("matmul: length assert (the reference traps here)")
    return out


def matmul_f32_rows(a, b, m, k, row0, row1, threads=1):
    a = _f32(a).ravel(); b = _f32(b).ravel(); out = np.empty((row1 - row0) * m, np.float32)
    lib().orc_matmul_f32_rows(_p(a), _p(b), m, k, row0, row1, _p(out), threads); return out


def gemm_bf16_rows(a_bits, bt_bits, N, K, row0, row1, threads=1, want_f32=False):
    """a_bits [M,K] uint16 (bf16 bits), bt_bits [N,K] uint16 -> bf16 bits [(row1-row0), N]."""
    a = np.ascontiguousarray(a_bits, dtype=np.uint16); bt = np.ascontiguousarray(bt_bits, dtype=np.uint16)
    c = np.empty(((row1 - row0), N), np.uint16)
    cf = np.empty(((row1 - row0), N), np.float32) if want_f32 else None
    lib().orc_gemm_bf16_rows(_p(a), _p(bt), N, K, row0, row1, _p(c), _p(cf), threads)
    return (c, cf) if want_f32 else c


def gemm_i8_rows(a, bt, N, K, row0, row1, threads=1):
    a = np.ascontiguousarray(a, dtype=np.int8); bt = np.ascontiguousarray(bt, dtype=np.int8)
    c = np.empty(((row1 - row0), N), np.int32)
    lib().orc_gemm_i8_rows(_p(a), _p(bt), N, K, row0, row1, _p(c), threads); return c


def attn_decode_bf16(q, k, v, B, Hq, Hkv, D, L, scale, unit0=0, unit1=None, threads=1, want_f32=False):
    """q [B,Hq,D], k/v [B,Hkv,L,D] as bf16 bit patterns (uint16) -> o bits [B,Hq,D]."""
    q = np.ascontiguousarray(q, dtype=np.uint16); k = np.ascontiguousarray(k, dtype=np.uint16)
    v = np.ascontiguousarray(v, dtype=np.uint16)
    if unit1 is None:
        unit1 = B * Hq
    o = np.zeros((B, Hq, D), np.uint16)
    of = np.zeros((B, Hq, D), np.float32) if want_f32 else None
    lib().orc_attn_decode_bf16(_p(q), _p(k), _p(v), B, Hq, Hkv, D, L, C.c_float(scale), unit0, unit1,
                               _p(o), _p(of), threads)
    return (o, of) if want_f32 else o


def _u16(a):
    return np.ascontiguousarray(a, dtype=np.uint16)


def embed_bf16(table, ids):
    table, ids = _u16(table), np.ascontiguousarray(ids, dtype=np.int32)
    out = np.empty((ids.size, table.shape[1]), np.uint16)
    lib().orc_embed_bf16(_p(table), _p(ids), _p(out), ids.size, table.shape[1])
    return out


def rmsnorm_rows_bf16(x, threads=1):
    x = _u16(x)
    y = np.empty_like(x)
    lib().orc_rmsnorm_rows_bf16(_p(x), _p(y), x.shape[0], x.shape[1], threads)
    return y


def rope_append_bf16(qkv, k_cache, v_cache, seq, pos0, hq, hkv, base):
    """qkv [tokens, (hq+2hkv)*128]; caches [batch, hkv, cap, 128] are updated in place; returns q [tokens, hq, 128]."""
    qkv = _u16(qkv)
    tokens, cap = qkv.shape[0], k_cache.shape[2]
    q = np.empty((tokens, hq, 128), np.uint16)
    lib().orc_rope_append_bf16(_p(qkv), _p(q), _p(k_cache), _p(v_cache), tokens, seq, pos0, hq, hkv, cap, C.c_float(base))
    return q


def attn_cached_bf16(q, k_cache, v_cache, batch, seq, pos0, hq, hkv, scale, threads=1, want_f32=False):
    """Token (b, s) attends to cache rows 0..pos0+s; q [batch*seq, hq, 128] -> out [batch*seq, hq*128] (bits)."""
    q = _u16(q)
    cap = k_cache.shape[2]
    out = np.empty((batch * seq, hq * 128), np.uint16)
    of = np.empty((batch * seq, hq * 128), np.float32) if want_f32 else None
    lib().orc_attn_cached_bf16(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(of), batch, seq, pos0, hq, hkv, cap,
                               C.c_float(scale), threads)
    return (out, of) if want_f32 else out


def swiglu_bf16(gu):
    gu = _u16(gu)
    out = np.empty((gu.shape[0], gu.shape[1] // 2), np.uint16)
    lib().orc_swiglu_bf16(_p(gu), _p(out), gu.shape[0], gu.shape[1] // 2)
    return out


def add_bf16(x, y):
    x, y = _u16(x), _u16(y)
    out = np.empty_like(x)
    lib().orc_add_bf16(_p(x), _p(y), _p(out), x.size)
    return out


def linear_bf16(x, w, res=None, threads=1):
    x, w = _u16(x), _u16(w)
    res = _u16(res) if res is not None else None
    y = np.empty((x.shape[0], w.shape[0]), np.uint16)
    lib().orc_linear_bf16(_p(x), _p(w), _p(res), _p(y), x.shape[0], w.shape[0], x.shape[1], threads)
    return y


def llama_block(cfg, weights, ids, batch, seq, pos0, k_cache, v_cache, threads=1):
    """cfg: dict(hidden, n_heads, n_kv_heads, ffn, max_len, rope_base); weights: dict of bf16-bit arrays
    (embedding, w_qkv, w_o, w_gate_up, w_down); caches [batch, n_kv_heads, max_len, 128] updated in place."""
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    out = np.empty((batch * seq, cfg["hidden"]), np.uint16)
    w = {k: _u16(v) for k, v in weights.items()}
    lib().orc_llama_block(cfg["hidden"], cfg["n_heads"], cfg["n_kv_heads"], cfg["ffn"], cfg["max_len"],
                          C.c_float(cfg["rope_base"]), _p(w["embedding"]), _p(w["w_qkv"]), _p(w["w_o"]),
                          _p(w["w_gate_up"]), _p(w["w_down"]), _p(ids), batch, seq, pos0, _p(k_cache), _p(v_cache),
                          _p(out), threads)
    return out


# operand and result kinds of the primitive table (codegen/gpu.rs:322-447): op -> ((inputs), output)
PRIM_KINDS = {
    "bool.not": (("bool",), "bool"), "bool.and": (("bool", "bool"), "bool"), "bool.or": (("bool", "bool"), "bool"),
    "u64.add": (("u64", "u64"), "u64"), "u64.sub": (("u64", "u64"), "u64"), "u64.mul": (("u64", "u64"), "u64"),
    "u64.ne": (("u64", "u64"), "bool"), "u64.lt": (("u64", "u64"), "bool"), "u64.lte": (("u64", "u64"), "bool"),
    "u64.gte": (("u64", "u64"), "bool"), "u64.eq": (("u64", "u64"), "bool"), "u64.gt": (("u64", "u64"), "bool"),
    "u32.add": (("u32", "u32"), "u32"), "u32.sub": (("u32", "u32"), "u32"), "u32.mul": (("u32", "u32"), "u32"),
    "u32.and": (("u32", "u32"), "u32"), "u32.or": (("u32", "u32"), "u32"), "u32.xor": (("u32", "u32"), "u32"),
    "u32.shl": (("u32", "u32"), "u32"), "u32.shr": (("u32", "u32"), "u32"), "u32.not": (("u32",), "u32"),
    "u32.eq": (("u32", "u32"), "bool"), "u32.ne": (("u32", "u32"), "bool"), "u32.lt": (("u32", "u32"), "bool"),
    "u32.gt": (("u32", "u32"), "bool"), "u32.lte": (("u32", "u32"), "bool"), "u32.gte": (("u32", "u32"), "bool"),
    "u32.to-f32": (("u32",), "f32"), "u64.to-f32": (("u64",), "f32"), "u32.bitcast-f32": (("u32",), "f32"),
    "f32.add": (("f32", "f32"), "f32"), "f32.sub": (("f32", "f32"), "f32"), "f32.mul": (("f32", "f32"), "f32"),
    "f32.div": (("f32", "f32"), "f32"), "f32.neg": (("f32",), "f32"), "f32.fma": (("f32", "f32", "f32"), "f32"),
    "f32.eq": (("f32", "f32"), "bool"), "f32.ne": (("f32", "f32"), "bool"), "f32.lt": (("f32", "f32"), "bool"),
    "f32.gt": (("f32", "f32"), "bool"), "f32.lte": (("f32", "f32"), "bool"), "f32.gte": (("f32", "f32"), "bool"),
    "f32.select": (("bool", "f32", "f32"), "f32"), "u32.select": (("bool", "u32", "u32"), "u32"),
    "u64.select": (("bool", "u64", "u64"), "u64"), "bool.select": (("bool", "bool", "bool"), "bool"),
    "f32.round-to-u32": (("f32",), "u32"), "f32.bitcast-u32": (("f32",), "u32"),
    "bool.t": ((), "bool"), "bool.f": ((), "bool"), "u64.zero": ((), "u64"), "u64.one": ((), "u64"), "u32.one": ((), "u32"),
    "f32.one": ((), "f32"),
}


def prim(op, *raw):
    """One primitive of the table on raw operand bits -> raw result bits (f32 values as their 32-bit patterns)."""
    known = C.c_int(0)
    a, b, c = (list(raw) + [0, 0, 0])[:3]
    r = lib().orc_prim(op.encode(), a, b, c, C.byref(known))
    if not known.value:
        raise KeyError(op)
    return int(r)


def f32_to_bf16_bits(x):
    """Round-to-nearest-even f32 -> bf16 bit patterns (numpy, same rule as the oracle)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
