"""CPU interpreter of the generic map kernel's register programs (test infrastructure): the same instruction semantics
as csrc/map_program.cu, one element at a time, so the compiler (map_program.py) can be tested without a GPU and the kernel
against something that is not the compiler's own reading of the program."""
import ctypes
import ctypes.util

import numpy as np

from catena_lang_b200.map_program import _OPS

M32, M64 = 0xFFFFFFFF, 0xFFFFFFFFFFFFFFFF
_libm = ctypes.CDLL(ctypes.util.find_library("m") or "libm.so.6")
_libm.fmaf.restype = ctypes.c_float
_libm.fmaf.argtypes = [ctypes.c_float] * 3


class Fault(Exception):
    pass


def _f(bits):
    return np.uint32(bits & M32).view(np.float32)


def _b(x):
    return int(np.float32(x).view(np.uint32))


def _u_to_f32(x):
    from catena_lang_b200.evaluator import u_to_f32
    return _b(u_to_f32(x))


def run(program, env, length, buffers_host):
    """out[i] for i < length.  `env` as for MapProgram.launch; `buffers_host`: one numpy uint8 array per buffer of env."""
    init, buffers = program.init_registers(env)
    assert len(buffers) == len(buffers_host)
    out = np.zeros(length, np.uint64 if program.elem_bytes == 8 else np.uint32)
    code = [(_OPS[c.op], c.dst, c.a, c.b, c.c, c.target) for c in program.code]
    with np.errstate(all="ignore"):
        for i in range(length):
            r = list(init) + [0] * (program.n_regs - len(init))
            r[program.index_reg] = i
            pc = steps = 0
            while True:
                op, dst, a, b, c, target = code[pc]
                pc += 1
                steps += 1
                assert steps < 10_000_000
                x, y = r[a], (r[b] if not op.startswith("LOAD") else None)
                if op == "HALT":
                    break
                elif op == "MOV": v = x
                elif op == "MOV32": v = (r[dst] & ~M32) | (x & M32)
                elif op == "JMP": pc = target; continue
                elif op == "JZ":
                    if x & M32 == 0: pc = target
                    continue
                elif op == "ASSERT":
                    if x & M32 == 0: raise Fault("assert")
                    continue
                elif op == "SELECT": v = y if x & M32 else r[c]
                elif op == "SELECT32": v = (r[dst] & ~M32) | ((y if x & M32 else r[c]) & M32)
                elif op == "BOOL_NOT": v = 0 if x else 1
                elif op == "BOOL_AND": v = 1 if (x and y) else 0
                elif op == "BOOL_OR": v = 1 if (x or y) else 0
                elif op == "U64_ADD": v = (x + y) & M64
                elif op == "U64_SUB": v = (x - y) & M64
                elif op == "U64_MUL": v = (x * y) & M64
                elif op in ("U64_DIV", "U64_REM"):
                    if y == 0: raise Fault("division by zero")
                    v = x // y if op == "U64_DIV" else x % y
                elif op in ("U64_EQ", "U32_EQ"): v = int(x == y)
                elif op in ("U64_NE", "U32_NE"): v = int(x != y)
                elif op in ("U64_LT", "U32_LT"): v = int(x < y)
                elif op in ("U64_LTE", "U32_LTE"): v = int(x <= y)
                elif op in ("U64_GT", "U32_GT"): v = int(x > y)
                elif op in ("U64_GTE", "U32_GTE"): v = int(x >= y)
                elif op in ("U64_TO_F32", "U32_TO_F32"): v = _u_to_f32(x)
                elif op == "U32_ADD": v = (x + y) & M32
                elif op == "U32_SUB": v = (x - y) & M32
                elif op == "U32_MUL": v = (x * y) & M32
                elif op == "U32_AND": v = x & y & M32
                elif op == "U32_OR": v = (x | y) & M32
                elif op == "U32_XOR": v = (x ^ y) & M32
                elif op == "U32_NOT": v = ~x & M32
                elif op in ("U32_SHL", "U32_SHR"):
                    if y >= 32: raise Fault("shift")
                    v = ((x << y) if op == "U32_SHL" else (x >> y)) & M32
                elif op == "F32_ADD": v = _b(_f(x) + _f(y))
                elif op == "F32_SUB": v = _b(_f(x) - _f(y))
                elif op == "F32_MUL": v = _b(_f(x) * _f(y))
                elif op == "F32_DIV": v = _b(_f(x) / _f(y))
                elif op == "F32_NEG": v = (x ^ 0x80000000) & M32
                elif op == "F32_FMA": v = _b(_libm.fmaf(float(_f(x)), float(_f(y)), float(_f(r[c]))))
                elif op == "F32_MULADD": v = _b(np.float32(_f(x) * _f(y)) + _f(r[c]))
                elif op == "F32_MULSUB": v = _b(np.float32(_f(x) * _f(y)) - _f(r[c]))
                elif op == "F32_SUBMUL": v = _b(_f(r[c]) - np.float32(_f(x) * _f(y)))
                elif op == "F32_EQ": v = int(_f(x) == _f(y))
                elif op == "F32_NE": v = int(_f(x) != _f(y))
                elif op == "F32_LT": v = int(_f(x) < _f(y))
                elif op == "F32_LTE": v = int(_f(x) <= _f(y))
                elif op == "F32_GT": v = int(_f(x) > _f(y))
                elif op == "F32_GTE": v = int(_f(x) >= _f(y))
                elif op == "F32_ROUND_TO_U32":
                    fx = _f(x)
                    if not (fx >= 0 and fx < np.float32(4294967296.0)): raise Fault("round-to-u32")
                    v = int(np.rint(fx))
                elif op in ("LOAD_U64", "LOAD_F32"):
                    view = buffers_host[b].view(np.uint64 if op == "LOAD_U64" else np.uint32)
                    if x >= view.size: raise Fault("index past the buffer")
                    v = int(view[x])
                else:
                    raise AssertionError(op)
                r[dst] = v
            out[i] = r[program.result_reg] & (M64 if program.elem_bytes == 8 else M32)
    return out
