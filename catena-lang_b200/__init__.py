"""catena_lang_b200 — host-side binding of libcatena_b200.so (hand-written sm_100a kernels behind
catena-lang's `program_*` calling convention).

The package directory is called ``catena-lang_b200``; import it as ``catena_lang_b200`` (the
repository root holds a one-file loader of that name).

This module holds the raw ctypes view of the C ABI (``lib()``, ``CatenaMem``) and small numpy
helpers.  The reference-shaped surface — ``Runtime.from_sources`` / ``Runtime.exec`` / ``Value`` /
``Mem`` / ``GpuDialect`` (catena-lang/src/runtime/runtime.rs:104-185, value.rs:5-21, mem.rs:38-70,
codegen/mod.rs:50-54) — lives in ``runtime.py`` and is re-exported here.

There is no CPU path: if the shared library is missing it must be built first
(``python catena-lang_b200/build.py``), and every compute call fails with a clear status when no
B200 is visible.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
# CATENA_B200_LIB overrides the location of the kernel library (for hosts that install it elsewhere)
LIB_PATH = os.environ.get("CATENA_B200_LIB") or os.path.join(_HERE, "libcatena_b200.so")

OK, E_ASSERT, E_CUDA, E_NO_DEVICE, E_BAD_ARG, E_TIMEOUT, E_TOO_LARGE, E_UNSUPPORTED = range(8)


class CatenaMem(C.Structure):
    """catena_mem_t {void* data; uint64_t len /*bytes*/} (codegen/prelude.rs:28-31)."""
    _fields_ = [("data", C.c_void_p), ("len", C.c_uint64)]


class Dim3(C.Structure):
    """catena_dim3_t (codegen/prelude.rs:13-17)."""
    _fields_ = [("x", C.c_uint32), ("y", C.c_uint32), ("z", C.c_uint32)]


class LaunchParams(C.Structure):
    """catena_launch_params_t {grid_dim, block_dim} (codegen/prelude.rs:23-26)."""
    _fields_ = [("grid_dim", Dim3), ("block_dim", Dim3)]


class LlamaBlockStruct(C.Structure):
    """catena_llama_block_t (include/catena_b200.h)."""
    _fields_ = [("hidden", C.c_uint64), ("n_heads", C.c_uint64), ("n_kv_heads", C.c_uint64), ("ffn", C.c_uint64),
                ("vocab", C.c_uint64), ("max_len", C.c_uint64), ("embedding", C.c_void_p), ("w_qkv", C.c_void_p),
                ("w_o", C.c_void_p), ("w_gate_up", C.c_void_p), ("w_down", C.c_void_p), ("rope_base", C.c_float)]


class CatenaError(RuntimeError):
    def __init__(self, status, what=""):
        self.status = int(status)
        super().__init__(f"catena_b200 status {self.status}: {status_string(self.status)} {what}".strip())


_lib = None


def lib():
    """Loads libcatena_b200.so and declares the prototypes of include/catena_b200.h."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(
            f"{LIB_PATH} is missing: build it with `python catena-lang_b200/build.py` "
            "(this package has no CPU or eager fallback)")
    L = C.CDLL(LIB_PATH)
    st, u64, f32, vp, mem = C.c_int32, C.c_uint64, C.c_float, C.c_void_p, CatenaMem
    pm, pf, pu = C.POINTER(CatenaMem), C.POINTER(C.c_float), C.POINTER(C.c_uint64)

    def proto(name, res, args):
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args

    proto("catena_b200_init", st, [C.c_int])
    proto("catena_b200_device_count", C.c_int, [])
    proto("catena_b200_current_device", C.c_int, [])
    proto("catena_b200_set_stream", st, [vp])
    proto("catena_b200_get_stream", vp, [])
    proto("catena_b200_set_blocking", None, [C.c_int])
    proto("catena_b200_sync", st, [])
    proto("catena_b200_last_status", st, [])
    proto("catena_b200_clear_status", None, [])
    proto("catena_b200_status_string", C.c_char_p, [st])
    proto("catena_b200_version", C.c_char_p, [])
    proto("catena_b200_launch_count", u64, [])
    proto("catena_b200_mem_alloc", st, [u64, pm])
    proto("catena_b200_mem_free", st, [mem])
    proto("catena_b200_mem_upload", st, [vp, u64, pm])
    proto("catena_b200_mem_download", st, [mem, vp, u64])
    proto("catena_b200_mem_write", st, [mem, vp, u64])
    proto("catena_b200_mem_trim", st, [])
    proto("catena_b200_ipc_export", st, [mem, vp, pu])
    proto("catena_b200_ipc_import", st, [vp, u64, u64, pm])
    proto("catena_b200_ipc_close", st, [mem, u64])
    for name in SCALAR_PROGRAMS:
        proto(symbol_for(name), None, [f32, pf])
    proto("program_math_powf", None, [f32, f32, pf])
    for base in ["program_nn_softmax", "program_nn_rmsnorm"]:
        proto(base, None, [mem, pm])
        proto(base + "_s", st, [mem, pm])
    for base in ["program_sum_f32", "program_mean_f32", "program_max_f32"]:
        proto(base, None, [mem, pf])
        proto(base + "_s", st, [mem, pf])
    proto("program_tensor_broadcast_f32", None, [f32, u64, pm])
    proto("program_tensor_broadcast_f32_s", st, [f32, u64, pm])
    proto("program_tensor_arange_f32", None, [u64, pm])
    proto("program_tensor_arange_f32_s", st, [u64, pm])
    proto("program_tensor_slice_f32", None, [mem, u64, u64, pm])
    proto("program_tensor_slice_f32_s", st, [mem, u64, u64, pm])
    proto("program_tensor_concat_f32", None, [mem, mem, pm])
    proto("program_tensor_concat_f32_s", st, [mem, mem, pm])
    proto("program_tensor_argmax_f32", None, [mem, pu])
    proto("program_tensor_argmax_f32_s", st, [mem, pu])
    proto("program_matmul_2x2_via_mem", None, [mem, mem, u64, u64, u64, u64, u64, u64, pm])
    proto("program_matmul_2x2_via_mem_s", st, [mem, mem, u64, u64, u64, u64, u64, u64, pm])
    proto("program_matmul_right_identity_2x2_via_mem", None, [mem, u64, u64, pm])
    proto("program_matmul_left_identity_2x2_via_mem", None, [mem, u64, u64, pm])
    for base, args in (("program_sum_u64", [mem, pu]), ("program_dot_u64", [mem, mem, pu]), ("program_array_head_u64", [mem, pu])):
        proto(base, None, args)
        proto(base + "_s", st, args)
    proto("catena_b200_map_f32_s", st, [C.c_char_p, mem, pm])
    proto("catena_b200_launch_len", u64, [LaunchParams])
    proto("catena_b200_gpu_materialize_f32_s", st, [C.c_char_p, LaunchParams, mem, pm])
    for base in ["program_gemm_bf16_rc", "program_gemm_i8_rc"]:
        proto(base, None, [mem, mem, u64, u64, u64, pm])
        proto(base + "_s", st, [mem, mem, u64, u64, u64, pm])
    proto("program_attn_decode_bf16", None, [mem, mem, mem, u64, u64, u64, u64, u64, pm])
    proto("program_attn_decode_bf16_s", st, [mem, mem, mem, u64, u64, u64, u64, u64, pm])
    proto("catena_b200_gemm_bf16_into", st, [vp, vp, vp, u64, u64, u64, u64])
    proto("catena_b200_gemm_i8_into", st, [vp, vp, vp, u64, u64, u64, u64])
    proto("catena_b200_matmul_f32_into", st, [vp, vp, vp, u64, u64, u64])
    proto("catena_b200_gemm_bf16_into_peers", st, [vp, vp, vp, u64, u64, u64, u64, C.POINTER(vp), C.c_uint32])
    proto("catena_b200_gemm_i8_into_peers", st, [vp, vp, vp, u64, u64, u64, u64, C.POINTER(vp), C.c_uint32])
    proto("catena_b200_attn_decode_bf16_into", st, [vp, vp, vp, vp, u64, u64, u64, u64, u64, u64, u64])
    proto("catena_b200_attn_decode_bf16_into_peers", st, [vp, vp, vp, vp, u64, u64, u64, u64, u64, u64, u64, C.POINTER(vp), C.c_uint32])
    proto("catena_b200_map_f32_into", st, [C.c_char_p, vp, vp, u64])
    proto("catena_b200_softmax_f32_into", st, [vp, vp, u64])
    proto("catena_b200_rmsnorm_f32_into", st, [vp, vp, u64])
    proto("catena_b200_check_device_errors", st, [])
    proto("catena_b200_map_program_s", st, [vp, C.c_uint32, vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, vp, C.c_uint32, C.c_uint32,
                                            u64, pm])
    proto("catena_b200_map_program_range_s", st, [vp, C.c_uint32, vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, vp, C.c_uint32, C.c_uint32,
                                                  u64, u64, pm])
    # compiled map kernels (csrc/map_jit.cu): code, n_insn, init, init_is_const, n_init, n_regs, index_reg, result_reg, n_buffers, elem_bytes
    spec = [vp, C.c_uint32, vp, vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]
    proto("catena_b200_map_ptx_s", st, spec + [vp, u64, C.POINTER(u64)])
    proto("catena_b200_map_compile_s", st, spec + [C.POINTER(vp)])
    proto("catena_b200_map_kernel_launch_s", st, [vp, vp, C.c_uint32, vp, C.c_uint32, u64, u64, pm])
    proto("catena_b200_map_kernel_release", None, [vp])
    pblk = C.POINTER(LlamaBlockStruct)
    proto("catena_b200_llama_workspace_bytes", u64, [pblk, u64])
    proto("catena_b200_llama_prefill", st, [pblk, vp, u64, u64, vp, vp, vp, vp, u64])
    proto("catena_b200_llama_decode", st, [pblk, vp, u64, u64, vp, vp, vp, vp, u64])
    proto("catena_b200_embed_bf16_into", st, [vp, vp, vp, u64, u64, u64])
    proto("catena_b200_rmsnorm_rows_bf16_into", st, [vp, vp, u64, u64])
    proto("catena_b200_rope_append_bf16_into", st, [vp, vp, vp, vp, u64, u64, u64, u64, u64, u64, f32])
    proto("catena_b200_attn_prefill_bf16_into", st, [vp, vp, vp, vp, u64, u64, u64, u64, u64])
    proto("catena_b200_attn_decode_bf16_cache_into", st, [vp, vp, vp, vp, u64, u64, u64, u64, u64, u64])
    proto("catena_b200_swiglu_bf16_into", st, [vp, vp, u64, u64])
    proto("catena_b200_add_bf16_into", st, [vp, vp, vp, u64])
    proto("catena_b200_linear_swiglu_bf16_into", st, [vp, vp, vp, vp, u64, u64, u64])
    proto("catena_b200_linear_bf16_into", st, [vp, vp, vp, vp, u64, u64, u64])
    proto("catena_b200_debug_set_cta_limit", None, [C.c_int])
    proto("catena_b200_sum_f32_noalloc", st, [vp, u64, vp])
    proto("catena_b200_debug_set_gemm_pair", None, [C.c_int])
    proto("catena_b200_debug_set_attn_tc", None, [C.c_int])
    proto("catena_b200_debug_attn_last_launch", None, [C.POINTER(C.c_uint32)])
    proto("catena_b200_debug_set_prefill_tc", None, [C.c_int])
    proto("catena_b200_debug_set_decode_fused", None, [C.c_int])
    proto("catena_b200_debug_rcp_check", C.c_int, [C.POINTER(C.c_uint64)])
    proto("catena_b200_debug_packed_f32x2_check", C.c_int, [C.POINTER(C.c_uint64)])
    proto("catena_b200_debug_set_wait_limit_ns", None, [u64])
    proto("catena_b200_debug_stall_next", None, [C.c_int, C.c_uint32])
    _lib = L
    return L


# hexpr names of the scalar stdlib programs (stdlib/math.hex, stdlib/nn.hex)
SCALAR_PROGRAMS = [
    "math.sin-approx", "math.cos-approx", "math.sin-approx-full-nonneg", "math.sin-approx-full",
    "math.log-approx", "math.exp-approx-nonneg", "math.exp-approx", "math.exp2-approx", "math.log2-approx",
    "math.sqrt", "nn.sigmoid", "nn.silu", "nn.tanh", "nn.gelu-approx",
]


def symbol_for(name):
    """Source name -> C symbol (codegen/mod.rs:379-388): `program_` + name, every
    non-alphanumeric character replaced by `_`."""
    out = "".join(ch if ch.isalnum() and ch.isascii() else "_" for ch in name)
    if out and out[0].isdigit():
        out = "_" + out
    return "program_" + out


def status_string(status):
    return lib().catena_b200_status_string(int(status)).decode()


def check(status, what=""):
    if status != OK:
        raise CatenaError(status, what)


def upload(array):
    """numpy array -> device catena_mem_t (raw bytes)."""
    a = np.ascontiguousarray(array)
    m = CatenaMem()
    check(lib().catena_b200_mem_upload(a.ctypes.data_as(C.c_void_p), a.nbytes, C.byref(m)), "mem_upload")
    return m


def download(mem, dtype, count=None, out=None):
    """device catena_mem_t -> numpy (into `out`, e.g. a pinned buffer, when given)."""
    dtype = np.dtype(dtype)
    n = mem.len // dtype.itemsize if count is None else count
    if out is None:
        out = np.empty(n, dtype)
    elif out.dtype != dtype or out.size < n or not out.flags.c_contiguous:
        raise ValueError("download: `out` must be a contiguous array of the requested dtype and size")
    if n:
        check(lib().catena_b200_mem_download(mem, out.ctypes.data_as(C.c_void_p), n * dtype.itemsize), "mem_download")
    return out


def free(mem):
    if mem.data:
        check(lib().catena_b200_mem_free(mem), "mem_free")


from .llama import LlamaBlock  # noqa: E402,F401
from .runtime import (ExecError, GpuDialect, InitError, Mem, Runtime, Value, ValueKind)  # noqa: E402,F401
