//! Raw bindings of `include/catena_b200.h`.
//!
//! The entry points keep the calling convention of the code catena-lang generates
//! (`catena-lang/src/codegen/gpu.rs:235-261`): inputs by value, one trailing pointer per output,
//! `mem` as the 16-byte `{pointer, u64 bytes}` struct of `catena-lang/src/runtime/executor.rs:14-19`.
//! `Executor::new` can therefore keep resolving `program_<name>` with `dlsym` and calling through
//! libffi; these declarations are for callers that prefer to link directly.
#![allow(non_camel_case_types)]

use core::ffi::{c_char, c_int, c_void};

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct catena_mem_t {
    pub data: *mut c_void,
    pub len: u64, // bytes
}

pub type catena_status_t = i32;
pub const CATENA_OK: catena_status_t = 0;
pub const CATENA_E_ASSERT: catena_status_t = 1;
pub const CATENA_E_CUDA: catena_status_t = 2;
pub const CATENA_E_NO_DEVICE: catena_status_t = 3;
pub const CATENA_E_BAD_ARG: catena_status_t = 4;
pub const CATENA_E_TIMEOUT: catena_status_t = 5;
pub const CATENA_E_TOO_LARGE: catena_status_t = 6;
pub const CATENA_E_UNSUPPORTED: catena_status_t = 7;

/// One instruction of a register program for the generic map kernel (`enum catena_b200_map_op` numbers the opcodes).
/// Opaque handle of a compiled map kernel.
#[repr(C)]
pub struct catena_b200_map_kernel_t {
    _private: [u8; 0],
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct catena_b200_map_insn_t {
    pub op: u16,
    pub dst: u16,
    pub a: u16,
    pub b: u16,
    pub c: u16,
    pub reserved: u16,
    pub target: u32,
}

extern "C" {
    // runtime
    pub fn catena_b200_init(device: c_int) -> catena_status_t;
    pub fn catena_b200_device_count() -> c_int;
    pub fn catena_b200_current_device() -> c_int;
    pub fn catena_b200_set_stream(stream: *mut c_void) -> catena_status_t;
    pub fn catena_b200_set_blocking(blocking: c_int);
    pub fn catena_b200_sync() -> catena_status_t;
    pub fn catena_b200_last_status() -> catena_status_t;
    pub fn catena_b200_clear_status();
    pub fn catena_b200_status_string(s: catena_status_t) -> *const c_char;
    // allocator (replaces GpuRuntime::{alloc, free}, catena-lang/src/runtime/mem.rs:152-190)
    pub fn catena_b200_mem_alloc(bytes: u64, out: *mut catena_mem_t) -> catena_status_t;
    pub fn catena_b200_mem_free(mem: catena_mem_t) -> catena_status_t;
    pub fn catena_b200_mem_upload(host: *const c_void, bytes: u64, out: *mut catena_mem_t) -> catena_status_t;
    pub fn catena_b200_mem_download(mem: catena_mem_t, host: *mut c_void, bytes: u64) -> catena_status_t;
    pub fn catena_b200_ipc_export(mem: catena_mem_t, handle64: *mut c_void, offset: *mut u64) -> catena_status_t;
    pub fn catena_b200_ipc_import(handle64: *const c_void, offset: u64, bytes: u64, out: *mut catena_mem_t) -> catena_status_t;
    // stdlib programs
    pub fn program_math_exp_approx(x: f32, out: *mut f32);
    pub fn program_math_sqrt(x: f32, out: *mut f32);
    pub fn program_math_powf(x: f32, y: f32, out: *mut f32);
    pub fn program_nn_sigmoid(x: f32, out: *mut f32);
    pub fn program_nn_silu(x: f32, out: *mut f32);
    pub fn program_nn_softmax(input: catena_mem_t, out: *mut catena_mem_t);
    pub fn program_nn_rmsnorm(input: catena_mem_t, out: *mut catena_mem_t);
    pub fn program_sum_f32(input: catena_mem_t, out: *mut f32);
    pub fn program_mean_f32(input: catena_mem_t, out: *mut f32);
    pub fn program_max_f32(input: catena_mem_t, out: *mut f32);
    pub fn program_tensor_broadcast_f32(v: f32, n: u64, out: *mut catena_mem_t);
    pub fn program_tensor_arange_f32(n: u64, out: *mut catena_mem_t);
    pub fn program_tensor_slice_f32(input: catena_mem_t, start: u64, len: u64, out: *mut catena_mem_t);
    pub fn program_tensor_concat_f32(l: catena_mem_t, r: catena_mem_t, out: *mut catena_mem_t);
    pub fn program_tensor_argmax_f32(input: catena_mem_t, out: *mut u64);
    // catena-lang/tests/cases/matrix/matmul.hex:2-15
    pub fn program_matmul_2x2_via_mem(a: catena_mem_t, b: catena_mem_t, n: u64, m: u64, k: u64, nk: u64, km: u64,
                                      nm: u64, out: *mut catena_mem_t);
    // catena-lang/tests/cases/reducec/basic.hex:27-58, :60-122; catena-lang/tests/runtime.rs:713-726
    // (catena-lang/smoketest/src/array_head.cpp:37-43 calls the last one directly)
    pub fn program_sum_u64(input: catena_mem_t, out: *mut u64);
    pub fn program_dot_u64(lhs: catena_mem_t, rhs: catena_mem_t, out: *mut u64);
    pub fn program_array_head_u64(input: catena_mem_t, out: *mut u64);
    pub fn program_sum_u64_s(input: catena_mem_t, out: *mut u64) -> catena_status_t;
    pub fn program_dot_u64_s(lhs: catena_mem_t, rhs: catena_mem_t, out: *mut u64) -> catena_status_t;
    pub fn program_array_head_u64_s(input: catena_mem_t, out: *mut u64) -> catena_status_t;
    // programs without a counterpart in catena-lang
    pub fn program_gemm_bf16_rc(a: catena_mem_t, b_colmajor: catena_mem_t, m: u64, n: u64, k: u64, c: *mut catena_mem_t);
    pub fn program_gemm_i8_rc(a: catena_mem_t, b_colmajor: catena_mem_t, m: u64, n: u64, k: u64, c: *mut catena_mem_t);
    pub fn program_attn_decode_bf16(q: catena_mem_t, k_cache: catena_mem_t, v_cache: catena_mem_t, batch: u64, hq: u64,
                                    hkv: u64, d: u64, kv_len: u64, o: *mut catena_mem_t);
    // sharded execution
    pub fn catena_b200_gemm_bf16_into(a: *const c_void, b: *const c_void, c: *mut c_void, m: u64, n: u64, k: u64,
                                      ldc: u64) -> catena_status_t;
    pub fn catena_b200_attn_decode_bf16_into(q: *const c_void, k: *const c_void, v: *const c_void, o: *mut c_void,
                                             batch: u64, hq: u64, hkv: u64, d: u64, kv_len: u64, unit0: u64,
                                             unit1: u64) -> catena_status_t;
    // the same launches fused with the gather of a sharded result: stores into peer-mapped copies of the output
    pub fn catena_b200_gemm_bf16_into_peers(a: *const c_void, b: *const c_void, c: *mut c_void, m: u64, n: u64, k: u64, ldc: u64,
                                            peer_c: *const *mut c_void, n_peers: u32) -> catena_status_t;
    pub fn catena_b200_gemm_i8_into_peers(a: *const c_void, b: *const c_void, c: *mut c_void, m: u64, n: u64, k: u64, ldc: u64,
                                          peer_c: *const *mut c_void, n_peers: u32) -> catena_status_t;
    pub fn catena_b200_attn_decode_bf16_into_peers(q: *const c_void, k: *const c_void, v: *const c_void, o: *mut c_void,
                                                   batch: u64, hq: u64, hkv: u64, d: u64, kv_len: u64, unit0: u64, unit1: u64,
                                                   peer_o: *const *mut c_void, n_peers: u32) -> catena_status_t;
    pub fn catena_b200_check_device_errors() -> catena_status_t;
    // generic map: out[i] = producer(env.., i) for a producer compiled to a register program (include/catena_b200.h)
    pub fn catena_b200_map_program_s(code: *const catena_b200_map_insn_t, n_insn: u32, init: *const u64, n_init: u32, n_regs: u32,
                                     index_reg: u32, result_reg: u32, buffers: *const catena_mem_t, n_buffers: u32,
                                     elem_bytes: u32, len: u64, out: *mut catena_mem_t) -> catena_status_t;
    pub fn catena_b200_map_program_range_s(code: *const catena_b200_map_insn_t, n_insn: u32, init: *const u64, n_init: u32, n_regs: u32,
                                           index_reg: u32, result_reg: u32, buffers: *const catena_mem_t, n_buffers: u32,
                                           elem_bytes: u32, index0: u64, len: u64, out: *mut catena_mem_t) -> catena_status_t;
    // compiled map kernels: PTX written by the library, compiled by the driver
    pub fn catena_b200_map_ptx_s(code: *const catena_b200_map_insn_t, n_insn: u32, init: *const u64, init_is_const: *const u8, n_init: u32,
                                 n_regs: u32, index_reg: u32, result_reg: u32, n_buffers: u32, elem_bytes: u32, text: *mut c_char,
                                 capacity: u64, length: *mut u64) -> catena_status_t;
    pub fn catena_b200_map_compile_s(code: *const catena_b200_map_insn_t, n_insn: u32, init: *const u64, init_is_const: *const u8, n_init: u32,
                                     n_regs: u32, index_reg: u32, result_reg: u32, n_buffers: u32, elem_bytes: u32,
                                     kernel: *mut *mut catena_b200_map_kernel_t) -> catena_status_t;
    pub fn catena_b200_map_kernel_launch_s(kernel: *const catena_b200_map_kernel_t, init: *const u64, n_init: u32, buffers: *const catena_mem_t,
                                           n_buffers: u32, index0: u64, len: u64, out: *mut catena_mem_t) -> catena_status_t;
    pub fn catena_b200_map_kernel_release(kernel: *mut catena_b200_map_kernel_t);
    pub fn catena_b200_sum_f32_noalloc(input: *const c_void, n: u64, out: *mut c_void) -> catena_status_t;
    // Llama-style block (device pointers throughout)
    pub fn catena_b200_llama_workspace_bytes(blk: *const catena_llama_block_t, tokens: u64) -> u64;
    pub fn catena_b200_llama_prefill(blk: *const catena_llama_block_t, ids: *const i32, batch: u64, seq: u64,
                                     k_cache: *mut c_void, v_cache: *mut c_void, out: *mut c_void, workspace: *mut c_void,
                                     workspace_bytes: u64) -> catena_status_t;
    pub fn catena_b200_llama_decode(blk: *const catena_llama_block_t, ids: *const i32, batch: u64, pos: u64,
                                    k_cache: *mut c_void, v_cache: *mut c_void, out: *mut c_void, workspace: *mut c_void,
                                    workspace_bytes: u64) -> catena_status_t;
    pub fn catena_b200_linear_bf16_into(x: *const c_void, w: *const c_void, residual: *const c_void, y: *mut c_void, m: u64,
                                        n: u64, k: u64) -> catena_status_t;

    // gpu.materialize (stdlib/gpu.hex:39-49) over the prebuilt scalar programs
    pub fn catena_b200_launch_len(params: catena_launch_params_t) -> u64;
    pub fn catena_b200_gpu_materialize_f32_s(op: *const c_char, params: catena_launch_params_t, input: catena_mem_t,
                                             out: *mut catena_mem_t) -> catena_status_t;
}

/// catena_dim3_t / catena_launch_params_t of the reference's prelude (src/codegen/prelude.rs:13-26).
#[repr(C)]
#[derive(Clone, Copy)]
#[allow(non_camel_case_types)]
pub struct catena_dim3_t {
    pub x: u32,
    pub y: u32,
    pub z: u32,
}
#[repr(C)]
#[derive(Clone, Copy)]
#[allow(non_camel_case_types)]
pub struct catena_launch_params_t {
    pub grid_dim: catena_dim3_t,
    pub block_dim: catena_dim3_t,
}

/// catena_llama_block_t of include/catena_b200.h.
#[repr(C)]
#[allow(non_camel_case_types)]
pub struct catena_llama_block_t {
    pub hidden: u64,
    pub n_heads: u64,
    pub n_kv_heads: u64,
    pub ffn: u64,
    pub vocab: u64,
    pub max_len: u64,
    pub embedding: *const c_void,
    pub w_qkv: *const c_void,
    pub w_o: *const c_void,
    pub w_gate_up: *const c_void,
    pub w_down: *const c_void,
    pub rope_base: f32,
}
