// `program_*` entry points: the C symbols the reference's Executor binds with dlsym + libffi
// (catena-lang/src/runtime/executor.rs:47-106), here selecting prebuilt sm_100a kernels instead
// of being generated and compiled per Runtime.  Calling convention, ownership and naming follow
// catena-lang/src/codegen/gpu.rs:235-261 and catena-lang/src/codegen/mod.rs:379-388:
// inputs by value, one trailing pointer per output, callee-allocated `mem` outputs
// (catena-lang/src/codegen/ops/materializec.rs:108-122), `{NULL, 0}` for empty results.
#include "catena_math.cuh"
#include "common.cuh"

using namespace catena;

namespace {

// Allocates an output of `bytes`, runs `body(ptr)`, frees the block again when the body fails.
template <class F>
catena_status_t with_output(uint64_t bytes, catena_mem_t* out, F body) {
    if (!out) return fail(CATENA_E_BAD_ARG, "null output pointer");
    out->data = nullptr;
    out->len = 0;
    CATENA_TRY(ensure_device());
    void* p = nullptr;
    CATENA_TRY(pool_alloc(bytes, &p));
    catena_status_t s = body(p);
    if (s == CATENA_OK) s = finish("program");
    if (s != CATENA_OK) {
        pool_free(p);
        return s;
    }
    out->data = p;
    out->len = bytes;
    return CATENA_OK;
}

// mem.cast.f32 (catena-lang/src/codegen/gpu.rs:768-782): len = bytes / sizeof(float)
inline uint64_t f32_len(catena_mem_t m) { return m.len / sizeof(float); }

inline catena_status_t check_mem(catena_mem_t m, const char* what) {
    if (m.len != 0 && !m.data) return fail(CATENA_E_BAD_ARG, what);
    return CATENA_OK;
}

}  // namespace

extern "C" {

// ---- scalar programs: host execution, like the reference's code outside materialize ----------
#define SCALAR1(sym, fn) \
    void sym(float x, float* out) { if (out) *out = cmath::fn(x); }
SCALAR1(program_math_sin_approx, sin_approx)
SCALAR1(program_math_cos_approx, cos_approx)
SCALAR1(program_math_sin_approx_full_nonneg, sin_full_nonneg)
SCALAR1(program_math_sin_approx_full, sin_full)
SCALAR1(program_math_log_approx, log_approx)
SCALAR1(program_math_exp_approx_nonneg, exp_nonneg)
SCALAR1(program_math_exp_approx, exp_approx)
SCALAR1(program_math_exp2_approx, exp2_approx)
SCALAR1(program_math_log2_approx, log2_approx)
SCALAR1(program_math_sqrt, sqrt_newton)
SCALAR1(program_nn_sigmoid, sigmoid)
SCALAR1(program_nn_silu, silu)
SCALAR1(program_nn_tanh, tanh_approx)
SCALAR1(program_nn_gelu_approx, gelu_approx)
#undef SCALAR1
void program_math_powf(float x, float y, float* out) { if (out) *out = cmath::powf_approx(x, y); }

// ---- softmax / rmsnorm ------------------------------------------------------------------------
catena_status_t program_nn_softmax_s(catena_mem_t in, catena_mem_t* out) {
    CATENA_TRY(check_mem(in, "nn.softmax: null input"));
    uint64_t n = f32_len(in);
    return with_output(n * 4, out, [&](void* p) { return launch_softmax((const float*)in.data, (float*)p, n); });
}
catena_status_t program_nn_rmsnorm_s(catena_mem_t in, catena_mem_t* out) {
    CATENA_TRY(check_mem(in, "nn.rmsnorm: null input"));
    uint64_t n = f32_len(in);
    return with_output(n * 4, out, [&](void* p) { return launch_rmsnorm((const float*)in.data, (float*)p, n); });
}
void program_nn_softmax(catena_mem_t in, catena_mem_t* out) { (void)program_nn_softmax_s(in, out); }
void program_nn_rmsnorm(catena_mem_t in, catena_mem_t* out) { (void)program_nn_rmsnorm_s(in, out); }

// ---- folds ---------------------------------------------------------------------------------------
catena_status_t program_sum_f32_s(catena_mem_t in, float* out) {
    if (!out) return fail(CATENA_E_BAD_ARG, "sum-f32: null out");
    *out = 0.0f;
    CATENA_TRY(check_mem(in, "sum-f32: null input"));
    return reduce_f32(RED_SUM, (const float*)in.data, f32_len(in), out);
}
catena_status_t program_mean_f32_s(catena_mem_t in, float* out) {
    if (!out) return fail(CATENA_E_BAD_ARG, "mean-f32: null out");
    *out = 0.0f;
    CATENA_TRY(check_mem(in, "mean-f32: null input"));
    float sum = 0.0f;
    CATENA_TRY(reduce_f32(RED_SUM, (const float*)in.data, f32_len(in), &sum));
    *out = cmath::div(sum, cmath::u64_to_f32(f32_len(in)));   // sum.hex:61-64 (0/0 for an empty input)
    return CATENA_OK;
}
catena_status_t program_max_f32_s(catena_mem_t in, float* out) {
    if (!out) return fail(CATENA_E_BAD_ARG, "max-f32: null out");
    *out = 0.0f;
    CATENA_TRY(check_mem(in, "max-f32: null input"));
    return reduce_f32(RED_MAX, (const float*)in.data, f32_len(in), out);
}
void program_sum_f32(catena_mem_t in, float* out) { (void)program_sum_f32_s(in, out); }
void program_mean_f32(catena_mem_t in, float* out) { (void)program_mean_f32_s(in, out); }
void program_max_f32(catena_mem_t in, float* out) { (void)program_max_f32_s(in, out); }

// ---- tensor programs -----------------------------------------------------------------------------
catena_status_t program_tensor_broadcast_f32_s(float v, uint64_t n, catena_mem_t* out) {
    return with_output(n * 4, out, [&](void* p) { return launch_broadcast(v, (float*)p, n); });
}
catena_status_t program_tensor_arange_f32_s(uint64_t n, catena_mem_t* out) {
    return with_output(n * 4, out, [&](void* p) { return launch_arange((float*)p, n); });
}
catena_status_t program_tensor_slice_f32_s(catena_mem_t in, uint64_t start, uint64_t len, catena_mem_t* out) {
    if (out) { out->data = nullptr; out->len = 0; }
    CATENA_TRY(check_mem(in, "tensor.slice-f32: null input"));
    // the producer asserts input_len > start + i for every element (tensor.hex:58-64); with len == 0
    // no element is produced and nothing is asserted
    uint64_t in_len = f32_len(in);
    if (len != 0 && (start >= in_len || len > in_len - start))
        return fail(CATENA_E_ASSERT, "tensor.slice-f32: slice reaches past the input");
    return with_output(len * 4, out, [&](void* p) { return launch_slice((const float*)in.data, start, (float*)p, len); });
}
catena_status_t program_tensor_concat_f32_s(catena_mem_t l, catena_mem_t r, catena_mem_t* out) {
    CATENA_TRY(check_mem(l, "tensor.concat-f32: null left"));
    CATENA_TRY(check_mem(r, "tensor.concat-f32: null right"));
    uint64_t nl = f32_len(l), nr = f32_len(r);
    return with_output((nl + nr) * 4, out, [&](void* p) {
        return launch_concat((const float*)l.data, nl, (const float*)r.data, nr, (float*)p);
    });
}
catena_status_t program_tensor_argmax_f32_s(catena_mem_t in, uint64_t* out) {
    if (!out) return fail(CATENA_E_BAD_ARG, "tensor.argmax-f32: null out");
    *out = 0;
    CATENA_TRY(check_mem(in, "tensor.argmax-f32: null input"));
    return argmax_f32((const float*)in.data, f32_len(in), out);
}
void program_tensor_broadcast_f32(float v, uint64_t n, catena_mem_t* out) { (void)program_tensor_broadcast_f32_s(v, n, out); }
void program_tensor_arange_f32(uint64_t n, catena_mem_t* out) { (void)program_tensor_arange_f32_s(n, out); }
void program_tensor_slice_f32(catena_mem_t in, uint64_t start, uint64_t len, catena_mem_t* out) {
    (void)program_tensor_slice_f32_s(in, start, len, out);
}
void program_tensor_concat_f32(catena_mem_t l, catena_mem_t r, catena_mem_t* out) { (void)program_tensor_concat_f32_s(l, r, out); }
void program_tensor_argmax_f32(catena_mem_t in, uint64_t* out) { (void)program_tensor_argmax_f32_s(in, out); }

// ---- f32 matmul --------------------------------------------------------------------------------
catena_status_t program_matmul_2x2_via_mem_s(catena_mem_t a, catena_mem_t b, uint64_t n, uint64_t m, uint64_t k,
                                             uint64_t nk, uint64_t km, uint64_t nm, catena_mem_t* out) {
    if (out) { out->data = nullptr; out->len = 0; }
    CATENA_TRY(check_mem(a, "matmul: null a"));
    CATENA_TRY(check_mem(b, "matmul: null b"));
    // runtime length asserts of the entry program (matmul.hex:18-27)
    if (f32_len(a) != nk) return fail(CATENA_E_ASSERT, "matmul: a.len/4 != n*k argument");
    if (f32_len(b) != km) return fail(CATENA_E_ASSERT, "matmul: b.len/4 != k*m argument");
    // the type-level products n*k, k*m, n*m are not re-checked by the reference; a mismatch there
    // would read out of bounds, so it is rejected here
    if (n * k != nk || k * m != km || n * m != nm) return fail(CATENA_E_BAD_ARG, "matmul: nk/km/nm do not match n, m, k");
    return with_output(nm * 4, out, [&](void* p) {
        return launch_matmul_f32((const float*)a.data, (const float*)b.data, (float*)p, n, m, k);
    });
}
void program_matmul_2x2_via_mem(catena_mem_t a, catena_mem_t b, uint64_t n, uint64_t m, uint64_t k, uint64_t nk,
                                uint64_t km, uint64_t nm, catena_mem_t* out) {
    (void)program_matmul_2x2_via_mem_s(a, b, n, m, k, nk, km, nm, out);
}
static catena_status_t identity_matmul(catena_mem_t a, uint64_t n, uint64_t nn, catena_mem_t* out, int left) {
    if (out) { out->data = nullptr; out->len = 0; }
    CATENA_TRY(check_mem(a, "matmul identity: null a"));
    if (f32_len(a) != nn) return fail(CATENA_E_ASSERT, "matmul identity: a.len/4 != n*n argument");
    if (n * n != nn) return fail(CATENA_E_BAD_ARG, "matmul identity: nn != n*n");
    return with_output(nn * 4, out, [&](void* p) { return launch_identity_matmul_f32((const float*)a.data, (float*)p, n, left); });
}
void program_matmul_right_identity_2x2_via_mem(catena_mem_t a, uint64_t n, uint64_t nn, catena_mem_t* out) {
    (void)identity_matmul(a, n, nn, out, 0);
}
void program_matmul_left_identity_2x2_via_mem(catena_mem_t a, uint64_t n, uint64_t nn, catena_mem_t* out) {
    (void)identity_matmul(a, n, nn, out, 1);
}

// ---- map ---------------------------------------------------------------------------------------------
catena_status_t catena_b200_map_f32_s(const char* op, catena_mem_t in, catena_mem_t* out) {
    int id = map_op_from_name(op);
    if (id < 0) return fail(CATENA_E_BAD_ARG, "map: unknown scalar program");
    CATENA_TRY(check_mem(in, "map: null input"));
    uint64_t n = f32_len(in);
    return with_output(n * 4, out, [&](void* p) { return launch_map_unary(id, (const float*)in.data, (float*)p, n); });
}
uint64_t catena_b200_launch_len(catena_launch_params_t p) {
    return (uint64_t)p.grid_dim.x * p.grid_dim.y * p.grid_dim.z * p.block_dim.x * p.block_dim.y * p.block_dim.z;
}
catena_status_t catena_b200_gpu_materialize_f32_s(const char* op, catena_launch_params_t params, catena_mem_t in, catena_mem_t* out) {
    if (out) { out->data = nullptr; out->len = 0; }
    int id = map_op_from_name(op);
    if (id < 0) return fail(CATENA_E_BAD_ARG, "gpu.materialize: unknown scalar program");
    // the product of six u32 dimensions can pass 2^64: refuse instead of wrapping
    const long double exact = (long double)params.grid_dim.x * params.grid_dim.y * params.grid_dim.z * (long double)params.block_dim.x *
                              params.block_dim.y * params.block_dim.z;
    if (exact > 9.0e18L) return fail(CATENA_E_TOO_LARGE, "gpu.materialize: launch length beyond 2^63");
    const uint64_t n = catena_b200_launch_len(params);
    if (n == 0) return with_output(0, out, [&](void*) { return CATENA_OK; });
    CATENA_TRY(check_mem(in, "gpu.materialize: null environment buffer"));
    if (f32_len(in) < n) return fail(CATENA_E_ASSERT, "gpu.materialize: environment buffer shorter than the launch length");
    return with_output(n * 4, out, [&](void* p) { return launch_map_unary(id, (const float*)in.data, (float*)p, n); });
}
catena_status_t catena_b200_map_f32_into(const char* op, const void* in, void* out, uint64_t n) {
    int id = map_op_from_name(op);
    if (id < 0) return fail(CATENA_E_BAD_ARG, "map: unknown scalar program");
    CATENA_TRY(ensure_device());
    if (n && (!in || !out)) return fail(CATENA_E_BAD_ARG, "map: null buffer");
    CATENA_TRY(launch_map_unary(id, (const float*)in, (float*)out, n));
    return finish("map");
}
catena_status_t catena_b200_softmax_f32_into(const void* in, void* out, uint64_t n) {
    CATENA_TRY(ensure_device());
    if (n && (!in || !out)) return fail(CATENA_E_BAD_ARG, "softmax: null buffer");
    CATENA_TRY(launch_softmax((const float*)in, (float*)out, n));
    return finish("softmax");
}
catena_status_t catena_b200_rmsnorm_f32_into(const void* in, void* out, uint64_t n) {
    CATENA_TRY(ensure_device());
    if (n && (!in || !out)) return fail(CATENA_E_BAD_ARG, "rmsnorm: null buffer");
    CATENA_TRY(launch_rmsnorm((const float*)in, (float*)out, n));
    return finish("rmsnorm");
}

// ---- tensor-core GEMMs ---------------------------------------------------------------------------------
static catena_status_t gemm_program(catena_mem_t a, catena_mem_t b, uint64_t m, uint64_t n, uint64_t k,
                                    catena_mem_t* c, int is_i8) {
    if (c) { c->data = nullptr; c->len = 0; }
    CATENA_TRY(check_mem(a, "gemm: null a"));
    CATENA_TRY(check_mem(b, "gemm: null b"));
    const uint64_t in_b = is_i8 ? 1 : 2, out_b = is_i8 ? 4 : 2;
    if (a.len != m * k * in_b) return fail(CATENA_E_ASSERT, "gemm: a.len does not match m*k");
    if (b.len != n * k * in_b) return fail(CATENA_E_ASSERT, "gemm: b.len does not match n*k");
    return with_output(m * n * out_b, c, [&](void* p) { return launch_gemm_tc(a.data, b.data, p, m, n, k, n, is_i8); });
}
catena_status_t program_gemm_bf16_rc_s(catena_mem_t a, catena_mem_t b, uint64_t m, uint64_t n, uint64_t k, catena_mem_t* c) {
    return gemm_program(a, b, m, n, k, c, 0);
}
catena_status_t program_gemm_i8_rc_s(catena_mem_t a, catena_mem_t b, uint64_t m, uint64_t n, uint64_t k, catena_mem_t* c) {
    return gemm_program(a, b, m, n, k, c, 1);
}
void program_gemm_bf16_rc(catena_mem_t a, catena_mem_t b, uint64_t m, uint64_t n, uint64_t k, catena_mem_t* c) {
    (void)gemm_program(a, b, m, n, k, c, 0);
}
void program_gemm_i8_rc(catena_mem_t a, catena_mem_t b, uint64_t m, uint64_t n, uint64_t k, catena_mem_t* c) {
    (void)gemm_program(a, b, m, n, k, c, 1);
}
catena_status_t catena_b200_gemm_bf16_into(const void* a, const void* b, void* c, uint64_t m, uint64_t n, uint64_t k,
                                           uint64_t ldc) {
    CATENA_TRY(launch_gemm_tc(a, b, c, m, n, k, ldc, 0));
    return finish("gemm_bf16");
}
catena_status_t catena_b200_gemm_i8_into(const void* a, const void* b, void* c, uint64_t m, uint64_t n, uint64_t k,
                                         uint64_t ldc) {
    CATENA_TRY(launch_gemm_tc(a, b, c, m, n, k, ldc, 1));
    return finish("gemm_i8");
}
catena_status_t catena_b200_gemm_bf16_into_peers(const void* a, const void* b, void* c, uint64_t m, uint64_t n, uint64_t k,
                                                 uint64_t ldc, void* const* peer_c, uint32_t n_peers) {
    CATENA_TRY(launch_gemm_tc_peers(a, b, c, m, n, k, ldc, 0, peer_c, n_peers));
    return finish("gemm_bf16_peers");
}
catena_status_t catena_b200_gemm_i8_into_peers(const void* a, const void* b, void* c, uint64_t m, uint64_t n, uint64_t k,
                                               uint64_t ldc, void* const* peer_c, uint32_t n_peers) {
    CATENA_TRY(launch_gemm_tc_peers(a, b, c, m, n, k, ldc, 1, peer_c, n_peers));
    return finish("gemm_i8_peers");
}
catena_status_t catena_b200_matmul_f32_into(const void* a, const void* b, void* c, uint64_t n, uint64_t m, uint64_t k) {
    CATENA_TRY(ensure_device());
    if (!a || !b || !c) return fail(CATENA_E_BAD_ARG, "matmul_f32_into: null operand");
    CATENA_TRY(launch_matmul_f32((const float*)a, (const float*)b, (float*)c, n, m, k));
    return finish("matmul_f32");
}

// ---- attention decode -------------------------------------------------------------------------------------
catena_status_t program_attn_decode_bf16_s(catena_mem_t q, catena_mem_t kc, catena_mem_t vc, uint64_t batch, uint64_t hq,
                                           uint64_t hkv, uint64_t d, uint64_t kv_len, catena_mem_t* o) {
    if (o) { o->data = nullptr; o->len = 0; }
    CATENA_TRY(check_mem(q, "attn: null q"));
    CATENA_TRY(check_mem(kc, "attn: null key cache"));
    CATENA_TRY(check_mem(vc, "attn: null value cache"));
    if (q.len != batch * hq * d * 2) return fail(CATENA_E_ASSERT, "attn: q.len does not match batch*hq*d");
    if (kc.len != batch * hkv * kv_len * d * 2 || vc.len != kc.len)
        return fail(CATENA_E_ASSERT, "attn: cache length does not match batch*hkv*kv_len*d");
    return with_output(batch * hq * d * 2, o, [&](void* p) {
        return launch_attn_decode(q.data, kc.data, vc.data, p, batch, hq, hkv, d, kv_len, kv_len, 0, batch * hkv);
    });
}
void program_attn_decode_bf16(catena_mem_t q, catena_mem_t kc, catena_mem_t vc, uint64_t batch, uint64_t hq, uint64_t hkv,
                              uint64_t d, uint64_t kv_len, catena_mem_t* o) {
    (void)program_attn_decode_bf16_s(q, kc, vc, batch, hq, hkv, d, kv_len, o);
}
catena_status_t catena_b200_attn_decode_bf16_into(const void* q, const void* kc, const void* vc, void* o, uint64_t batch,
                                                  uint64_t hq, uint64_t hkv, uint64_t d, uint64_t kv_len, uint64_t unit0,
                                                  uint64_t unit1) {
    CATENA_TRY(launch_attn_decode(q, kc, vc, o, batch, hq, hkv, d, kv_len, kv_len, unit0, unit1));
    return finish("attn_decode");
}

catena_status_t catena_b200_attn_decode_bf16_into_peers(const void* q, const void* kc, const void* vc, void* o, uint64_t batch,
                                                        uint64_t hq, uint64_t hkv, uint64_t d, uint64_t kv_len, uint64_t unit0,
                                                        uint64_t unit1, void* const* peer_o, uint32_t n_peers) {
    CATENA_TRY(launch_attn_decode(q, kc, vc, o, batch, hq, hkv, d, kv_len, kv_len, unit0, unit1, peer_o, n_peers));
    return finish("attn_decode");
}

void catena_b200_debug_set_cta_limit(int limit) {
    gemm_tc_set_cta_limit(limit);
    attn_set_cluster_limit(limit > 0 ? (limit >= 8 ? limit / 8 : 1) : 0);
}

void catena_b200_debug_set_gemm_pair(int on) { gemm_tc_set_pair_mode(on); }
void catena_b200_debug_set_attn_tc(int on) { attn_set_tc_mode(on); }
void catena_b200_debug_set_decode_fused(int mode) { decode_fused_set_mode(mode); }
void catena_b200_debug_attn_last_launch(uint32_t out[4]) { attn_last_launch(out); }
catena_status_t catena_b200_debug_rcp_check(uint64_t out[2]) {
    if (!out) return fail(CATENA_E_BAD_ARG, "rcp check: null argument");
    CATENA_TRY(ensure_device());
    return attn_prefill_rcp_check(out);
}

catena_status_t catena_b200_debug_packed_f32x2_check(uint64_t out[3]) {
    if (!out) return fail(CATENA_E_BAD_ARG, "packed f32x2 check: null argument");
    CATENA_TRY(ensure_device());
    return packed_f32x2_check(out);
}

catena_status_t catena_b200_check_device_errors(void) {
    CATENA_TRY(gemm_tc_check_errors());
    CATENA_TRY(decode_fused_check_errors());
    CATENA_TRY(map_program_check_errors());
    return attn_check_errors();
}

}  // extern "C"
