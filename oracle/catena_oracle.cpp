// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// A plain C++ restatement of what catena-lang's code generator prints for the
// data-parallel hot path, evaluated on the host.  Nothing in the shipped library links,
// loads or calls this file: it exists so that the parity tests, the smoke check and the
// reported CPU baseline have an independent answer to compare the CUDA kernels with.
//
// Build (oracle/Makefile):  g++ -O2 -ffp-contract=off -pthread -shared -fPIC
// `-ffp-contract=off` is mandatory: the reference compiles device code with
// `--fmad=false` (catena-lang/src/runtime/artifact.rs:59-80), so `f32.mul` followed by
// `f32.add` is two roundings, and only `f32.fma` fuses (codegen/gpu.rs:589-604).
//
// Parity status:
//   * everything under "reference programs" follows in-tree reference sources line by
//     line and is pinned by the known-answer vectors of the reference's own tests
//     (tests/runtime.rs, tests/cases/*.rs) — see tests/test_oracle_golden.py;
//   * the bf16 / int8 GEMM and the cached-attention decode have NO counterpart in the
//     reference (it has no bf16, int8 or attention): they are composed from the
//     reference's rules (ascending-k left fold, unfused mul/add, its softmax program) and
//     are "parity unpinned".
//
// Each function cites the reference file:line it restates.

#include <cmath>
#include <cstdint>
#include <cstring>
#include <cstdlib>
#include <string>
#include <thread>
#include <vector>

namespace {

// ---- codegen/prelude.rs:64-80 : bit casts ------------------------------------------
inline float bits_f32(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }
inline uint32_t f32_bits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }

// ---- codegen/gpu.rs:322-447 : primitive table (one C expression each) ----------------
inline float f32_add(float a, float b) { return a + b; }
inline float f32_sub(float a, float b) { return a - b; }
inline float f32_mul(float a, float b) { return a * b; }
inline float f32_div(float a, float b) { return a / b; }
inline float f32_neg(float a) { return -a; }
inline float f32_select(bool c, float t, float f) { return c ? t : f; }       // gpu.rs:624-640
inline uint32_t f32_round_to_u32(float x) { return (uint32_t)nearbyintf(x); } // gpu.rs:642-655
inline float u32_to_f32(uint32_t x) { return (float)x; }
inline float u64_to_f32(uint64_t x) { return (float)x; }

// ---- stdlib/math.hex:3-23 ------------------------------------------------------------
float sin_approx(float x) {
    float x2 = f32_mul(x, x);
    float x3 = f32_mul(x2, x);
    float x5 = f32_mul(x3, x2);
    float x7 = f32_mul(x5, x2);
    float f3 = u32_to_f32(0x6u), f5 = u32_to_f32(0x78u), f7 = u32_to_f32(0x13B0u);
    float t3 = f32_div(x3, f3), t5 = f32_div(x5, f5), t7 = f32_div(x7, f7);
    float p1 = f32_sub(x, t3);
    float p2 = f32_add(p1, t5);
    return f32_sub(p2, t7);
}

// ---- stdlib/math.hex:27-47 -----------------------------------------------------------
float cos_approx(float x) {
    float x2 = f32_mul(x, x);
    float x4 = f32_mul(x2, x2);
    float x6 = f32_mul(x4, x2);
    float f2 = u32_to_f32(2u), f4 = u32_to_f32(0x18u), f6 = u32_to_f32(0x2D0u), one = u32_to_f32(1u);
    float t2 = f32_div(x2, f2), t4 = f32_div(x4, f4), t6 = f32_div(x6, f6);
    float p1 = f32_sub(one, t2);
    float p2 = f32_add(p1, t4);
    return f32_sub(p2, t6);
}

// ---- stdlib/math.hex:52-87 -----------------------------------------------------------
float sin_full_nonneg(float x) {
    float inv_pio2 = bits_f32(0x3F22F983u), hi = bits_f32(0x3FC90FDAu), lo = bits_f32(0x33A22168u);
    float scaled = f32_mul(x, inv_pio2);
    uint32_t n = f32_round_to_u32(scaled);
    float nf = u32_to_f32(n);
    float r1 = f32_sub(x, f32_mul(nf, hi));
    float r = f32_sub(r1, f32_mul(nf, lo));
    float s = sin_approx(r), c = cos_approx(r);
    float ns = f32_neg(s), nc = f32_neg(c);
    uint32_t q = n & 3u;
    float q23 = f32_select(q == 2u, ns, nc);
    float q123 = f32_select(q == 1u, c, q23);
    return f32_select(q == 0u, s, q123);
}

// ---- stdlib/math.hex:91-103 ----------------------------------------------------------
float sin_full(float x) {
    float zero = u32_to_f32(0u);
    bool neg = x < zero;
    float mag = f32_select(neg, f32_neg(x), x);
    float base = sin_full_nonneg(mag);
    return f32_select(neg, f32_neg(base), base);
}

// ---- stdlib/math.hex:110-144 ---------------------------------------------------------
float log_approx(float x) {
    float ln2 = bits_f32(0x3F317218u);
    float c0 = bits_f32(0xC00BE629u), c1 = bits_f32(0x4087355Au), c2 = bits_f32(0xC03AA687u),
          c3 = bits_f32(0x3F60A4E1u);
    uint32_t xb = f32_bits(x);
    uint32_t eb = xb >> 0x17u;
    uint32_t fb = xb & 0x007FFFFFu;
    float m = bits_f32(fb + 0x3F000000u);
    float e = f32_sub(u32_to_f32(eb), u32_to_f32(0x7Eu));
    float p2 = f32_add(c2, f32_mul(m, c3));
    float p1 = f32_add(c1, f32_mul(m, p2));
    float poly = f32_add(c0, f32_mul(m, p1));
    return f32_add(poly, f32_mul(e, ln2));
}

// ---- stdlib/math.hex:148-183 ---------------------------------------------------------
float exp_nonneg(float x) {
    float inv_ln2 = bits_f32(0x3FB8AA3Bu), hi = bits_f32(0x3F317200u), lo = bits_f32(0x35BFBE8Eu);
    float c0 = bits_f32(0x3F7FF8FCu), c1 = bits_f32(0x3F809C7Eu), c2 = bits_f32(0x3EEF1187u),
          c3 = bits_f32(0x3E738A8Bu);
    float scaled = f32_mul(x, inv_ln2);
    uint32_t k = f32_round_to_u32(scaled);
    float kf = u32_to_f32(k);
    float r1 = f32_sub(x, f32_mul(kf, hi));
    float xr = f32_sub(r1, f32_mul(kf, lo));
    float p2 = f32_add(c2, f32_mul(xr, c3));
    float p1 = f32_add(c1, f32_mul(xr, p2));
    float poly = f32_add(c0, f32_mul(xr, p1));
    uint32_t pow2_bits = (k + 0x7Fu) * 0x00800000u;  // u32 wraparound, math.hex:174-178
    return f32_mul(poly, bits_f32(pow2_bits));
}

// ---- stdlib/math.hex:185-199 ---------------------------------------------------------
float exp_approx(float x) {
    float zero = u32_to_f32(0u), one = bits_f32(0x3F800000u);
    bool neg = x < zero;
    float mag = f32_select(neg, f32_neg(x), x);
    float base = exp_nonneg(mag);
    float recip = f32_div(one, base);
    return f32_select(neg, recip, base);
}

// ---- stdlib/math.hex:202-231 ---------------------------------------------------------
float exp2_approx(float x) { return exp_approx(f32_mul(x, bits_f32(0x3F317218u))); }
float log2_approx(float x) { return f32_mul(log_approx(x), bits_f32(0x3FB8AA3Bu)); }
float powf_approx(float x, float y) { return exp2_approx(f32_mul(y, log2_approx(x))); }

// ---- stdlib/math.hex:235-272 ---------------------------------------------------------
float sqrt_newton(float x) {
    float zero = u32_to_f32(0u), one = bits_f32(0x3F800000u), half = bits_f32(0x3F000000u);
    float g = f32_select(x < one, one, x);
    for (int it = 0; it < 6; ++it) g = f32_mul(f32_add(g, f32_div(x, g)), half);
    return f32_select(x <= zero, zero, g);
}

// ---- stdlib/nn.hex:2-56 --------------------------------------------------------------
float sigmoid(float x) {
    float one = 1.0f;  // f32.one
    return f32_div(one, f32_add(one, exp_approx(f32_neg(x))));
}
float silu(float x) { return f32_mul(x, sigmoid(x)); }
float tanh_approx(float x) {
    float one = 1.0f, two = bits_f32(0x40000000u);
    return f32_sub(f32_mul(sigmoid(f32_mul(x, two)), two), one);
}
float gelu_approx(float x) {
    float one = 1.0f, half = bits_f32(0x3F000000u), s2pi = bits_f32(0x3F4C422Au),
          cc = bits_f32(0x3D372713u);
    float x3 = f32_mul(f32_mul(x, x), x);
    float inner = f32_add(x, f32_mul(x3, cc));
    float shaped = tanh_approx(f32_mul(inner, s2pi));
    return f32_mul(f32_mul(x, f32_add(one, shaped)), half);
}

// ---- codegen/ops/reducec.rs:75-131 : acc = zero; for i in 0..n: acc = add(acc, get(i)) --
template <class Acc, class Get, class Add>
inline Acc reducec(Acc zero, uint64_t n, Get get, Add add) {
    Acc acc = zero;
    for (uint64_t i = 0; i < n; ++i) {
        auto v = get(i);
        Acc next = add(acc, v);
        acc = next;
    }
    return acc;
}

// stdlib/sum.hex:73-84 : keep the accumulator when acc >= value
inline float max_env(float acc, float v) { return f32_select(acc >= v, acc, v); }

// ---- codegen/ops/materializec.rs:36-145 : out[i] = f(env, i), i in [0, len) -----------
// The kernel's elements are independent, so splitting [0,len) over host threads is
// semantically the reference's launch; `threads <= 1` keeps the literal single-thread order.
template <class F>
inline void parallel_for(uint64_t len, int threads, F body) {
    if (threads <= 1 || len < 2) {
        for (uint64_t i = 0; i < len; ++i) body(i);
        return;
    }
    uint64_t nt = (uint64_t)threads < len ? (uint64_t)threads : len;
    std::vector<std::thread> pool;
    for (uint64_t t = 0; t < nt; ++t) {
        uint64_t lo = len * t / nt, hi = len * (t + 1) / nt;
        pool.emplace_back([=, &body]() { for (uint64_t i = lo; i < hi; ++i) body(i); });
    }
    for (auto& th : pool) th.join();
}
template <class T, class F>
inline void materializec(T* out, uint64_t len, int threads, F f) {
    parallel_for(len, threads, [&](uint64_t i) { out[i] = f(i); });
}

// bf16 helpers for the beyond-reference programs: exact upcast, RNE downcast.
inline float bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }
inline uint16_t f32_to_bf16_rne(float f) {
    uint32_t u = f32_bits(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u);  // quiet NaN
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7FFFu + lsb;
    return (uint16_t)(u >> 16);
}

}  // namespace

extern "C" {

int orc_max_threads(void) {
    unsigned n = std::thread::hardware_concurrency();
    return n ? (int)n : 1;
}

// ---- scalar programs (Appendix of entry points: `void program_math_<name>(float, float*)`) ----
float orc_math_sin_approx(float x) { return sin_approx(x); }
float orc_math_cos_approx(float x) { return cos_approx(x); }
float orc_math_sin_approx_full_nonneg(float x) { return sin_full_nonneg(x); }
float orc_math_sin_approx_full(float x) { return sin_full(x); }
float orc_math_log_approx(float x) { return log_approx(x); }
float orc_math_exp_approx_nonneg(float x) { return exp_nonneg(x); }
float orc_math_exp_approx(float x) { return exp_approx(x); }
float orc_math_exp2_approx(float x) { return exp2_approx(x); }
float orc_math_log2_approx(float x) { return log2_approx(x); }
float orc_math_powf(float x, float y) { return powf_approx(x, y); }
float orc_math_sqrt(float x) { return sqrt_newton(x); }
float orc_nn_sigmoid(float x) { return sigmoid(x); }
float orc_nn_silu(float x) { return silu(x); }
float orc_nn_tanh(float x) { return tanh_approx(x); }
float orc_nn_gelu_approx(float x) { return gelu_approx(x); }
// codegen/gpu.rs:589-604 : f32.fma = fmaf (pinned by tests/runtime.rs:333-363)
float orc_f32_fma(float a, float b, float c) { return fmaf(a, b, c); }
// unfused counterpart (`f32.mul` then `f32.add`)
float orc_f32_mul_add(float a, float b, float c) { return f32_add(f32_mul(a, b), c); }

// elementwise application of a scalar program over a buffer (for bulk parity checks)
// op ids follow the order of the list above (0 = sin_approx ... 13 = gelu_approx; 9 = powf is binary)
void orc_map_unary(int op, const float* x, float* y, uint64_t n, int threads) {
    typedef float (*fn_t)(float);
    static const fn_t table[] = {sin_approx, cos_approx, sin_full_nonneg, sin_full, log_approx,
                                 exp_nonneg, exp_approx, exp2_approx, log2_approx, nullptr,
                                 sqrt_newton, sigmoid, silu, tanh_approx, gelu_approx};
    if (op < 0 || op > 14 || !table[op]) return;
    fn_t f = table[op];
    materializec(y, n, threads, [&](uint64_t i) { return f(x[i]); });
}

// ---- stdlib/sum.hex:29-44, 47-67, 86-101 ---------------------------------------------
float orc_sum_f32(const float* x, uint64_t n) {
    return reducec(bits_f32(0x00000000u), n, [&](uint64_t i) { return x[i]; }, f32_add);
}
float orc_mean_f32(const float* x, uint64_t n) { return f32_div(orc_sum_f32(x, n), u64_to_f32(n)); }
float orc_max_f32(const float* x, uint64_t n) {
    return reducec(bits_f32(0xFF800000u), n, [&](uint64_t i) { return x[i]; }, max_env);
}

// integer folds used by the reference's reducec tests (tests/cases/reducec.rs:6-48)
uint64_t orc_sum_u64(const uint64_t* x, uint64_t n) {
    return reducec((uint64_t)0, n, [&](uint64_t i) { return x[i]; },
                   [](uint64_t a, uint64_t b) { return a + b; });
}
uint64_t orc_dot_u64(const uint64_t* x, const uint64_t* y, uint64_t n) {
    return reducec((uint64_t)0, n, [&](uint64_t i) { return x[i] * y[i]; },
                   [](uint64_t a, uint64_t b) { return a + b; });
}

// ---- stdlib/tensor.hex:171-227 : argmax, pair accumulator, ties keep the first ---------
// returns UINT64_MAX for an empty input (the reference asserts, i.e. traps).
uint64_t orc_tensor_argmax_f32(const float* x, uint64_t n) {
    if (n == 0) return UINT64_MAX;
    struct P { uint64_t pos; float v; };
    P init{0, x[0]};
    P r = reducec(init, n, [&](uint64_t i) { return P{i, x[i]}; },
                  [](P acc, P v) {
                      bool keep = acc.v >= v.v;
                      return P{keep ? acc.pos : v.pos, f32_select(keep, acc.v, v.v)};
                  });
    return r.pos;
}

// ---- stdlib/nn.hex:93-122 : softmax = host fold max, host fold sum(exp~), map kernel ----
void orc_nn_softmax(const float* x, float* y, uint64_t n, int threads) {
    float max_x = orc_max_f32(x, n);
    float denom = reducec(bits_f32(0u), n,
                          [&](uint64_t i) { return exp_approx(f32_sub(x[i], max_x)); }, f32_add);
    materializec(y, n, threads,
                 [&](uint64_t i) { return f32_div(exp_approx(f32_sub(x[i], max_x)), denom); });
}

// ---- stdlib/nn.hex:154-182 : rmsnorm = fold sum x*x, /len, +eps, sqrt~, map x/rms ------
void orc_nn_rmsnorm(const float* x, float* y, uint64_t n, int threads) {
    float ss = reducec(bits_f32(0u), n, [&](uint64_t i) { return f32_mul(x[i], x[i]); }, f32_add);
    float mean_sq = f32_div(ss, u64_to_f32(n));
    float rms = sqrt_newton(f32_add(mean_sq, bits_f32(0x3727C5ACu)));
    materializec(y, n, threads, [&](uint64_t i) { return f32_div(x[i], rms); });
}

// ---- stdlib/tensor.hex:10-21, 35-46, 49-82, 109-168 ----------------------------------
void orc_tensor_broadcast_f32(float v, uint64_t n, float* y) {
    materializec(y, n, 1, [&](uint64_t) { return v; });
}
void orc_tensor_arange_f32(uint64_t n, float* y) {
    materializec(y, n, 1, [&](uint64_t i) { return u64_to_f32(i); });
}
// returns 0 on success, 1 where the reference's per-element bounds assert would trap
int orc_tensor_slice_f32(const float* x, uint64_t in_len, uint64_t start, uint64_t len, float* y) {
    for (uint64_t i = 0; i < len; ++i) {
        uint64_t j = start + i;
        if (!(in_len > j)) return 1;
        y[i] = x[j];
    }
    return 0;
}
void orc_tensor_concat_f32(const float* l, uint64_t nl, const float* r, uint64_t nr, float* y) {
    materializec(y, nl + nr, 1, [&](uint64_t i) {
        bool use_left = i < nl;
        return use_left ? l[i - 0] : r[i - nl];  // tensor.ref.f32.at-offset, tensor.hex:85-106
    });
}

// ---- stdlib/matrix.hex:210-327 + tests/cases/matrix/matmul.hex:2-63 --------------------
// C[i,j] = (((+0 + a_i0*b_0j) + a_i1*b_1j) + ...), mul and add rounded separately, k ascending;
// i = flat / m, j = flat % m (codegen/ops/row_major.rs:30-68); A index i*k+kk, B index kk*m+j.
// Returns 1 where the entry program's length asserts would trap (matmul.hex:18-27).
int orc_matmul_f32(const float* a, uint64_t a_len, const float* b, uint64_t b_len, uint64_t n,
                   uint64_t m, uint64_t k, uint64_t nk, uint64_t km, uint64_t nm, float* out,
                   int threads) {
    if (nk != a_len || km != b_len) return 1;
    materializec(out, nm, threads, [&](uint64_t flat) {
        uint64_t i = flat / m, j = flat % m;
        return reducec(bits_f32(0u), k,
                       [&](uint64_t kk) { return f32_mul(a[i * k + kk], b[kk * m + j]); }, f32_add);
    });
    return 0;
}

// Row slab [row0, row1) of the same product, for bounded CPU timing of large shapes.
void orc_matmul_f32_rows(const float* a, const float* b, uint64_t m, uint64_t k, uint64_t row0,
                         uint64_t row1, float* out_rows, int threads) {
    uint64_t cnt = (row1 - row0) * m;
    materializec(out_rows, cnt, threads, [&](uint64_t f) {
        uint64_t i = row0 + f / m, j = f % m;
        return reducec(bits_f32(0u), k,
                       [&](uint64_t kk) { return f32_mul(a[i * k + kk], b[kk * m + j]); }, f32_add);
    });
}

// ===== beyond-reference programs (parity unpinned; rules inherited as stated) ============

// bf16 GEMM, A row-major [M,K], B column-major (stored as [N,K], K contiguous), fp32 left fold
// over ascending k with separately rounded mul/add (the matrix.hex:236-256 rule), bf16 RNE output.
// Computes rows [row0,row1) only; c_rows has (row1-row0)*N entries.
void orc_gemm_bf16_rows(const uint16_t* a, const uint16_t* bt, uint64_t N, uint64_t K, uint64_t row0,
                        uint64_t row1, uint16_t* c_rows, float* c_rows_f32, int threads) {
    uint64_t cnt = (row1 - row0) * N;
    std::vector<float> af((row1 - row0) * K);
    for (uint64_t t = 0; t < af.size(); ++t) af[t] = bf16_to_f32(a[row0 * K + t]);
    auto cell = [&](uint64_t f) {
        uint64_t i = f / N, j = f % N;
        const uint16_t* bj = bt + j * K;
        const float* ai = af.data() + i * K;
        return reducec(bits_f32(0u), K,
                       [&](uint64_t kk) { return f32_mul(ai[kk], bf16_to_f32(bj[kk])); }, f32_add);
    };
    parallel_for(cnt, threads, [&](uint64_t f) {
        float v = cell(f);
        if (c_rows_f32) c_rows_f32[f] = v;
        if (c_rows) c_rows[f] = f32_to_bf16_rne(v);
    });
}

// int8 x int8 -> int32 GEMM, same layouts; integer sums are order-free and cannot overflow
// for K <= 131071 (|a*b| <= 16384).
void orc_gemm_i8_rows(const int8_t* a, const int8_t* bt, uint64_t N, uint64_t K, uint64_t row0,
                      uint64_t row1, int32_t* c_rows, int threads) {
    uint64_t cnt = (row1 - row0) * N;
    materializec(c_rows, cnt, threads, [&](uint64_t f) {
        uint64_t i = row0 + f / N, j = f % N;
        const int8_t* ai = a + i * K;
        const int8_t* bj = bt + j * K;
        int32_t acc = 0;
        for (uint64_t kk = 0; kk < K; ++kk) acc += (int32_t)ai[kk] * (int32_t)bj[kk];
        return acc;
    });
}

// Cached-attention decode for one new token, composed from reference programs:
//   s_j   = (fold_d q_d*k_jd, ascending d, unfused) * scale          (matrix.hex cell-dot rule)
//   w     = nn.softmax(s)  (global max, exp~, left-fold denominator, p/denom; nn.hex:93-122)
//   o_d   = fold_j w_j * v_jd, ascending j, unfused                   (cell-dot rule again)
// q [B,Hq,D] bf16, k/v cache [B,Hkv,L,D] bf16, o [B,Hq,D] bf16 (and optional fp32 copy).
// Query head h reads KV head h / (Hq/Hkv).  Only units [unit0, unit1) of the B*Hq (batch, head)
// pairs are computed; o / o_f32 are indexed by absolute unit.
void orc_attn_decode_bf16(const uint16_t* q, const uint16_t* kc, const uint16_t* vc, uint64_t B,
                          uint64_t Hq, uint64_t Hkv, uint64_t D, uint64_t L, float scale,
                          uint64_t unit0, uint64_t unit1, uint16_t* o, float* o_f32, int threads) {
    (void)B;
    uint64_t group = Hq / Hkv;
    parallel_for(unit1 - unit0, threads, [&](uint64_t uu) {
        uint64_t u = unit0 + uu;
        uint64_t b = (uint64_t)u / Hq, h = (uint64_t)u % Hq, kvh = h / group;
        const uint16_t* qv = q + (uint64_t)u * D;
        const uint16_t* kb = kc + ((b * Hkv + kvh) * L) * D;
        const uint16_t* vb = vc + ((b * Hkv + kvh) * L) * D;
        std::vector<float> s(L), w(L);
        for (uint64_t j = 0; j < L; ++j) {
            float dot = reducec(bits_f32(0u), D, [&](uint64_t d) {
                return f32_mul(bf16_to_f32(qv[d]), bf16_to_f32(kb[j * D + d]));
            }, f32_add);
            s[j] = f32_mul(dot, scale);
        }
        orc_nn_softmax(s.data(), w.data(), L, 1);
        for (uint64_t d = 0; d < D; ++d) {
            float acc = reducec(bits_f32(0u), L, [&](uint64_t j) {
                return f32_mul(w[j], bf16_to_f32(vb[j * D + d]));
            }, f32_add);
            if (o_f32) o_f32[(uint64_t)u * D + d] = acc;
            if (o) o[(uint64_t)u * D + d] = f32_to_bf16_rne(acc);
        }
    });
}

// ---- Llama-style block, composed from reference programs (no counterpart in the reference) ----
// Rules: nn.rmsnorm without gain (nn.hex:125-182) over the bf16 row; projections = orc_gemm_bf16_rows;
// rotary angle = pos * powf~(base, -2i/128), sin = sin-approx-full, cos(x) = sin-approx-full(x + pi/2)
// (math.hex:91-103, 202-231), pairs (i, i+64); attention = nn.softmax over the visible cache rows followed
// by the cell-dot fold with the values; SwiGLU = nn.silu(gate) * up; residual = f32.add of two bf16 values.

void orc_embed_bf16(const uint16_t* table, const int32_t* ids, uint16_t* out, uint64_t tokens, uint64_t hidden) {
    for (uint64_t t = 0; t < tokens; ++t) std::memcpy(out + t * hidden, table + (uint64_t)ids[t] * hidden, hidden * 2);
}

void orc_rmsnorm_rows_bf16(const uint16_t* x, uint16_t* y, uint64_t rows, uint64_t hidden, int threads) {
    parallel_for(rows, threads, [&](uint64_t r) {
        const uint16_t* xr = x + r * hidden;
        float s = reducec(bits_f32(0u), hidden, [&](uint64_t i) { float v = bf16_to_f32(xr[i]); return f32_mul(v, v); }, f32_add);
        float rms = sqrt_newton(f32_add(f32_div(s, u64_to_f32(hidden)), bits_f32(0x3727C5ACu)));
        for (uint64_t i = 0; i < hidden; ++i) y[r * hidden + i] = f32_to_bf16_rne(f32_div(bf16_to_f32(xr[i]), rms));
    });
}

void orc_rope_append_bf16(const uint16_t* qkv, uint16_t* q_out, uint16_t* k_cache, uint16_t* v_cache, uint64_t tokens,
                          uint64_t seq, uint64_t pos0, uint64_t hq, uint64_t hkv, uint64_t cap, float base) {
    const uint64_t heads = hq + 2 * hkv, D = 128;
    float inv[64];
    for (uint32_t i = 0; i < 64; ++i) inv[i] = powf_approx(base, f32_neg(f32_div(u32_to_f32(2 * i), 128.0f)));
    for (uint64_t t = 0; t < tokens; ++t) {
        const uint64_t b = t / seq, pos = pos0 + t % seq;
        for (uint64_t h = 0; h < heads; ++h) {
            const uint16_t* src = qkv + (t * heads + h) * D;
            if (h >= hq + hkv) {
                std::memcpy(v_cache + ((b * hkv + (h - hq - hkv)) * cap + pos) * D, src, D * 2);
                continue;
            }
            uint16_t* dst = h < hq ? q_out + (t * hq + h) * D : k_cache + ((b * hkv + (h - hq)) * cap + pos) * D;
            for (uint32_t i = 0; i < 64; ++i) {
                const float x1 = bf16_to_f32(src[i]), x2 = bf16_to_f32(src[i + 64]);
                const float angle = f32_mul(u32_to_f32((uint32_t)pos), inv[i]);
                const float sn = sin_full(angle), cs = sin_full(f32_add(angle, bits_f32(0x3FC90FDBu)));
                dst[i] = f32_to_bf16_rne(f32_sub(f32_mul(x1, cs), f32_mul(x2, sn)));
                dst[i + 64] = f32_to_bf16_rne(f32_add(f32_mul(x2, cs), f32_mul(x1, sn)));
            }
        }
    }
}

// Token (b, s) of q [batch*seq, hq, 128] attends to cache rows 0 .. pos0 + s of sequence b.
void orc_attn_cached_bf16(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache, uint16_t* out, float* out_f32,
                          uint64_t batch, uint64_t seq, uint64_t pos0, uint64_t hq, uint64_t hkv, uint64_t cap, float scale,
                          int threads) {
    const uint64_t D = 128, group = hq / hkv;
    parallel_for(batch * seq * hq, threads, [&](uint64_t u) {
        const uint64_t t = u / hq, h = u % hq, b = t / seq, L = pos0 + t % seq + 1, kvh = h / group;
        const uint16_t* qv = q + u * D;
        const uint16_t* kb = k_cache + (b * hkv + kvh) * cap * D;
        const uint16_t* vb = v_cache + (b * hkv + kvh) * cap * D;
        std::vector<float> sc(L), w(L);
        for (uint64_t j = 0; j < L; ++j) {
            float dot = reducec(bits_f32(0u), D, [&](uint64_t d) { return f32_mul(bf16_to_f32(qv[d]), bf16_to_f32(kb[j * D + d])); }, f32_add);
            sc[j] = f32_mul(dot, scale);
        }
        orc_nn_softmax(sc.data(), w.data(), L, 1);
        for (uint64_t d = 0; d < D; ++d) {
            float acc = reducec(bits_f32(0u), L, [&](uint64_t j) { return f32_mul(w[j], bf16_to_f32(vb[j * D + d])); }, f32_add);
            if (out_f32) out_f32[u * D + d] = acc;
            out[u * D + d] = f32_to_bf16_rne(acc);
        }
    });
}

void orc_swiglu_bf16(const uint16_t* gu, uint16_t* a, uint64_t tokens, uint64_t ffn) {
    for (uint64_t t = 0; t < tokens; ++t)
        for (uint64_t c = 0; c < ffn; ++c)
            a[t * ffn + c] = f32_to_bf16_rne(f32_mul(silu(bf16_to_f32(gu[t * 2 * ffn + c])), bf16_to_f32(gu[t * 2 * ffn + ffn + c])));
}

void orc_add_bf16(const uint16_t* x, const uint16_t* y, uint16_t* out, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) out[i] = f32_to_bf16_rne(f32_add(bf16_to_f32(x[i]), bf16_to_f32(y[i])));
}

// y [m, n] = x [m, k] w[n, k]^T, rounded to bf16, then + res (optional)
void orc_linear_bf16(const uint16_t* x, const uint16_t* w, const uint16_t* res, uint16_t* y, uint64_t m, uint64_t n, uint64_t k,
                     int threads) {
    orc_gemm_bf16_rows(x, w, n, k, 0, m, y, nullptr, threads);
    if (res) orc_add_bf16(y, res, y, m * n);
}

// The whole block for batch*seq tokens at positions pos0 .. pos0+seq-1 (prefill: pos0 = 0; decode: seq = 1).
void orc_llama_block(uint64_t hidden, uint64_t hq, uint64_t hkv, uint64_t ffn, uint64_t cap, float rope_base,
                     const uint16_t* embedding, const uint16_t* w_qkv, const uint16_t* w_o, const uint16_t* w_gate_up,
                     const uint16_t* w_down, const int32_t* ids, uint64_t batch, uint64_t seq, uint64_t pos0,
                     uint16_t* k_cache, uint16_t* v_cache, uint16_t* out, int threads) {
    const uint64_t T = batch * seq, D = 128, qkv_cols = (hq + 2 * hkv) * D;
    std::vector<uint16_t> x(T * hidden), nrm(T * hidden), qkv(T * qkv_cols), q(T * hq * D), att(T * hq * D), x2(T * hidden),
        gu(T * 2 * ffn), act(T * ffn);
    orc_embed_bf16(embedding, ids, x.data(), T, hidden);
    orc_rmsnorm_rows_bf16(x.data(), nrm.data(), T, hidden, threads);
    orc_linear_bf16(nrm.data(), w_qkv, nullptr, qkv.data(), T, qkv_cols, hidden, threads);
    orc_rope_append_bf16(qkv.data(), q.data(), k_cache, v_cache, T, seq, pos0, hq, hkv, cap, rope_base);
    orc_attn_cached_bf16(q.data(), k_cache, v_cache, att.data(), nullptr, batch, seq, pos0, hq, hkv, cap,
                         0.08838834764831845f /* 1/sqrt(128) rounded to f32, as the kernels pass it */, threads);
    orc_linear_bf16(att.data(), w_o, x.data(), x2.data(), T, hidden, hq * D, threads);
    orc_rmsnorm_rows_bf16(x2.data(), nrm.data(), T, hidden, threads);
    orc_linear_bf16(nrm.data(), w_gate_up, nullptr, gu.data(), T, 2 * ffn, hidden, threads);
    orc_swiglu_bf16(gu.data(), act.data(), T, ffn);
    orc_linear_bf16(act.data(), w_down, x2.data(), out, T, hidden, ffn, threads);
}

// ---- codegen/gpu.rs:322-447 : the primitive table, one generated C expression per operation ----------
// `op` is the hexpr name; operands and result travel as raw bits (an f32 in the low 32 bits, a bool as 0 / 1).  The body
// of each case is the expression the renderer prints for that primitive (gpu.rs file:line beside each group), compiled by
// the host compiler exactly as the reference's generated code would be (uint32_t / uint64_t / float / uint8_t operands,
// the usual C conversions, no contraction).  Returns 0 and sets *known = 0 for a name outside the table.
uint64_t orc_prim(const char* op, uint64_t a, uint64_t b, uint64_t c, int* known) {
    const std::string o(op);
    const uint32_t a32 = (uint32_t)a, b32 = (uint32_t)b, c32 = (uint32_t)c;
    const float af = bits_f32(a32), bf = bits_f32(b32), cf = bits_f32(c32);
    const uint8_t ab = a ? 1 : 0, bb = b ? 1 : 0;
    auto F = [](float x) { return (uint64_t)f32_bits(x); };
    if (known) *known = 1;
    // gpu.rs:327-369 (bool)
    if (o == "bool.t") return 1;
    if (o == "bool.f") return 0;
    if (o == "bool.not") return (uint8_t)(!ab);
    if (o == "bool.id") return ab;
    if (o == "bool.and") return (uint8_t)(ab && bb);
    if (o == "bool.or") return (uint8_t)(ab || bb);
    // gpu.rs:379-389 (u64), :402-403, :697-733 (u64.eq / u64.gt: the flag output)
    if (o == "u64.zero") return 0;
    if (o == "u64.one") return 1;
    if (o == "u64.add") return a + b;
    if (o == "u64.sub") return a - b;
    if (o == "u64.mul") return a * b;
    if (o == "u64.ne") return a != b;
    if (o == "u64.lt") return a < b;
    if (o == "u64.lte") return a <= b;
    if (o == "u64.gte") return a >= b;
    if (o == "u64.eq") return a == b;
    if (o == "u64.gt") return a > b;
    if (o == "u64.name" || o == "ix.to-u64") return a;
    // gpu.rs:390-412 (u32)
    if (o == "u32.one") return 1;
    if (o == "u32.add") return (uint32_t)(a32 + b32);
    if (o == "u32.sub") return (uint32_t)(a32 - b32);
    if (o == "u32.mul") return (uint32_t)(a32 * b32);
    if (o == "u32.and") return (uint32_t)(a32 & b32);
    if (o == "u32.or") return (uint32_t)(a32 | b32);
    if (o == "u32.xor") return (uint32_t)(a32 ^ b32);
    if (o == "u32.shl") return (uint32_t)(a32 << b32);      // defined for shifts below 32 only
    if (o == "u32.shr") return (uint32_t)(a32 >> b32);
    if (o == "u32.not") return (uint32_t)(~a32);
    if (o == "u32.eq") return a32 == b32;
    if (o == "u32.ne") return a32 != b32;
    if (o == "u32.lt") return a32 < b32;
    if (o == "u32.gt") return a32 > b32;
    if (o == "u32.lte") return a32 <= b32;
    if (o == "u32.gte") return a32 >= b32;
    if (o == "u32.to-f32") return F((float)(a32));                       // gpu.rs:535-548
    if (o == "u64.to-f32") return F((float)(a));                         // gpu.rs:550-563
    if (o == "u32.bitcast-f32") return F(bits_f32(a32));                 // gpu.rs:565-578, prelude.rs:64-71
    // gpu.rs:418-436 (f32)
    if (o == "f32.one") return F(1.0);
    if (o == "f32.add") return F(af + bf);
    if (o == "f32.sub") return F(af - bf);
    if (o == "f32.neg") return F(-af);
    if (o == "f32.mul") return F(af * bf);
    if (o == "f32.div") return F(af / bf);
    if (o == "f32.fma") return F(fmaf(af, bf, cf));                      // gpu.rs:589-604
    if (o == "f32.eq") return af == bf;
    if (o == "f32.ne") return af != bf;
    if (o == "f32.lt") return af < bf;
    if (o == "f32.gt") return af > bf;
    if (o == "f32.lte") return af <= bf;
    if (o == "f32.gte") return af >= bf;
    if (o == "f32.select") return F(ab ? bf : cf);                       // gpu.rs:624-640
    if (o == "u32.select") return ab ? b32 : c32;
    if (o == "u64.select") return ab ? b : c;
    if (o == "bool.select") return ab ? (uint8_t)(b != 0) : (uint8_t)(c != 0);
    if (o == "f32.round-to-u32") return (uint32_t)nearbyintf(af);        // gpu.rs:642-655, defined for 0 <= x < 2^32
    if (o == "f32.bitcast-u32") return f32_bits(af);                     // gpu.rs:657-670, prelude.rs:73-80
    // ops/row_major.rs:9-68 with (cols, row, col) / (cols, flat)
    if (o == "row-major-index") return b * a + c;
    if (o == "row-major-row") return b / a;
    if (o == "row-major-col") return b % a;
    if (known) *known = 0;
    return 0;
}

uint16_t orc_f32_to_bf16(float f) { return f32_to_bf16_rne(f); }
float orc_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }

}  // extern "C"
