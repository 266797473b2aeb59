/*
 * oracle.c - CPU restatement of the reference's numeric contracts for the quantized
 * transformer-decode path.  TEST INFRASTRUCTURE ONLY: it is linked by tests/, by
 * __graft_entry__.smoke() and by bench.py's CPU-baseline legs as the checker and the
 * timed CPU baseline; the product (libb200backend.so) never links or calls it.
 *
 * Parity status, piece by piece:
 *   - pinned by the reference's own vectors (see tests/test_oracle_golden.py): the FMA GEMM
 *     order, the int8 x int8 -> int32 wrapping accumulate, bf16 round-to-nearest-even, the
 *     composite tolerance judge, the paged KV append / attention loop (MHA, f32), the greedy
 *     first-max argmax, RMSNorm with an f64 sum of squares, the two-branch sigmoid.
 *   - PARITY UNPINNED (the reference has no code or vectors for them; the rule comes from the
 *     benchmark configuration text): int8 / FP8-E4M3 quantisation rules, the dequant epilogue,
 *     SiLU-gate, GQA head mapping with bf16 K/V, RoPE, the Llama-style layer wiring.
 *
 * The reference is Rust and cannot be compiled in this environment; each function cites
 * the reference file:line it follows.  Build: see oracle/Makefile (-ffp-contract=off so that
 * only the fmaf() calls written below fuse).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* Loops over fewer elements than this run on the calling thread: a parallel region costs more than they do. */
#define SMALL_WORK ((int64_t)1 << 18)

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Sets the number of threads of the parallel loops (a launcher may have exported OMP_NUM_THREADS=1). */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ------------------------------------------------------------------ bf16
 * IEEE round-to-nearest-even f32 -> bf16 and exact widening, the behaviour of the `half`
 * crate (=2.7.1) that the reference relies on (crates/backend-cpu/src/typed_bf16.rs:72,86;
 * tie example 1 + 2^-8 -> 1.0 at typed_bf16.rs:359-380). */
uint16_t orc_f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40u); /* NaN stays NaN */
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
float orc_bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
void orc_f32_to_bf16_array(const float* x, int64_t n, uint16_t* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = orc_f32_to_bf16(x[i]);
}
void orc_bf16_to_f32_array(const uint16_t* x, int64_t n, float* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = orc_bf16_to_f32(x[i]);
}

/* ------------------------------------------------------------------ composite judge
 * pass iff rel < 1e-3 || abs < 1e-5, rel = |a-b| / max(|a|, |b|, 1e-12); non-finite fails
 * (crates/tensor-core/src/tolerance.rs:29-37). */
int orc_composite_close(float actual, float reference) {
    double a = (double)actual, r = (double)reference;
    double diff = fabs(a - r);
    double scale = fmax(fmax(fabs(a), fabs(r)), 1e-12);
    double rel = diff / scale;
    return (rel < 1e-3) || (diff < 1e-5);
}
/* Returns the number of failing elements; writes max abs / max rel error of the finite pairs. */
int64_t orc_compare(const float* actual, const float* reference, int64_t n, double* max_abs, double* max_rel) {
    int64_t fails = 0;
    double ma = 0.0, mr = 0.0;
    for (int64_t i = 0; i < n; ++i) {
        if (!orc_composite_close(actual[i], reference[i])) ++fails;
        double diff = fabs((double)actual[i] - (double)reference[i]);
        double scale = fmax(fmax(fabs((double)actual[i]), fabs((double)reference[i])), 1e-12);
        if (isfinite(diff)) {
            if (diff > ma) ma = diff;
            if (diff / scale > mr) mr = diff / scale;
        }
    }
    if (max_abs) *max_abs = ma;
    if (max_rel) *max_rel = mr;
    return fails;
}

/* ------------------------------------------------------------------ GEMM contracts */

/* c[i][j] = fma(a[i][p], b[p][j], c[i][j]) for p ascending; c must be zeroed by the caller.
 * a: [m,k], b: [k,n] (crates/backend-cpu/src/parity.rs:340-361). */
void orc_matmul_reference_fma(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m; ++i) {
        const float* a_row = a + i * k;
        float* c_row = c + i * n;
        for (int64_t p = 0; p < k; ++p) {
            const float a_ip = a_row[p];
            const float* b_row = b + p * n;
            for (int64_t j = 0; j < n; ++j) c_row[j] = fmaf(a_ip, b_row[j], c_row[j]);
        }
    }
}

/* acc[i][j] = sum_p a[i][p] * w[j][p] in wrapping int32 (the host model of the reference's
 * int8 MMA probe: crates/backend-cuda/tests/int8_mma_probe_real_device.rs:196-238).
 * a: [m,k] int8, w: [n,k] int8 (K-major weight rows). */
void orc_gemm_i8_s32(const int8_t* a, const int8_t* w, int64_t m, int64_t n, int64_t k, int32_t* acc) {
#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t i = 0; i < m; ++i) {
        for (int64_t j = 0; j < n; ++j) {
            const int8_t* ar = a + i * k;
            const int8_t* wr = w + j * k;
            uint32_t s = 0; /* unsigned arithmetic = two's complement wrap without UB */
            for (int64_t p = 0; p < k; ++p) s += (uint32_t)((int32_t)ar[p] * (int32_t)wr[p]);
            acc[i * n + j] = (int32_t)s;
        }
    }
}

/* ------------------------------------------------------------------ FP8 E4M3 (OCP "FN": no inf, max 448)
 * PARITY UNPINNED.  Software encode with round-to-nearest-even and saturation to +-448,
 * NaN -> 0x7F | sign; decode is exact. */
float orc_e4m3_to_f32(uint8_t v) {
    const uint32_t sign = v >> 7, e = (v >> 3) & 0xF, m = v & 7;
    float r;
    if (e == 0xF && m == 7) r = NAN;
    else if (e == 0) r = ldexpf((float)m, -9);               /* subnormal: m * 2^-3 * 2^-6 */
    else r = ldexpf(1.0f + (float)m / 8.0f, (int)e - 7);
    return sign ? -r : r;
}
uint8_t orc_f32_to_e4m3(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    const uint8_t sign = (uint8_t)((u >> 31) << 7);
    if (f != f) return (uint8_t)(sign | 0x7F);
    float a = fabsf(f);
    if (a >= 448.0f) {
        /* values above the largest finite code saturate, including the round-up region and inf */
        return (uint8_t)(sign | 0x7E);
    }
    if (a < ldexpf(1.0f, -6)) {
        /* subnormal range: code = rne(a / 2^-9), may round up to the first normal (8) */
        float q = rintf(ldexpf(a, 9));
        return (uint8_t)(sign | (uint8_t)q);
    }
    int e;
    float mant = frexpf(a, &e);          /* a = mant * 2^e, mant in [0.5, 1) */
    /* a = (2*mant) * 2^(e-1); 3 fraction bits */
    float scaled = ldexpf(mant, 4);      /* in [8, 16) */
    float r = rintf(scaled);             /* RNE (default rounding mode) */
    int exp = e - 1;
    if (r >= 16.0f) { r = 8.0f; exp += 1; }
    int code = ((exp + 7) << 3) | ((int)r - 8);
    if (code > 0x7E) code = 0x7E;
    return (uint8_t)(sign | (uint8_t)code);
}
void orc_e4m3_to_f32_array(const uint8_t* q, int64_t n, float* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = orc_e4m3_to_f32(q[i]);
}

/* acc[i][j] = fma-chain over p ascending of decode(a[i][p]) * decode(b[j][p]), f32
 * (order of crates/backend-cpu/src/parity.rs:340-361 applied to the decoded operands). */
void orc_gemm_fp8_f32(const uint8_t* a, const uint8_t* b, int64_t m, int64_t n, int64_t k, float* acc) {
    float lut[256];
    for (int i = 0; i < 256; ++i) lut[i] = orc_e4m3_to_f32((uint8_t)i);
#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t i = 0; i < m; ++i) {
        for (int64_t j = 0; j < n; ++j) {
            const uint8_t* ar = a + i * k;
            const uint8_t* br = b + j * k;
            float s = 0.0f;
            for (int64_t p = 0; p < k; ++p) s = fmaf(lut[ar[p]], lut[br[p]], s);
            acc[i * n + j] = s;
        }
    }
}

/* ------------------------------------------------------------------ quantisers (PARITY UNPINNED)
 * scale = amax(row) / 127, q = rne(x / scale) clamped to [-127, 127]; amax == 0 -> scale 0, q 0. */
void orc_quantize_i8_per_row(const float* x, int64_t rows, int64_t cols, int8_t* q, float* scale) {
#pragma omp parallel for schedule(static) if (rows * cols > SMALL_WORK)
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * cols;
        float amax = 0.0f;
        for (int64_t c = 0; c < cols; ++c) amax = fmaxf(amax, fabsf(xr[c]));
        const float s = amax / 127.0f;
        scale[r] = s;
        for (int64_t c = 0; c < cols; ++c) {
            float v = 0.0f;
            if (s != 0.0f) {
                v = rintf(xr[c] / s);
                v = fminf(fmaxf(v, -127.0f), 127.0f);
            }
            q[r * cols + c] = (int8_t)v;
        }
    }
}
void orc_dequantize_i8_per_row(const int8_t* q, const float* scale, int64_t rows, int64_t cols, float* x) {
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < cols; ++c) x[r * cols + c] = (float)q[r * cols + c] * scale[r];
}
/* scale = amax / 448, q = e4m3(x / scale). */
void orc_quantize_fp8_per_tensor(const float* x, int64_t n, uint8_t* q, float* scale) {
    float amax = 0.0f;
    for (int64_t i = 0; i < n; ++i) amax = fmaxf(amax, fabsf(x[i]));
    const float s = amax / 448.0f;
    scale[0] = s;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) q[i] = orc_f32_to_e4m3(s == 0.0f ? 0.0f : x[i] / s);
}

/* Per-row form (the FP8 decoder's activations and weights): scale[r] = amax(row r) / 448, q = e4m3(x / scale[r]). */
void orc_quantize_fp8_per_row(const float* x, int64_t rows, int64_t cols, uint8_t* q, float* scale) {
#pragma omp parallel for schedule(static) if (rows * cols > SMALL_WORK)
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * cols;
        float amax = 0.0f;
        for (int64_t c = 0; c < cols; ++c) amax = fmaxf(amax, fabsf(xr[c]));
        const float s = amax / 448.0f;
        scale[r] = s;
        for (int64_t c = 0; c < cols; ++c) q[r * cols + c] = orc_f32_to_e4m3(s == 0.0f ? 0.0f : xr[c] / s);
    }
}

/* ------------------------------------------------------------------ activations
 * Two-branch sigmoid and SiLU = x * sigmoid(x) (crates/tensor-core/src/scalar_op.rs:355,666-673). */
float orc_sigmoid_stable(float x) {
    if (x >= 0.0f) return 1.0f / (1.0f + expf(-x));
    float e = expf(x);
    return e / (1.0f + e);
}
float orc_silu(float x) { return x * orc_sigmoid_stable(x); }

/* ------------------------------------------------------------------ fused epilogue
 * y = act(fma(acc, sa * sb, bias)) (+ residual): bias, then activation, once after the full-K
 * sum (crates/tensor-core/src/backend_ops.rs:4111-4127; crates/backend-cuda/src/kernels.rs:456-475).
 * acc_is_int: acc points at int32 (converted with round-to-nearest) else f32.
 * act: 0 none, 1 relu, 2 silu, 3 silu-gate (columns [0,n/2) gate, [n/2,n) up -> n/2 outputs).
 * out_bf16: store bf16 (uint16) instead of f32. */
void orc_epilogue(const void* acc, int acc_is_int, int64_t m, int64_t n, const float* a_scale, int a_per_row,
                  const float* b_scale, int b_per_col, const float* bias, int act, const float* residual,
                  void* out, int out_bf16) {
    const int gate = act == 3;
    const int64_t n_out = gate ? n / 2 : n;
#pragma omp parallel for schedule(static) if (m * n > SMALL_WORK)
    for (int64_t i = 0; i < m; ++i) {
        const float sa = a_scale[a_per_row ? i : 0];
        for (int64_t j = 0; j < n_out; ++j) {
            float y;
            if (!gate) {
                const float t = acc_is_int ? (float)((const int32_t*)acc)[i * n + j] : ((const float*)acc)[i * n + j];
                y = fmaf(t, sa * b_scale[b_per_col ? j : 0], bias ? bias[j] : 0.0f);
                if (act == 1) y = fmaxf(y, 0.0f);
                else if (act == 2) y = orc_silu(y);
            } else {
                const int64_t ju = n_out + j;
                const float tg = acc_is_int ? (float)((const int32_t*)acc)[i * n + j] : ((const float*)acc)[i * n + j];
                const float tu = acc_is_int ? (float)((const int32_t*)acc)[i * n + ju] : ((const float*)acc)[i * n + ju];
                const float g = fmaf(tg, sa * b_scale[b_per_col ? j : 0], bias ? bias[j] : 0.0f);
                const float u = fmaf(tu, sa * b_scale[b_per_col ? ju : 0], bias ? bias[ju] : 0.0f);
                y = orc_silu(g) * u;
            }
            if (residual) y = y + residual[i * n_out + j];
            if (out_bf16) ((uint16_t*)out)[i * n_out + j] = orc_f32_to_bf16(y);
            else ((float*)out)[i * n_out + j] = y;
        }
    }
}

/* ------------------------------------------------------------------ RMSNorm
 * sum of squares in f64 (fma), one downcast for rstd, out = x * rstd * w
 * (crates/backend-cpu/src/rmsnorm.rs:203-228). */
void orc_rmsnorm(const float* x, const float* w, float eps, int64_t rows, int64_t hidden, float* out) {
#pragma omp parallel for schedule(static) if (rows * hidden > SMALL_WORK)
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * hidden;
        double acc = 0.0;
        for (int64_t i = 0; i < hidden; ++i) {
            const double v = (double)xr[i];
            acc = fma(v, v, acc);
        }
        const float inv_n = 1.0f / (float)hidden;
        const float rstd = (float)(1.0 / sqrt(fma(acc, (double)inv_n, (double)eps)));
        for (int64_t i = 0; i < hidden; ++i) out[r * hidden + i] = w ? xr[i] * rstd * w[i] : xr[i] * rstd;
    }
}

/* ------------------------------------------------------------------ RoPE (PARITY UNPINNED)
 * Rotate-half form on one head vector: for i < d/2,
 *   out[i]       = fma(x[i],       cos[i], -(x[i + d/2] * sin[i]))
 *   out[i + d/2] = fma(x[i + d/2], cos[i],   x[i]       * sin[i])
 * cos/sin come from a table [pos][d/2] computed in f64 (angle = pos * theta^(-2i/d)). */
void orc_rope_table(int64_t max_pos, int64_t head_dim, double theta, float* cos_t, float* sin_t) {
    const int64_t half = head_dim / 2;
    for (int64_t p = 0; p < max_pos; ++p)
        for (int64_t i = 0; i < half; ++i) {
            const double inv = pow(theta, -2.0 * (double)i / (double)head_dim);
            const double ang = (double)p * inv;
            cos_t[p * half + i] = (float)cos(ang);
            sin_t[p * half + i] = (float)sin(ang);
        }
}
void orc_rope_apply(float* x, int64_t heads, int64_t head_dim, const float* cos_row, const float* sin_row) {
    const int64_t half = head_dim / 2;
    for (int64_t h = 0; h < heads; ++h) {
        float* v = x + h * head_dim;
        for (int64_t i = 0; i < half; ++i) {
            const float x1 = v[i], x2 = v[i + half];
            v[i] = fmaf(x1, cos_row[i], -(x2 * sin_row[i]));
            v[i + half] = fmaf(x2, cos_row[i], x1 * sin_row[i]);
        }
    }
}

/* ------------------------------------------------------------------ greedy argmax
 * first index of the maximum, strict '>' (crates/autodiff/src/generate/mod.rs:333-343). */
int64_t orc_greedy_argmax(const float* row, int64_t n) {
    int64_t best = 0;
    float bv = row[0];
    for (int64_t i = 1; i < n; ++i)
        if (row[i] > bv) { bv = row[i]; best = i; }
    return best;
}

/* ------------------------------------------------------------------ paged KV
 * Pools are [num_blocks, block_size, E_kv] row-major; a token row is block_id * block_size +
 * pos % block_size.  kv_bf16 != 0: pools hold bf16 (uint16) and incoming f32 rows are rounded
 * (RNE) on append; else f32 as in the reference. */

/* copy row r of k_new / v_new [rows, e] to pool row slot_mapping[r]
 * (crates/backend-cpu/src/paged_kv.rs:33-66).  Returns 0, or -1 on an out-of-range slot. */
int orc_paged_kv_append(const float* k_new, const float* v_new, void* k_pool, void* v_pool, const uint32_t* slots,
                        int64_t rows, int64_t e, int64_t pool_rows, int kv_bf16) {
    for (int64_t r = 0; r < rows; ++r) {
        const int64_t dst = (int64_t)slots[r];
        if (dst >= pool_rows) return -1;
        for (int64_t c = 0; c < e; ++c) {
            if (kv_bf16) {
                ((uint16_t*)k_pool)[dst * e + c] = orc_f32_to_bf16(k_new[r * e + c]);
                ((uint16_t*)v_pool)[dst * e + c] = orc_f32_to_bf16(v_new[r * e + c]);
            } else {
                ((float*)k_pool)[dst * e + c] = k_new[r * e + c];
                ((float*)v_pool)[dst * e + c] = v_new[r * e + c];
            }
        }
    }
    return 0;
}

static inline float kv_at(const void* pool, int64_t idx, int kv_bf16) {
    return kv_bf16 ? orc_bf16_to_f32(((const uint16_t*)pool)[idx]) : ((const float*)pool)[idx];
}

/* out[b, i, h, :] = softmax_j((q * scale) . k_j) . v_j over j <= seq_len - l_new + i, keys found
 * through the block table; one sequential loop per query row: scores with fma over Dh, running
 * max, exp(s - max) summed in order, normalised weights fma-accumulated in order
 * (crates/backend-cpu/src/paged_kv.rs:96-178).  Generalised (PARITY UNPINNED) to GQA:
 * kv head = q head / (num_q_heads / num_kv_heads); q / out are [B, l_new, Hq * Dh].
 * Returns 0, -1 on an invalid block id, -2 on seq_len < l_new. */
int orc_paged_attention(const float* q, const void* k_pool, const void* v_pool, const uint32_t* block_tables,
                        const uint32_t* seq_lens, int64_t batch, int64_t l_new, int64_t num_q_heads,
                        int64_t num_kv_heads, int64_t head_dim, int64_t block_size, int64_t num_blocks,
                        int64_t max_blocks_per_seq, float scale, int kv_bf16, float* out) {
    const int64_t eq = num_q_heads * head_dim;
    const int64_t ekv = num_kv_heads * head_dim;
    const int64_t group = num_q_heads / num_kv_heads;
    int status = 0;
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (int64_t b = 0; b < batch; ++b) {
        for (int64_t h = 0; h < num_q_heads; ++h) {
            const int64_t s_total = (int64_t)seq_lens[b];
            if (s_total < l_new) { status = -2; continue; }
            const int64_t s_prev = s_total - l_new;
            const int64_t kvh = h / group;
            float* weights = (float*)malloc((size_t)(s_total > 0 ? s_total : 1) * sizeof(float));
            for (int64_t i = 0; i < l_new; ++i) {
                const float* q_row = q + (b * l_new + i) * eq + h * head_dim;
                float* o_row = out + (b * l_new + i) * eq + h * head_dim;
                const int64_t limit = s_prev + i + 1;
                float mx = -INFINITY;
                int bad = 0;
                for (int64_t j = 0; j < limit; ++j) {
                    const uint32_t blk = block_tables[b * max_blocks_per_seq + j / block_size];
                    if ((int64_t)blk >= num_blocks) { bad = 1; break; }
                    const int64_t off = ((int64_t)blk * block_size + j % block_size) * ekv + kvh * head_dim;
                    float acc = 0.0f;
                    for (int64_t d = 0; d < head_dim; ++d) acc = fmaf(q_row[d] * scale, kv_at(k_pool, off + d, kv_bf16), acc);
                    weights[j] = acc;
                    if (acc > mx) mx = acc;
                }
                if (bad) { status = -1; continue; }
                float sum = 0.0f;
                for (int64_t j = 0; j < limit; ++j) {
                    weights[j] = expf(weights[j] - mx);
                    sum += weights[j];
                }
                for (int64_t d = 0; d < head_dim; ++d) o_row[d] = 0.0f;
                for (int64_t j = 0; j < limit; ++j) {
                    const float p = weights[j] / sum;
                    const uint32_t blk = block_tables[b * max_blocks_per_seq + j / block_size];
                    const int64_t off = ((int64_t)blk * block_size + j % block_size) * ekv + kvh * head_dim;
                    for (int64_t d = 0; d < head_dim; ++d) o_row[d] = fmaf(p, kv_at(v_pool, off + d, kv_bf16), o_row[d]);
                }
            }
            free(weights);
        }
    }
    return status;
}

/* ====================================================================================================
 * Kernel-order restatements (PARITY UNPINNED, like every piece the reference has no code for).
 *
 * The functions above follow the reference's sequential loops.  The CUDA kernels of the decoder sum in
 * another, fixed, order (lanes, warps, blocks) and use their own exponential; upstream of a per-token int8
 * quantiser a last-bit difference can flip a code, so a free-running greedy comparison needs the CPU side
 * to round exactly as the kernels do.  The functions below restate that order with the same correctly
 * rounded operations (this file is compiled with -ffp-contract=off: only the fmaf()/fma() written here
 * fuse).  The tests check each of them against its sequential counterpart above within the composite
 * tolerance on the same inputs.
 * ==================================================================================================== */

/* e^x from multiply, fused multiply-add, add, round-to-integer and exponent arithmetic only: x = n ln2 + r
 * (ln2 in two parts), degree-5 polynomial on top of 1 + r, result scaled by 2^n in two multiplications. */
float orc_exp_det(float x) {
    if (!(x > -104.0f)) return x != x ? x : 0.0f;
    if (x > 88.8f) return INFINITY;
    const float n = rintf(x * 1.44269504088896341f);
    float r = fmaf(n, -0.693359375f, x);
    r = fmaf(n, 2.12194440e-4f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    float y = fmaf(p, r * r, r) + 1.0f;
    const int32_t ni = (int32_t)n;
    const int32_t a = (ni - (ni & 1)) / 2, b = ni - a;
    union { uint32_t u; float f; } s1, s2;
    s1.u = (uint32_t)(a + 127) << 23;
    s2.u = (uint32_t)(b + 127) << 23;
    y = y * s1.f;
    return y * s2.f;
}
void orc_exp_det_array(const float* x, int64_t n, float* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = orc_exp_det(x[i]);
}
float orc_sigmoid_det(float x) {
    if (x >= 0.0f) return 1.0f / (1.0f + orc_exp_det(-x));
    const float e = orc_exp_det(x);
    return e / (1.0f + e);
}
float orc_silu_det(float x) { return x * orc_sigmoid_det(x); }

/* orc_epilogue with the kernels' exponential inside SiLU (act 2 and 3); no bf16 output. */
void orc_epilogue_det(const int32_t* acc, int64_t m, int64_t n, const float* a_scale, const float* b_scale,
                      int act, float* out) {
    const int gate = act == 3;
    const int64_t n_out = gate ? n / 2 : n;
#pragma omp parallel for schedule(static) if (m * n > SMALL_WORK)
    for (int64_t i = 0; i < m; ++i) {
        const float sa = a_scale[i];
        for (int64_t j = 0; j < n_out; ++j) {
            float y;
            if (!gate) {
                y = fmaf((float)acc[i * n + j], sa * b_scale[j], 0.0f);
                if (act == 1) y = fmaxf(y, 0.0f);
                else if (act == 2) y = orc_silu_det(y);
            } else {
                const float g = fmaf((float)acc[i * n + j], sa * b_scale[j], 0.0f);
                const float u = fmaf((float)acc[i * n + n_out + j], sa * b_scale[n_out + j], 0.0f);
                y = orc_silu_det(g) * u;
            }
            out[i * n_out + j] = y;
        }
    }
}

/* Sum over a warp the way `v += shfl_xor(v, o)` for o = 16, 8, 4, 2, 1 does: a butterfly whose result is the
 * same in every lane because addition is commutative. */
static double butterfly_sum_d(double* v) {
    for (int o = 16; o > 0; o >>= 1) {
        double t[32];
        for (int l = 0; l < 32; ++l) t[l] = v[l] + v[l ^ o];
        memcpy(v, t, sizeof t);
    }
    return v[0];
}
static float butterfly_sum_f(float* v) {
    for (int o = 16; o > 0; o >>= 1) {
        float t[32];
        for (int l = 0; l < 32; ++l) t[l] = v[l] + v[l ^ o];
        memcpy(v, t, sizeof t);
    }
    return v[0];
}

/* f64 sum of squares of x[0, n) in the order of a CTA of `threads` threads (a multiple of 32):
 *   mode 0 ("wide"): thread t owns the groups of four columns g = t + k * threads, k = 0 .. vpt - 1, and chains
 *                    fma(v, v, acc) over its columns in ascending order;
 *   mode 1 ("strided"): thread t owns the columns t, t + threads, ... in ascending order;
 * then a butterfly over each warp and the warps added in ascending order. */
static double sumsq_block(const float* x, int64_t n, int threads, int vpt, int mode) {
    double total = 0.0;
    for (int w = 0; w < threads / 32; ++w) {
        double lane[32];
        for (int l = 0; l < 32; ++l) {
            const int t = w * 32 + l;
            double acc = 0.0;
            if (mode == 0) {
                for (int k = 0; k < vpt; ++k) {
                    const int64_t g = t + (int64_t)k * threads;
                    if (g < n / 4)
                        for (int e = 0; e < 4; ++e) {
                            const double v = (double)x[4 * g + e];
                            acc = fma(v, v, acc);
                        }
                }
            } else {
                for (int64_t i = t; i < n; i += threads) {
                    const double v = (double)x[i];
                    acc = fma(v, v, acc);
                }
            }
            lane[l] = acc;
        }
        total += butterfly_sum_d(lane);
    }
    return total;
}

/* RMSNorm with the sum of squares taken in kernel order; the rest is orc_rmsnorm's arithmetic.
 *   mode 0: one wide CTA per row (`threads` threads, `vpt` groups of four columns per thread);
 *   mode 1: the row cut into `cl` chunks of hidden / cl columns, one CTA of 256 threads each (strided), the
 *           chunk sums added in chunk order starting from 0.0. */
void orc_rmsnorm_kernel_order(const float* x, const float* w, float eps, int64_t rows, int64_t hidden, int mode,
                              int threads, int vpt_or_cl, float* out) {
#pragma omp parallel for schedule(static) if (rows * hidden > SMALL_WORK)
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * hidden;
        double acc;
        if (mode == 0) {
            acc = sumsq_block(xr, hidden, threads, vpt_or_cl, 0);
        } else {
            const int64_t nc = hidden / vpt_or_cl;
            acc = 0.0;
            for (int c = 0; c < vpt_or_cl; ++c) acc += sumsq_block(xr + c * nc, nc, 256, 0, 1);
        }
        const float inv_n = 1.0f / (float)hidden;
        const float rstd = (float)(1.0 / sqrt(fma(acc, (double)inv_n, (double)eps)));
        for (int64_t i = 0; i < hidden; ++i) out[r * hidden + i] = xr[i] * rstd * w[i];
    }
}

/* orc_paged_attention in the order of the general-shape CUDA kernel (head_dim <= 256): four warps walk the
 * keys j = warp, warp + 4, ...; lane l holds the dims l, l + 32, ...; per key
 *   s  = butterfly over lanes of the fma chain over a lane's dims of (q[d] * scale) * k[d]
 *   m' = max(m, s); c = exp(m - m'); p = exp(s - m'); l = fma(l, c, p); o[d] = fma(p, v[d], o[d] * c)
 * then the warps are merged in order: g = exp(m_w - max m); L = fma(l_w, g, L); O[d] = fma(o_w[d], g, O[d]);
 * out[d] = O[d] / L.  exp is orc_exp_det.  Same arguments and return codes as orc_paged_attention. */
int orc_paged_attention_kernel_order(const float* q, const void* k_pool, const void* v_pool,
                                     const uint32_t* block_tables, const uint32_t* seq_lens, int64_t batch,
                                     int64_t l_new, int64_t num_q_heads, int64_t num_kv_heads, int64_t head_dim,
                                     int64_t block_size, int64_t num_blocks, int64_t max_blocks_per_seq, float scale,
                                     int kv_bf16, float* out) {
    if (head_dim > 256) return -3;
    const int64_t eq = num_q_heads * head_dim;
    const int64_t ekv = num_kv_heads * head_dim;
    const int64_t group = num_q_heads / num_kv_heads;
    int status = 0;
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (int64_t row = 0; row < batch * l_new; ++row) {
        for (int64_t h = 0; h < num_q_heads; ++h) {
            const int64_t b = row / l_new, i = row % l_new;
            const int64_t s_total = (int64_t)seq_lens[b];
            if (s_total < l_new) { status = -2; continue; }
            const int64_t limit = s_total - l_new + i + 1;
            const int64_t kvh = h / group;
            const float* q_row = q + row * eq + h * head_dim;
            float* o_row = out + row * eq + h * head_dim;
            float qs[256];
            for (int64_t d = 0; d < head_dim; ++d) qs[d] = q_row[d] * scale;
            float wm[4], wl[4], wo[4][256];
            int bad = 0;
            for (int w = 0; w < 4 && !bad; ++w) {
                float m = -INFINITY, l = 0.0f;
                float* acc = wo[w];
                for (int64_t d = 0; d < head_dim; ++d) acc[d] = 0.0f;
                for (int64_t j = w; j < limit; j += 4) {
                    const uint32_t blk = block_tables[b * max_blocks_per_seq + j / block_size];
                    if ((int64_t)blk >= num_blocks) { bad = 1; break; }
                    const int64_t off = ((int64_t)blk * block_size + j % block_size) * ekv + kvh * head_dim;
                    float lane[32];
                    for (int ln = 0; ln < 32; ++ln) {
                        float s = 0.0f;
                        for (int64_t d = ln; d < head_dim; d += 32) s = fmaf(qs[d], kv_at(k_pool, off + d, kv_bf16), s);
                        lane[ln] = s;
                    }
                    const float s = butterfly_sum_f(lane);
                    const float m_new = fmaxf(m, s);
                    const float corr = orc_exp_det(m - m_new);
                    const float p = orc_exp_det(s - m_new);
                    l = fmaf(l, corr, p);
                    for (int64_t d = 0; d < head_dim; ++d) acc[d] = fmaf(p, kv_at(v_pool, off + d, kv_bf16), acc[d] * corr);
                    m = m_new;
                }
                wm[w] = m;
                wl[w] = l;
            }
            if (bad) { status = -1; continue; }
            const float mm = fmaxf(fmaxf(wm[0], wm[1]), fmaxf(wm[2], wm[3]));
            float g[4], ll = 0.0f;
            for (int w = 0; w < 4; ++w) {
                g[w] = wm[w] == -INFINITY ? 0.0f : orc_exp_det(wm[w] - mm);
                ll = fmaf(wl[w], g[w], ll);
            }
            for (int64_t d = 0; d < head_dim; ++d) {
                float o = 0.0f;
                for (int w = 0; w < 4; ++w) o = fmaf(wo[w][d], g[w], o);
                o_row[d] = limit > 0 ? o / ll : 0.0f;
            }
        }
    }
    return status;
}

/* ====================================================================================================
 * Block-scale INT8 contract proposed by the reference for its quantisation backend
 * (docs/int8-quant-grade-up-verification-plan.md:177-241).  PARITY UNPINNED beyond the accumulator vectors the
 * reference holds (K = 128 chain of 127 * 127 = 2 064 512, K_safe = 133 144): the document is a pre-registered
 * contract without code; this is its literal restatement.
 *   delta = pow2ceil(max(amax_block, 1e-4) / 127),  q = rne(x / delta)            blocks of 128 along K
 *   per block: s32 partial -> f32 (exact) -> * (delta_a * delta_b) once -> widen to f64
 *   blocks added in ascending order in f64, one narrowing to f32
 * ==================================================================================================== */
#define ORC_QBLOCK 128

float orc_pow2ceil(float x) {
    uint32_t b;
    memcpy(&b, &x, 4);
    if ((b & 0x7FFFFFu) == 0u) return x;
    b = ((b >> 23) + 1u) << 23;
    float r;
    memcpy(&r, &b, 4);
    return r;
}

/* x [rows, cols] -> q int8 [rows, cols], delta [rows, nb] (transposed == 0) or [nb, rows] (transposed != 0).
 * Returns 1 when a value was not finite (its block gets delta 1 and zero codes), else 0. */
int orc_quantize_i8_block(const float* x, int64_t rows, int64_t cols, int transposed, int8_t* q, float* delta) {
    const int64_t nb = (cols + ORC_QBLOCK - 1) / ORC_QBLOCK;
    int bad = 0;
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t b = 0; b < nb; ++b) {
            const int64_t c0 = b * ORC_QBLOCK, c1 = c0 + ORC_QBLOCK < cols ? c0 + ORC_QBLOCK : cols;
            float amax = 0.0f;
            int finite = 1;
            for (int64_t c = c0; c < c1; ++c) {
                const float v = x[r * cols + c];
                if (!isfinite(v)) finite = 0;
                amax = fmaxf(amax, fabsf(v));
            }
            float d = 1.0f;
            if (finite) d = orc_pow2ceil(fmaxf(amax, 1e-4f) / 127.0f);
            else bad = 1;
            delta[transposed ? b * rows + r : r * nb + b] = d;
            for (int64_t c = c0; c < c1; ++c) q[r * cols + c] = finite ? (int8_t)(int)rintf(x[r * cols + c] / d) : (int8_t)0;
        }
    return bad;
}

void orc_dequantize_i8_block(const int8_t* q, const float* delta, int64_t rows, int64_t cols, int transposed, float* x) {
    const int64_t nb = (cols + ORC_QBLOCK - 1) / ORC_QBLOCK;
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < cols; ++c) {
            const int64_t b = c / ORC_QBLOCK;
            x[r * cols + c] = (float)q[r * cols + c] * delta[transposed ? b * rows + r : r * nb + b];
        }
}

/* a [m, k] int8 with da [m, nb]; w [n, k] int8 with dw [nb, n]; out [m, n] f32.
 * Returns 1 when a result is not finite after the narrowing, else 0. */
int orc_gemm_i8_block_scaled(const int8_t* a, const float* da, const int8_t* w, const float* dw, int64_t m, int64_t n,
                             int64_t k, float* out) {
    const int64_t nb = (k + ORC_QBLOCK - 1) / ORC_QBLOCK;
    int bad = 0;
#pragma omp parallel for schedule(static) collapse(2) reduction(|| : bad)
    for (int64_t i = 0; i < m; ++i)
        for (int64_t j = 0; j < n; ++j) {
            double acc = 0.0;
            for (int64_t b = 0; b < nb; ++b) {
                const int64_t p0 = b * ORC_QBLOCK, p1 = p0 + ORC_QBLOCK < k ? p0 + ORC_QBLOCK : k;
                int32_t part = 0;
                for (int64_t p = p0; p < p1; ++p) part += (int32_t)a[i * k + p] * (int32_t)w[j * k + p];
                const float dout = da[i * nb + b] * dw[b * n + j];      /* composed scale first */
                const float val = (float)part * dout;                    /* one multiplication */
                acc += (double)val;                                      /* widen, ascending blocks */
            }
            const float y = (float)acc;                                  /* one narrowing */
            if (!isfinite(y)) bad = 1;
            out[i * n + j] = y;
        }
    return bad;
}
