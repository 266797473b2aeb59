// Host-callable launchers of the non-GEMM kernels (quantisers, paged KV, decoder glue).
// All of them only enqueue work on the given stream.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// ---- quant.cu
cudaError_t quantize_i8_per_row(const float* x, int64_t rows, int64_t cols, int8_t* q, float* scale, cudaStream_t s);
cudaError_t dequantize_i8_per_row(const int8_t* q, const float* scale, int64_t rows, int64_t cols, float* x,
                                  cudaStream_t s);
// `amax_scratch` is one uint32 of device memory owned by the context.
cudaError_t quantize_fp8_per_tensor(const float* x, int64_t n, uint8_t* q, float* scale, uint32_t* amax_scratch,
                                    cudaStream_t s);

// Block-scale contract: one power-of-two scale per 128 values of a row.  `transposed` selects the layout of the scale
// array: [rows, nb] (0) or [nb, rows] (1).  `status` is a device word: bit 0 is set when an input value is not finite.
cudaError_t quantize_i8_block_pow2(const float* x, int64_t rows, int64_t cols, int8_t* q, float* delta, int transposed,
                                   uint32_t* status, cudaStream_t s);
cudaError_t dequantize_i8_block(const int8_t* q, const float* delta, int64_t rows, int64_t cols, int transposed, float* x,
                                cudaStream_t s);

// ---- paged_kv.cu
struct PagedAttnShape {
    int batch, l_new, num_q_heads, num_kv_heads, head_dim, block_size, num_blocks, max_blocks_per_seq;
    float scale;
};
struct PagedAttnPlan {
    PagedAttnShape shape;
    int kv_bf16;
    int fast;           // TMA split-K path (head_dim 128, bf16, block 16, 1/2/4/8 q heads per kv head)
    int chunk_blocks;   // blocks per split
    int max_chunks;     // splits reserved per query row
    CUtensorMap tma_k, tma_v;
};
// Copies row r of k_new / v_new [rows, e] (f32) to pool row slots_dev[r], rounding to bf16 when kv_bf16.
cudaError_t paged_kv_append(const float* k_new, const float* v_new, void* k_pool, void* v_pool, const uint32_t* slots_dev,
                            int64_t rows, int64_t e, int64_t pool_rows, int kv_bf16, uint32_t* err, cudaStream_t s);
bool paged_attention_fast_path(const PagedAttnShape& sh, int kv_bf16);
// max_seq_len bounds the number of splits a row can need; want_chunk_blocks <= 0 picks the default.
cudaError_t paged_attention_make_plan(PagedAttnPlan* plan, const PagedAttnShape& sh, int kv_bf16, const void* k_pool,
                                      const void* v_pool, int max_seq_len, int want_chunk_blocks);
size_t paged_attention_scratch_bytes(const PagedAttnPlan& plan);
// q, out: [batch, l_new, num_q_heads * head_dim] f32.  tables/seq_lens are device arrays.
cudaError_t paged_attention_launch(const PagedAttnPlan& plan, const float* q, const void* k_pool, const void* v_pool,
                                   const uint32_t* tables_dev, const uint32_t* seq_lens_dev, float* out, void* scratch,
                                   unsigned int* work_counter, int sm_count, uint32_t* err, cudaStream_t stream,
                                   int8_t* xq_out = nullptr, float* sx_out = nullptr, int fp8 = 0);
// True when the launch can also emit the per-token quantisation of the output rows (xq_out / sx_out; int8 under
// amax / 127, or with fp8 != 0 E4M3 under amax / 448): `out` may then be null.  The caller must also pass a 16-byte
// aligned q.
bool paged_attention_can_quantize(const PagedAttnPlan& plan);

// Device address (for the given, current device) and size of the file-scope static scratch array that
// stands in for `scratch` when the caller must not allocate.  The first call on a device looks the address
// up with cudaGetSymbolAddress; it allocates nothing.
cudaError_t paged_attention_static_scratch(int device, void** out);
size_t paged_attention_static_scratch_capacity();

// ---- decode_kernels.cu (one CTA per token row; `raw` = split-K planes [splits][M][N] of int32)
cudaError_t embed_norm_quant(const int* ids, const float* table, int vocab, int M, int d, const float* norm_w, float eps,
                             float* h, int8_t* xq, float* sx, uint32_t* err, cudaStream_t s);
// `pre` != nullptr: the already dequantised (and, under tensor parallelism, all-reduced) GEMM output
// [M, d] is used instead of raw / sx_in / sw.
cudaError_t resid_norm_quant(const int* raw, int splits, int M, int d, const float* sx_in, const float* sw,
                             const float* pre, const float* norm_w, float eps, float* h, int8_t* xq, float* sx_out,
                             cudaStream_t s);
cudaError_t gate_quant(const int* raw, int splits, int M, int F, const float* sx_in, const float* sw, int8_t* xq,
                       float* sx_out, cudaStream_t s);
// ---- decode_rows.cu: the same operations with one wide CTA per row (or one cluster per row for the once-per-step
// kernels); they fall back to the kernels above for rows wider than 16384 columns.
// fp8 != 0 selects the FP8 form of the decoder: `raw` holds f32 accumulators (bit patterns, summed over the planes in
// plane order) and the rows are emitted as E4M3 codes under the per-token scale amax / 448 instead of int8 under
// amax / 127.  It exists in the wide / cluster kernels only (invalid-value error for other row widths).
cudaError_t embed_norm_quant_auto(const int* ids, const float* table, int vocab, int M, int d, const float* norm_w,
                                  float eps, float* h, int8_t* xq, float* sx, uint32_t* err, cudaStream_t s, int fp8 = 0);
cudaError_t resid_norm_quant_auto(const int* raw, int splits, int M, int d, const float* sx_in, const float* sw,
                                  const float* pre, const float* norm_w, float eps, float* h, int8_t* xq, float* sx_out,
                                  cudaStream_t s, int fp8 = 0);
cudaError_t gate_quant_auto(const int* raw, int splits, int M, int F, const float* sx_in, const float* sw, int8_t* xq,
                            float* sx_out, cudaStream_t s, int fp8 = 0);
cudaError_t quantize_rows_auto(const float* x, int M, int n, int8_t* xq, float* sx_out, cudaStream_t s, int fp8 = 0);
cudaError_t argmax_rows_auto(const float* logits, int M, int vocab, int* out_ids, cudaStream_t s);
// `active` (null: all rows) marks the rows whose K / V are appended; the others only get their q row.
cudaError_t qkv_rope_append_auto(const int* raw, int splits, int M, int hq, int hkv, int dh, const float* sx_in,
                                 const float* sw, const float* cos_t, const float* sin_t, int max_pos,
                                 const uint32_t* positions, const uint32_t* active, const uint32_t* block_tables,
                                 int max_blocks_per_seq, int block_size, int num_blocks, float* q_out, uint16_t* k_pool,
                                 uint16_t* v_pool, uint32_t* err, cudaStream_t s, int rows_per_seq = 1, int fp8 = 0);
// Prefill: `rows_per_seq` consecutive token rows belong to one sequence (row m uses table row m / rows_per_seq).
// positions[m] = seq_lens[m / l_new] + m % l_new for m < count * l_new ...
cudaError_t prefill_positions(const uint32_t* seq_lens, uint32_t* positions, int count, int l_new, cudaStream_t s);
// ... and afterwards seq_lens[b] += l_new for b < count.
cudaError_t prefill_advance(uint32_t* seq_lens, int count, int l_new, cudaStream_t s);

// y[m, n] = sum_planes(raw)[m, n] * (sx[m] * sw[n]) as f32 (the addend of a cross-rank sum)
cudaError_t dequant_planes(const int* raw, int splits, int M, int N, const float* sx, const float* sw, float* y,
                           cudaStream_t s);
// positions[i] = seq_lens[i]; seq_lens[i] += 1
cudaError_t begin_step(uint32_t* seq_lens, uint32_t* positions, const uint32_t* active, int n, cudaStream_t s);
cudaError_t argmax_rows(const float* logits, int M, int vocab, int* out_ids, cudaStream_t s);
cudaError_t fill_normal(float* out, int64_t n, uint64_t seed, uint64_t stream_id, float std, cudaStream_t s);
cudaError_t fill_normal_bf16(uint16_t* out, int64_t n, uint64_t seed, uint64_t stream_id, float std, cudaStream_t s);
cudaError_t slice_cols_i8(const int8_t* src, int64_t rows, int64_t ld, int64_t c0, int64_t cols, int8_t* dst,
                          cudaStream_t s);

// Rows quantised under a scale that comes from outside (tensor parallelism with exact integer sums: the row maximum
// is merged across the ranks between the two calls).  Rows of up to 16384 columns, a multiple of 4.
bool rows_scaled_supported(int n);
cudaError_t rows_amax(const float* x, int M, int n, float* amax_out, cudaStream_t s);
cudaError_t quantize_rows_with_amax(const float* x, int M, int n, const float* amax, int8_t* xq, float* sx_out, cudaStream_t s);
// a = silu(gate) * up of the columns [0, F) / [F, 2F) of the raw planes as f32 [M, F], and the row maxima of |a|
cudaError_t gate_rows_f32(const int* raw, int splits, int M, int F, const float* sx_in, const float* sw, float* out,
                          float* amax_out, cudaStream_t s);

// Tensor-parallel finish of a row-parallel GEMM over the ranks' exchange blocks (decode_rows.cu): sums the f32
// partials of the rows this rank owns over all ranks, adds the residual, applies RMSNorm and the per-token int8
// quantisation and delivers the int8 rows and scales to every rank.  `peers` is a device array of the tp block
// bases; a block starts with 512 bytes of flags (ready[tp] at +0, delivered[tp] at +256).  The kernel waits for the
// peers' partials but not for their rows: the consumer of the delivered rows waits for the delivered flags.
// Needs one GPU per rank unless the flags are raised beforehand.
// Scattered form (push_tiles != 0): the ranks' GEMMs have stored the partials of this rank's rows straight into its
// block as planes [tp][rows][d] at o_part and count their launches in count[tp] at o_count (GemmPush); the kernel
// waits until every count has grown by push_tiles (1: one count per launch) since the call before (*push_target
// keeps the sum) and reads only its own memory.
constexpr uint64_t kCrossGpuWaitNs = 2000000000ull;      // default bound of a cross-GPU wait (two seconds)
bool tp_finish_supported(int d);
cudaError_t tp_finish(uint8_t* const* peers, size_t o_sx, size_t o_xq, size_t o_part, int tp, int rank, int rows, int d,
                      const float* norm_w, float eps, float* h, uint32_t* epoch, unsigned int* arrived, uint32_t* err,
                      cudaStream_t s, uint64_t timeout_ns = 0,    // 0: the default bound of a cross-GPU wait
                      size_t o_count = 0, uint32_t push_tiles = 0, uint32_t* push_target = nullptr, int fp8 = 0);

}  // namespace b200
