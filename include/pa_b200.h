/*
 * pa_b200.h -- C-ABI of libpa_b200.so: the B200 (sm_100a) implementation of the
 * reference's decode hot path (paged attention over the tiled KV cache + INT8
 * quantise / dequantise / int8 matmul).  Plain pointers and sizes only; every
 * pointer named d_* (and every tensor argument unless stated otherwise) is a
 * DEVICE pointer; `stream` is a cudaStream_t passed as void*.
 *
 * Every entry point returns an int status: 0 = PA_OK, <0 = PA_ERR_* (argument /
 * support errors, nothing launched), >0 = a cudaError_t from the launch.
 * pa_error_string() renders any of them.  There is no CPU fallback anywhere.
 *
 * Each declaration cites the reference interface it replaces (paths relative to
 * the reference repository root).
 */
#ifndef PA_B200_H_
#define PA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PA_OK 0
#define PA_ERR_INVALID_ARG (-1)  /* null pointer, non-positive size, misaligned buffer */
#define PA_ERR_UNSUPPORTED (-2)  /* head_dim / tile_size / activation outside the built set */
#define PA_ERR_WORKSPACE (-3)    /* workspace too small; see pa_decode_workspace_bytes */
#define PA_ERR_NO_DEVICE (-4)    /* no sm_100 device is current */
#define PA_ERR_NCCL (-5)         /* an NCCL call failed (pa_nccl_*) */

#define PA_ACT_NONE 0
#define PA_ACT_RELU 1
#define PA_ACT_GELU 2 /* gelu_erf, dnnl_matmul_int8.cpp:48-49 */

typedef void* pa_stream_t; /* cudaStream_t */

/* ---------------------------------------------------------------- runtime */
int pa_version(void);
const char* pa_error_string(int status);
/* sm count / compute capability of the current device. */
int pa_device_info(int* sm_count, int* cc_major, int* cc_minor);

/* ------------------------------------------------------------- page table */
/* kv_cache/page_table.cpp:14-26,41-47  PageTable::init / clear:
 * every entry := -1 (unmapped). */
int pa_page_table_clear(int32_t* d_table, int64_t n_entries, pa_stream_t stream);

/* kv_cache/page_table.cpp:49-53 PageTable::assign and :64-67 remove, batched:
 * d_table[d_idx[i]] = d_page[i] for i < n (page -1 == remove).  Replaces the
 * reference's one blocking 4-byte cudaMemcpy per entry.  idx is the flat index
 * beam*(H*Tiles) + head*Tiles + tile (page_table.hpp:39-42); out-of-range
 * indices are ignored (the reference asserts). */
int pa_page_table_update(int32_t* d_table, int64_t n_entries, const int32_t* d_idx,
                         const int32_t* d_page, int n, pa_stream_t stream);

/* kv_cache/page_table.hpp:44-49 PageTable::lookup (device), batched: d_out[i] =
 * table entry of (d_beam[i], d_head[i], d_tile[i]) or -1 when the flat index
 * is out of range. */
int pa_page_table_lookup(const int32_t* d_table, int num_beams, int num_heads, int num_tiles,
                         const int32_t* d_beam, const int32_t* d_head, const int32_t* d_tile,
                         int32_t* d_out, int n, pa_stream_t stream);

/* -------------------------------------------------------- page pool: gather */
/* kv_cache/kv_tile_cache.hpp:21-26 KVTileCache<T>::get, materialised: copies
 * the pages of rows r < R (table row = d_beam_ids ? d_beam_ids[r] : r) of one
 * pool into dense [R, H, num_tiles*tile_size, D]; unmapped / out-of-range pages
 * are filled with `fill_byte`.  elem_bytes = sizeof(T) (1, 2 or 4).
 * Bit-exact byte mover. */
int pa_kv_gather(const void* d_pool, void* d_dense, const int32_t* d_table, int num_beams,
                 int num_heads, int num_tiles, int total_pages, int tile_size, int head_dim,
                 int elem_bytes, const int32_t* d_beam_ids, int R, int fill_byte,
                 pa_stream_t stream);

/* -------------------------------------------------------- page pool: append */
/* kv_cache/kv_tile_cache.hpp:29-34 KVTileCache<T>::get_write_ptr + the row
 * write the caller performs: row (d_positions[r] % tile_size) of page
 * (beam, head, d_positions[r] / tile_size) := new_k/new_v[r, head, :].
 * Unmapped pages are skipped.  new_k/new_v are [R, H, D].
 *   _f16      : new rows already fp16, byte copy.
 *   _f32_f16  : new rows fp32, rounded to nearest-even fp16 on write.
 *   _f32_i8   : new rows fp32; per (row, head) scale = compute_minmax_scale
 *               (int8_quant.cpp:59-64), q = batch_quantize (int8_quant.cpp:15-28);
 *               scale stored at d_*_scales[page*tile_size + row_in_page]. */
int pa_kv_append_f16(void* d_k_pool, void* d_v_pool, const int32_t* d_table, int num_beams,
                     int num_heads, int num_tiles, int total_pages, int tile_size, int head_dim,
                     const void* d_new_k, const void* d_new_v, const int32_t* d_beam_ids,
                     const int32_t* d_positions, int R, pa_stream_t stream);
/* fp32 rows into an fp32 pool (KVTileCache<float>): raw copy. */
int pa_kv_append_f32(float* d_k_pool, float* d_v_pool, const int32_t* d_table, int num_beams,
                     int num_heads, int num_tiles, int total_pages, int tile_size, int head_dim,
                     const float* d_new_k, const float* d_new_v, const int32_t* d_beam_ids,
                     const int32_t* d_positions, int R, pa_stream_t stream);
int pa_kv_append_f32_f16(void* d_k_pool, void* d_v_pool, const int32_t* d_table, int num_beams,
                         int num_heads, int num_tiles, int total_pages, int tile_size,
                         int head_dim, const float* d_new_k, const float* d_new_v,
                         const int32_t* d_beam_ids, const int32_t* d_positions, int R,
                         pa_stream_t stream);
int pa_kv_append_f32_i8(int8_t* d_k_pool, int8_t* d_v_pool, float* d_k_scales, float* d_v_scales,
                        const int32_t* d_table, int num_beams, int num_heads, int num_tiles,
                        int total_pages, int tile_size, int head_dim, const float* d_new_k,
                        const float* d_new_v, const int32_t* d_beam_ids,
                        const int32_t* d_positions, int R, pa_stream_t stream);

/* Copy-on-write support for beam search over shared-prefix pages (north star; no
 * reference implementation): pool[d_dst_pages[i]] := pool[d_src_pages[i]] for the K and V
 * pools (and the int8 scale rows when given), i < n.  Bit-exact byte mover. */
int pa_kv_copy_pages(void* d_k_pool, void* d_v_pool, float* d_k_scales, float* d_v_scales,
                     const int32_t* d_src_pages, const int32_t* d_dst_pages, int n, int total_pages,
                     int tile_size, int head_dim, int elem_bytes, pa_stream_t stream);

/* ------------------------------------------------ paged decode attention */
/* Bytes of scratch the decode entry points need for B rows x H heads of head_dim D over a
 * page table of num_tiles tiles of tile_size tokens. */
size_t pa_decode_workspace_bytes(int B, int num_heads, int head_dim, int num_tiles, int tile_size);

/*
 * attention/paged_flash_attention_kernel_fused.cu:5-90 (launched by
 * attention/attention_tile_launcher.hpp:35-90, dispatched by
 * attention/attention_cuda.cu:41-95), with the math of
 * attention_cpu/cpu_attention_kernel.cpp:36-129 (global softmax):
 * for every (b, h)
 *     beam   = d_beam_ids ? d_beam_ids[b] : b
 *     s[t]   = dot(q[b,h,:], K[beam,h,t,:]) / temperature      t < ctx(b)
 *     p      = exp(s - max s) / (sum exp(s - max s) + 1e-6)
 *     out[b,h,:] = sum_t p[t] * V[beam,h,t,:]
 * K/V rows come from pages: page = table[beam][h][t / tile_size]; unmapped or
 * out-of-range pages contribute nothing.  ctx(b) = d_ctx_lens ? d_ctx_lens[b] : T.
 * q, out: [B, H, D] f32 (out may alias q).  Pools: [total_pages][tile_size][D].
 * d_rope: optional [D] interleaved cos/sin, pairwise rotation of q
 * (cpu_attention_kernel.cpp:13-19); NULL = off.  d_lse_out: optional [B, H]
 * log-sum-exp of the scaled scores (replaces the racy rerank_scores side
 * output, ...fused.cu:53-55).  head_dim in {64, 128}; tile_size % 16 == 0.
 *
 * _f16: fp16 K/V pages, split-KV grid kernel, 128-bit page-indirect global
 *       loads, warp-shuffle online softmax, LSE combine.
 * _f16_overlap: paged_flash_attention_kernel_fused_overlap.cu:5-91 -- same
 *       results through the persistent kernel that stages pages into shared
 *       memory with the TMA bulk-copy engine (multi-stage mbarrier ring) so
 *       loads and math overlap.
 * _i8 / _i8_overlap: int8 K/V pages with per-(page,row) f32 scales, dequantised
 *       in the kernel as q/scale (int8_quant.cpp:46-57).
 * _f32 / _f32_overlap: fp32 K/V pages -- KVTileCache<float>, the instantiation
 *       AttentionCUDA::forward takes (attention_config.hpp:15, kv_tile_cache.cpp:127);
 *       the same kernels on 4-byte elements.
 */
int pa_paged_decode_f16(const float* d_q, float* d_out, const void* d_k_pool, const void* d_v_pool,
                        const int32_t* d_table, int num_beams, int num_heads, int num_tiles,
                        int total_pages, const int32_t* d_beam_ids, const int32_t* d_ctx_lens,
                        int B, int T, int head_dim, int tile_size, float temperature,
                        const float* d_rope, float* d_lse_out, void* d_workspace,
                        size_t workspace_bytes, pa_stream_t stream);
int pa_paged_decode_f16_overlap(const float* d_q, float* d_out, const void* d_k_pool,
                                const void* d_v_pool, const int32_t* d_table, int num_beams,
                                int num_heads, int num_tiles, int total_pages,
                                const int32_t* d_beam_ids, const int32_t* d_ctx_lens, int B,
                                int T, int head_dim, int tile_size, float temperature,
                                const float* d_rope, float* d_lse_out, void* d_workspace,
                                size_t workspace_bytes, pa_stream_t stream);
int pa_paged_decode_i8(const float* d_q, float* d_out, const int8_t* d_k_pool,
                       const int8_t* d_v_pool, const float* d_k_scales, const float* d_v_scales,
                       const int32_t* d_table, int num_beams, int num_heads, int num_tiles,
                       int total_pages, const int32_t* d_beam_ids, const int32_t* d_ctx_lens,
                       int B, int T, int head_dim, int tile_size, float temperature,
                       const float* d_rope, float* d_lse_out, void* d_workspace,
                       size_t workspace_bytes, pa_stream_t stream);
int pa_paged_decode_i8_overlap(const float* d_q, float* d_out, const int8_t* d_k_pool,
                               const int8_t* d_v_pool, const float* d_k_scales,
                               const float* d_v_scales, const int32_t* d_table, int num_beams,
                               int num_heads, int num_tiles, int total_pages,
                               const int32_t* d_beam_ids, const int32_t* d_ctx_lens, int B, int T,
                               int head_dim, int tile_size, float temperature,
                               const float* d_rope, float* d_lse_out, void* d_workspace,
                               size_t workspace_bytes, pa_stream_t stream);

int pa_paged_decode_f32(const float* d_q, float* d_out, const float* d_k_pool, const float* d_v_pool,
                        const int32_t* d_table, int num_beams, int num_heads, int num_tiles,
                        int total_pages, const int32_t* d_beam_ids, const int32_t* d_ctx_lens,
                        int B, int T, int head_dim, int tile_size, float temperature,
                        const float* d_rope, float* d_lse_out, void* d_workspace,
                        size_t workspace_bytes, pa_stream_t stream);
int pa_paged_decode_f32_overlap(const float* d_q, float* d_out, const float* d_k_pool,
                                const float* d_v_pool, const int32_t* d_table, int num_beams,
                                int num_heads, int num_tiles, int total_pages,
                                const int32_t* d_beam_ids, const int32_t* d_ctx_lens, int B,
                                int T, int head_dim, int tile_size, float temperature,
                                const float* d_rope, float* d_lse_out, void* d_workspace,
                                size_t workspace_bytes, pa_stream_t stream);

/* Decode attention WITH the reference's in-attention top-k / top-p filter and its optional side outputs: the CPU
 * kernel's algorithm stage by stage (attention_cpu/cpu_attention_kernel.cpp:61-126) -- K pass, softmax over all T
 * scores (softmax_lut.cpp:203-231), apply_topk_topp_filter (rank-based zeroing, no renormalisation,
 * softmax_lut.cpp:233-256), V pass.  The filter needs a row's every probability before any is used, so this is
 * the explicit three-stage form, not the one-pass kernels above; callers use it only when top_k > 0, top_p < 1
 * or a side output is wanted (cpu_attention_kernel.hpp:20-21 defaults keep the hot path).
 *   kv_kind: 0 fp16 pages, 1 int8 pages + scales, 2 fp32 pages.
 *   d_logits_out  (optional) [B,H,T]: pre-softmax scores, -1e9 for unmapped tiles (CPUAttentionOutput::logits),
 *                 -inf past a row's context;  d_weights_out (optional) [B,H,T]: post-filter probabilities
 *                 (CPUAttentionOutput::attention_weights).  Whichever is NULL lives in d_workspace
 *                 (>= pa_attention_filtered_workspace_bytes(B, num_heads, T)).  Temperature applied once (D3). */
size_t pa_attention_filtered_workspace_bytes(int B, int num_heads, int T);
int pa_paged_attention_filtered(const float* d_q, float* d_out, const void* d_k_pool, const void* d_v_pool,
                                const float* d_k_scales, const float* d_v_scales, int kv_kind,
                                const int32_t* d_table, int num_beams, int num_heads, int num_tiles,
                                int total_pages, const int32_t* d_beam_ids, const int32_t* d_ctx_lens, int B,
                                int T, int head_dim, int tile_size, float temperature, const float* d_rope,
                                int top_k, float top_p, float* d_logits_out, float* d_weights_out,
                                void* d_workspace, size_t workspace_bytes, pa_stream_t stream);

/* Beam-aware shared-prefix decode (north star; the reference's only hook is the
 * beam_ids[b] -> page-table-row indirection, ...fused.cu:22).  Rows b = g*beam_width ..
 * g*beam_width + beam_width-1 form beam group g.  Same results as pa_paged_decode_f16, but
 * a K/V page whose id is the same for several beams of a group (shared prefix /
 * not-yet-copied copy-on-write page) is read from HBM ONCE per group and applied to all
 * those beams' queries on the tensor cores (mma.sync m16n8k16, fp16 operands split hi/lo so
 * scores and outputs keep fp32 accuracy).  Pages that differ are staged per distinct id.
 * Requires head_dim == 128, beam_width <= 4, B % beam_width == 0; otherwise
 * PA_ERR_UNSUPPORTED and the caller uses pa_paged_decode_f16[_overlap].  d_ctx_lens (optional)
 * gives every row its own context length (tokens at or past it are masked for that row only):
 * with consecutive query positions as the rows of a group this is causal prefill, 4 queries
 * per K/V byte. */
int pa_paged_decode_f16_group(const float* d_q, float* d_out, const void* d_k_pool,
                              const void* d_v_pool, const int32_t* d_table, int num_beams,
                              int num_heads, int num_tiles, int total_pages,
                              const int32_t* d_beam_ids, const int32_t* d_ctx_lens, int B, int T,
                              int head_dim, int tile_size, float temperature, const float* d_rope,
                              int beam_width, float* d_lse_out, void* d_workspace,
                              size_t workspace_bytes, pa_stream_t stream);

/* Beam groups over INT8 pages: the per-row streaming kernel through the beam_ids indirection (the tensor-core group
 * kernel is fp16-only).  Same results as pa_paged_decode_i8_overlap; shared-prefix pages are served from L2 after
 * their first read (evict_first is off when d_beam_ids is given), so HBM sees roughly the unique bytes. */
int pa_paged_decode_i8_group(const float* d_q, float* d_out, const int8_t* d_k_pool, const int8_t* d_v_pool,
                             const float* d_k_scales, const float* d_v_scales, const int32_t* d_table,
                             int num_beams, int num_heads, int num_tiles, int total_pages,
                             const int32_t* d_beam_ids, const int32_t* d_ctx_lens, int B, int T, int head_dim,
                             int tile_size, float temperature, const float* d_rope, int beam_width,
                             float* d_lse_out, void* d_workspace, size_t workspace_bytes, pa_stream_t stream);

/* Split-KV across GPUs (north-star long-context mode): same computation over
 * this rank's pages only, emitting UN-normalised partials for an LSE combine:
 *   d_part_m[b,h] = max_t s[t] (natural-log units; -inf if no key)
 *   d_part_l[b,h] = sum_t exp(s[t]-m),  d_part_o[b,h,:] = sum_t exp(s[t]-m) V[t,:]
 * (no positional term enters the math, so a rank needs no token offset: its page-table rows simply hold
 * its own tile range).  One launch: the streaming kernel merges each row when its last chunk finishes.
 * _i8: int8 pages with per-(page,row) scales. */
int pa_paged_decode_f16_partial(const float* d_q, float* d_part_m, float* d_part_l,
                                float* d_part_o, const void* d_k_pool, const void* d_v_pool,
                                const int32_t* d_table, int num_beams, int num_heads,
                                int num_tiles, int total_pages, const int32_t* d_beam_ids,
                                const int32_t* d_ctx_lens, int B, int T, int head_dim,
                                int tile_size, float temperature, const float* d_rope,
                                void* d_workspace, size_t workspace_bytes, pa_stream_t stream);
int pa_paged_decode_i8_partial(const float* d_q, float* d_part_m, float* d_part_l, float* d_part_o,
                               const int8_t* d_k_pool, const int8_t* d_v_pool, const float* d_k_scales,
                               const float* d_v_scales, const int32_t* d_table, int num_beams,
                               int num_heads, int num_tiles, int total_pages, const int32_t* d_beam_ids,
                               const int32_t* d_ctx_lens, int B, int T, int head_dim, int tile_size,
                               float temperature, const float* d_rope, void* d_workspace,
                               size_t workspace_bytes, pa_stream_t stream);

/* LSE combine of n_parts partials (layout [n_parts][rows] for m/l and
 * [n_parts][rows][D] for o, as gathered from n_parts ranks):
 *   M = max_i m_i; w_i = exp(m_i - M); out = sum w_i o_i / (sum w_i l_i + 1e-6). */
int pa_lse_combine(const float* d_part_m, const float* d_part_l, const float* d_part_o,
                   int n_parts, int rows, int head_dim, float* d_out, float* d_lse_out,
                   pa_stream_t stream);

/* --------------------------------------------------------------- int8_quant */
/* attention_cpu/int8_quant.cpp:5-13  q = clamp(round_half_away(x*scale),-128,127) */
int pa_quantize_i8(const float* d_x, int64_t n, float scale, int8_t* d_q, pa_stream_t stream);
/* attention_cpu/int8_quant.cpp:15-28 per-row scale, x [rows, dim] */
int pa_batch_quantize_i8(const float* d_x, const float* d_scales, int rows, int dim, int8_t* d_q,
                         pa_stream_t stream);
/* attention_cpu/int8_quant.cpp:30-36 -> *d_out (one float, device) */
int pa_absmax(const float* d_x, int64_t n, float* d_out, pa_stream_t stream);
/* attention_cpu/int8_quant.cpp:59-64 127/(absmax+1e-6) -> *d_out */
int pa_minmax_scale(const float* d_x, int64_t n, float* d_out, pa_stream_t stream);
/* the same, one scale per row of x [rows, dim] -> d_scales[rows] */
int pa_batch_minmax_scale(const float* d_x, int rows, int dim, float* d_scales, pa_stream_t stream);
/* attention_cpu/int8_quant.cpp:38-44  x = (float)q / scale (IEEE division) */
int pa_dequantize_i8(const int8_t* d_q, int64_t n, float scale, float* d_x, pa_stream_t stream);
/* attention_cpu/int8_quant.cpp:46-57 */
int pa_batch_dequantize_i8(const int8_t* d_q, const float* d_scales, int rows, int dim, float* d_x,
                           pa_stream_t stream);

/* ------------------------------------------------------------ int8 matmul */
/* attention_cpu/dnnl_matmul_int8.cpp:7-76:
 *   acc[b,m,n] = sum_k A[b,m,k] * B[b,k,n]              (s8 x s8 -> s32, exact)
 *   C_s8       = sat_s8(rne(act(alpha*acc + bias[n]))),  alpha = scaleA*scaleB/scaleC
 * A [BATCH,M,K], B [BATCH,K,N], C [BATCH,M,N] row-major (format_tag::abc).
 * d_C_s8 and/or d_C_s32 may be NULL (at least one must be given); d_C_s32
 * receives the raw int32 accumulators (the bit-exact parity target).
 * tcgen05 kind::i8 tensor-core kernel; K % 16 == 0 and N % 16 == 0 required.
 * d_workspace: caller-owned scratch for split-K partial tiles, at least
 * pa_gemm_i8_workspace_bytes(BATCH, M, N, K) bytes (0 = this shape never splits), 16-byte aligned.  The
 * library owns no growable scratch (a pointer captured in a CUDA graph must stay valid; streams must not share
 * it): NULL or too small a workspace makes the GEMM run unsplit -- same result, fewer CTAs. */
size_t pa_gemm_i8_workspace_bytes(int BATCH, int M, int N, int K);
int pa_gemm_i8(const int8_t* d_A, const int8_t* d_B, int8_t* d_C_s8, int32_t* d_C_s32, int BATCH,
               int M, int N, int K, float scaleA, float scaleB, float scaleC, const float* d_bias,
               int act, void* d_workspace, size_t workspace_bytes, pa_stream_t stream);

/* Dynamic-quantisation form of the same GEMM, used by the INT8 decoder MLP ("int8_quant ->
 * dnnl_matmul_int8 -> dequant", attention_cpu/README.md:80-86):
 *   C_f32[b,m,n] = act(alpha_row*acc + bias[n]),  alpha_row = b_dequant / d_a_qscales[b*M+m]
 * d_a_qscales [BATCH*M] are the DEVICE-resident per-row quantisation scales of A in the
 * int8_quant.cpp convention (A_s8 = batch_quantize(x, scales, K), int8_quant.cpp:15-28,
 * so x ~ A_s8 / scale); b_dequant is the dequantisation multiplier of the weights
 * (w ~ B_s8 * b_dequant).  No host synchronisation: the scales produced by
 * pa_batch_minmax_scale feed this call directly. */
int pa_gemm_i8_dequant(const int8_t* d_A, const int8_t* d_B, float* d_C_f32, int BATCH, int M, int N,
                       int K, const float* d_a_qscales, float b_dequant, const float* d_bias, int act,
                       void* d_workspace, size_t workspace_bytes,
                       pa_stream_t stream);

/* The same GEMM with the DYNAMIC ROW QUANTISATION of its output fused into the epilogue -- the
 * "fc1 -> int8_quant -> fc2" hand-off of the INT8 decoder MLP (attention_cpu/README.md:80-86) in one kernel:
 *   v[b,m,n]       = act(alpha_row*acc + bias[n])                  (as pa_gemm_i8_dequant; act none / relu)
 *   d_c_qscale[bm] = 127 / (max_n |v| + 1e-6)                      (compute_minmax_scale, int8_quant.cpp:59-64)
 *   C_s8[b,m,n]    = clamp(round_half_away(v * d_c_qscale[bm]))    (batch_quantize, int8_quant.cpp:15-28)
 * bit-identical to pa_gemm_i8_dequant followed by pa_row_quantize_dynamic_i8, without the f32 round trip (the
 * accumulators wait in TMEM while the row maxima cross the grid).  Needs the whole grid resident at once:
 * PA_ERR_UNSUPPORTED for M <= 128, for more CTA pairs than SMs / 2, for shapes that would split K, and for gelu --
 * callers then use the two separate calls.  d_workspace: >= pa_gemm_i8_dynquant_workspace_bytes(BATCH, M, N) bytes,
 * 16-byte aligned, DEDICATED to this function and ZERO-FILLED ONCE by the caller (its first 16 bytes are the
 * self-resetting counters of the grid barrier; one stream at a time per workspace). */
size_t pa_gemm_i8_dynquant_workspace_bytes(int BATCH, int M, int N);
int pa_gemm_i8_dynquant(const int8_t* d_A, const int8_t* d_B, int8_t* d_C_s8, float* d_c_qscale, int BATCH,
                        int M, int N, int K, const float* d_a_qscale, float b_dequant, const float* d_bias,
                        int act, void* d_workspace, size_t workspace_bytes, pa_stream_t stream);

/* ------------------------------------------------- decoder glue (row a14) */
/* decoder/token_embedding.hpp:19-26: d_out[r,:] = E[d_ids[r],:] (ids outside [0,vocab) give
 * zeros; the reference reads out of bounds).  _i8: int8 table dequantised as q/qscale
 * (int8_quant.cpp:38-44). */
int pa_embedding_f32(const float* d_E, const int32_t* d_ids, int rows, int hidden, int vocab,
                     float* d_out, pa_stream_t stream);
int pa_embedding_i8(const int8_t* d_E, float qscale, const int32_t* d_ids, int rows, int hidden,
                    int vocab, float* d_out, pa_stream_t stream);
/* decoder/layer_norm.hpp:20-37: biased variance, inv_std = 1/sqrt(var+eps), y = (x-mean)*inv_std*gamma+beta.
 * d_out may alias d_x. */
int pa_layer_norm_f32(const float* d_x, const float* d_gamma, const float* d_beta, int rows,
                      int hidden, float eps, float* d_out, pa_stream_t stream);
/* decoder/mlp.hpp:23-41, one layer of the float MLP: out[r,n] = act(bias[n] + sum_k x[r,k]*W[k*N+n]),
 * act in {PA_ACT_NONE, PA_ACT_RELU}.  d_out must not alias d_x.  d_workspace: caller-owned scratch for the
 * K-slice partials, >= pa_linear_workspace_bytes(rows, K, N) bytes (NULL / too small: unsliced, same result
 * up to the summation order).
 * Arithmetic: layers with >= 16 rows, N % 4 == 0, K % 4 == 0, 16-byte aligned operands and >= 5e7 MACs run on
 * the tensor cores (tcgen05 kind::tf32 with every operand split into hi + lo: x.W ~= x_hi.W_lo + x_lo.W_hi +
 * x_hi.W_hi, fp32 accumulation; error <= 1e-5 * sum_k |x||W| stated, <= 1.1e-6 measured -- the fp32 SIMT
 * kernels: 1-3e-7); everything else, and everything with PA_LINEAR_TC=0 in the environment, in fp32 FMA
 * arithmetic proper (only the summation order differs from the reference's scalar loop). */
size_t pa_linear_workspace_bytes(int rows, int K, int N);
int pa_linear_f32(const float* d_x, const float* d_W, const float* d_bias, int rows, int K, int N,
                  int act, float* d_out, void* d_workspace, size_t workspace_bytes, pa_stream_t stream);
/* pa_linear_f32 restricted to the fp32 FMA kernels whatever the size: products and sums in IEEE float. */
int pa_linear_f32_exact(const float* d_x, const float* d_W, const float* d_bias, int rows, int K, int N,
                        int act, float* d_out, void* d_workspace, size_t workspace_bytes, pa_stream_t stream);
/* The same layer on weights repacked ONCE (at load) into the tensor-core kernel's own order:
 * [ceil(N/128) feature tiles][ceil(K/32) K blocks][32 k][128 n] f32, zero padded, so that every block the
 * kernel streams is one contiguous 16 KB run (whole DRAM pages instead of 512-byte rows 4*N bytes apart).
 * pa_linear_pack_bytes: size of the packed copy; pa_linear_pack_f32: W [K, N] -> d_W_packed.
 * pa_linear_f32_packed: any rows >= 1, any N; K % 4 == 0 and 16-byte aligned d_x (else PA_ERR_UNSUPPORTED);
 * workspace as pa_linear_workspace_bytes(rows, K, N); same arithmetic and bits as pa_linear_f32 on the
 * tensor-core kernel (PA_LINEAR_TC=1). */
size_t pa_linear_pack_bytes(int K, int N);
int pa_linear_pack_f32(const float* d_W, float* d_W_packed, int K, int N, pa_stream_t stream);
int pa_linear_f32_packed(const float* d_x, const float* d_W_packed, const float* d_bias, int rows, int K,
                         int N, int act, float* d_out, void* d_workspace, size_t workspace_bytes,
                         pa_stream_t stream);
/* logits[r,v] = dot(x[r,:], E[v,:]) against the (tied) embedding table E [vocab, hidden]
 * (the reference reads logits out of the hidden state, cuda_decoder.cu:58). */
int pa_logits_f32(const float* d_x, const float* d_E, int rows, int hidden, int vocab,
                  float* d_logits, pa_stream_t stream);
int pa_logits_i8(const float* d_x, const int8_t* d_E, float qscale, int rows, int hidden, int vocab,
                 float* d_logits, pa_stream_t stream);
/* decoder/cuda_decoder.cu:7-14 sample_from_logits (divide=1: argmax logits/T) and
 * decoder/int8_decoder.cpp:97-104 sample_from_int8_logits (divide=0: argmax logits*T);
 * first maximum wins (std::max_element). */
int pa_argmax_f32(const float* d_logits, int rows, int vocab, float temperature, int divide,
                  int32_t* d_out_ids, pa_stream_t stream);
/* pa_logits_* followed by pa_argmax_f32 in ONE pass over the embedding table: the sampler is folded
 * into the logits kernel as an atomicMax on an order-preserving 64-bit key (first maximum wins).
 * d_best: [rows] u64 scratch, zero-initialised once by the caller, reset by every call.
 * elem_bytes 4: d_E f32; elem_bytes 1: d_E int8 dequantised as q / qscale. */
int pa_logits_argmax(const float* d_x, const void* d_E, int elem_bytes, float qscale, int rows, int hidden,
                     int vocab, float temperature, int divide, float* d_logits,
                     unsigned long long* d_best, int32_t* d_out_ids, pa_stream_t stream);
/* LayerNorm (decoder/layer_norm.hpp:20-37) fused with the dynamic row quantisation that follows it in the INT8
 * decoder (compute_minmax_scale + batch_quantize per row, int8_quant.cpp:59-64, 15-28): d_scales[row], d_q [rows,
 * hidden]; d_out_f32 (optional) also receives the normalised f32 rows.  Bit-identical to pa_layer_norm_f32 followed
 * by pa_row_quantize_dynamic_i8. */
int pa_layer_norm_quantize_i8(const float* d_x, const float* d_gamma, const float* d_beta, int rows, int hidden,
                              float eps, float* d_out_f32, float* d_scales, int8_t* d_q, pa_stream_t stream);
/* compute_minmax_scale + batch_quantize of every row of x [rows, dim] in one kernel
 * (attention_cpu/int8_quant.cpp:59-64, 15-28); bit-identical to pa_batch_minmax_scale followed by
 * pa_batch_quantize_i8. */
int pa_row_quantize_dynamic_i8(const float* d_x, int rows, int dim, float* d_scales, int8_t* d_q,
                               pa_stream_t stream);
/* attention/attention_kernel_utils.cuh:20-35 apply_rotary_embedding for whole batches: d_q and/or d_k
 * [rows, num_heads, head_dim] f32 are rotated pairwise in place with the interleaved table
 * d_rope[token * head_dim + d] = cos, [.. + d + 1] = sin at token = d_positions[row] (apply_on_k = d_k
 * given).  Rows whose position is outside [0, T) are left untouched.  Bit-exact (same operation order). */
int pa_apply_rope_f32(float* d_q, float* d_k, const float* d_rope, const int32_t* d_positions, int rows,
                      int num_heads, int head_dim, int T, pa_stream_t stream);
/* positions[r] += 1 (and ctx_lens[r] += 1 when given): advances the decode step on the device. */
int pa_advance_positions(int32_t* d_positions, int32_t* d_ctx_lens, int rows, pa_stream_t stream);

/* ------------------------------------------------ sampling */
/* attention_cpu/softmax_lut.cpp:203-231 softmax_lut_vec over vocabulary logits [rows, vocab]:
 * p = exp((x - max)/temperature) / (sum + 1e-6). */
int pa_softmax_temperature(const float* d_logits, int rows, int vocab, float temperature, float* d_probs,
                           pa_stream_t stream);
/* attention_cpu/softmax_lut.cpp:60-100 fused_softmax_lut_inplace / softmax_batch_parallel over int32
 * logits [rows, n] with the exp table of build_exp_lut (:11-18, d_lut [resolution], max_x = 10):
 * BIT-EXACT (table index by truncation, sum in the reference's sequential order). */
int pa_softmax_lut_i32(const int32_t* d_logits, int rows, int n, float scale, const float* d_lut,
                       int resolution, float* d_probs, pa_stream_t stream);
/* attention_cpu/softmax_lut.cpp:233-256 apply_topk_topp_filter, in place: rank entries by
 * (prob, index) descending (ties: larger index first), zero those with rank >= top_k (top_k > 0)
 * or whose higher-ranked probability mass is >= top_p (top_p < 1), no renormalisation; then the
 * EOS rule (probs[eos] > eos_thresh zeroes everything else).  Replaces the serial thread-0 top-k of
 * attention/top_k_top_p_filter.cuh:55-111 by a radix select. */
int pa_topk_topp_filter(float* d_probs, int rows, int vocab, int top_k, float top_p, int eos_token_id,
                        float eos_thresh, pa_stream_t stream);
/* Inverse-CDF sample in index order: first index whose inclusive prefix sum of d_probs exceeds
 * d_uniform[row] * total (uniform numbers in [0,1) supplied by the caller; the reference calls the
 * host rand() from device code, top_k_top_p_filter.cuh:109). */
int pa_sample_from_probs(const float* d_probs, int rows, int vocab, const float* d_uniform,
                         int32_t* d_out_ids, pa_stream_t stream);

/* ------------------------------------------------ prefill */
/* The multi-query form the reference's headers promise (q/out [B, H, T, D] and `is_prefill`,
 * attention/attention_config.hpp:8-9,17; causal rule attention/attention_kernel_utils.cuh:70-79)
 * but do not implement: query t of row b attends the cached keys [0, ctx_start[b] + t] of
 * table row (d_beam_ids ? d_beam_ids[b] : b).  d_q, d_out: [B, num_heads, Tq, head_dim] f32.
 * d_ctx_start: [B] tokens cached BEFORE this chunk (NULL = 0: plain prefill); the Tq new
 * tokens' K/V must already be appended.  Same softmax semantics as pa_paged_decode_*. */
size_t pa_prefill_workspace_bytes(int B, int Tq, int num_heads, int head_dim, int num_tiles, int tile_size);
int pa_paged_prefill_f16(const float* d_q, float* d_out, const void* d_k_pool, const void* d_v_pool,
                         const int32_t* d_table, int num_beams, int num_heads, int num_tiles,
                         int total_pages, const int32_t* d_beam_ids, const int32_t* d_ctx_start, int B,
                         int Tq, int head_dim, int tile_size, float temperature, void* d_workspace,
                         size_t workspace_bytes, pa_stream_t stream);
int pa_paged_prefill_i8(const float* d_q, float* d_out, const int8_t* d_k_pool, const int8_t* d_v_pool,
                        const float* d_k_scales, const float* d_v_scales, const int32_t* d_table,
                        int num_beams, int num_heads, int num_tiles, int total_pages,
                        const int32_t* d_beam_ids, const int32_t* d_ctx_start, int B, int Tq,
                        int head_dim, int tile_size, float temperature, void* d_workspace,
                        size_t workspace_bytes, pa_stream_t stream);

/* Token-major prefill: d_q, d_out are [B, Tq, num_heads, head_dim] f32 -- the layout the decoders' QKV
 * projection leaves the activations in (CUDADecoder.py:75-80 reshapes [B, n, hidden] into heads), so the
 * caller needs no permute + copy either side of the attention.  The strides are folded into the tcgen05
 * kernel's Q loads and O stores; everything else as pa_paged_prefill_f16/_i8.  No workspace.  Returns
 * PA_ERR_UNSUPPORTED where that kernel does not apply (head_dim other than 64 / 128, pages that are not
 * 16 << k tokens, pools not 128-byte aligned, d_q == d_out): permute and call the [B, H, Tq, D] entry then. */
int pa_paged_prefill_f16_tokmajor(const float* d_q, float* d_out, const void* d_k_pool, const void* d_v_pool,
                                  const int32_t* d_table, int num_beams, int num_heads, int num_tiles,
                                  int total_pages, const int32_t* d_beam_ids, const int32_t* d_ctx_start,
                                  int B, int Tq, int head_dim, int tile_size, float temperature,
                                  pa_stream_t stream);
int pa_paged_prefill_i8_tokmajor(const float* d_q, float* d_out, const int8_t* d_k_pool, const int8_t* d_v_pool,
                                 const float* d_k_scales, const float* d_v_scales, const int32_t* d_table,
                                 int num_beams, int num_heads, int num_tiles, int total_pages,
                                 const int32_t* d_beam_ids, const int32_t* d_ctx_start, int B, int Tq,
                                 int head_dim, int tile_size, float temperature, pa_stream_t stream);

/* --------------------------------- inter-GPU split-KV exchange over peer memory */
/* Exchange buffers: one per rank, pa_splitkv_exchange_bytes(world, rows, head_dim) bytes
 * (uint4 [2 parity][world][rows][head_dim/2 + 1] flag-in-data packets, csrc/xchg.cuh).
 * pa_p2p_alloc: cudaMalloc'd, zero-filled exchange buffer + its 64-byte CUDA IPC handle;
 * pa_p2p_open: map a peer process's buffer (NVLink P2P); pa_p2p_close / pa_p2p_free. */
size_t pa_splitkv_exchange_bytes(int world, int rows, int head_dim);
int pa_p2p_alloc(size_t bytes, void** d_ptr, unsigned char* handle64);
int pa_p2p_open(const unsigned char* handle64, void** d_peer_ptr);
int pa_p2p_close(void* d_peer_ptr);
int pa_p2p_free(void* d_ptr);
/* Decode + row merge + exchange + combine in ONE launch: the streaming kernel over this rank's
 * pages; the warp that finishes the last chunk of a row merges it and stores it into slot `rank`
 * of every peer's exchange buffer (d_peer_bufs: device array [world] of mapped buffer pointers,
 * this rank's own buffer at index `rank`) as 16-byte packets that carry their own epoch flag --
 * sending never blocks; at the end of the same kernel every row's `world` partials are received
 * from the local buffer and LSE-combined into d_out [B, H, D] (identical on every rank).
 * d_epochs [2*B*H] u32: per-row step counters (first half) and self-resetting row-completion counters (second
 * half) in device memory, zero-initialised ONCE by the caller (the launch is CUDA-graph replayable); *d_status is set to 1, the row written as NaN and its epoch NOT advanced if a
 * peer does not arrive within ~2 s.  Exchange buffers must be sized for rows = B*num_heads. */
int pa_paged_decode_f16_splitkv(const float* d_q, float* d_out, const void* d_k_pool,
                                const void* d_v_pool, const int32_t* d_table, int num_beams,
                                int num_heads, int num_tiles, int total_pages,
                                const int32_t* d_beam_ids, const int32_t* d_ctx_lens, int B, int T,
                                int head_dim, int tile_size, float temperature, const float* d_rope,
                                float* d_lse_out, void* d_workspace, size_t workspace_bytes,
                                void* const* d_peer_bufs, int rank, int world, uint32_t* d_epochs,
                                int* d_status, pa_stream_t stream);
int pa_paged_decode_i8_splitkv(const float* d_q, float* d_out, const int8_t* d_k_pool,
                               const int8_t* d_v_pool, const float* d_k_scales, const float* d_v_scales,
                               const int32_t* d_table, int num_beams, int num_heads, int num_tiles,
                               int total_pages, const int32_t* d_beam_ids, const int32_t* d_ctx_lens,
                               int B, int T, int head_dim, int tile_size, float temperature,
                               const float* d_rope, float* d_lse_out, void* d_workspace,
                               size_t workspace_bytes, void* const* d_peer_bufs, int rank, int world,
                               uint32_t* d_epochs, int* d_status, pa_stream_t stream);
/* The same packet exchange as a stand-alone kernel after pa_paged_decode_*_partial: phase 1 sends
 * every row (never blocks), phase 2 receives and combines.  head_dim in {64, 128}, world <= 32. */
int pa_splitkv_exchange_combine(const float* d_part_m, const float* d_part_l, const float* d_part_o,
                                void* const* d_peer_bufs, int rank, int world, int rows,
                                int head_dim, uint32_t* d_epochs, float* d_out, float* d_lse_out,
                                int* d_status, pa_stream_t stream);

/* The two halves of pa_splitkv_exchange_combine on their own: _send stores this rank's rows into every peer's
 * buffer and never waits; _recv polls until every rank's packets of the current step are in this rank's buffer,
 * combines and advances the epochs. */
int pa_splitkv_exchange_send(const float* d_part_m, const float* d_part_l, const float* d_part_o,
                             void* const* d_peer_bufs, int rank, int world, int rows, int head_dim,
                             const uint32_t* d_epochs, pa_stream_t stream);
int pa_splitkv_exchange_recv(void* const* d_peer_bufs, int rank, int world, int rows, int head_dim,
                             uint32_t* d_epochs, float* d_out, float* d_lse_out, int* d_status,
                             pa_stream_t stream);

/* --------------------------------- NCCL form of the exchange (the north star's baseline) */
/* NCCL is loaded at run time (dlopen "libnccl.so.2"); PA_ERR_UNSUPPORTED when it is absent.
 * pa_nccl_unique_id: rank 0 creates the 128-byte ncclUniqueId, the application distributes it;
 * pa_nccl_init: ncclCommInitRank on the current device; pa_nccl_destroy.
 * pa_nccl_allgather_combine: ncclAllGather of this rank's (m [rows], l [rows], O [rows, D]) into
 * d_gather_ws (>= pa_nccl_gather_bytes) in the [n_parts][rows] layout of pa_lse_combine, then the
 * combine kernel, all on `stream`. */
int pa_nccl_unique_id(unsigned char* id128);
int pa_nccl_init(const unsigned char* id128, int rank, int world, void** comm);
int pa_nccl_destroy(void* comm);
size_t pa_nccl_gather_bytes(int world, int rows, int head_dim);
int pa_nccl_allgather_combine(void* comm, int world, const float* d_part_m, const float* d_part_l,
                              const float* d_part_o, int rows, int head_dim, void* d_gather_ws,
                              size_t gather_bytes, float* d_out, float* d_lse_out, pa_stream_t stream);

/* ------------------------------------------------------------------------------------------------------------
 * Ragged-batch sequence ops (no counterpart in the reference: decoder stacks with a float residual stream,
 * per-sequence recurrent state and routed experts).  A step's rows are the concatenated PORTIONS of several
 * sequences (prompt chunks and single decoded tokens).  `elem` is the activation element size: 4 = float,
 * 2 = bfloat16; norms, recurrences, softmax and the residual are float either way.
 * ------------------------------------------------------------------------------------------------------------ */
/* x[r] = table[ids[r]] (table in the activation type) as float; out-of-range ids give zeros. */
int pa_embedding_rows(const void* d_table, int elem, const int32_t* d_ids, int rows, int width, int vocab,
                      float* d_out, pa_stream_t stream);
/* The same rows multiplied by `scale`. */
int pa_embedding_rows_scaled(const void* d_table, int elem, const int32_t* d_ids, int rows, int width, int vocab,
                             float scale, float* d_out, pa_stream_t stream);
/* RMS norm h = x / sqrt(mean(x^2) + eps) * g with g = d_gain_vec[j] (per channel) or the scalar `gain`
 * (d_gain_vec NULL), written to d_out (may be NULL).  With d_shift and d_out_shifted: token shift
 * hs = h + (h' - h) * shift[j], h' = the normalised row d_row_prev[r] of this batch, or, for d_row_prev[r] < 0,
 * the row d_state[d_row_slot[r]] (the previous portion's last h; zeros for a new sequence). */
int pa_rms_norm_shift(const float* d_x, int rows, int width, float eps, float gain, const float* d_gain_vec,
                      const float* d_shift, const int32_t* d_row_prev, const int32_t* d_row_slot,
                      const float* d_state, void* d_out, void* d_out_shifted, int elem, pa_stream_t stream);
/* d_state[slot of portion s] = normalised last row of portion s (call after pa_rms_norm_shift of the same x). */
int pa_rms_norm_state_store(const float* d_x, int width, float eps, float gain, const float* d_gain_vec,
                            const int32_t* d_seq_start, const int32_t* d_seq_len, const int32_t* d_seq_slot,
                            int num_seqs, float* d_state, pa_stream_t stream);
/* minGRU over every portion: rows of d_zxg are [z | u | g] pre-activations (3 * width);
 * z = sigmoid(z + z_bias), c = u + x_bias >= 0 ? . + 1/2 : sigmoid(.), S = (1 - z) S + z c from d_state[slot],
 * y = S * silu(g); d_state[slot] is left at the portion's last S.  _chunked: the same result (up to float
 * rounding) as a three-pass scan over host-listed chunks, for long portions. */
int pa_mingru_scan(const void* d_zxg, const float* d_z_bias, const float* d_x_bias, int width,
                   const int32_t* d_seq_start, const int32_t* d_seq_len, const int32_t* d_seq_slot, int num_seqs,
                   float* d_state, void* d_y, int elem, pa_stream_t stream);
size_t pa_mingru_chunked_workspace_bytes(int num_chunks, int width);
int pa_mingru_scan_chunked(const void* d_zxg, const float* d_z_bias, const float* d_x_bias, int width,
                           const int32_t* d_chunk_start, const int32_t* d_chunk_len, int num_chunks,
                           const int32_t* d_seq_chunk0, const int32_t* d_seq_nchunks, const int32_t* d_seq_slot,
                           int num_seqs, float* d_state, void* d_y, int elem, void* d_workspace,
                           size_t workspace_bytes, pa_stream_t stream);
/* x = gelu_erf(x) in place; out[r, j] = silu(gu[r, j]) * gu[r, ff + j]. */
int pa_gelu_inplace(void* d_x, int64_t n, int elem, pa_stream_t stream);
int pa_silu_mul(const void* d_gate_up, int64_t rows, int ff, void* d_out, int elem, pa_stream_t stream);
/* out[r, j] = act(gu[r, j]) * gu[r, ff + j]; act 0 = silu, 1 = relu, 2 = tanh-form gelu. */
int pa_act_mul(const void* d_gate_up, int64_t rows, int ff, int act, void* d_out, int elem, pa_stream_t stream);
/* x += mult * (mix + dense + sum_k routed[r * top + k] + shared_gate[r] * shared); every term optional. */
int pa_residual_combine(float* d_x, int64_t rows, int width, float mult, const void* d_mix, const void* d_dense,
                        const float* d_routed, int top, const void* d_shared, const float* d_shared_gate,
                        int elem, pa_stream_t stream);
int pa_gather_rows_f32(const float* d_src, const int32_t* d_rows, int n, int width, float* d_dst,
                       pa_stream_t stream);
/* Norm on a sublayer's OUTPUT: s = y (activation type, optional) + sum_k sel_w[r, k] * routed[r * top + k] (float
 * rows of the chosen experts, optional; d_sel_w NULL: weights 1); x[r] += s / sqrt(mean(s^2) + eps) * d_gain[j].
 * d_next (optional): the new x rounded to the activation type, the operand of the next sublayer's products. */
int pa_residual_add_norm(float* d_x, int64_t rows, int width, float eps, const float* d_gain, const void* d_y,
                         const float* d_routed, const float* d_sel_w, int top, void* d_next, int elem,
                         pa_stream_t stream);
/* out[i] = x[i] in the activation type. */
int pa_cast_rows(const float* d_x, int64_t n, void* d_out, int elem, pa_stream_t stream);

/* K/V rows of a projection buffer -> page pools with separate key and value widths (K pages
 * [total_pages][tile_size][k_dim], V pages [..][v_dim]); row r goes to position d_row_pos[r] of table row
 * d_row_slot[r]; the key of kv head g starts at column k_off + g * k_dim of the source row. */
int pa_kv_append_rows(void* d_k_pool, void* d_v_pool, const int32_t* d_table, int num_slots, int num_kv_heads,
                      int num_tiles, int total_pages, int tile_size, int k_dim, int v_dim, const void* d_src,
                      int64_t src_stride, int k_off, int v_off, const int32_t* d_row_slot,
                      const int32_t* d_row_pos, int rows, int elem, pa_stream_t stream);
/* Differential attention (two softmax maps per head over one value tensor, out = headwise_rms(a1 - lambda a2) *
 * out_mult) with a position-dependent query temperature 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1),
 * causal, over the paged pools.  d_q_tiles [num_q_tiles][4] = (first row, tokens, slot, first position): runs of
 * at most pa_diff_attention_tile_tokens(heads, kv_heads) consecutive tokens of one portion.  nsplit > 1 cuts
 * the keys of every tile into that many parts (workspace: pa_diff_attention_workspace_bytes).
 * tile_kind 0: the float tile kernel (any shape, both element types).  tile_kind 1 promises that every tile holds ONE
 * token (decode): those run on a kernel that streams the keys straight from the pools, 8 warps across each tile's
 * context.  tile_kind 2: bfloat16 only, tiles of up to pa_diff_attention_mma_tile_tokens(dim, vdim, elem) tokens
 * (0 = this shape is not served) on the tensor cores, one query head per CTA, nsplit = 1; PA_ERR_UNSUPPORTED if the
 * shape or an alignment (16-byte q rows and pools) rules it out.  tile_kind 3: the same kernel for tiles of ONE token
 * each, the CTA's rows being the query heads of one key/value head (pa_diff_attention_mma_head_rows != 0: bfloat16,
 * a served shape, at most 64 heads per key/value head); nsplit = 1, so it wants a batch of many sequences. */
int pa_diff_attention_tile_tokens(int heads, int kv_heads);
int pa_diff_attention_mma_tile_tokens(int dim, int vdim, int elem);
int pa_diff_attention_mma_head_rows(int heads, int kv_heads, int dim, int vdim, int elem);
size_t pa_diff_attention_workspace_bytes(int num_q_tiles, int heads, int kv_heads, int vdim, int nsplit);
int pa_diff_attention(const void* d_q, int64_t q_stride, int q_off, const void* d_k_pool, const void* d_v_pool,
                      const int32_t* d_table, int num_slots, int num_kv_heads, int num_tiles, int total_pages,
                      int tile_size, const int32_t* d_q_tiles, int num_q_tiles, int heads, int dim, int vdim,
                      float scale, float temp_coef, int temp_every, float lambda, float out_mult, float eps,
                      void* d_out, int elem, int nsplit, int tile_kind, void* d_workspace,
                      size_t workspace_bytes, pa_stream_t stream);

/* Router: float logits h . w_router[e] (+ d_bias[e], optional), score_fn 0 = sigmoid / 1 = softmax over all experts,
 * the `top` largest (ties: lower id), optionally renormalised; score_fn 2: the `top` largest LOGITS, weights = softmax
 * over the chosen logits only.  d_w_shared_gate (optional): shared_gate[r] = sigmoid(h . w). */
int pa_router_topk(const void* d_h, const float* d_w_router, const float* d_bias, const float* d_w_shared_gate,
                   int rows, int width, int experts, int top, int score_fn, int renorm, int32_t* d_sel_id,
                   float* d_sel_w, float* d_shared_gate, int elem, pa_stream_t stream);
/* Group the rows * top (row, choice) pairs by expert: d_order [pairs], d_meta [pa_moe_meta_ints] (offsets and
 * the row tiles of the grouped products: pa_moe_tile_rows() pairs each, or 16 where pairs <= 32 * experts, the
 * regime in which the bfloat16 products stream the weights straight into the MMA fragments). */
int pa_moe_tile_rows(void);
int pa_moe_max_tiles(int pairs, int experts);
size_t pa_moe_meta_ints(int pairs, int experts);
int pa_moe_sort(const int32_t* d_sel_id, int pairs, int experts, int32_t* d_order, int32_t* d_meta,
                pa_stream_t stream);
/* act[i] = silu(W_gate[e] a) * (W_up[e] a), a = h[row(i)] * sel_w (input scaling; d_sel_w NULL: none), weights
 * [experts][2 * ff][width] (gate rows, then up rows); sorted pair order. */
int pa_moe_gate_up(const void* d_h, int64_t ldh, const void* d_w_gate_up, int width, int ff, int experts,
                   const int32_t* d_order, const float* d_sel_w, int top, const int32_t* d_meta, int pairs,
                   void* d_act, int elem, pa_stream_t stream);
/* pa_moe_gate_up with the gate's activation chosen: 0 = silu, 1 = relu, 2 = relu squared. */
int pa_moe_gate_up_act(const void* d_h, int64_t ldh, const void* d_w_gate_up, int width, int ff, int experts,
                       const int32_t* d_order, const float* d_sel_w, int top, const int32_t* d_meta, int pairs,
                       int act, void* d_act, int elem, pa_stream_t stream);
/* Experts without a gate: act[i] = act(W_up[e] a), weights [experts][ff][width]; same a, order and act codes. */
int pa_moe_up(const void* d_h, int64_t ldh, const void* d_w_up, int width, int ff, int experts,
              const int32_t* d_order, const float* d_sel_w, int top, const int32_t* d_meta, int pairs, int act,
              void* d_act, int elem, pa_stream_t stream);
/* out_pairs[row * top + choice] = W_down[e] act[i] as float, weights [experts][width][ff]. */
int pa_moe_down(const void* d_act, const void* d_w_down, int ff, int width, int experts, const int32_t* d_order,
                const int32_t* d_meta, int pairs, float* d_out_pairs, int elem, pa_stream_t stream);


/* ---- attention through a low-rank latent (latent_attention.cu) --------------------------------------------------
 * The pool keeps ONE row [c (kv_rank) | kr (rot_dim)] per token for all heads (a KVTileCache with one key/value head
 * and no value pool); keys and values of head h are Wuk_h c and Wuv_h c and are never materialised: the queries are
 * mapped into the latent (ql_h = Wuk_h^T qp_h, pa_head_linear) and the weighted sums of c are mapped out (Wuv_h).
 *
 * pa_rope_table: d_table [rows][dims / 2][cos, sin] of the angles d_row_pos[r] * base^(-2i / dims).
 * pa_rope_rows: rotates, in place, the interleaved pairs (2i, 2i + 1), i < dims / 2, that start at column
 *   off + h * head_stride of every row, h < heads.
 * pa_latent_kv_append: source row r holds [c_raw (kv_rank) | kr_raw (rot_dim)] from column c_off; the pool row at
 *   position d_row_pos[r] of table row d_row_slot[r] becomes [c_raw / rms(c_raw) * d_gain | kr_raw with its first
 *   rot_dims entries rotated].
 * pa_rms_norm_rows: dst[r, :width] = src[r, off : off + width] / rms * d_gain (rows in the activation type).
 * pa_head_linear: out[r, h, :N] = x[r, h, :K] . W[h] with W [heads][K][N]; x and out addressed by row and head strides.
 * pa_head_gate: out[r, h * vdim + v] = in[r, h, v] * sigmoid(gate[r * gate_row_stride + h]).
 * pa_latent_attention: causal softmax attention of `heads` query rows per token, [ql_h | qr_h] . [c_j | kr_j] * scale,
 *   out[r, h, :kv_rank] = sum_j p_j c_j.  d_q_tiles [num_q_tiles][4] = (first row, tokens, slot, first position): runs of
 *   at most pa_latent_attention_tile_tokens(heads) consecutive tokens of one portion (tile_kind 0: the float tile
 *   kernel, any shape, both element types; nsplit > 1 cuts the keys of every tile into that many parts, workspace
 *   pa_latent_attention_workspace_bytes) or of at most pa_latent_attention_mma_tile_tokens(...) tokens (tile_kind 2:
 *   bfloat16 on the tensor cores; 0 = this shape is not served; PA_ERR_UNSUPPORTED where a shape or an alignment rules
 *   it out).  tile_kind 3: tile_kind 2 with the promise that every tile holds ONE token (decoded tokens): with at most 16
 *   heads the warps of the tensor-core kernel then split the keys of a step instead of the rows. */
int pa_rope_table(const int32_t* d_row_pos, int rows, int dims, float base, float* d_table, pa_stream_t stream);
int pa_rope_rows(void* d_x, int64_t stride, int off, int head_stride, int heads, int dims, const float* d_table,
                 int rows, int elem, pa_stream_t stream);
int pa_latent_kv_append(void* d_pool, const int32_t* d_table, int num_slots, int num_tiles, int total_pages,
                        int tile_size, int kv_rank, int rot_dim, int rot_dims, const void* d_src, int64_t src_stride,
                        int c_off, const float* d_gain, float eps, const float* d_rope_table,
                        const int32_t* d_row_slot, const int32_t* d_row_pos, int rows, int elem, pa_stream_t stream);
int pa_rms_norm_rows(const void* d_src, int64_t src_stride, int off, int width, float eps, const float* d_gain,
                     void* d_dst, int64_t dst_stride, int rows, int elem, pa_stream_t stream);
int pa_head_linear(const void* d_x, int64_t x_row_stride, int64_t x_head_stride, const void* d_W, int heads, int K,
                   int N, int rows, void* d_out, int64_t o_row_stride, int64_t o_head_stride, int elem,
                   pa_stream_t stream);
int pa_head_gate(const void* d_in, int64_t in_row_stride, int64_t in_head_stride, const void* d_gate,
                 int64_t gate_row_stride, int heads, int vdim, int64_t rows, void* d_out, int elem, pa_stream_t stream);
int pa_latent_attention_tile_tokens(int heads);
int pa_latent_attention_mma_tile_tokens(int heads, int kv_rank, int rot_dim, int elem);
size_t pa_latent_attention_workspace_bytes(int num_q_tiles, int heads, int kv_rank, int nsplit);
int pa_latent_attention(const void* d_q_lat, int64_t ql_row_stride, int64_t ql_head_stride, const void* d_q_rot,
                        int64_t qr_row_stride, int64_t qr_head_stride, const void* d_pool, const int32_t* d_table,
                        int num_slots, int num_tiles, int total_pages, int tile_size, const int32_t* d_q_tiles,
                        int num_q_tiles, int heads, int kv_rank, int rot_dim, float scale, void* d_out,
                        int64_t o_row_stride, int64_t o_head_stride, int elem, int nsplit, int tile_kind,
                        void* d_workspace, size_t workspace_bytes, pa_stream_t stream);

/* ---- pre-norm wiring, looped blocks (seq_ops.cu) ---------------------------------------------------------------------
 * pa_residual_add_prenorm: x[r] += y_scale * y + y2_scale * y2 + sum_k sel_w[r, k] * routed[(r, k)] + shared + bias
 *   (every addend optional; y, y2, shared in the activation type, routed float pairs, bias one float row), then, when
 *   d_next is given, next[r] = x[r] / sqrt(mean(x[r]^2) + eps) * d_gain in the activation type.
 * pa_concat_rows: out[r] = [a[r] | b[r]] (two float row sets of equal width) in the activation type.
 * pa_router_topk_grouped: pa_router_topk where the experts form `ngroups` equal groups of neighbours and only experts
 *   of the `keep` groups with the largest maxima can be chosen. */
int pa_residual_add_prenorm(float* d_x, int64_t rows, int width, const void* d_y, float y_scale, const void* d_y2,
                            float y2_scale, const float* d_routed, const float* d_sel_w, int top, const void* d_shared,
                            const float* d_bias, float eps, const float* d_gain, void* d_next, int elem,
                            pa_stream_t stream);
int pa_concat_rows(const float* d_a, const float* d_b, int64_t rows, int width, void* d_out, int elem,
                   pa_stream_t stream);
int pa_router_topk_grouped(const void* d_h, const float* d_w_router, const float* d_bias, const float* d_w_shared_gate,
                           int rows, int width, int experts, int top, int score_fn, int renorm, int ngroups, int keep,
                           int32_t* d_sel_id, float* d_sel_w, float* d_shared_gate, int elem, pa_stream_t stream);

/* ---- softmax attention with score modifiers and visibility rules (masked_attention.cu) ------------------------------
 * Grouped key/value heads over the pools pa_kv_append_rows fills (key rows of `dim`, value rows of `vdim`), no rotation.
 * score = (q . k) * scale; softcap > 0: softcap * tanh(score / softcap); bias_kind 1: - d_bias[h] * (i - j);
 * bias_kind 2: + d_bias[min(i - j, bias_len - 1) * heads + h].  mask_kind 0: causal; 1: 0 <= i - j < mask_size;
 * 2: j <= i in the same block of mask_size positions (blocks counted from position 0 of the sequence).
 * d_q_tiles as for pa_diff_attention: runs of at most pa_masked_attention_tile_tokens(heads, kv_heads) tokens
 * (tile_kind 0 or 1: the float kernels, any shape, both element types), or of at most
 * pa_masked_attention_mma_tile_tokens(dim, vdim, elem) tokens (tile_kind 2: bfloat16 on the tensor cores; 0 = not
 * served; PA_ERR_UNSUPPORTED where a stride or an alignment rules it out). */
int pa_masked_attention_tile_tokens(int heads, int kv_heads);
int pa_masked_attention_mma_tile_tokens(int dim, int vdim, int elem);
int pa_masked_attention(const void* d_q, int64_t q_stride, int q_off, const void* d_k_pool, const void* d_v_pool,
                        const int32_t* d_table, int num_slots, int num_kv_heads, int num_tiles, int total_pages,
                        int tile_size, const int32_t* d_q_tiles, int num_q_tiles, int heads, int dim, int vdim,
                        float scale, float softcap, int mask_kind, int mask_size, int bias_kind, const float* d_bias,
                        int bias_len, void* d_out, int elem, int tile_kind, pa_stream_t stream);
/* pa_masked_attention with a temperature per head, a sink and turned values: score *= d_head_scale[h] right after the
 * scale (NULL: none); mask_kind 1 with mask_keep > 0 also keeps the first mask_keep positions of the sequence visible;
 * d_sink [heads] (NULL: none): exp(d_sink[h]) joins head h's softmax denominator (no key, no value; zeros add one to the
 * denominator); d_out_rot [rows][vdim / 2][cos, sin] (NULL: none; a pa_rope_table over vdim): the neighbouring pairs of
 * every head's output are turned back by the row's angle, in float, before the result is rounded. */
/* pa_rope_kv_append: the rotation of one step's q | k | v rows and their append in one launch.  Query head h (columns
 * q_off + h * dim of the row) is rotated in place over its first rot_dims dimensions (neighbouring pairs, d_rope
 * [rows][rot_dims / 2][cos, sin]); with pools given, the key of kv head g (k_off + g * dim) goes to the row's place in
 * the pool rotated the same way and its value (v_off + g * vdim) turned over all of vdim by d_value_rope
 * [rows][vdim / 2][cos, sin] (NULL: as it is).  d_k_pool NULL: a layer that reads another layer's pool. */
int pa_rope_kv_append(void* d_src, int64_t src_stride, int q_off, int k_off, int v_off, int heads, int kv_heads, int dim,
                      int vdim, int rot_dims, const float* d_rope, const float* d_value_rope, void* d_k_pool,
                      void* d_v_pool, const int32_t* d_table, int num_slots, int num_tiles, int total_pages, int tile_size,
                      const int32_t* d_row_slot, const int32_t* d_row_pos, int rows, int elem, pa_stream_t stream);
int pa_masked_attention_sink(const void* d_q, int64_t q_stride, int q_off, const void* d_k_pool, const void* d_v_pool,
                             const int32_t* d_table, int num_slots, int num_kv_heads, int num_tiles, int total_pages,
                             int tile_size, const int32_t* d_q_tiles, int num_q_tiles, int heads, int dim, int vdim,
                             float scale, float softcap, int mask_kind, int mask_size, int mask_keep, int bias_kind,
                             const float* d_bias, int bias_len, const float* d_head_scale, const float* d_sink,
                             const float* d_out_rot, void* d_out, int elem, int tile_kind, pa_stream_t stream);

/* ---- the parallel wiring with two norms, polynomial activation, capped logits, biased choice (seq_ops.cu, moe_ops.cu)
 * pa_residual_add_norm2: x[r] += y + y2 + sum_k sel_w[r, k] * e_k (every addend optional; y, y2 in the activation
 *   type); e_k is the float row routed[(r, k)], or, where d_sel_id is given and sel_id[r, k] >= experts, the row
 *   d_ident[r] (activation type: an identity expert returns the feed-forward's input).  Then next1[r] = x[r] / rms(x[r])
 *   * d_gain1 and next2[r] = x[r] / rms(x[r]) * d_gain2 (each optional) in the activation type.
 * pa_poly_norm: out[r] = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3 over rows of `ff` values, powers element by element,
 *   N(u) = u / sqrt(mean(u^2) + eps); d_coef: four floats on the device.
 * pa_logit_softcap: z <- cap * tanh(scale * z / cap) in place (cap 0: only the scale).
 * pa_router_topk_biased: pa_router_topk_grouped with d_choice_bias [experts] (NULL: none) added to the scores for the
 *   choice only; renorm divides the chosen scores by their sum + 1e-20.
 * pa_causal_conv: pa_causal_conv_silu with the activation chosen (0: none, 1: silu) and an optional bias. */
int pa_residual_add_norm2(float* d_x, int64_t rows, int width, const void* d_y, const void* d_y2, const float* d_routed,
                          const float* d_sel_w, const int32_t* d_sel_id, int top, int experts, const void* d_ident,
                          float eps, const float* d_gain1, void* d_next1, const float* d_gain2, void* d_next2, int elem,
                          pa_stream_t stream);
int pa_poly_norm(const void* d_z, int64_t rows, int ff, const float* d_coef, float eps, void* d_out, int elem,
                 pa_stream_t stream);
int pa_logit_softcap(float* d_logits, int64_t n, float scale, float cap, pa_stream_t stream);
int pa_router_topk_biased(const void* d_h, const float* d_w_router, const float* d_bias, const float* d_w_shared_gate,
                          int rows, int width, int experts, int top, int score_fn, int renorm, int ngroups, int keep,
                          const float* d_choice_bias, int32_t* d_sel_id, float* d_sel_w, float* d_shared_gate, int elem,
                          pa_stream_t stream);
int pa_causal_conv(const void* d_in, int64_t in_stride, int in_off, int channels, int taps, const float* d_weight,
                   const float* d_bias, int act, const float* d_state, const int32_t* d_chunks, int num_chunks, void* d_out,
                   int64_t out_stride, int elem, pa_stream_t stream);

/* ---- matrix-state recurrences (recurrence_ops.cu) --------------------------------------------------------------------
 * pa_causal_conv_silu: out[r, c] = silu(bias[c] + sum_i w[c, i] * in(t - (taps - 1 - i))[c]) over the tokens of a
 *   sequence (weights [channels][taps], taps <= 8); inputs before a portion's first token come from the state slot
 *   [slots][taps - 1][channels] (float).  d_chunks [num_chunks][4] = (first row, tokens, slot, offset of the first token
 *   within its portion).  pa_conv_state_update then leaves the portion's last taps - 1 inputs in the slot.
 * pa_decay_scan: per head S_t = a_t S_{t-1} + k_t (s_t v_t)^T, o_t = S_t^T q_t + skip[h] * v_t, S [dim][vdim] float in
 *   d_state [slots][heads][dim][vdim].  q / k of head h are read at off + (h / (heads / groups)) * dim, v at
 *   off + h * vdim; act 1: q, k, v pass silu.  d_dt == NULL: a_t = d_decay[h], s_t = 1.  Else dt = softplus(raw + d_dt_bias[h])
 *   (raw at dt_off + h), a_t = exp(-exp(d_a_log[h]) * dt), s_t = dt.  d_out: float rows [heads * vdim].
 *   chunked 0: d_items [num_items][4] = one item per portion (first row, tokens, slot, -), walked in order from / to the
 *   slot.  chunked 1: items are chunks of portions in portion order, d_seq_chunk0 / d_seq_nchunks / d_seq_slot describe
 *   the portions; three passes (fold, chain, replay) with pa_decay_scan_workspace_bytes(num_items, ...) of workspace.
 * pa_gated_rms_norm: out[r] = RMS norm of the float row y[r] in `groups` equal parts (each by its own mean square)
 *   times d_weight; gate_mode 1: y is first multiplied by silu(gate); gate_mode 2: the result by sigmoid(gate). */
int pa_causal_conv_silu(const void* d_in, int64_t in_stride, int in_off, int channels, int taps, const float* d_weight,
                        const float* d_bias, const float* d_state, const int32_t* d_chunks, int num_chunks, void* d_out,
                        int64_t out_stride, int elem, pa_stream_t stream);
int pa_conv_state_update(const void* d_in, int64_t in_stride, int in_off, int channels, int taps,
                         const int32_t* d_seq_start, const int32_t* d_seq_len, const int32_t* d_seq_slot, int num_seqs,
                         float* d_state, int elem, pa_stream_t stream);
size_t pa_decay_scan_workspace_bytes(int num_chunks, int heads, int dim, int vdim);
int pa_decay_scan(const void* d_q, int64_t q_stride, int q_off, const void* d_k, int64_t k_stride, int k_off,
                  const void* d_v, int64_t v_stride, int v_off, int heads, int groups, int dim, int vdim, int act,
                  const float* d_decay, const void* d_dt, int64_t dt_stride, int dt_off, const float* d_dt_bias,
                  const float* d_a_log, const float* d_skip, float* d_state, float* d_out, int64_t out_stride,
                  const int32_t* d_items, int num_items, const int32_t* d_seq_chunk0, const int32_t* d_seq_nchunks,
                  const int32_t* d_seq_slot, int num_seqs, int chunked, void* d_workspace, size_t workspace_bytes,
                  int elem, pa_stream_t stream);
int pa_gated_rms_norm(const float* d_y, int64_t rows, int inner, int groups, const void* d_gate, int64_t gate_stride,
                      int gate_off, int gate_mode, const float* d_weight, float eps, void* d_out, int elem,
                      pa_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* PA_B200_H_ */
