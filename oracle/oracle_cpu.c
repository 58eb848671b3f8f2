/*
 * oracle_cpu.c -- TEST INFRASTRUCTURE ONLY.
 *
 * CPU restatement of the reference's decode hot path (paged attention over the
 * tiled KV cache, page-table gather/append addressing, INT8 quantise /
 * dequantise, LUT softmax family, s8 x s8 -> s32 matmul with the oneDNN-style
 * epilogue).  Every function cites the reference file:line it follows
 * (paths relative to the reference tree).
 *
 * Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline /
 * --impl reference legs may load this.  The product path (libpa_b200.so) never
 * links or calls it.
 *
 * Parity pinning: the int8_quant, softmax_lut and KVTileCacheCPU restatements
 * are pinned bit-for-bit against the reference's own objects (oracle/_ref,
 * built from the unmodified reference sources) in tests/test_oracle_pinning.py
 * and against hand-computed known answers.  The attention restatement
 * follows cpu_attention_kernel.cpp, which does not compile as shipped;
 * its softmax / filter stages are pinned against the
 * reference objects, its loop structure is a line-by-line restatement.
 * The oneDNN epilogue is "parity unpinned" (third-party, un-vendored,
 * un-pinned oneDNN < 3.0): only the int32 accumulators are a
 * bit-exact target.
 *
 * Build: gcc -O2 -fopenmp -ffp-contract=off -fno-fast-math (see oracle/Makefile).
 * -ffp-contract=off matters: the reference is built without FMA contraction
 * flags (CMakeLists.txt:4-9 sets no -march), so products and sums round
 * separately.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ */
/* Page table + page pool addressing                                   */
/* ------------------------------------------------------------------ */

/* kv_cache/page_table.hpp:39-42  PageTable::index */
ORC_API int orc_pt_index(int beam, int head, int tile, int num_heads, int num_tiles) {
    return beam * (num_heads * num_tiles) + head * num_tiles + tile;
}

/* kv_cache/page_table.hpp:44-49  PageTable::lookup (device) */
ORC_API int orc_pt_lookup(const int32_t* table, int total_entries, int beam, int head,
                          int tile, int num_heads, int num_tiles) {
    int idx = orc_pt_index(beam, head, tile, num_heads, num_tiles);
    if (idx < 0 || idx >= total_entries) return -1;
    return table[idx];
}

/* kv_cache/kv_tile_cache.hpp:21-26  KVTileCache<T>::get address math.
 * Returns the ELEMENT offset of the page start in the K (or V) pool, or -1
 * for "nullptr".  64-bit offset. */
ORC_API int64_t orc_kv_page_offset(const int32_t* table, int total_entries, int beam,
                                   int head, int tile, int num_heads, int num_tiles,
                                   int total_pages, int tile_size, int head_dim) {
    int page = orc_pt_lookup(table, total_entries, beam, head, tile, num_heads, num_tiles);
    if (page < 0 || page >= total_pages) return -1;
    return (int64_t)page * tile_size * head_dim;
}

/* Page gather: copy every mapped page of (beam,head) rows into a dense
 * [R, H, num_tiles*tile_size, D] buffer of elem_bytes-sized elements; unmapped
 * pages are filled with `fill` bytes.  Addressing per kv_tile_cache.hpp:21-26. */
ORC_API void orc_gather_pages(const uint8_t* pool, uint8_t* dense, const int32_t* table,
                              int num_beams, int num_heads, int num_tiles, int total_pages,
                              int tile_size, int head_dim, int elem_bytes,
                              const int32_t* beam_ids, int R, uint8_t fill) {
    const int total_entries = num_beams * num_heads * num_tiles;
    const size_t page_bytes = (size_t)tile_size * head_dim * elem_bytes;
    for (int r = 0; r < R; ++r) {
        int beam = beam_ids ? beam_ids[r] : r;
        for (int h = 0; h < num_heads; ++h)
            for (int t = 0; t < num_tiles; ++t) {
                int64_t off = orc_kv_page_offset(table, total_entries, beam, h, t, num_heads,
                                                 num_tiles, total_pages, tile_size, head_dim);
                uint8_t* dst = dense + (((size_t)r * num_heads + h) * num_tiles + t) * page_bytes;
                if (off < 0) memset(dst, fill, page_bytes);
                else memcpy(dst, pool + (size_t)off * elem_bytes, page_bytes);
            }
    }
}

/* KV append: the reference has no append; the storage layout and
 * get_write_ptr (kv_tile_cache.hpp:29-34) define it: the row of token `pos`
 * lives at page(beam,head,pos/tile_size) + (pos % tile_size)*head_dim.
 * new_k/new_v: [R, H, D] elements of elem_bytes.  Rows whose page is unmapped
 * are skipped (get_write_ptr returns nullptr). */
ORC_API void orc_kv_append(uint8_t* k_pool, uint8_t* v_pool, const int32_t* table,
                           int num_beams, int num_heads, int num_tiles, int total_pages,
                           int tile_size, int head_dim, int elem_bytes,
                           const uint8_t* new_k, const uint8_t* new_v,
                           const int32_t* beam_ids, const int32_t* positions, int R) {
    const int total_entries = num_beams * num_heads * num_tiles;
    const size_t row_bytes = (size_t)head_dim * elem_bytes;
    for (int r = 0; r < R; ++r) {
        int beam = beam_ids ? beam_ids[r] : r;
        int pos = positions[r];
        /* deliberate deviation: a position past the table's capacity, or a beam outside
         * it, writes nothing; the reference's flat-index bound (page_table.hpp:44-49) would alias into another
         * head's / beam's entry and overwrite its page. */
        if (pos < 0 || pos / tile_size >= num_tiles || beam < 0 || beam >= num_beams) continue;
        for (int h = 0; h < num_heads; ++h) {
            int64_t off = orc_kv_page_offset(table, total_entries, beam, h, pos / tile_size,
                                             num_heads, num_tiles, total_pages, tile_size, head_dim);
            if (off < 0) continue;
            size_t dst = (size_t)off * elem_bytes + (size_t)(pos % tile_size) * row_bytes;
            size_t src = ((size_t)r * num_heads + h) * row_bytes;
            memcpy(k_pool + dst, new_k + src, row_bytes);
            memcpy(v_pool + dst, new_v + src, row_bytes);
        }
    }
}

/* ------------------------------------------------------------------ */
/* int8_quant (attention_cpu/int8_quant.cpp)                            */
/* ------------------------------------------------------------------ */

static inline int8_t orc_q1(float x, float scale) {
    /* int8_quant.cpp:8-10: static_cast<int32_t>(std::round(x*scale)), clamp.
     * std::round = half away from zero = roundf.  The float->int32 cast of an
     * out-of-range value is UB in C++; on x86 it yields INT_MIN, which the
     * clamp maps to -128.  We clamp in float first for +big to stay defined and
     * mirror the x86 result only where it is defined: callers in tests keep
     * |x*scale| < 2^31. */
    float r = roundf(x * scale);
    int32_t q;
    if (r >= 2147483648.0f || r < -2147483648.0f || r != r) q = INT32_MIN;
    else q = (int32_t)r;
    if (q > 127) q = 127;
    if (q < -128) q = -128;
    return (int8_t)q;
}

/* int8_quant.cpp:5-13 */
ORC_API void orc_quantize_to_int8(const float* x, int64_t n, float scale, int8_t* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = orc_q1(x[i], scale);
}

/* int8_quant.cpp:15-28 */
ORC_API void orc_batch_quantize(const float* x, const float* scales, int rows, int dim,
                                int8_t* out) {
    for (int b = 0; b < rows; ++b) {
        float s = scales[b];
        for (int i = 0; i < dim; ++i) {
            int64_t idx = (int64_t)b * dim + i;
            out[idx] = orc_q1(x[idx], s);
        }
    }
}

/* int8_quant.cpp:30-36 */
ORC_API float orc_compute_absmax(const float* x, int64_t n) {
    float m = 0.f;
    for (int64_t i = 0; i < n; ++i) {
        float a = fabsf(x[i]);
        m = (m < a) ? a : m; /* std::max(max_val, abs(v)): returns a only if m < a */
    }
    return m;
}

/* int8_quant.cpp:38-44 */
ORC_API void orc_dequantize_from_int8(const int8_t* q, int64_t n, float scale, float* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = (float)q[i] / scale;
}

/* int8_quant.cpp:46-57 */
ORC_API void orc_batch_dequantize(const int8_t* q, const float* scales, int rows, int dim,
                                  float* out) {
    for (int b = 0; b < rows; ++b) {
        float s = scales[b];
        for (int i = 0; i < dim; ++i) {
            int64_t idx = (int64_t)b * dim + i;
            out[idx] = (float)q[idx] / s;
        }
    }
}

/* int8_quant.cpp:59-64 */
ORC_API float orc_compute_minmax_scale(const float* x, int64_t n) {
    float mn = x[0], mx = x[0];
    for (int64_t i = 1; i < n; ++i) {
        if (x[i] < mn) mn = x[i];
        if (mx < x[i]) mx = x[i];
    }
    float a = fabsf(mn), b = fabsf(mx);
    float am = (a < b) ? b : a;
    return 127.f / (am + 1e-6f);
}

/* Row-wise minmax scale: one scale per row of `dim` (the per-(token,head)
 * granularity used for the INT8 KV cache). */
ORC_API void orc_batch_minmax_scale(const float* x, int rows, int dim, float* scales) {
    for (int b = 0; b < rows; ++b) scales[b] = orc_compute_minmax_scale(x + (int64_t)b * dim, dim);
}

/* ------------------------------------------------------------------ */
/* softmax_lut family (attention_cpu/softmax_lut.cpp)                   */
/* ------------------------------------------------------------------ */

/* softmax_lut.cpp:11-18.  `2 * max_x * i` is float*int -> float, then
 * / (resolution-1) int->float. */
ORC_API void orc_build_exp_lut(int resolution, float max_x, float* lut) {
    for (int i = 0; i < resolution; ++i) {
        float x = -max_x + 2 * max_x * i / (resolution - 1);
        lut[i] = expf(x);
    }
}

/* softmax_lut.cpp:60-82 fused_softmax_lut_inplace (scalar form; the Vec form
 * at :21-57 is bit-identical only in exp values -- its sum is chunked by 8,
 * see orc_softmax_lut). */
ORC_API void orc_fused_softmax_lut(const int32_t* logits, int64_t n, float scale,
                                   const float* lut, int resolution, float* out) {
    const float max_x = 10.0f;
    int32_t max_val = logits[0];
    for (int64_t i = 1; i < n; ++i)
        if (logits[i] > max_val) max_val = logits[i];
    float inv_range = (resolution - 1) / (2 * max_x);
    float sum = 0.0f;
    for (int64_t i = 0; i < n; ++i) {
        /* static_cast<float>(logits[i]) - max_val : float - int32 -> float */
        float x = ((float)logits[i] - (float)max_val) * scale;
        x = fmaxf(-max_x, fminf(max_x, x));
        int idx = (int)((x + max_x) * inv_range);
        out[i] = lut[idx];
        sum += out[i];
    }
    float inv = 1.0f / (sum + 1e-6f);
    for (int64_t i = 0; i < n; ++i) out[i] *= inv;
}

/* softmax_lut.cpp:21-57 softmax_lut (8-wide Vec form: sum accumulated as
 * per-chunk partial sums).  n must be a multiple of 8 (the reference overruns
 * otherwise). */
ORC_API void orc_softmax_lut(const int32_t* logits, int64_t n, float scale, const float* lut,
                             int resolution, float* out) {
    const float max_x = 10.0f;
    const float inv_range = (resolution - 1) / (2 * max_x);
    int32_t max_val = logits[0];
    for (int64_t i = 1; i < n; ++i)
        if (logits[i] > max_val) max_val = logits[i];
    for (int64_t i = 0; i < n; ++i) {
        float x = ((float)logits[i] - (float)max_val) * scale;
        x = fmaxf(-max_x, fminf(max_x, x));
        int idx = (int)((x + max_x) * inv_range);
        out[i] = lut[idx];
    }
    float sum = 0.0f;
    for (int64_t i = 0; i < n; i += 8) {
        float s = 0.f;
        for (int j = 0; j < 8 && i + j < n; ++j) s += out[i + j];
        sum += s;
    }
    float inv = 1.0f / (sum + 1e-6f);
    for (int64_t i = 0; i < n; ++i) out[i] = out[i] * inv;
}

/* softmax_lut.cpp:85-100 softmax_batch_parallel (OpenMP over rows) */
ORC_API void orc_softmax_batch_parallel(const int32_t* logits, int rows, int64_t n, float scale,
                                        const float* lut, int resolution, float* out) {
#pragma omp parallel for
    for (int r = 0; r < rows; ++r)
        orc_fused_softmax_lut(logits + (int64_t)r * n, n, scale, lut, resolution,
                              out + (int64_t)r * n);
}

/* softmax_lut.cpp:203-231 softmax_lut_vec: ignores the LUT; exact expf;
 * max init -1e9; (x-max)/temperature; chunked-by-8 sum; *inv.
 * len must be a multiple of 8 for the reference; we allow a ragged tail and
 * treat it as the reference would a zero-padded chunk EXCEPT that padded
 * lanes are not summed (the reference would read past the end). */
ORC_API void orc_softmax_lut_vec(const float* scores, int len, float temperature, float* out) {
    float maxval = -1e9f;
    for (int i = 0; i < len; ++i) maxval = (maxval < scores[i]) ? scores[i] : maxval;
    float sum = 0.0f;
    for (int i = 0; i < len; i += 8) {
        float s = 0.f;
        for (int j = 0; j < 8 && i + j < len; ++j) {
            float x = (scores[i + j] - maxval) / temperature;
            x = expf(x);
            out[i + j] = x;
            s += x;
        }
        sum += s;
    }
    float inv = 1.0f / (sum + 1e-6f);
    for (int i = 0; i < len; ++i) out[i] = out[i] * inv;
}

/* softmax_lut.cpp:162-201 softmax_lut_tile without the memo cache (the cache
 * only short-circuits repeated inputs; values are the exact softmax). */
ORC_API void orc_softmax_tile(const float* scores, int len, float temperature, float* out) {
    float maxval = -1e9f;
    for (int i = 0; i < len; ++i) maxval = (maxval < scores[i]) ? scores[i] : maxval;
    float sum = 0.0f;
    for (int i = 0; i < len; ++i) {
        out[i] = expf((scores[i] - maxval) / temperature);
        sum += out[i];
    }
    for (int i = 0; i < len; ++i) out[i] = out[i] / (sum + 1e-6f);
}

typedef struct { float p; int i; } orc_pi;
static int orc_pi_desc(const void* a, const void* b) {
    /* std::sort(..., std::greater<>()) on pair<float,int>: descending by p,
     * ties by descending index. */
    const orc_pi* x = (const orc_pi*)a; const orc_pi* y = (const orc_pi*)b;
    if (x->p > y->p) return -1;
    if (x->p < y->p) return 1;
    if (x->i > y->i) return -1;
    if (x->i < y->i) return 1;
    return 0;
}

/* softmax_lut.cpp:233-256 apply_topk_topp_filter: rank-based zeroing, no
 * renormalisation, EOS hard threshold. */
ORC_API void orc_apply_topk_topp_filter(float* probs, int len, int top_k, float top_p,
                                        int eos_token_id, float eos_thresh) {
    orc_pi* sorted = (orc_pi*)malloc(sizeof(orc_pi) * (size_t)(len > 0 ? len : 1));
    for (int i = 0; i < len; ++i) { sorted[i].p = probs[i]; sorted[i].i = i; }
    qsort(sorted, (size_t)len, sizeof(orc_pi), orc_pi_desc);
    float cum = 0.0f;
    for (int i = 0; i < len; ++i) {
        int idx = sorted[i].i;
        if ((top_k > 0 && i >= top_k) || (top_p < 1.0f && cum >= top_p)) probs[idx] = 0.0f;
        cum += sorted[i].p;
    }
    if (eos_token_id >= 0 && eos_token_id < len && probs[eos_token_id] > eos_thresh)
        for (int i = 0; i < len; ++i)
            if (i != eos_token_id) probs[i] = 0.0f;
    free(sorted);
}

/* ------------------------------------------------------------------ */
/* Paged decode attention (attention_cpu/cpu_attention_kernel.cpp:36-129) */
/* ------------------------------------------------------------------ */

/* cpu_attention_kernel.cpp:13-19 pairwise RoPE on q, rope[d]=cos, rope[d+1]=sin,
 * no position offset. */
static void orc_rope_q(float* q, const float* rope, int D) {
    for (int d = 0; d + 1 < D; d += 2) {
        float c = rope[d], s = rope[d + 1];
        float q0 = q[d], q1 = q[d + 1];
        q[d] = q0 * c - q1 * s;
        q[d + 1] = q0 * s + q1 * c;
    }
}

/* Generic element fetch: kv_kind 0 = float32 pool, 1 = int8 pool with per
 * (page, token) f32 scales (dequant per int8_quant.cpp:46-57: q / scale),
 * 2 = int8 pool raw cast (the literal CPUAttention<int8_t> path: Vec load
 * "will decode if int8_t", cpu_attention_kernel.cpp:51-53,80). */
static inline void orc_load_row(float* dst, const void* pool, const float* scales, int kv_kind,
                                int64_t page_off, int page, int tile_size, int t, int D) {
    if (kv_kind == 0) {
        memcpy(dst, (const float*)pool + page_off + (int64_t)t * D, sizeof(float) * (size_t)D);
    } else {
        const int8_t* src = (const int8_t*)pool + page_off + (int64_t)t * D;
        if (kv_kind == 1) {
            float s = scales[(int64_t)page * tile_size + t];
            for (int d = 0; d < D; ++d) dst[d] = (float)src[d] / s;
        } else {
            for (int d = 0; d < D; ++d) dst[d] = (float)src[d];
        }
    }
}

/*
 * q, out: [B, H, D] f32.  Pools: [total_pages][tile_size][D].
 * table: dense int32 [num_beams][H][num_tiles], -1 = unmapped.
 * ctx_lens: per-row T (NULL -> T for every row; the reference has one T).
 * double_temperature: reproduce the CPU path's second division by
 *   temperature inside softmax_lut_vec; 0 = GPU semantics.
 * probs_out / logits_out: optional [B, H, T] (CPUAttentionOutput, hpp:34-39).
 */
ORC_API void orc_paged_attention(const float* q, float* out, const void* k_pool,
                                 const void* v_pool, const float* k_scales,
                                 const float* v_scales, int kv_kind, const int32_t* table,
                                 int num_beams, int H, int num_tiles, int total_pages,
                                 const int32_t* beam_ids, const int32_t* ctx_lens, int B, int T,
                                 int D, int tile_size, float temperature,
                                 int double_temperature, const float* rope, int top_k,
                                 float top_p, float* probs_out, float* logits_out) {
    const int total_entries = num_beams * H * num_tiles;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < B; ++b) {
        for (int h = 0; h < H; ++h) {
            /* :50 */
            const int beam = beam_ids ? beam_ids[b] : b;
            const int Tb = ctx_lens ? ctx_lens[b] : T;
            const int ntiles = (Tb + tile_size - 1) / tile_size; /* :45 */
            float* qv = (float*)malloc(sizeof(float) * (size_t)D * 2);
            float* row = qv + D;
            memcpy(qv, q + ((int64_t)b * H + h) * D, sizeof(float) * (size_t)D); /* :51-53 */
            if (rope) orc_rope_q(qv, rope, D);                                   /* :56-59 */

            int Tal = Tb > 0 ? Tb : 1;
            float* scores = (float*)malloc(sizeof(float) * (size_t)Tal * 2);
            float* probs = scores + Tal;
            for (int t = 0; t < Tb; ++t) { scores[t] = -1e9f; probs[t] = 0.f; } /* :61-62 */

            /* K pass :68-87 */
            for (int tile = 0; tile < ntiles; ++tile) {
                int tile_start = tile * tile_size;
                int tile_len = tile_size < Tb - tile_start ? tile_size : Tb - tile_start;
                int page = orc_pt_lookup(table, total_entries, beam, h, tile, H, num_tiles);
                if (page < 0 || page >= total_pages) continue; /* :73, kv_tile_cache.hpp:23 */
                int64_t off = (int64_t)page * tile_size * D;
                for (int t = 0; t < tile_len; ++t) {
                    orc_load_row(row, k_pool, k_scales, kv_kind, off, page, tile_size, t, D);
                    float dot = 0.0f;
                    for (int d = 0; d < D; ++d) dot += qv[d] * row[d]; /* :82-83 */
                    scores[tile_start + t] = dot / temperature;       /* :85, causal=false (D7) */
                }
            }

            /* softmax over all T :90 (softmax_lut.cpp:203-231) */
            orc_softmax_lut_vec(scores, Tb, double_temperature ? temperature : 1.0f, probs);

            /* filter :93-97; defaults top_k=0, top_p=1 make it a no-op */
            if (top_k > 0 || top_p < 1.0f)
                orc_apply_topk_topp_filter(probs, Tb, top_k, top_p, -1, 0.0f);

            /* V pass :103-117 */
            float* o = out + ((int64_t)b * H + h) * D;
            float* acc = (float*)calloc((size_t)D, sizeof(float));
            for (int tile = 0; tile < ntiles; ++tile) {
                int tile_start = tile * tile_size;
                int tile_len = tile_size < Tb - tile_start ? tile_size : Tb - tile_start;
                int page = orc_pt_lookup(table, total_entries, beam, h, tile, H, num_tiles);
                if (page < 0 || page >= total_pages) continue;
                int64_t off = (int64_t)page * tile_size * D;
                for (int t = 0; t < tile_len; ++t) {
                    orc_load_row(row, v_pool, v_scales, kv_kind, off, page, tile_size, t, D);
                    float p = probs[tile_start + t];
                    for (int d = 0; d < D; ++d) acc[d] += p * row[d];
                }
            }
            memcpy(o, acc, sizeof(float) * (size_t)D); /* :120 */
            free(acc);

            if (probs_out)
                memcpy(probs_out + ((int64_t)b * H + h) * T, probs, sizeof(float) * (size_t)Tb);
            if (logits_out)
                memcpy(logits_out + ((int64_t)b * H + h) * T, scores, sizeof(float) * (size_t)Tb);
            free(scores);
            free(qv);
        }
    }
}

/* Split-KV partial + LSE combine restatement (north-star addition; the math is
 * the exact decomposition of the global softmax above): partial over tokens
 * [t0,t1) gives m = max score, l = sum exp(s-m), O = sum exp(s-m) V.
 * Combine: M = max m_i; out = sum w_i O_i / (sum w_i l_i + 1e-6), w_i = exp(m_i-M). */
ORC_API void orc_lse_combine(const float* part_m, const float* part_l, const float* part_o,
                             int n_parts, int rows, int D, float* out) {
    for (int r = 0; r < rows; ++r) {
        float M = -INFINITY;
        for (int i = 0; i < n_parts; ++i) {
            float m = part_m[(int64_t)i * rows + r];
            if (m > M) M = m;
        }
        float L = 0.f;
        for (int d = 0; d < D; ++d) out[(int64_t)r * D + d] = 0.f;
        for (int i = 0; i < n_parts; ++i) {
            float m = part_m[(int64_t)i * rows + r];
            float w = (m == -INFINITY) ? 0.f : expf(m - M);
            L += w * part_l[(int64_t)i * rows + r];
            const float* o = part_o + ((int64_t)i * rows + r) * D;
            for (int d = 0; d < D; ++d) out[(int64_t)r * D + d] += w * o[d];
        }
        for (int d = 0; d < D; ++d) out[(int64_t)r * D + d] /= (L + 1e-6f);
    }
}

/* ------------------------------------------------------------------ */
/* INT8 matmul (attention_cpu/dnnl_matmul_int8.cpp:7-76)                */
/* ------------------------------------------------------------------ */

/* Exact s8 x s8 -> s32 accumulation; A [BATCH,M,K], B [BATCH,K,N], row-major
 * (format_tag::abc, :25-27).  Bit-exact target. */
ORC_API void orc_gemm_s8s8s32(const int8_t* A, const int8_t* Bm, int32_t* C, int BATCH, int M,
                              int N, int K) {
#pragma omp parallel for collapse(2)
    for (int b = 0; b < BATCH; ++b)
        for (int m = 0; m < M; ++m) {
            int32_t* c = C + ((int64_t)b * M + m) * N;
            for (int n = 0; n < N; ++n) c[n] = 0;
            const int8_t* a = A + ((int64_t)b * M + m) * K;
            for (int k = 0; k < K; ++k) {
                int32_t av = a[k];
                const int8_t* brow = Bm + ((int64_t)b * K + k) * N;
                for (int n = 0; n < N; ++n) c[n] += av * (int32_t)brow[n];
            }
        }
}

static inline float orc_gelu_erf(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f)); }

/* Epilogue (:39-56): alpha = scaleA*scaleB/scaleC (:40); dst = sat_s8(rne(
 * act(alpha*acc + bias))).  act: 0 none, 1 relu, 2 gelu_erf.  PARITY
 * UNPINNED (oneDNN < 3.0 not available); s8 outputs compared +-1 LSB. */
ORC_API void orc_matmul_int8_epilogue(const int32_t* acc, int8_t* C, int64_t rows, int N,
                                      float scaleA, float scaleB, float scaleC,
                                      const float* bias, int act) {
    float alpha = scaleA * scaleB / scaleC;
    for (int64_t r = 0; r < rows; ++r)
        for (int n = 0; n < N; ++n) {
            float v = alpha * (float)acc[r * N + n];
            if (bias) v += bias[n];
            if (act == 1) v = v > 0.f ? v : 0.f;
            else if (act == 2) v = orc_gelu_erf(v);
            float r_ = nearbyintf(v); /* round-half-even under default FE_TONEAREST */
            if (r_ > 127.f) r_ = 127.f;
            if (r_ < -128.f) r_ = -128.f;
            C[r * N + n] = (int8_t)r_;
        }
}

ORC_API int orc_dnnl_matmul_int8(const int8_t* A, const int8_t* Bm, int8_t* C, int BATCH, int M,
                                 int N, int K, float scaleA, float scaleB, float scaleC,
                                 const float* bias, int act) {
    int32_t* acc = (int32_t*)malloc(sizeof(int32_t) * (size_t)BATCH * M * N);
    if (!acc) return 0;
    orc_gemm_s8s8s32(A, Bm, acc, BATCH, M, N, K);
    orc_matmul_int8_epilogue(acc, C, (int64_t)BATCH * M, N, scaleA, scaleB, scaleC, bias, act);
    free(acc);
    return 1;
}

/* ------------------------------------------------------------------ */
/* Decoder glue (decoder/layer_norm.hpp:20-37, decoder/mlp.hpp:23-41)    */
/* ------------------------------------------------------------------ */

ORC_API void orc_layer_norm(const float* in, float* out, const float* gamma, const float* beta,
                            int rows, int hidden, float eps) {
    for (int i = 0; i < rows; ++i) {
        const float* x = in + (int64_t)i * hidden;
        float* y = out + (int64_t)i * hidden;
        float mean = 0;
        for (int j = 0; j < hidden; ++j) mean += x[j];
        mean /= hidden;
        float var = 0;
        for (int j = 0; j < hidden; ++j) var += (x[j] - mean) * (x[j] - mean);
        var /= hidden;
        /* `T inv_std = 1.0 / std::sqrt(var + epsilon_)` with T = float: std::sqrt picks the FLOAT overload (the
         * root is rounded to f32 first), the division by the double literal 1.0 is done in double, the quotient
         * is rounded to f32 (pinned bit-exact against the compiled header, tests/test_oracle_pinning.py) */
        float inv_std = (float)(1.0 / (double)sqrtf(var + eps));
        for (int j = 0; j < hidden; ++j) y[j] = (x[j] - mean) * inv_std * gamma[j] + beta[j];
    }
}

/* mlp.hpp:23-41, float instantiation; fc1_w [hidden][inter] (j*inter+i), ReLU. */
ORC_API void orc_mlp_f32(const float* in, float* out, const float* fc1_w, const float* fc1_b,
                         const float* fc2_w, const float* fc2_b, int rows, int hidden, int inter) {
#pragma omp parallel for
    for (int b = 0; b < rows; ++b) {
        float* mid = (float*)malloc(sizeof(float) * (size_t)inter);
        for (int i = 0; i < inter; ++i) {
            float sum = fc1_b[i];
            for (int j = 0; j < hidden; ++j) sum += in[(int64_t)b * hidden + j] * fc1_w[(int64_t)j * inter + i];
            mid[i] = sum > 0.f ? sum : 0.f;
        }
        for (int i = 0; i < hidden; ++i) {
            float sum = fc2_b[i];
            for (int j = 0; j < inter; ++j) sum += mid[j] * fc2_w[(int64_t)j * hidden + i];
            out[(int64_t)b * hidden + i] = sum;
        }
        free(mid);
    }
}


/* ------------------------------------------------------------------ */
/* INT8Decoder::quantize_weights arithmetic (decoder/int8_decoder.cpp:52-56,  */
/* also INT8Quantizer::quantize :20-25): scale = *max_element (signed max),   */
/* int8 = static_cast<int8_t>(fp32 / scale * 127): truncation, no clamp.      */
/* ------------------------------------------------------------------ */
ORC_API float orc_quantize_weights_file(const float* w, int64_t n, int8_t* out) {
    float scale = w[0];
    for (int64_t i = 1; i < n; ++i)
        if (w[i] > scale) scale = w[i];
    for (int64_t i = 0; i < n; ++i) out[i] = (int8_t)(int32_t)(w[i] / scale * 127);
    return scale;
}

/* attention/attention_kernel_utils.cuh:20-35 apply_rotary_embedding, float version, one (row, head) vector:
 * cos = rotary_emb[token*D + d], sin = rotary_emb[token*D + d + 1]. */
ORC_API void orc_apply_rotary_embedding(float* q, float* k, const float* rotary_emb, int head_dim, int token_idx,
                                        int apply_on_k) {
    for (int d = 0; d < head_dim; d += 2) {
        float c = rotary_emb[(int64_t)token_idx * head_dim + d];
        float s = rotary_emb[(int64_t)token_idx * head_dim + d + 1];
        float q0 = q[d], q1 = q[d + 1];
        q[d] = q0 * c - q1 * s;
        q[d + 1] = q0 * s + q1 * c;
        if (apply_on_k) {
            float k0 = k[d], k1 = k[d + 1];
            k[d] = k0 * c - k1 * s;
            k[d + 1] = k0 * s + k1 * c;
        }
    }
}

/* Thread count of the OpenMP loops (bench.py sets it to the box's core count: under torchrun the environment
 * carries OMP_NUM_THREADS=1, which would otherwise make the CPU baseline single-threaded). */
ORC_API void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
