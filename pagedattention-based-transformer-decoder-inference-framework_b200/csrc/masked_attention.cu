// masked_attention.cu -- softmax attention with grouped key/value heads over the paged KV pools for a RAGGED batch
// (prompt portions and single decoded tokens in one launch), with the score modifiers and visibility rules a design
// picks by parameter:
//
//   score   s = (q . k) * scale;  softcap > 0: s <- softcap * tanh(s / softcap);  then a distance bias is added:
//           bias_kind 1: - slope[h] * (i - j)            (one slope per query head)
//           bias_kind 2: + table[min(i - j, len - 1)][h] (a table over the distance, one column per query head)
//   mask    mask_kind 0: causal (j <= i);  1: sliding window (0 <= i - j < size);  2: chunks (j <= i and
//           floor(i / size) == floor(j / size), chunks counted from position 0 of the sequence)
//
// No rotation: positions enter through the bias and the mask only.  Scores, the modifiers, softmax weights and the
// weighted sums are float; K/V pages are stored in the activation type (float or bfloat16).  Only the key steps a
// tile's rows can see are visited, so the work per token is bounded by the window or chunk size.
//
// Pools: K pages [total_pages][tile_size][dim], V pages [total_pages][tile_size][vdim]; a (slot, kv head, tile) entry
// of the page table names the page of both (appended by pa_kv_append_rows).
#include "seq_common.cuh"

namespace pa {

constexpr int kMaRows = 32;     // (token, head) rows per CTA
constexpr int kMaWarps = 8;
constexpr int kMaRpw = kMaRows / kMaWarps;
constexpr int kMaKeys = 32;     // keys staged per step

struct MaskAttnParams {
    const void* q;              // rows of the projection buffer; the query of head h starts at q_off + h * dim
    int64_t q_stride;
    int q_off;
    const void* k_pool;
    const void* v_pool;
    const int32_t* table;
    int num_slots, num_kv_heads, num_tiles, total_pages, tile_size;
    const int32_t* tiles;       // [ntiles][4]: first row, tokens, slot, position of the first token
    int heads, dim, vdim;
    float scale, softcap;
    int mask_kind, mask_size;
    int bias_kind, bias_len;
    const float* bias;          // kind 1: [heads]; kind 2: [bias_len][heads]
    void* out;                  // [rows][heads * vdim]
    int head_rows;              // tensor-core kernel: every tile is ONE token and the rows are the heads of a kv head
};

__device__ __forceinline__ int ma_first_key(const MaskAttnParams& p, int pos) {
    if (p.mask_kind == 1) return max(0, pos - p.mask_size + 1);
    if (p.mask_kind == 2) return pos / p.mask_size * p.mask_size;
    return 0;
}

__device__ __forceinline__ bool ma_visible(const MaskAttnParams& p, int i, int j) {
    if (j > i) return false;
    if (p.mask_kind == 1) return i - j < p.mask_size;
    if (p.mask_kind == 2) return i / p.mask_size == j / p.mask_size;
    return true;
}

// the float score of (query position i, key position j, query head h) from the raw dot product
__device__ __forceinline__ float ma_score(const MaskAttnParams& p, float dot, int i, int j, int h, float slope) {
    float s = dot * p.scale;
    if (p.softcap > 0.f) s = p.softcap * tanhf(s / p.softcap);
    if (p.bias_kind == 1) s -= slope * (float)(i - j);
    else if (p.bias_kind == 2) s += p.bias[(int64_t)min(i - j, p.bias_len - 1) * p.heads + h];
    return s;
}

__device__ __forceinline__ void ma_geometry(int heads, int kv_heads, int& hpg, int& hc, int& nchunk) {
    hpg = heads / kv_heads;
    hc = hpg < kMaRows ? hpg : kMaRows;
    nchunk = (hpg + hc - 1) / hc;
}

// CTA of 8 warps = 32 (token, head) rows that read the SAME key/value head: up to 32 / hc consecutive tokens of one
// portion x hc = min(32, heads per kv head) query heads.  Keys are staged 32 at a time (one key per lane for the
// scores; lanes switch to value columns for the weighted sums).
template <typename T, int NV>
__global__ void __launch_bounds__(kMaWarps * 32) masked_attention_kernel(const MaskAttnParams p) {
    extern __shared__ float smem[];
    const int kd = p.dim, kds = kd + 1;
    float* Qs = smem;                              // [32][kd]
    float* Ks = Qs + kMaRows * kd;                 // [32][kd + 1]
    float* Vs = Ks + kMaKeys * kds;                // [32][vdim]
    __shared__ int64_t page_row[kMaKeys];          // pool row of the staged key, or -1

    int hpg, hc, nchunk;
    ma_geometry(p.heads, p.num_kv_heads, hpg, hc, nchunk);
    const int bq = kMaRows / hc;
    const int* tile = p.tiles + 4 * blockIdx.x;
    const int row0 = tile[0], ntok = tile[1], slot = tile[2], pos0 = tile[3];
    const int g = blockIdx.y / nchunk, chunk = blockIdx.y % nchunk;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* kp = static_cast<const T*>(p.k_pool);
    const T* vp = static_cast<const T*>(p.v_pool);

    for (int idx = threadIdx.x; idx < kMaRows * kd; idx += blockDim.x) {
        const int r = idx / kd, d = idx % kd;
        const int tok = r / hc, hh = chunk * hc + r % hc;
        float v = 0.f;
        if (tok < bq && tok < ntok && hh < hpg)
            v = to_f32<T>(static_cast<const T*>(p.q)[(int64_t)(row0 + tok) * p.q_stride + p.q_off + (int64_t)(g * hpg + hh) * kd + d]);
        Qs[idx] = v;
    }

    int rpos[kMaRpw], rhead[kMaRpw];   // position of the row's token (-1: unused row) and its query head
    float slope[kMaRpw], m[kMaRpw], l[kMaRpw], acc[kMaRpw][NV];
#pragma unroll
    for (int r = 0; r < kMaRpw; ++r) {
        const int row = warp * kMaRpw + r;
        const int tok = row / hc, hh = chunk * hc + row % hc;
        const bool used = tok < bq && tok < ntok && hh < hpg;
        rpos[r] = used ? pos0 + tok : -1;
        rhead[r] = used ? g * hpg + hh : 0;
        slope[r] = p.bias_kind == 1 ? p.bias[rhead[r]] : 0.f;
        m[r] = -INFINITY;
        l[r] = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) acc[r][i] = 0.f;
    }

    const int last_tok = min(ntok, bq) - 1;
    const int total = pos0 + last_tok + 1;                 // keys any row of the tile may see
    const int s_begin = ma_first_key(p, pos0) / kMaKeys;
    const int s_end = (total + kMaKeys - 1) / kMaKeys;

    for (int st = s_begin; st < s_end; ++st) {
        const int c0 = st * kMaKeys;
        __syncthreads();                                   // the previous step's tiles are consumed (and Qs is written)
        if (threadIdx.x < kMaKeys) {
            const int j = c0 + threadIdx.x;
            int64_t pr = -1;
            if (j < total && j / p.tile_size < p.num_tiles) {
                const int page = p.table[((int64_t)slot * p.num_kv_heads + g) * p.num_tiles + j / p.tile_size];
                if (page >= 0 && page < p.total_pages) pr = (int64_t)page * p.tile_size + j % p.tile_size;
            }
            page_row[threadIdx.x] = pr;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < kMaKeys * kd; idx += blockDim.x) {
            const int key = idx / kd, d = idx % kd;
            const int64_t pr = page_row[key];
            Ks[key * kds + d] = pr >= 0 ? to_f32<T>(kp[pr * kd + d]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < kMaKeys * p.vdim; idx += blockDim.x) {
            const int key = idx / p.vdim, d = idx % p.vdim;
            const int64_t pr = page_row[key];
            Vs[idx] = pr >= 0 ? to_f32<T>(vp[pr * p.vdim + d]) : 0.f;
        }
        __syncthreads();

        // ---- scores: lane = key
        float s[kMaRpw];
#pragma unroll
        for (int r = 0; r < kMaRpw; ++r) s[r] = 0.f;
        const float* kr = Ks + lane * kds;
        const float* qb = Qs + warp * kMaRpw * kd;
        for (int d = 0; d < kd; ++d) {
            const float kv = kr[d];
#pragma unroll
            for (int r = 0; r < kMaRpw; ++r) s[r] = fmaf(qb[r * kd + d], kv, s[r]);
        }
        const int j = c0 + lane;
        const bool mapped = page_row[lane] >= 0;
        float w[kMaRpw];
#pragma unroll
        for (int r = 0; r < kMaRpw; ++r) {
            const bool vis = mapped && rpos[r] >= 0 && ma_visible(p, rpos[r], j);
            const float v = vis ? ma_score(p, s[r], rpos[r], j, rhead[r], slope[r]) : -INFINITY;
            const float n = fmaxf(m[r], warp_max(v));
            const float c = n == -INFINITY ? 1.f : expf(m[r] - n);
            w[r] = vis ? expf(v - n) : 0.f;
            l[r] = l[r] * c + warp_sum(w[r]);
            m[r] = n;
#pragma unroll
            for (int i = 0; i < NV; ++i) acc[r][i] *= c;
        }
        // ---- weighted sums: lane = value column
        const int nk = min(kMaKeys, total - c0);
        for (int jj = 0; jj < nk; ++jj) {
            float v[NV];
#pragma unroll
            for (int i = 0; i < NV; ++i) v[i] = lane + 32 * i < p.vdim ? Vs[jj * p.vdim + lane + 32 * i] : 0.f;
#pragma unroll
            for (int r = 0; r < kMaRpw; ++r) {
                const float wj = __shfl_sync(0xffffffffu, w[r], jj);
#pragma unroll
                for (int i = 0; i < NV; ++i) acc[r][i] = fmaf(wj, v[i], acc[r][i]);
            }
        }
    }

#pragma unroll
    for (int r = 0; r < kMaRpw; ++r) {
        if (rpos[r] < 0) continue;
        const int row = warp * kMaRpw + r;
        T* dst = static_cast<T*>(p.out) + (int64_t)(row0 + row / hc) * p.heads * p.vdim + (int64_t)rhead[r] * p.vdim;
        const float inv = 1.0f / l[r];
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (lane + 32 * i < p.vdim) dst[lane + 32 * i] = from_f32<T>(acc[r][i] * inv);
    }
}

template <typename T, int NV>
static int ma_launch(const MaskAttnParams& p, int ntiles, cudaStream_t st) {
    int hpg, hc, nchunk;
    hpg = p.heads / p.num_kv_heads;
    hc = hpg < kMaRows ? hpg : kMaRows;
    nchunk = (hpg + hc - 1) / hc;
    const size_t smem = ((size_t)kMaRows * p.dim + (size_t)kMaKeys * (p.dim + 1) + (size_t)kMaKeys * p.vdim) * sizeof(float);
    if (smem > 200 * 1024) return PA_ERR_UNSUPPORTED;
    cudaError_t e = cudaFuncSetAttribute(masked_attention_kernel<T, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((unsigned)ntiles, (unsigned)(p.num_kv_heads * nchunk));
    masked_attention_kernel<T, NV><<<grid, kMaWarps * 32, smem, st>>>(p);
    PA_RETURN_LAUNCH_STATUS();
}

template <typename T>
static int ma_dispatch(const MaskAttnParams& p, int ntiles, cudaStream_t st) {
    const int nv = (p.vdim + 31) / 32;
    switch (nv) {
        case 1: return ma_launch<T, 1>(p, ntiles, st);
        case 2: return ma_launch<T, 2>(p, ntiles, st);
        case 3: return ma_launch<T, 3>(p, ntiles, st);
        case 4: return ma_launch<T, 4>(p, ntiles, st);
        case 5: case 6: return ma_launch<T, 6>(p, ntiles, st);
        case 7: case 8: return ma_launch<T, 8>(p, ntiles, st);
        default: return PA_ERR_UNSUPPORTED;
    }
}

}  // namespace pa

using namespace pa;

PA_API int pa_masked_attention_tile_tokens(int heads, int kv_heads) {
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads) return 0;
    const int hpg = heads / kv_heads;
    return kMaRows / (hpg < kMaRows ? hpg : kMaRows);
}

PA_API int pa_masked_attention(const void* d_q, int64_t q_stride, int q_off, const void* d_k_pool, const void* d_v_pool,
                               const int32_t* d_table, int num_slots, int num_kv_heads, int num_tiles, int total_pages,
                               int tile_size, const int32_t* d_q_tiles, int num_q_tiles, int heads, int dim, int vdim,
                               float scale, float softcap, int mask_kind, int mask_size, int bias_kind,
                               const float* d_bias, int bias_len, void* d_out, int elem, int tile_kind,
                               pa_stream_t stream) {
    PA_CHECK_ARG(d_q && d_k_pool && d_v_pool && d_table && d_q_tiles && d_out && num_q_tiles >= 0);
    PA_CHECK_ARG(num_slots > 0 && num_kv_heads > 0 && num_tiles > 0 && total_pages > 0 && tile_size > 0);
    PA_CHECK_ARG(heads > 0 && heads % num_kv_heads == 0 && dim > 0 && vdim > 0 && softcap >= 0.f);
    PA_CHECK_ARG(mask_kind >= 0 && mask_kind <= 2 && (mask_kind == 0 || mask_size > 0));
    PA_CHECK_ARG(bias_kind >= 0 && bias_kind <= 2 && (bias_kind == 0 || d_bias) && (bias_kind != 2 || bias_len > 0));
    if (num_q_tiles == 0) return PA_OK;
    MaskAttnParams p;
    p.q = d_q; p.q_stride = q_stride; p.q_off = q_off; p.k_pool = d_k_pool; p.v_pool = d_v_pool; p.table = d_table;
    p.num_slots = num_slots; p.num_kv_heads = num_kv_heads; p.num_tiles = num_tiles; p.total_pages = total_pages;
    p.tile_size = tile_size; p.tiles = d_q_tiles; p.heads = heads; p.dim = dim; p.vdim = vdim; p.scale = scale;
    p.softcap = softcap; p.mask_kind = mask_kind; p.mask_size = mask_size; p.bias_kind = bias_kind; p.bias = d_bias;
    p.bias_len = bias_len; p.out = d_out; p.head_rows = 0;
    if (elem != 4 && elem != 2) return PA_ERR_UNSUPPORTED;
    (void)tile_kind;
    if (elem == 4) return ma_dispatch<float>(p, num_q_tiles, as_stream(stream));
    return ma_dispatch<bf16_t>(p, num_q_tiles, as_stream(stream));
}

PA_API int pa_masked_attention_mma_tile_tokens(int dim, int vdim, int elem) {
    (void)dim; (void)vdim; (void)elem;
    return 0;
}
