// masked_attention.cu -- softmax attention with grouped key/value heads over the paged KV pools for a RAGGED batch
// (prompt portions and single decoded tokens in one launch), with the score modifiers and visibility rules a design
// picks by parameter:
//
//   score   s = (q . k) * scale;  softcap > 0: s <- softcap * tanh(s / softcap);  then a distance bias is added:
//           bias_kind 1: - slope[h] * (i - j)            (one slope per query head)
//           bias_kind 2: + table[min(i - j, len - 1)][h] (a table over the distance, one column per query head)
//           head_scale != null: s <- s * head_scale[h] right after the scale (a temperature per query head)
//   mask    mask_kind 0: causal (j <= i);  1: sliding window (0 <= i - j < size), which with mask_keep > 0 also keeps the
//           first mask_keep positions of the sequence visible (at their true positions);  2: chunks (j <= i and
//           floor(i / size) == floor(j / size), chunks counted from position 0 of the sequence)
//   sink    sink != null: exp(sink[h]) joins the softmax denominator of head h (a logit without key or value; zeros
//           give the "one added to the denominator" form)
//   output  out_rot != null: [rows][vdim / 2][cos, sin] of the batch rows; the neighbouring pairs (2m, 2m + 1) of every
//           head's output are turned BACK by the row's angle (values that were cached turned by their own position), in
//           float, before the result is rounded
//

// No rotation: positions enter through the bias and the mask only.  Scores, the modifiers, softmax weights and the
// weighted sums are float; K/V pages are stored in the activation type (float or bfloat16).  Only the key steps a
// tile's rows can see are visited, so the work per token is bounded by the window or chunk size.
//
// Pools: K pages [total_pages][tile_size][dim], V pages [total_pages][tile_size][vdim]; a (slot, kv head, tile) entry
// of the page table names the page of both (appended by pa_kv_append_rows).
#include "seq_common.cuh"

namespace pa {

// ---- rotation of this step's q | k | v rows fused with the append ----------------------------------------------------
// One warp per (row, unit): units [0, heads) are the query heads, rotated in place over their first rot_dims dimensions;
// units [heads, heads + kv_heads) are the key/value heads of a layer with a pool of its own: the key goes to its place in
// the pool rotated the same way, the value turned over all of vdim (vrot != null) or as it is.  Pairs are neighbours
// (2m, 2m + 1); the tables hold [rows][dims / 2][cos, sin] of the batch rows.
template <typename T>
__device__ __forceinline__ void ma_turn_copy(const T* __restrict__ src, T* __restrict__ dst, int n, int dims,
                                             const float* __restrict__ t, int lane) {
    for (int d = 2 * lane; d < n; d += 64) {
        float u = to_f32<T>(src[d]), v = d + 1 < n ? to_f32<T>(src[d + 1]) : 0.f;
        if (t && d + 1 < dims) {
            const float c = t[d], sn = t[d + 1];          // pair d / 2: entries (d / 2) * 2 and + 1
            const float u0 = u;
            u = u0 * c - v * sn;
            v = v * c + u0 * sn;
        }
        dst[d] = from_f32<T>(u);
        if (d + 1 < n) dst[d + 1] = from_f32<T>(v);
    }
}

template <typename T>
__global__ void rope_kv_append_kernel(T* __restrict__ src, int64_t stride, int q_off, int k_off, int v_off, int heads,
                                      int kv_heads, int dim, int vdim, int rot_dims, const float* __restrict__ rope,
                                      const float* __restrict__ vrot, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                      const int32_t* __restrict__ table, int num_slots, int num_tiles, int total_pages,
                                      int tile_size, const int32_t* __restrict__ row_slot,
                                      const int32_t* __restrict__ row_pos, int rows) {
    const int lane = threadIdx.x & 31;
    const int units = heads + (k_pool ? kv_heads : 0);
    const int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (w >= (int64_t)rows * units) return;
    const int u = (int)(w % units);
    const int64_t r = w / units;
    T* row = src + r * stride;
    const float* rt = rope ? rope + r * (rot_dims >> 1) * 2 : nullptr;
    if (u < heads) {
        if (rt) ma_turn_copy<T>(row + q_off + (int64_t)u * dim, row + q_off + (int64_t)u * dim, rot_dims, rot_dims, rt, lane);
        return;
    }
    const int g = u - heads;
    const int slot = row_slot[r], pos = row_pos[r];
    if (pos < 0 || pos / tile_size >= num_tiles || (unsigned)slot >= (unsigned)num_slots) return;
    const int page = table[((int64_t)slot * kv_heads + g) * num_tiles + pos / tile_size];
    if (page < 0 || page >= total_pages) return;
    const int64_t prow = (int64_t)page * tile_size + pos % tile_size;
    ma_turn_copy<T>(row + k_off + (int64_t)g * dim, k_pool + prow * dim, dim, rot_dims, rt, lane);
    ma_turn_copy<T>(row + v_off + (int64_t)g * vdim, v_pool + prow * vdim, vdim, vdim,
                    vrot ? vrot + r * (vdim >> 1) * 2 : nullptr, lane);
}

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
    const float* head_scale;    // [heads] or null
    const float* sink;          // [heads] or null
    int mask_keep;              // window masks: the first mask_keep positions stay visible
    const float* out_rot;       // [rows][vdim / 2][2] or null
    int head_rows;              // tensor-core kernel: every tile is ONE token and the rows are the heads of a kv head
};

__device__ __forceinline__ int ma_first_key(const MaskAttnParams& p, int pos) {
    if (p.mask_kind == 1) return max(0, pos - p.mask_size + 1);
    if (p.mask_kind == 2) return pos / p.mask_size * p.mask_size;
    return 0;
}

__device__ __forceinline__ bool ma_visible(const MaskAttnParams& p, int i, int j) {
    if (j > i) return false;
    if (p.mask_kind == 1) return i - j < p.mask_size || j < p.mask_keep;
    if (p.mask_kind == 2) return i / p.mask_size == j / p.mask_size;
    return true;
}

// The key steps (runs of `keys` positions) the rows of a tile can see, in order: the steps of the kept first positions,
// then the steps from the first key of the tile's first token (ma_first_key) to its last token.  `first` = that first
// key, `total` = keys up to the tile's last token.
struct MaSteps {
    int head, body0, count;
    __device__ __forceinline__ int step(int n) const { return n < head ? n : body0 + n - head; }
};
__device__ __forceinline__ MaSteps ma_steps(const MaskAttnParams& p, int first, int total, int keys) {
    MaSteps s;
    s.body0 = first / keys;
    s.head = 0;
    if (p.mask_kind == 1 && p.mask_keep > 0) s.head = min(s.body0, (min(p.mask_keep, total) + keys - 1) / keys);
    s.count = s.head + (total + keys - 1) / keys - s.body0;
    return s;
}

// the softmax denominator with the sink of head h: returns the factor for the accumulated sums (and updates l)
__device__ __forceinline__ float ma_sink(const MaskAttnParams& p, int h, float m, float& l) {
    if (!p.sink) return 1.f;
    const float sk = p.sink[h];
    const float n = fmaxf(m, sk);
    const float c = m == -INFINITY ? 0.f : expf(m - n);
    l = l * c + expf(sk - n);
    return c;
}

// turns the pair (u, v) = columns (2m, 2m + 1) of batch row `row` back by the row's angle; even = this thread holds u
__device__ __forceinline__ float ma_unturn(const MaskAttnParams& p, int64_t row, int col, float mine, float other) {
    const float* t = p.out_rot + (row * (p.vdim >> 1) + (col >> 1)) * 2;
    return (col & 1) ? mine * t[0] - other * t[1] : mine * t[0] + other * t[1];
}

// the float score of (query position i, key position j, query head h) from the raw dot product
__device__ __forceinline__ float ma_score(const MaskAttnParams& p, float dot, int i, int j, int h, float slope) {
    float s = dot * p.scale;
    if (p.head_scale) s *= p.head_scale[h];
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
    const MaSteps steps = ma_steps(p, ma_first_key(p, pos0), total, kMaKeys);

    for (int sn = 0; sn < steps.count; ++sn) {
        const int c0 = steps.step(sn) * kMaKeys;
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
        float ll = l[r];
        const float inv = ma_sink(p, rhead[r], m[r], ll) / ll;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int col = lane + 32 * i;
            float v = acc[r][i] * inv;
            if (p.out_rot) {                           // the partner column sits in the neighbouring lane (vdim is even)
                const float o = __shfl_xor_sync(0xffffffffu, v, 1);
                if (col < p.vdim) v = ma_unturn(p, row0 + row / hc, col, v, o);
            }
            if (col < p.vdim) dst[col] = from_f32<T>(v);
        }
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


// ---- single-token tiles (decode) ------------------------------------------------------------------------------------
// One CTA = one token x one key/value head; its R >= heads-per-kv-head rows are the query heads of the group.  Nothing is
// staged: each of the kMaDecWarps warps takes every kMaDecWarps-th run of 32 keys of the visible range, a lane reads ITS key's row with 16-byte
// loads straight into the dot products of every row (queries broadcast from shared memory), the warp does the online
// softmax, then lanes switch to value columns and read each key's value row coalesced.  The warps' (m, l, acc) are
// merged through shared memory.  Needs dim a multiple of the 16-byte vector and R <= 8 (else the tile kernel serves).
template <typename T> struct MaVec { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void ma_load16(const T* __restrict__ p, float (&f)[MaVec<T>::N]) {
    const uint4 v = ldg_stream_128(p);
    if (sizeof(T) == 4) {
        f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
    } else {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
}

// NV consecutive values of a row starting at element lane * NV, in one load where NV * sizeof(T) is 4, 8 or a multiple of 16
template <typename T, int NV>
__device__ __forceinline__ void ma_load_packed(const T* __restrict__ p, float (&f)[NV]) {
    constexpr int BYTES = NV * sizeof(T);
    if (BYTES % 16 == 0) {
#pragma unroll
        for (int c = 0; c < BYTES / 16; ++c) {
            float t[MaVec<T>::N];
            ma_load16<T>(p + c * MaVec<T>::N, t);
#pragma unroll
            for (int i = 0; i < MaVec<T>::N; ++i) f[c * MaVec<T>::N + i] = t[i];
        }
    } else if (BYTES == 8 && sizeof(T) == 2) {
        const uint2 v = ldg_stream_64(p);
        f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
        f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    } else if (BYTES == 8) {
        const uint2 v = ldg_stream_64(p);
        f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    } else if (BYTES == 4 && sizeof(T) == 2) {
        const uint32_t v = *reinterpret_cast<const uint32_t*>(p);
        f[0] = __uint_as_float(v << 16); f[1] = __uint_as_float(v & 0xffff0000u);
    } else {
#pragma unroll
        for (int i = 0; i < NV; ++i) f[i] = to_f32<T>(p[i]);
    }
}

// value column held in slot i of a lane: lane + 32 i, or (PACKED: vdim == 32 NV) lane * NV + i
template <int NV, bool PACKED>
__device__ __forceinline__ int ma_col(int lane, int i) { return PACKED ? lane * NV + i : lane + 32 * i; }

constexpr int kMaDecWarps = 16;   // a window of ~1000 keys leaves each warp two steps: the chain of dependent loads stays short

template <typename T, int R, int NV, bool PACKED>
__global__ void __launch_bounds__(kMaDecWarps * 32) masked_attention_decode_kernel(const MaskAttnParams p) {
    extern __shared__ float smem[];
    constexpr int VN = MaVec<T>::N;
    const int kd = p.dim;
    float* Qs = smem;                                   // [R][kd]
    float* Ps = Qs + R * kd;                            // [warps][R][2 + vdim]
    const int pstride = 2 + p.vdim;
    const int hpg = p.heads / p.num_kv_heads;
    const int* tile = p.tiles + 4 * blockIdx.x;
    const int row0 = tile[0], slot = tile[2], pos = tile[3];
    const int g = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* kp = static_cast<const T*>(p.k_pool);
    const T* vp = static_cast<const T*>(p.v_pool);
    for (int idx = threadIdx.x; idx < R * kd; idx += blockDim.x) {
        const int r = idx / kd, d = idx % kd;
        Qs[idx] = r < hpg ? to_f32<T>(static_cast<const T*>(p.q)[(int64_t)row0 * p.q_stride + p.q_off + (int64_t)(g * hpg + r) * kd + d]) : 0.f;
    }
    __syncthreads();
    float m[R], l[R], acc[R][NV], slope[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        m[r] = -INFINITY;
        l[r] = 0.f;
        slope[r] = p.bias_kind == 1 && r < hpg ? p.bias[g * hpg + r] : 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) acc[r][i] = 0.f;
    }
    const int total = pos + 1;
    const MaSteps steps = ma_steps(p, ma_first_key(p, pos), total, kMaKeys);
    const int32_t* trow = p.table + ((int64_t)slot * p.num_kv_heads + g) * p.num_tiles;
    for (int sn = warp; sn < steps.count; sn += kMaDecWarps) {
        const int st = steps.step(sn);
        const int j = st * kMaKeys + lane;
        int prow = -1;                                  // pool row of this lane's key
        if (j < total && ma_visible(p, pos, j) && j / p.tile_size < p.num_tiles) {
            const int page = trow[j / p.tile_size];
            if (page >= 0 && page < p.total_pages) prow = page * p.tile_size + j % p.tile_size;
        }
        float s[R];
#pragma unroll
        for (int r = 0; r < R; ++r) s[r] = 0.f;
        if (prow >= 0) {
            const T* kr = kp + (int64_t)prow * kd;
#pragma unroll 8
            for (int d0 = 0; d0 < kd; d0 += VN) {
                float kv[VN];
                ma_load16<T>(kr + d0, kv);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float* q = Qs + r * kd + d0;
#pragma unroll
                    for (int i = 0; i < VN; ++i) s[r] = fmaf(q[i], kv[i], s[r]);
                }
            }
        }
        const bool vis = prow >= 0;
        float w[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float v = vis && r < hpg ? ma_score(p, s[r], pos, j, g * hpg + r, slope[r]) : -INFINITY;
            const float n = fmaxf(m[r], warp_max(v));
            const float c = n == -INFINITY ? 1.f : expf(m[r] - n);
            w[r] = v == -INFINITY ? 0.f : expf(v - n);
            l[r] = l[r] * c + warp_sum(w[r]);
            m[r] = n;
#pragma unroll
            for (int i = 0; i < NV; ++i) acc[r][i] *= c;
        }
        const int nk = min(kMaKeys, total - st * kMaKeys);
#pragma unroll 8
        for (int jj = 0; jj < nk; ++jj) {
            const int pr = __shfl_sync(0xffffffffu, prow, jj);
            float v[NV];
#pragma unroll
            for (int i = 0; i < NV; ++i) v[i] = 0.f;
            if (pr >= 0) {
                const T* vr = vp + (int64_t)pr * p.vdim;
                if (PACKED) {
                    ma_load_packed<T, NV>(vr + lane * NV, v);
                } else {
#pragma unroll
                    for (int i = 0; i < NV; ++i) v[i] = lane + 32 * i < p.vdim ? to_f32<T>(vr[lane + 32 * i]) : 0.f;
                }
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float wj = __shfl_sync(0xffffffffu, w[r], jj);
#pragma unroll
                for (int i = 0; i < NV; ++i) acc[r][i] = fmaf(wj, v[i], acc[r][i]);
            }
        }
    }
    // ---- the warps' partials -> shared memory, merged by warp r for row r
#pragma unroll
    for (int r = 0; r < R; ++r) {
        float* dst = Ps + ((int64_t)warp * R + r) * pstride;
        if (lane == 0) { dst[0] = m[r]; dst[1] = l[r]; }
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (ma_col<NV, PACKED>(lane, i) < p.vdim) dst[2 + ma_col<NV, PACKED>(lane, i)] = acc[r][i];
    }
    __syncthreads();
    for (int r = warp; r < R; r += kMaDecWarps) {
        if (r >= hpg) continue;
        float M = -INFINITY;
        for (int w = 0; w < kMaDecWarps; ++w) M = fmaxf(M, Ps[((int64_t)w * R + r) * pstride]);
        if (p.sink) M = fmaxf(M, p.sink[g * hpg + r]);
        float L = p.sink ? expf(p.sink[g * hpg + r] - M) : 0.f, b[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) b[i] = 0.f;
        for (int w = 0; w < kMaDecWarps; ++w) {
            const float* pw = Ps + ((int64_t)w * R + r) * pstride;
            const float f = pw[0] == -INFINITY ? 0.f : expf(pw[0] - M);
            L = fmaf(f, pw[1], L);
#pragma unroll
            for (int i = 0; i < NV; ++i)
                if (ma_col<NV, PACKED>(lane, i) < p.vdim) b[i] = fmaf(f, pw[2 + ma_col<NV, PACKED>(lane, i)], b[i]);
        }
        T* dst = static_cast<T*>(p.out) + (int64_t)row0 * p.heads * p.vdim + (int64_t)(g * hpg + r) * p.vdim;
        const float inv = 1.0f / L;
#pragma unroll
        for (int i = 0; i < NV; ++i) b[i] *= inv;
        if (p.out_rot) {          // the partner column: the neighbouring slot of this lane (packed pairs) or the neighbouring lane
            float o[NV];
#pragma unroll
            for (int i = 0; i < NV; ++i) o[i] = (PACKED && NV > 1) ? b[i ^ 1] : __shfl_xor_sync(0xffffffffu, b[i], 1);
#pragma unroll
            for (int i = 0; i < NV; ++i)
                if (ma_col<NV, PACKED>(lane, i) < p.vdim) b[i] = ma_unturn(p, row0, ma_col<NV, PACKED>(lane, i), b[i], o[i]);
        }
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (ma_col<NV, PACKED>(lane, i) < p.vdim) dst[ma_col<NV, PACKED>(lane, i)] = from_f32<T>(b[i]);
    }
}

template <typename T, int R, int NV>
static int ma_decode_launch(const MaskAttnParams& p, int ntiles, cudaStream_t st) {
    const size_t smem = ((size_t)R * p.dim + (size_t)kMaDecWarps * R * (2 + p.vdim)) * sizeof(float);
    if (smem > 200 * 1024) return PA_ERR_UNSUPPORTED;
    // one load per lane and value row where the row is exactly 32 lanes x NV values and the pool is aligned for it
    const bool packed = p.vdim == 32 * NV && (uintptr_t)p.v_pool % 16 == 0 &&
                        ((NV * sizeof(T)) % 16 == 0 || NV * sizeof(T) == 8 || (NV * sizeof(T) == 4 && sizeof(T) == 2));
    auto kern = packed ? masked_attention_decode_kernel<T, R, NV, true> : masked_attention_decode_kernel<T, R, NV, false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((unsigned)ntiles, (unsigned)p.num_kv_heads);
    kern<<<grid, kMaDecWarps * 32, smem, st>>>(p);
    PA_RETURN_LAUNCH_STATUS();
}

// PA_ERR_UNSUPPORTED: this shape stays on the tile kernel
template <typename T>
static int ma_decode_dispatch(const MaskAttnParams& p, int ntiles, cudaStream_t st) {
    const int hpg = p.heads / p.num_kv_heads, nv = (p.vdim + 31) / 32;
    if (p.dim % MaVec<T>::N || hpg > 8 || nv > 8) return PA_ERR_UNSUPPORTED;
    if ((uintptr_t)p.k_pool % 16) return PA_ERR_UNSUPPORTED;
    const int NVc = nv <= 1 ? 1 : nv <= 2 ? 2 : nv <= 4 ? 4 : 8;
#define PA_MA_DEC(RR)                                                   \
    switch (NVc) {                                                      \
        case 1: return ma_decode_launch<T, RR, 1>(p, ntiles, st);       \
        case 2: return ma_decode_launch<T, RR, 2>(p, ntiles, st);       \
        case 4: return ma_decode_launch<T, RR, 4>(p, ntiles, st);       \
        default: if (RR <= 4) return ma_decode_launch<T, (RR <= 4 ? RR : 4), 8>(p, ntiles, st); return PA_ERR_UNSUPPORTED; \
    }
    if (hpg <= 2) { PA_MA_DEC(2) }
    if (hpg <= 4) { PA_MA_DEC(4) }
    PA_MA_DEC(8)
#undef PA_MA_DEC
}

// ---- prompt portions on the tensor cores (bfloat16) -------------------------------------------------------------------
// One CTA = up to 64 consecutive tokens of one portion x ONE query head; 4 warps, warp w owns rows 16 w .. 16 w + 15:
// a flash-attention (mma.sync m16n8k16, bfloat16 operands, float accumulators) over staged key and value tiles of 64 keys,
// located through the page table and brought in with 16-byte cp.async copies into two buffers (the copies of step t + 1
// fly while step t is multiplied).  Only the key steps between the first key the tile's first token sees and its last
// token are visited; a warp skips steps none of its rows can see.  The dot products are raw q . k; scale, soft cap and
// distance bias are applied to the float score.  Scores, the running maximum, the exponentials and their sum are float;
// the weights enter the second product rounded to bfloat16, like every other matrix operand of this precision.
// DIM and VDIM are the PADDED sizes (32, 64 or 128): the real dim / vdim values (any multiple of 8) sit at the start of
// the columns and the rest is zero; 16-wide steps that are all padding are skipped.  A bias table of up to kMmBiasMax
// distances is staged (this head's column) in shared memory.
constexpr int kMmRows = 64, kMmKeys = 64, kMmThreads = 128, kMmPad = 8, kMmStages = 2, kMmBiasMax = 4096;

__device__ __forceinline__ float ma_tanh(float x) {        // 1 - 2 / (e^{2x} + 1), relative error ~1e-6
    const float e = __expf(2.0f * x);
    return 1.0f - __fdividef(2.0f, e + 1.0f);
}

template <int DIM, int VDIM>
__global__ void __launch_bounds__(kMmThreads) masked_attention_mma_kernel(const MaskAttnParams p) {
    constexpr int KS = DIM + kMmPad, VS = VDIM + kMmPad, NT = VDIM / 8, NST = kMmStages;
    extern __shared__ __align__(16) unsigned char mm_smem[];
    bf16_t* Qs = reinterpret_cast<bf16_t*>(mm_smem);         // [64][KS]
    bf16_t* Ks = Qs + kMmRows * KS;                           // [NST][64][KS]
    bf16_t* Vs = Ks + NST * kMmKeys * KS;                     // [NST][64][VS]
    float* Bs = reinterpret_cast<float*>(Vs + NST * kMmKeys * VS);   // [bias_len] (bias_kind 2, bias_len <= kMmBiasMax)
    __shared__ int key_ok[NST][kMmKeys];

    const int* tile = p.tiles + 4 * blockIdx.x;
    const int row0 = tile[0], ntok = tile[1], slot = tile[2], pos0 = tile[3];
    const int head = blockIdx.y, hpg = p.heads / p.num_kv_heads, g = head / hpg;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rbase = warp * 16;
    const bool active = rbase < ntok;
    const bf16_t* kp = static_cast<const bf16_t*>(p.k_pool);
    const bf16_t* vp = static_cast<const bf16_t*>(p.v_pool);
    const int32_t* trow = p.table + ((int64_t)slot * p.num_kv_heads + g) * p.num_tiles;
    const int total = pos0 + ntok;
    const MaSteps steps = ma_steps(p, ma_first_key(p, pos0), total, kMmKeys);
    const int keep = p.mask_kind == 1 ? p.mask_keep : 0;
    const int dim = p.dim, vdim = p.vdim;
    const bool bias_smem = p.bias_kind == 2 && p.bias_len <= kMmBiasMax;

    for (int c = tid; c < kMmRows * (DIM / 8); c += kMmThreads) {
        const int r = c / (DIM / 8), cv = (c % (DIM / 8)) * 8;
        const bool ok = r < ntok && cv < dim;
        const bf16_t* src = static_cast<const bf16_t*>(p.q) + (ok ? (int64_t)(row0 + r) * p.q_stride + p.q_off + (int64_t)head * dim + cv : 0);
        cp_async_16(smem_u32(Qs + r * KS + cv), src, ok);
    }
    if (bias_smem)
        for (int d = tid; d < p.bias_len; d += kMmThreads) Bs[d] = p.bias[(int64_t)d * p.heads + head];
    auto pool_row = [&](int j) -> int64_t {
        if (j < total && j / p.tile_size < p.num_tiles) {
            const int page = trow[j / p.tile_size];
            if (page >= 0 && page < p.total_pages) return (int64_t)page * p.tile_size + j % p.tile_size;
        }
        return -1;
    };
    // two threads per key: ONE page look-up per thread and step; a thread copies every second 16-byte piece of its key's
    // row and of its value row
    auto load_tile = [&](int kt, int buf) {
        const int key = tid >> 1, q2 = tid & 1;
        const int64_t pr = pool_row(kt * kMmKeys + key);
        if (q2 == 0) key_ok[buf][key] = pr >= 0;
        bf16_t* kdst = Ks + (buf * kMmKeys + key) * KS;
        const bf16_t* ksrc = kp + (pr >= 0 ? pr * dim : 0);
#pragma unroll
        for (int i = 0; i < DIM / 16; ++i) {
            const int cv = (q2 + 2 * i) * 8;
            const bool ok = pr >= 0 && cv < dim;
            cp_async_16(smem_u32(kdst + cv), ok ? ksrc + cv : kp, ok);
        }
        bf16_t* vdst = Vs + (buf * kMmKeys + key) * VS;
        const bf16_t* vsrc = vp + (pr >= 0 ? pr * vdim : 0);
#pragma unroll
        for (int i = 0; i < VDIM / 16; ++i) {
            const int cv = (q2 + 2 * i) * 8;
            const bool ok = pr >= 0 && cv < vdim;
            cp_async_16(smem_u32(vdst + cv), ok ? vsrc + cv : vp, ok);
        }
    };
#pragma unroll
    for (int t = 0; t < NST - 1; ++t) {
        if (t < steps.count) load_tile(steps.step(t), t);
        cp_async_commit();
    }

    float o[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[t][c] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    int rpos[2], rlo[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        rpos[i] = pos0 + rbase + (lane >> 2) + 8 * i;
        rlo[i] = ma_first_key(p, rpos[i]);
    }
    // the warp's rows together see keys [wlo, whi]
    const int wlo = ma_first_key(p, pos0 + rbase), whi = pos0 + min(rbase + 15, ntok - 1);
    const float slope = p.bias_kind == 1 ? p.bias[head] : 0.f;
    const float hscale = p.head_scale ? p.head_scale[head] : 1.f;
    const float inv_cap = p.softcap > 0.f ? 1.0f / p.softcap : 0.f;
    constexpr float kLog2e = 1.4426950408889634f;

    for (int sn = 0; sn < steps.count; ++sn) {
        const int buf = sn % NST, c0 = steps.step(sn) * kMmKeys;
        if (sn + NST - 1 < steps.count) load_tile(steps.step(sn + NST - 1), (sn + NST - 1) % NST);
        cp_async_commit();
        cp_async_wait<NST - 1>();
        __syncthreads();
        if (active && ((c0 + kMmKeys - 1 >= wlo && c0 <= whi) || c0 < keep)) {
        float s[8][4];
#pragma unroll
        for (int t = 0; t < 8; ++t)
#pragma unroll
            for (int c = 0; c < 4; ++c) s[t][c] = 0.f;
#pragma unroll
        for (int ks = 0; ks < DIM; ks += 16) {
            if (ks >= dim) continue;                         // all padding
            uint32_t a[4];
            ldsm_x4(smem_u32(Qs + (rbase + (lane & 15)) * KS + ks + (lane >> 4) * 8), a[0], a[1], a[2], a[3]);
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(smem_u32(Ks + (buf * kMmKeys + np * 16 + (lane & 7) + ((lane >> 4) << 3)) * KS + ks + ((lane >> 3) & 1) * 8),
                        b0, b1, b2, b3);
                mma_bf16_16816(s[2 * np], a, b0, b1);
                mma_bf16_16816(s[2 * np + 1], a, b2, b3);
            }
        }
        // ---- float scores -> weights (log2 domain)
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            const int col = t * 8 + 2 * (lane & 3);
            const int2 okk = *reinterpret_cast<const int2*>(&key_ok[buf][col]);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int i = c >> 1, j = c0 + col + (c & 1);
                const bool vis = ((c & 1) ? okk.y : okk.x) && j <= rpos[i] && (j >= rlo[i] || j < keep);
                float v = s[t][c] * p.scale;
                if (p.head_scale) v *= hscale;
                if (p.softcap > 0.f) v = p.softcap * ma_tanh(v * inv_cap);
                if (p.bias_kind == 1) v -= slope * (float)(rpos[i] - j);
                else if (p.bias_kind == 2 && vis) {
                    const int dist = min(rpos[i] - j, p.bias_len - 1);
                    v += bias_smem ? Bs[dist] : p.bias[(int64_t)dist * p.heads + head];
                }
                s[t][c] = vis ? v * kLog2e : -INFINITY;
                mx[i] = fmaxf(mx[i], s[t][c]);
            }
        }
        float ref[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
            const float mn = fmaxf(m[i], mx[i]);
            ref[i] = mn == -INFINITY ? 0.f : mn;
            const float corr = exp2f(m[i] - ref[i]);         // m = -inf: 0 (nothing accumulated yet)
            m[i] = mn;
            l[i] *= corr;
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                o[t][2 * i] *= corr;
                o[t][2 * i + 1] *= corr;
            }
        }
#pragma unroll
        for (int t = 0; t < 8; ++t)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                s[t][c] = exp2f(s[t][c] - ref[c >> 1]);
                l[c >> 1] += s[t][c];
            }
        // ---- weighted sums
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t a[4];
            a[0] = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                if (np * 16 >= vdim) continue;               // all padding
                uint32_t b0, b1, b2, b3;
                ldsm_x4_trans(smem_u32(Vs + (buf * kMmKeys + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + np * 16 + (lane >> 4) * 8),
                              b0, b1, b2, b3);
                mma_bf16_16816(o[2 * np], a, b0, b1);
                mma_bf16_16816(o[2 * np + 1], a, b2, b3);
            }
        }
        }
        __syncthreads();                                     // this buffer is free for the copies of step kt + NST
    }
    cp_async_wait<0>();
    if (!active) return;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
        const int r = rbase + (lane >> 2) + 8 * i;
        if (r >= ntok) continue;
        float inv = 1.0f / l[i];
        if (p.sink) {                                        // the running maximum is in the log2 domain
            const float sk = p.sink[head] * kLog2e, mn = fmaxf(m[i], sk);
            const float corr = exp2f(m[i] - mn);
            inv = corr / (l[i] * corr + exp2f(sk - mn));
        }
        bf16_t* dst = static_cast<bf16_t*>(p.out) + (int64_t)(row0 + r) * p.heads * vdim + (int64_t)head * vdim + 2 * (lane & 3);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            if (t * 8 >= vdim) continue;
            float u = o[t][2 * i] * inv, v = o[t][2 * i + 1] * inv;
            if (p.out_rot) {                                 // a thread holds both columns of a pair
                const int col = t * 8 + 2 * (lane & 3);
                const float u0 = u;
                u = ma_unturn(p, row0 + r, col, u0, v);
                v = ma_unturn(p, row0 + r, col + 1, v, u0);
            }
            *reinterpret_cast<uint32_t*>(dst + t * 8) = pack_bf16x2(u, v);
        }
    }
}

template <int DIM, int VDIM>
static int mm_launch(const MaskAttnParams& p, int ntiles, cudaStream_t st) {
    size_t smem = ((size_t)(kMmRows + kMmStages * kMmKeys) * (DIM + kMmPad) + (size_t)kMmStages * kMmKeys * (VDIM + kMmPad)) * sizeof(bf16_t);
    if (p.bias_kind == 2 && p.bias_len <= kMmBiasMax) smem += (size_t)p.bias_len * sizeof(float);
    auto kern = masked_attention_mma_kernel<DIM, VDIM>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((unsigned)ntiles, (unsigned)p.heads);
    kern<<<grid, kMmThreads, smem, st>>>(p);
    PA_RETURN_LAUNCH_STATUS();
}

static bool mm_shape_ok(int dim, int vdim) { return dim % 8 == 0 && dim <= 128 && vdim % 8 == 0 && vdim <= 128; }
static int mm_padded(int n) { return n <= 32 ? 32 : n <= 64 ? 64 : 128; }

// PA_ERR_UNSUPPORTED: this shape or these pointers stay on the float kernel
static int mm_dispatch(const MaskAttnParams& p, int ntiles, cudaStream_t st) {
    if (!mm_shape_ok(p.dim, p.vdim) || p.q_stride % 8 || p.q_off % 8) return PA_ERR_UNSUPPORTED;
    if ((uintptr_t)p.q % 16 || (uintptr_t)p.k_pool % 16 || (uintptr_t)p.v_pool % 16 || (uintptr_t)p.out % 4) return PA_ERR_UNSUPPORTED;
    const int dp = mm_padded(p.dim), vp = mm_padded(p.vdim);
#define PA_MM_CASE(D, V) if (dp == D && vp == V) return mm_launch<D, V>(p, ntiles, st)
    PA_MM_CASE(32, 32); PA_MM_CASE(32, 64); PA_MM_CASE(32, 128);
    PA_MM_CASE(64, 32); PA_MM_CASE(64, 64); PA_MM_CASE(64, 128);
    PA_MM_CASE(128, 32); PA_MM_CASE(128, 64); PA_MM_CASE(128, 128);
#undef PA_MM_CASE
    return PA_ERR_UNSUPPORTED;
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
    return pa_masked_attention_sink(d_q, q_stride, q_off, d_k_pool, d_v_pool, d_table, num_slots, num_kv_heads, num_tiles,
                                    total_pages, tile_size, d_q_tiles, num_q_tiles, heads, dim, vdim, scale, softcap,
                                    mask_kind, mask_size, 0, bias_kind, d_bias, bias_len, nullptr, nullptr, nullptr, d_out,
                                    elem, tile_kind, stream);
}

PA_API int pa_masked_attention_sink(const void* d_q, int64_t q_stride, int q_off, const void* d_k_pool, const void* d_v_pool,
                                    const int32_t* d_table, int num_slots, int num_kv_heads, int num_tiles, int total_pages,
                                    int tile_size, const int32_t* d_q_tiles, int num_q_tiles, int heads, int dim, int vdim,
                                    float scale, float softcap, int mask_kind, int mask_size, int mask_keep, int bias_kind,
                                    const float* d_bias, int bias_len, const float* d_head_scale, const float* d_sink,
                                    const float* d_out_rot, void* d_out, int elem, int tile_kind, pa_stream_t stream) {
    PA_CHECK_ARG(mask_keep >= 0 && (mask_keep == 0 || mask_kind == 1) && (!d_out_rot || vdim % 2 == 0));
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
    p.head_scale = d_head_scale; p.sink = d_sink; p.mask_keep = mask_keep; p.out_rot = d_out_rot;
    if (elem != 4 && elem != 2) return PA_ERR_UNSUPPORTED;
    if (tile_kind == 2) {       // on the tensor cores: tiles of up to pa_masked_attention_mma_tile_tokens tokens
        if (elem != 2) return PA_ERR_UNSUPPORTED;
        return mm_dispatch(p, num_q_tiles, as_stream(stream));
    }
    if (tile_kind == 1) {       // every tile is one token: the streaming kernel, where it serves the shape
        const int st = elem == 4 ? ma_decode_dispatch<float>(p, num_q_tiles, as_stream(stream))
                                 : ma_decode_dispatch<bf16_t>(p, num_q_tiles, as_stream(stream));
        if (st != PA_ERR_UNSUPPORTED) return st;
    }
    if (elem == 4) return ma_dispatch<float>(p, num_q_tiles, as_stream(stream));
    return ma_dispatch<bf16_t>(p, num_q_tiles, as_stream(stream));
}

PA_API int pa_rope_kv_append(void* d_src, int64_t src_stride, int q_off, int k_off, int v_off, int heads, int kv_heads,
                             int dim, int vdim, int rot_dims, const float* d_rope, const float* d_value_rope,
                             void* d_k_pool, void* d_v_pool, const int32_t* d_table, int num_slots, int num_tiles,
                             int total_pages, int tile_size, const int32_t* d_row_slot, const int32_t* d_row_pos, int rows,
                             int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_src && rows >= 0 && heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0);
    PA_CHECK_ARG(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dim && (rot_dims == 0 || d_rope));
    PA_CHECK_ARG(!d_value_rope || vdim % 2 == 0);
    PA_CHECK_ARG(!d_k_pool || (d_v_pool && d_table && d_row_slot && d_row_pos && num_slots > 0 && num_tiles > 0 &&
                               total_pages > 0 && tile_size > 0));
    if (rows == 0) return PA_OK;
    const int64_t threads = (int64_t)rows * (heads + (d_k_pool ? kv_heads : 0)) * 32;
    PA_DISPATCH_ELEM(elem, rope_kv_append_kernel<T><<<(unsigned)((threads + 255) / 256), 256, 0, as_stream(stream)>>>(
                               static_cast<T*>(d_src), src_stride, q_off, k_off, v_off, heads, kv_heads, dim, vdim, rot_dims,
                               rot_dims ? d_rope : nullptr, d_value_rope, static_cast<T*>(d_k_pool),
                               static_cast<T*>(d_v_pool), d_table, num_slots, num_tiles, total_pages, tile_size, d_row_slot,
                               d_row_pos, rows));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_masked_attention_mma_tile_tokens(int dim, int vdim, int elem) {
    return elem == 2 && mm_shape_ok(dim, vdim) ? kMmRows : 0;
}
