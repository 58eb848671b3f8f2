// moe_ops.cu -- routed feed-forward experts for a batch of token rows.
//
//   router_topk_kernel       float router logits (+ optional bias), score function (sigmoid, softmax over all experts, or
//                            softmax over the chosen logits only), the `top` largest per row, optional renormalisation
//                            of the chosen scores, and an optional per-row shared-expert gate
//   moe_sort_kernel          groups the (row, choice) pairs by expert (counting sort) and lists the row tiles of the
//                            grouped matrix products
//   grouped_linear_kernel    out[i] = f(A[src(i)] * s(i)) . W[expert(i)]^T over the sorted pairs, one CTA per
//                            (row tile of one expert, column strip); float accumulation; three epilogues: gate/up pair
//                            with act(gate) * up, a single up product with act(up), or plain rows scattered back to the
//                            (row, choice) order as float
//
// Weights are [experts][out][in] in the activation type.  Where the design scales the expert's INPUT by the routing
// weight (instead of its output), `a_scale` carries the weight and the scaled row is rounded to the activation type
// before the product, like any other operand.
#include "seq_common.cuh"

namespace pa {

// ---- router ---------------------------------------------------------------------------------------------------------
// One warp per row.  score_fn: 0 = sigmoid, 1 = softmax over the experts, 2 = the largest LOGITS are chosen and the
// weights are the softmax over the chosen logits only.  Ties go to the lower expert id.  With ngroups > 1 the experts
// form ngroups equal groups of neighbours, a group's score is its largest score, and only experts of the `keep` best
// groups (ties: lower group) can be chosen.  choice_bias (optional, one float per expert) is added to the scores for the
// CHOICE only: the weights are the chosen experts' scores without it.  renorm divides the weights by their sum (+ 1e-20).
// The expert ids are not interpreted here: a caller may route over more outputs than it has expert weights (identity
// experts) and sort only the ids below its expert count.
// The dot products run over groups of kRtGroup weight vectors (the experts' rows and, last, the shared-expert gate's):
// a lane takes 16-byte pieces of the token row and multiplies each into the whole group, so the row is read once per
// group and the weights with 16-byte loads (VEC; rows whose width or alignment does not allow it go element by element).
constexpr int kRtGroup = 8;

template <typename T>
__device__ __forceinline__ void rt_load(const T* p, float (&f)[16 / sizeof(T)]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
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

template <typename T, bool VEC>
__global__ void __launch_bounds__(128) router_topk_kernel(const T* __restrict__ h, const float* __restrict__ w_router,
                                                          const float* __restrict__ bias,
                                                          const float* __restrict__ w_shared_gate, int rows, int width,
                                                          int experts, int top, int score_fn, int renorm,
                                                          int ngroups, int keep, const float* __restrict__ choice_bias,
                                                          int32_t* __restrict__ sel_id, float* __restrict__ sel_w,
                                                          float* __restrict__ shared_gate) {
    extern __shared__ float sc[];                     // [warps][experts]
    constexpr int VN = 16 / sizeof(T);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= rows) return;
    float* s = sc + warp * experts;
    const T* hr = h + (int64_t)row * width;
    const int nvec = experts + (w_shared_gate ? 1 : 0);
    for (int e0 = 0; e0 < nvec; e0 += kRtGroup) {
        float acc[kRtGroup];
        const float* wr[kRtGroup];
#pragma unroll
        for (int c = 0; c < kRtGroup; ++c) {
            acc[c] = 0.f;
            const int e = e0 + c;
            wr[c] = e < experts ? w_router + (int64_t)e * width : e < nvec ? w_shared_gate : nullptr;
        }
        if (VEC) {
            for (int j = lane * VN; j < width; j += 32 * VN) {
                float hv[VN];
                rt_load<T>(hr + j, hv);
#pragma unroll
                for (int c = 0; c < kRtGroup; ++c) {
                    if (!wr[c]) continue;
#pragma unroll
                    for (int i = 0; i < VN; i += 4) {
                        const float4 w4 = *reinterpret_cast<const float4*>(wr[c] + j + i);
                        acc[c] = fmaf(hv[i], w4.x, acc[c]);
                        acc[c] = fmaf(hv[i + 1], w4.y, acc[c]);
                        acc[c] = fmaf(hv[i + 2], w4.z, acc[c]);
                        acc[c] = fmaf(hv[i + 3], w4.w, acc[c]);
                    }
                }
            }
        } else {
            for (int j = lane; j < width; j += 32) {
                const float hv = to_f32<T>(hr[j]);
#pragma unroll
                for (int c = 0; c < kRtGroup; ++c)
                    if (wr[c]) acc[c] = fmaf(hv, wr[c][j], acc[c]);
            }
        }
#pragma unroll
        for (int c = 0; c < kRtGroup; ++c) {
            const int e = e0 + c;
            if (e >= nvec) continue;
            const float v = warp_sum(acc[c]);
            if (lane == 0) {
                if (e < experts) s[e] = bias ? v + bias[e] : v;
                else shared_gate[row] = sigmoid_f32(v);
            }
        }
    }
    __syncwarp();
    if (lane == 0) {
        if (score_fn == 0) {
            for (int e = 0; e < experts; ++e) s[e] = sigmoid_f32(s[e]);
        } else if (score_fn == 1) {
            float m = -INFINITY, z = 0.f;
            for (int e = 0; e < experts; ++e) m = fmaxf(m, s[e]);
            for (int e = 0; e < experts; ++e) { s[e] = expf(s[e] - m); z += s[e]; }
            for (int e = 0; e < experts; ++e) s[e] /= z;
        }
        if (ngroups > 1 && keep < ngroups) {          // only the experts of the `keep` groups with the largest maxima stay
            const int gsz = experts / ngroups;
            unsigned long long kept = 0ull;           // ngroups <= 64
            for (int k = 0; k < keep; ++k) {
                int bg = -1;
                float bv = -INFINITY;
                for (int gi = 0; gi < ngroups; ++gi) {
                    if (kept >> gi & 1ull) continue;
                    float gm = -INFINITY;
                    for (int e = gi * gsz; e < (gi + 1) * gsz; ++e) gm = fmaxf(gm, s[e]);
                    if (bg < 0 || gm > bv) { bv = gm; bg = gi; }
                }
                kept |= 1ull << bg;
            }
            for (int e = 0; e < experts; ++e)
                if (!(kept >> (e / gsz) & 1ull)) s[e] = -INFINITY;
        }
        float total = 0.f;
        for (int k = 0; k < top; ++k) {
            int best = 0;
            float bv = -INFINITY;
            for (int e = 0; e < experts; ++e) {
                const float v = choice_bias ? s[e] + choice_bias[e] : s[e];
                if (v > bv) { bv = v; best = e; }
            }
            sel_id[(int64_t)row * top + k] = best;
            sel_w[(int64_t)row * top + k] = s[best];
            total += s[best];
            s[best] = -INFINITY;
        }
        if (score_fn == 2) {                          // softmax over the chosen logits (the first chosen is the largest)
            const float m = sel_w[(int64_t)row * top];
            total = 0.f;
            for (int k = 0; k < top; ++k) {
                const float ex = expf(sel_w[(int64_t)row * top + k] - m);
                sel_w[(int64_t)row * top + k] = ex;
                total += ex;
            }
        }
        if (renorm || score_fn == 2)
            for (int k = 0; k < top; ++k) sel_w[(int64_t)row * top + k] /= total + 1e-20f;
    }
}

// ---- grouping -------------------------------------------------------------------------------------------------------
// One CTA.  meta layout (int32): [0, E] exclusive offsets of the experts' pair ranges; then `max_tiles` entries of
// (expert, first sorted pair, pairs) -- expert = -1 marks an unused tile.  order[i] = the (row * top + choice) index of
// sorted pair i.  Pairs of one expert keep no particular order: every output row depends on its own input row only.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int32_t* __restrict__ sel_id, int n, int experts, int tile_rows,
                                                        int max_tiles, int32_t* __restrict__ order,
                                                        int32_t* __restrict__ meta) {
    extern __shared__ int sh[];                       // [experts] counts, [experts + 1] offsets, [experts] cursors
    int* cnt = sh;
    int* off = sh + experts;
    int* cur = off + experts + 1;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int e = sel_id[i];
        if (e >= 0 && e < experts) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0, t = 0;
        int32_t* tiles = meta + experts + 1;
        for (int e = 0; e < experts; ++e) {
            off[e] = acc;
            cur[e] = acc;
            meta[e] = acc;
            for (int r = 0; r < cnt[e] && t < max_tiles; r += tile_rows, ++t) {
                tiles[3 * t] = e;
                tiles[3 * t + 1] = acc + r;
                tiles[3 * t + 2] = min(tile_rows, cnt[e] - r);
            }
            acc += cnt[e];
        }
        off[experts] = acc;
        meta[experts] = acc;
        for (; t < max_tiles; ++t) { tiles[3 * t] = -1; tiles[3 * t + 1] = 0; tiles[3 * t + 2] = 0; }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int e = sel_id[i];
        if (e >= 0 && e < experts) order[atomicAdd(&cur[e], 1)] = i;
    }
}

// ---- grouped product ------------------------------------------------------------------------------------------------
constexpr int kGlBM = 64, kGlBN = 64, kGlBK = 32;   // kGlBM is also the row tile of the tensor-core kernel

// MODE 0: A rows gathered from the token rows (order[i] / top), scaled by a_scale[order[i]]; W[e] = [2 * n_out][K]
//         (gate rows, then up rows); out[i][n] = silu(gate) * up in the activation type, sorted order.
// MODE 1: A rows = sorted rows i; W[e] = [n_out][K]; out_f32[order[i]][n] (scatter to the (row, choice) order).
// MODE 2: A rows as MODE 0; W[e] = [n_out][K]; out[i][n] = act(product) in the activation type, sorted order.
// act (MODE 0: of the gate, MODE 2: of the product): 0 = silu, 1 = relu, 2 = relu squared.
__device__ __forceinline__ float expert_act(float v, int act) {
    if (act == 1) return fmaxf(v, 0.f);
    if (act == 2) { const float r = fmaxf(v, 0.f); return r * r; }
    return silu_f32(v);
}

template <typename T, int MODE>
__global__ void __launch_bounds__(256) grouped_linear_kernel(const T* __restrict__ A, int64_t lda, const T* __restrict__ W,
                                                             int K, int n_out, const int32_t* __restrict__ order,
                                                             const float* __restrict__ a_scale, int top,
                                                             const int32_t* __restrict__ tiles, T* __restrict__ out,
                                                             float* __restrict__ out_f32, int act) {
    __shared__ float As[kGlBK][kGlBM + 1];
    __shared__ float Bs[kGlBK][kGlBN + 1];
    __shared__ float Bu[MODE == 0 ? kGlBK : 1][kGlBN + 1];
    __shared__ int src_row[kGlBM];
    __shared__ float src_scale[kGlBM];
    const int e = tiles[3 * blockIdx.x];
    if (e < 0) return;
    const int i0 = tiles[3 * blockIdx.x + 1], nr = tiles[3 * blockIdx.x + 2];
    const int n0 = blockIdx.y * kGlBN;
    const int w_rows = MODE == 0 ? 2 * n_out : n_out;
    const T* We = W + (int64_t)e * w_rows * K;
    if (threadIdx.x < kGlBM) {
        const int r = threadIdx.x;
        int sr = -1;
        float sc = 1.f;
        if (r < nr) {
            const int pair = order[i0 + r];
            if (MODE != 1) {
                sr = pair / top;
                if (a_scale) sc = a_scale[pair];
            } else {
                sr = i0 + r;
            }
        }
        src_row[r] = sr;
        src_scale[r] = sc;
    }
    constexpr int RT = kGlBM / 16;                            // rows per thread
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;   // rows ty*RT .. +RT-1, columns tx*4 .. +3
    float acc[RT][4], accu[RT][4];
#pragma unroll
    for (int a = 0; a < RT; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = accu[a][b] = 0.f;
    for (int k0 = 0; k0 < K; k0 += kGlBK) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < kGlBM * kGlBK; idx += 256) {
            const int r = idx / kGlBK, kk = idx % kGlBK;
            float v = 0.f;
            const int sr = src_row[r];
            if (sr >= 0 && k0 + kk < K) {
                v = to_f32<T>(A[(int64_t)sr * lda + k0 + kk]);
                if (MODE != 1 && a_scale) v = to_f32<T>(from_f32<T>(v * src_scale[r]));
            }
            As[kk][r] = v;
        }
        for (int idx = threadIdx.x; idx < kGlBN * kGlBK; idx += 256) {
            const int n = idx / kGlBK, kk = idx % kGlBK;
            float v = 0.f, u = 0.f;
            if (n0 + n < n_out && k0 + kk < K) {
                v = to_f32<T>(We[(int64_t)(n0 + n) * K + k0 + kk]);
                if (MODE == 0) u = to_f32<T>(We[(int64_t)(n_out + n0 + n) * K + k0 + kk]);
            }
            Bs[kk][n] = v;
            if (MODE == 0) Bu[kk][n] = u;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < kGlBK; ++kk) {
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const float w = Bs[kk][tx * 4 + b];
                const float u = MODE == 0 ? Bu[kk][tx * 4 + b] : 0.f;
#pragma unroll
                for (int a = 0; a < RT; ++a) {
                    const float av = As[kk][ty * RT + a];
                    acc[a][b] = fmaf(av, w, acc[a][b]);
                    if (MODE == 0) accu[a][b] = fmaf(av, u, accu[a][b]);
                }
            }
        }
    }
#pragma unroll
    for (int a = 0; a < RT; ++a) {
        const int r = ty * RT + a;
        if (r >= nr) continue;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int n = n0 + tx * 4 + b;
            if (n >= n_out) continue;
            if (MODE == 0) {
                // the two products leave the accumulator in the activation type, like every other projection
                const float gte = to_f32<T>(from_f32<T>(acc[a][b])), up = to_f32<T>(from_f32<T>(accu[a][b]));
                out[(int64_t)(i0 + r) * n_out + n] = from_f32<T>(expert_act(gte, act) * up);
            } else if (MODE == 2) {
                out[(int64_t)(i0 + r) * n_out + n] = from_f32<T>(expert_act(to_f32<T>(from_f32<T>(acc[a][b])), act));
            } else {
                out_f32[(int64_t)order[i0 + r] * n_out + n] = acc[a][b];
            }
        }
    }
}

// ---- the same product on the tensor cores (bfloat16 operands, float accumulation) -------------------------------------
// CTA = 4 warps on a 64-row x 128-weight-row tile, K in steps of 32.  The weight tile comes through a ring of three
// shared-memory buffers filled by 16-byte cp.async copies two steps ahead; the token rows (gathered, and scaled in MODE
// 0) go through registers into two buffers, one step ahead.  MODE 0: weight rows [n0, n0 + 64) (gate) and the matching up
// rows, so a thread holds gate and up of the same output and applies silu(gate) * up itself; MODE 1: 128 output columns.
// Operands reach the mma.sync.m16n8k16 fragments through ldmatrix from rows padded to 80 bytes (conflict-free).
// Needs K % 8 == 0 and 16-byte aligned rows (the dispatcher falls back to the kernel above otherwise).
constexpr int kMmBK = 32, kMmLd = 40, kMmBRows = 128, kMmStages = 3;

__device__ __forceinline__ uint4 scale_bf16x8(uint4 v, float sc) {
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(p[i]);
        p[i] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
    }
    return v;
}

template <int MODE>
__global__ void __launch_bounds__(128) grouped_mma_kernel(const bf16_t* __restrict__ A, int64_t lda,
                                                          const bf16_t* __restrict__ W, int K, int n_out,
                                                          const int32_t* __restrict__ order,
                                                          const float* __restrict__ a_scale, int top,
                                                          const int32_t* __restrict__ tiles, bf16_t* __restrict__ out,
                                                          float* __restrict__ out_f32, int act) {
    __shared__ __align__(16) bf16_t As[2][kGlBM][kMmLd];
    __shared__ __align__(16) bf16_t Bs[kMmStages][kMmBRows][kMmLd];
    __shared__ int src_row[kGlBM];
    __shared__ float src_scale[kGlBM];
    const int e = tiles[3 * blockIdx.x];
    if (e < 0) return;
    const int i0 = tiles[3 * blockIdx.x + 1], nr = tiles[3 * blockIdx.x + 2];
    constexpr int NCOL = MODE == 0 ? 64 : 128;                     // outputs per CTA
    const int n0 = blockIdx.y * NCOL;
    const int w_rows = MODE == 0 ? 2 * n_out : n_out;
    const bf16_t* We = W + (int64_t)e * w_rows * K;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < kGlBM) {
        int sr = -1;
        float sc = 1.f;
        if (tid < nr) {
            const int pair = order[i0 + tid];
            if (MODE != 1) {
                sr = pair / top;
                if (a_scale) sc = a_scale[pair];
            } else {
                sr = i0 + tid;
            }
        }
        src_row[tid] = sr;
        src_scale[tid] = sc;
    }
    __syncthreads();
    // loaders: A tile 64 rows x 4 vectors of 8 -> 2 per thread; B tile 128 rows x 4 vectors -> 4 per thread
    const int lv = tid & 3;                                        // vector (8 elements) within the K step
    uint4 ra[2];
    auto load_regs = [&](int k0) {
        const int k = k0 + lv * 8;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int r = (tid >> 2) + j * 32;
            const int sr = src_row[r];
            uint4 v = make_uint4(0, 0, 0, 0);
            if (sr >= 0 && k < K) {
                v = *reinterpret_cast<const uint4*>(A + (int64_t)sr * lda + k);
                if (MODE != 1 && a_scale) v = scale_bf16x8(v, src_scale[r]);
            }
            ra[j] = v;
        }
    };
    auto store_regs = [&](int buf) {
#pragma unroll
        for (int j = 0; j < 2; ++j) *reinterpret_cast<uint4*>(&As[buf][(tid >> 2) + j * 32][lv * 8]) = ra[j];
    };
    auto copy_weights = [&](int k0, int buf) {                    // 128 weight rows x 4 pieces -> 4 per thread
        const int k = k0 + lv * 8;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int r = (tid >> 2) + j * 32;                    // tile row 0..127
            int wr;                                               // weight row
            if (MODE == 0) wr = r < 64 ? n0 + r : n_out + n0 + (r - 64);
            else wr = n0 + r;
            const bool ok = (MODE == 0 ? (r < 64 ? n0 + r : n0 + r - 64) : n0 + r) < n_out && k < K;
            cp_async_16(smem_u32(&Bs[buf][r][lv * 8]), ok ? We + (int64_t)wr * K + k : We, ok);
        }
    };
    const int wm = warp & 1, wn = warp >> 1;                       // 32 rows x (MODE 0: 32 gate + 32 up | MODE 1: 64 columns)
    float acc[2][8][4];
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[a][b][c] = 0.f;
    const int nk = (K + kMmBK - 1) / kMmBK;
#pragma unroll
    for (int t = 0; t < kMmStages - 1; ++t) {
        if (t < nk) copy_weights(t * kMmBK, t);
        cp_async_commit();
    }
    load_regs(0);
    store_regs(0);
    for (int kt = 0; kt < nk; ++kt) {
        const int buf = kt & 1, wb = kt % kMmStages;
        if (kt + kMmStages - 1 < nk) copy_weights((kt + kMmStages - 1) * kMmBK, (kt + kMmStages - 1) % kMmStages);
        cp_async_commit();
        if (kt + 1 < nk) load_regs((kt + 1) * kMmBK);
        cp_async_wait<kMmStages - 1>();
        __syncthreads();                                           // weights of step kt have landed; As[buf] is written
#pragma unroll
        for (int ks = 0; ks < kMmBK; ks += 16) {
            uint32_t af[2][4];
#pragma unroll
            for (int a = 0; a < 2; ++a)
                ldsm_x4(smem_u32(&As[buf][wm * 32 + a * 16 + (lane & 15)][ks + (lane >> 4) * 8]), af[a][0], af[a][1], af[a][2], af[a][3]);
#pragma unroll
            for (int bp = 0; bp < 4; ++bp) {                      // pairs of 8-column tiles
                int brow;
                if (MODE == 0) brow = (bp < 2 ? 0 : 64) + wn * 32 + (bp & 1) * 16;
                else brow = wn * 64 + bp * 16;
                uint32_t b0, b1, b2, b3;
                ldsm_x4(smem_u32(&Bs[wb][brow + (lane & 7) + ((lane >> 4) << 3)][ks + ((lane >> 3) & 1) * 8]), b0, b1, b2, b3);
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    mma_bf16_16816(acc[a][bp * 2], af[a], b0, b1);
                    mma_bf16_16816(acc[a][bp * 2 + 1], af[a], b2, b3);
                }
            }
        }
        if (kt + 1 < nk) store_regs(buf ^ 1);
        __syncthreads();
    }
    // epilogue: c0,c1 -> row lane/4, columns 2*(lane%4) + {0,1}; c2,c3 -> row + 8
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            const int r = wm * 32 + a * 16 + hrow * 8 + (lane >> 2);
            if (r >= nr) continue;
            if (MODE == 0) {
#pragma unroll
                for (int t = 0; t < 4; ++t)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int n = n0 + wn * 32 + t * 8 + 2 * (lane & 3) + c;
                        if (n >= n_out) continue;
                        const float gte = __bfloat162float(__float2bfloat16_rn(acc[a][t][hrow * 2 + c]));
                        const float up = __bfloat162float(__float2bfloat16_rn(acc[a][t + 4][hrow * 2 + c]));
                        out[(int64_t)(i0 + r) * n_out + n] = __float2bfloat16_rn(expert_act(gte, act) * up);
                    }
            } else if (MODE == 2) {
                bf16_t* dst = out + (int64_t)(i0 + r) * n_out;
#pragma unroll
                for (int t = 0; t < 8; ++t)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int n = n0 + wn * 64 + t * 8 + 2 * (lane & 3) + c;
                        if (n < n_out)
                            dst[n] = __float2bfloat16_rn(expert_act(__bfloat162float(__float2bfloat16_rn(acc[a][t][hrow * 2 + c])), act));
                    }
            } else {
                float* dst = out_f32 + (int64_t)order[i0 + r] * n_out;
#pragma unroll
                for (int t = 0; t < 8; ++t)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int n = n0 + wn * 64 + t * 8 + 2 * (lane & 3) + c;
                        if (n < n_out) dst[n] = acc[a][t][hrow * 2 + c];
                    }
            }
        }
}

// ---- few rows per expert (decoding): the weights are the traffic -------------------------------------------------------
// With few pairs per expert (skinny_ok) the sort cuts the experts' ranges into row tiles of 16.  CTA = 4 warps on one
// such tile x 32 weight rows (MODE 0: 16 gate rows and the matching 16 up rows; MODE 1: 32 output columns).  Nothing is
// staged: the warps split K into interleaved pieces of 32, and a lane reads 16 bytes (8 consecutive k) of ITS weight
// row and of its two token rows straight into the mma.sync.m16n8k16 fragments.  The sum over k does not care about
// order, so the 8 values a lane holds stand for k slots {2t, 2t+1, 2t+8, 2t+9} of two consecutive MMAs -- the same
// assignment on both operands.  All loads of a step (16 weight and 8 token pieces per lane) are issued before its first
// MMA; many small CTAs keep the whole chip's memory system busy.  The warps' partial sums meet in shared memory.
// Same argument rules as the kernel above.
constexpr int kSkRows = 16, kSkChunk = 32, kSkUnroll = 4, kSkWarps = 4, kSkCols = 32;

static bool skinny_ok(int pairs, int experts) { return pairs <= 32 * experts; }
static int moe_tile_rows(int pairs, int experts) { return skinny_ok(pairs, experts) ? kSkRows : kGlBM; }

template <int MODE>
__global__ void __launch_bounds__(kSkWarps * 32) grouped_skinny_kernel(const bf16_t* __restrict__ A, int64_t lda,
                                                                       const bf16_t* __restrict__ W, int K, int n_out,
                                                                       const int32_t* __restrict__ order,
                                                                       const float* __restrict__ a_scale, int top,
                                                                       const int32_t* __restrict__ tiles,
                                                                       bf16_t* __restrict__ out, float* __restrict__ out_f32,
                                                                       int act) {
    __shared__ float red[kSkWarps][kSkRows][kSkCols + 1];
    const int e = tiles[3 * blockIdx.x];
    if (e < 0) return;
    const int i0 = tiles[3 * blockIdx.x + 1], nr = tiles[3 * blockIdx.x + 2];
    constexpr int NCOL = MODE == 0 ? 16 : 32;                      // outputs per CTA
    const int n0 = blockIdx.y * NCOL;
    const int w_rows = MODE == 0 ? 2 * n_out : n_out;
    const bf16_t* We = W + (int64_t)e * w_rows * K;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    // this lane's two token rows (g and g + 8 of the tile) and their input factors
    const bf16_t* arow[2];
    float asc[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = g + 8 * i;
        arow[i] = nullptr;
        asc[i] = 1.f;
        if (r < nr) {
            const int pair = order[i0 + r];
            arow[i] = A + (int64_t)(MODE != 1 ? pair / top : i0 + r) * lda;
            if (MODE != 1 && a_scale) asc[i] = a_scale[pair];
        }
    }
    // this lane's weight row of each of the 4 column tiles (nullptr: past the end)
    const bf16_t* wrow[4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
        int col, wr;
        if (MODE == 0) { col = n0 + (nt & 1) * 8 + g; wr = (nt < 2 ? 0 : n_out) + col; }
        else { col = n0 + nt * 8 + g; wr = col; }
        wrow[nt] = col < n_out ? We + (int64_t)wr * K : nullptr;
    }
    float acc[4][4];
#pragma unroll
    for (int b = 0; b < 4; ++b)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[b][c] = 0.f;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int kc = warp * kSkChunk; kc < K; kc += kSkWarps * kSkChunk * kSkUnroll) {
        uint4 wv[kSkUnroll][4], av[kSkUnroll][2];
#pragma unroll
        for (int u = 0; u < kSkUnroll; ++u) {
            const int k = kc + u * kSkWarps * kSkChunk + 8 * t;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) wv[u][nt] = (wrow[nt] && k < K) ? ldg_stream_128(wrow[nt] + k) : zero;
#pragma unroll
            for (int i = 0; i < 2; ++i) av[u][i] = (arow[i] && k < K) ? *reinterpret_cast<const uint4*>(arow[i] + k) : zero;
        }
#pragma unroll
        for (int u = 0; u < kSkUnroll; ++u) {
            uint4 x = av[u][0], y = av[u][1];
            if (MODE != 1 && a_scale) {
                x = scale_bf16x8(x, asc[0]);
                y = scale_bf16x8(y, asc[1]);
            }
            const uint32_t a_lo[4] = {x.x, y.x, x.y, y.y}, a_hi[4] = {x.z, y.z, x.w, y.w};
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                mma_bf16_16816(acc[nt], a_lo, wv[u][nt].x, wv[u][nt].y);
                mma_bf16_16816(acc[nt], a_hi, wv[u][nt].z, wv[u][nt].w);
            }
        }
    }
    // c0,c1 -> row g, columns 2t + {0,1} of the column tile; c2,c3 -> row g + 8
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) red[warp][g + (c >> 1) * 8][nt * 8 + 2 * t + (c & 1)] = acc[nt][c];
    __syncthreads();
    for (int idx = tid; idx < nr * NCOL; idx += kSkWarps * 32) {
        const int r = idx / NCOL, c = idx % NCOL;
        if (n0 + c >= n_out) continue;
        if (MODE == 0) {
            float gte = 0.f, up = 0.f;
#pragma unroll
            for (int w = 0; w < kSkWarps; ++w) { gte += red[w][r][c]; up += red[w][r][16 + c]; }
            gte = __bfloat162float(__float2bfloat16_rn(gte));
            up = __bfloat162float(__float2bfloat16_rn(up));
            out[(int64_t)(i0 + r) * n_out + n0 + c] = __float2bfloat16_rn(expert_act(gte, act) * up);
        } else if (MODE == 2) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < kSkWarps; ++w) v += red[w][r][c];
            out[(int64_t)(i0 + r) * n_out + n0 + c] = __float2bfloat16_rn(expert_act(__bfloat162float(__float2bfloat16_rn(v)), act));
        } else {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < kSkWarps; ++w) v += red[w][r][c];
            out_f32[(int64_t)order[i0 + r] * n_out + n0 + c] = v;
        }
    }
}

static bool mma_ok(const void* A, int64_t lda, const void* W, int K) {
    return K % 8 == 0 && lda % 8 == 0 && (uintptr_t)A % 16 == 0 && (uintptr_t)W % 16 == 0;
}

}  // namespace pa

using namespace pa;

PA_API int pa_router_topk_grouped(const void* d_h, const float* d_w_router, const float* d_bias,
                                  const float* d_w_shared_gate, int rows, int width, int experts, int top, int score_fn,
                                  int renorm, int ngroups, int keep, int32_t* d_sel_id, float* d_sel_w,
                                  float* d_shared_gate, int elem, pa_stream_t stream) {
    return pa_router_topk_biased(d_h, d_w_router, d_bias, d_w_shared_gate, rows, width, experts, top, score_fn, renorm,
                                 ngroups, keep, nullptr, d_sel_id, d_sel_w, d_shared_gate, elem, stream);
}

PA_API int pa_router_topk_biased(const void* d_h, const float* d_w_router, const float* d_bias,
                                 const float* d_w_shared_gate, int rows, int width, int experts, int top, int score_fn,
                                 int renorm, int ngroups, int keep, const float* d_choice_bias, int32_t* d_sel_id,
                                 float* d_sel_w, float* d_shared_gate, int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_h && d_w_router && d_sel_id && d_sel_w && rows >= 0 && width > 0 && experts > 0);
    PA_CHECK_ARG(ngroups >= 1 && ngroups <= 64 && experts % ngroups == 0 && keep >= 1 && keep <= ngroups);
    PA_CHECK_ARG((int64_t)keep * (experts / ngroups) >= top);
    PA_CHECK_ARG(top > 0 && top <= experts && score_fn >= 0 && score_fn <= 2 && (!d_w_shared_gate || d_shared_gate));
    if (rows == 0) return PA_OK;
    if (experts > 2048) return PA_ERR_UNSUPPORTED;
    const size_t smem = (size_t)4 * experts * sizeof(float);
    // 16-byte pieces: every row of the tokens and of the float weight vectors must start on a 16-byte boundary
    const bool vec = width % 8 == 0 && (uintptr_t)d_h % 16 == 0 && (uintptr_t)d_w_router % 16 == 0 &&
                     (uintptr_t)d_w_shared_gate % 16 == 0;
#define PA_ROUTER(VEC)                                                                                                 \
    PA_DISPATCH_ELEM(elem, (router_topk_kernel<T, VEC><<<(unsigned)((rows + 3) / 4), 128, smem, as_stream(stream)>>>(  \
                               static_cast<const T*>(d_h), d_w_router, d_bias, d_w_shared_gate, rows, width, experts, top, \
                               score_fn, renorm, ngroups, keep, d_choice_bias, d_sel_id, d_sel_w, d_shared_gate)))
    if (vec) PA_ROUTER(true);
    else PA_ROUTER(false);
#undef PA_ROUTER
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_router_topk(const void* d_h, const float* d_w_router, const float* d_bias, const float* d_w_shared_gate,
                          int rows, int width, int experts, int top, int score_fn, int renorm, int32_t* d_sel_id,
                          float* d_sel_w, float* d_shared_gate, int elem, pa_stream_t stream) {
    return pa_router_topk_grouped(d_h, d_w_router, d_bias, d_w_shared_gate, rows, width, experts, top, score_fn, renorm, 1,
                                  1, d_sel_id, d_sel_w, d_shared_gate, elem, stream);
}

PA_API int pa_moe_tile_rows(void) { return kGlBM; }

PA_API int pa_moe_max_tiles(int pairs, int experts) {
    if (pairs <= 0 || experts <= 0) return 0;
    const int tr = moe_tile_rows(pairs, experts);
    return (pairs + tr - 1) / tr + experts;
}

PA_API size_t pa_moe_meta_ints(int pairs, int experts) {
    return (size_t)experts + 1 + 3 * (size_t)pa_moe_max_tiles(pairs, experts);
}

PA_API int pa_moe_sort(const int32_t* d_sel_id, int pairs, int experts, int32_t* d_order, int32_t* d_meta,
                       pa_stream_t stream) {
    PA_CHECK_ARG(d_sel_id && d_order && d_meta && pairs >= 0 && experts > 0);
    if (pairs == 0) return PA_OK;
    if (experts > 4096) return PA_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(3 * experts + 1) * sizeof(int);
    moe_sort_kernel<<<1, 1024, smem, as_stream(stream)>>>(d_sel_id, pairs, experts, moe_tile_rows(pairs, experts), pa_moe_max_tiles(pairs, experts),
                                                         d_order, d_meta);
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_moe_gate_up_act(const void* d_h, int64_t ldh, const void* d_w_gate_up, int width, int ff, int experts,
                              const int32_t* d_order, const float* d_sel_w, int top, const int32_t* d_meta, int pairs,
                              int act, void* d_act, int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_h && d_w_gate_up && d_order && d_meta && d_act && width > 0 && ff > 0 && experts > 0 && top > 0);
    PA_CHECK_ARG(act >= 0 && act <= 2);
    if (pairs <= 0) return PA_OK;
    dim3 grid((unsigned)pa_moe_max_tiles(pairs, experts), (unsigned)((ff + kGlBN - 1) / kGlBN));
    const int32_t* tiles = d_meta + experts + 1;
    if (elem == 2 && mma_ok(d_h, ldh, d_w_gate_up, width) && skinny_ok(pairs, experts)) {
        dim3 gs((unsigned)pa_moe_max_tiles(pairs, experts), (unsigned)((ff + 15) / 16));
        grouped_skinny_kernel<0><<<gs, kSkWarps * 32, 0, as_stream(stream)>>>(
            static_cast<const bf16_t*>(d_h), ldh, static_cast<const bf16_t*>(d_w_gate_up), width, ff, d_order, d_sel_w, top,
            tiles, static_cast<bf16_t*>(d_act), nullptr, act);
        PA_RETURN_LAUNCH_STATUS();
    }
    if (elem == 2 && mma_ok(d_h, ldh, d_w_gate_up, width)) {
        grouped_mma_kernel<0><<<grid, 128, 0, as_stream(stream)>>>(
            static_cast<const bf16_t*>(d_h), ldh, static_cast<const bf16_t*>(d_w_gate_up), width, ff, d_order, d_sel_w, top,
            tiles, static_cast<bf16_t*>(d_act), nullptr, act);
        PA_RETURN_LAUNCH_STATUS();
    }
    PA_DISPATCH_ELEM(elem, grouped_linear_kernel<T, 0><<<grid, 256, 0, as_stream(stream)>>>(
                               static_cast<const T*>(d_h), ldh, static_cast<const T*>(d_w_gate_up), width, ff, d_order,
                               d_sel_w, top, tiles, static_cast<T*>(d_act), nullptr, act));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_moe_gate_up(const void* d_h, int64_t ldh, const void* d_w_gate_up, int width, int ff, int experts,
                          const int32_t* d_order, const float* d_sel_w, int top, const int32_t* d_meta, int pairs,
                          void* d_act, int elem, pa_stream_t stream) {
    return pa_moe_gate_up_act(d_h, ldh, d_w_gate_up, width, ff, experts, d_order, d_sel_w, top, d_meta, pairs, 0, d_act, elem,
                              stream);
}

PA_API int pa_moe_up(const void* d_h, int64_t ldh, const void* d_w_up, int width, int ff, int experts,
                     const int32_t* d_order, const float* d_sel_w, int top, const int32_t* d_meta, int pairs, int act,
                     void* d_act, int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_h && d_w_up && d_order && d_meta && d_act && width > 0 && ff > 0 && experts > 0 && top > 0);
    PA_CHECK_ARG(act >= 0 && act <= 2);
    if (pairs <= 0) return PA_OK;
    const unsigned nt = (unsigned)pa_moe_max_tiles(pairs, experts);
    const int32_t* tiles = d_meta + experts + 1;
    if (elem == 2 && mma_ok(d_h, ldh, d_w_up, width) && skinny_ok(pairs, experts)) {
        grouped_skinny_kernel<2><<<dim3(nt, (unsigned)((ff + kSkCols - 1) / kSkCols)), kSkWarps * 32, 0, as_stream(stream)>>>(
            static_cast<const bf16_t*>(d_h), ldh, static_cast<const bf16_t*>(d_w_up), width, ff, d_order, d_sel_w, top, tiles,
            static_cast<bf16_t*>(d_act), nullptr, act);
        PA_RETURN_LAUNCH_STATUS();
    }
    if (elem == 2 && mma_ok(d_h, ldh, d_w_up, width)) {
        grouped_mma_kernel<2><<<dim3(nt, (unsigned)((ff + 127) / 128)), 128, 0, as_stream(stream)>>>(
            static_cast<const bf16_t*>(d_h), ldh, static_cast<const bf16_t*>(d_w_up), width, ff, d_order, d_sel_w, top, tiles,
            static_cast<bf16_t*>(d_act), nullptr, act);
        PA_RETURN_LAUNCH_STATUS();
    }
    PA_DISPATCH_ELEM(elem, grouped_linear_kernel<T, 2><<<dim3(nt, (unsigned)((ff + kGlBN - 1) / kGlBN)), 256, 0, as_stream(stream)>>>(
                               static_cast<const T*>(d_h), ldh, static_cast<const T*>(d_w_up), width, ff, d_order, d_sel_w, top,
                               tiles, static_cast<T*>(d_act), nullptr, act));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_moe_down(const void* d_act, const void* d_w_down, int ff, int width, int experts, const int32_t* d_order,
                       const int32_t* d_meta, int pairs, float* d_out_pairs, int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_act && d_w_down && d_order && d_meta && d_out_pairs && width > 0 && ff > 0 && experts > 0);
    if (pairs <= 0) return PA_OK;
    dim3 grid((unsigned)pa_moe_max_tiles(pairs, experts), (unsigned)((width + kGlBN - 1) / kGlBN));
    const int32_t* tiles = d_meta + experts + 1;
    if (elem == 2 && mma_ok(d_act, ff, d_w_down, ff) && skinny_ok(pairs, experts)) {
        dim3 gs((unsigned)pa_moe_max_tiles(pairs, experts), (unsigned)((width + kSkCols - 1) / kSkCols));
        grouped_skinny_kernel<1><<<gs, kSkWarps * 32, 0, as_stream(stream)>>>(
            static_cast<const bf16_t*>(d_act), (int64_t)ff, static_cast<const bf16_t*>(d_w_down), ff, width, d_order, nullptr, 1,
            tiles, nullptr, d_out_pairs, 0);
        PA_RETURN_LAUNCH_STATUS();
    }
    if (elem == 2 && mma_ok(d_act, ff, d_w_down, ff)) {
        dim3 g2((unsigned)pa_moe_max_tiles(pairs, experts), (unsigned)((width + 127) / 128));
        grouped_mma_kernel<1><<<g2, 128, 0, as_stream(stream)>>>(
            static_cast<const bf16_t*>(d_act), (int64_t)ff, static_cast<const bf16_t*>(d_w_down), ff, width, d_order, nullptr, 1,
            tiles, nullptr, d_out_pairs, 0);
        PA_RETURN_LAUNCH_STATUS();
    }
    PA_DISPATCH_ELEM(elem, grouped_linear_kernel<T, 1><<<grid, 256, 0, as_stream(stream)>>>(
                               static_cast<const T*>(d_act), (int64_t)ff, static_cast<const T*>(d_w_down), ff, width,
                               d_order, nullptr, 1, tiles, nullptr, d_out_pairs, 0));
    PA_RETURN_LAUNCH_STATUS();
}
