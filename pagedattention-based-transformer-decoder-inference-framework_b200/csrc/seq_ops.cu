// seq_ops.cu -- per-token ops of decoder stacks that keep a float residual stream and per-sequence recurrent state,
// over a RAGGED batch: the rows of one step are the concatenated portions of several sequences (a portion is a run of
// consecutive tokens of one sequence: a prompt chunk, or a single decoded token).  A portion is described by
// (first row, length, state slot); a row by (state slot, position, row of the previous token or -1).
//
//   embedding_rows_kernel     x[r] = table[id[r]] as float
//   rms_shift_kernel          RMS norm (scalar or per-channel gain) + optional token shift against the previous token's
//                             normalised row (from the batch, or from the sequence's state slot at a portion's start)
//   rms_state_store_kernel    state slot <- normalised row of a portion's last token
//   mingru_scan_kernel        minGRU recurrence S_t = (1 - z_t) S_{t-1} + z_t c_t with the output gate, state in float
//   mingru_chunk_* kernels    the same recurrence for long portions as a three-pass chunked scan
//   gelu / silu-mul           activations between two matrix products
//   residual_combine_kernel   x += m * (mixer + dense ff + sum of routed expert rows + gate * shared expert)
//   residual_add_norm_kernel  x += rms_norm(y + sum_k w_k * routed expert rows) * gain  (norm on the sublayer's OUTPUT),
//                             optionally leaving the new x in the activation type for the next sublayer's products
//   residual_add_prenorm_kernel  x += a * y + b * y2 + sum_k w_k * routed expert rows + shared + bias, then the NEXT
//                             sublayer's operand h = x / rms(x) * gain in the activation type (pre-norm wiring: the
//                             residual add of one sublayer fused with the norm in front of the next)
//   concat_rows_kernel        [x | x0] of two float row sets in the activation type (input of a looped block)
//   residual_add_norm2_kernel  the parallel wiring with two norms: x += the sublayers' outputs (routed experts by weight,
//                             identity experts = the feed-forward's own input row), then BOTH operands of the next layer,
//                             x / rms(x) * gain1 and x / rms(x) * gain2, from one mean square
//   poly_norm_kernel          a N(z) + b N(z^2) + c N(z^3) + e per row, N = division by the root mean square of the row
//   logit_softcap_kernel      cap * tanh(scale * z / cap) on float logits
//
// Norms, the recurrence with its gates, and the residual sum are computed in float whatever the activation type.
#include "seq_common.cuh"

namespace pa {

template <typename T>
__global__ void embedding_rows_kernel(const T* __restrict__ table, const int32_t* __restrict__ ids, int rows, int width,
                                      int vocab, float scale, float* __restrict__ out) {
    const int r = blockIdx.x;
    const int id = ids[r];
    const bool ok = id >= 0 && id < vocab;
    const T* src = table + (int64_t)(ok ? id : 0) * width;
    for (int j = threadIdx.x; j < width; j += blockDim.x) out[(int64_t)r * width + j] = ok ? to_f32<T>(src[j]) * scale : 0.f;
}

__device__ __forceinline__ float row_inv_rms(const float* __restrict__ xr, int width, float eps, float* sm) {
    float s = 0.f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) s = fmaf(xr[j], xr[j], s);
    s = block_sum(s, sm);
    return 1.0f / sqrtf(s / (float)width + eps);
}

template <typename T>
__global__ void __launch_bounds__(256) rms_shift_kernel(const float* __restrict__ x, int width, float eps, float g_scalar,
                                                        const float* __restrict__ g_vec, const float* __restrict__ shift,
                                                        const int32_t* __restrict__ row_prev,
                                                        const int32_t* __restrict__ row_slot,
                                                        const float* __restrict__ state, T* __restrict__ out_h,
                                                        T* __restrict__ out_hs) {
    __shared__ float sm[32];
    const int row = blockIdx.x;
    const float* xr = x + (int64_t)row * width;
    const float r = row_inv_rms(xr, width, eps, sm);
    const bool shifted = shift != nullptr && out_hs != nullptr;
    const int prev = shifted ? row_prev[row] : -1;
    const float* xp = nullptr;
    const float* sp = nullptr;
    float rp = 0.f;
    if (shifted) {
        if (prev >= 0) {
            xp = x + (int64_t)prev * width;
            rp = row_inv_rms(xp, width, eps, sm);
        } else {
            sp = state + (int64_t)row_slot[row] * width;
        }
    }
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        const float g = g_vec ? g_vec[j] : g_scalar;
        const float h = xr[j] * r * g;
        if (out_h) out_h[(int64_t)row * width + j] = from_f32<T>(h);
        if (shifted) {
            const float hp = xp ? xp[j] * rp * g : sp[j];
            out_hs[(int64_t)row * width + j] = from_f32<T>(h + (hp - h) * shift[j]);
        }
    }
}

__global__ void __launch_bounds__(256) rms_state_store_kernel(const float* __restrict__ x, int width, float eps,
                                                              float g_scalar, const float* __restrict__ g_vec,
                                                              const int32_t* __restrict__ seq_start,
                                                              const int32_t* __restrict__ seq_len,
                                                              const int32_t* __restrict__ seq_slot,
                                                              float* __restrict__ state) {
    __shared__ float sm[32];
    const int s = blockIdx.x;
    if (seq_len[s] <= 0) return;
    const float* xr = x + (int64_t)(seq_start[s] + seq_len[s] - 1) * width;
    const float r = row_inv_rms(xr, width, eps, sm);
    float* dst = state + (int64_t)seq_slot[s] * width;
    for (int j = threadIdx.x; j < width; j += blockDim.x) dst[j] = xr[j] * r * (g_vec ? g_vec[j] : g_scalar);
}

// ---- minGRU ---------------------------------------------------------------------------------------------------------
// zxg row layout: [z pre-activation | candidate pre-activation | output-gate pre-activation], each `width` wide.
// A thread owns V adjacent channels (V = 2 where the width is even: one 4- or 8-byte load per row and field) and
// walks its tokens in order; the loads of the next tokens do not depend on the state and are issued ahead (unrolled).
template <typename T, int V> struct MinGruVec;
template <typename T> struct MinGruVec<T, 1> {
    static __device__ __forceinline__ void load(const T* p, float (&f)[1]) { f[0] = to_f32<T>(*p); }
    static __device__ __forceinline__ void store(T* p, const float (&f)[1]) { *p = from_f32<T>(f[0]); }
};
template <> struct MinGruVec<float, 2> {
    static __device__ __forceinline__ void load(const float* p, float (&f)[2]) {
        const float2 v = *reinterpret_cast<const float2*>(p);
        f[0] = v.x; f[1] = v.y;
    }
    static __device__ __forceinline__ void store(float* p, const float (&f)[2]) { *reinterpret_cast<float2*>(p) = make_float2(f[0], f[1]); }
};
template <> struct MinGruVec<bf16_t, 2> {
    static __device__ __forceinline__ void load(const bf16_t* p, float (&f)[2]) {
        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
        f[0] = v.x; f[1] = v.y;
    }
    static __device__ __forceinline__ void store(bf16_t* p, const float (&f)[2]) {
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(f[0], f[1]);
    }
};

// The logistic function of the scan.  float rows: the exact expf and division.  bfloat16 rows: ex2.approx and
// rcp.approx -- still float arithmetic, relative error ~1e-6, three orders below the rounding of the projections that
// feed it; the exact forms cost more instructions than the scan has memory time for.
template <typename T> __device__ __forceinline__ float mingru_sigmoid(float v) {
    return sizeof(T) == 2 ? __fdividef(1.0f, 1.0f + __expf(-v)) : sigmoid_f32(v);
}

template <typename T, int V>
struct MinGruStep {
    float a[V], b[V], gate[V];
    __device__ __forceinline__ MinGruStep(const T* __restrict__ row, int width, int c, const float (&zb)[V], const float (&xb)[V]) {
        float zr[V], ur[V], gr[V];
        MinGruVec<T, V>::load(row + c, zr);
        MinGruVec<T, V>::load(row + width + c, ur);
        MinGruVec<T, V>::load(row + 2 * width + c, gr);
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const float z = mingru_sigmoid<T>(zr[i] + zb[i]);
            const float u = ur[i] + xb[i];
            const float cand = u >= 0.f ? u + 0.5f : mingru_sigmoid<T>(u);
            a[i] = 1.0f - z;
            b[i] = z * cand;
            gate[i] = gr[i] * mingru_sigmoid<T>(gr[i]);
        }
    }
};

template <int V>
__device__ __forceinline__ void mingru_biases(const float* z_bias, const float* x_bias, int c, float (&zb)[V], float (&xb)[V]) {
#pragma unroll
    for (int i = 0; i < V; ++i) {
        zb[i] = z_bias ? z_bias[c + i] : 0.f;
        xb[i] = x_bias ? x_bias[c + i] : 0.f;
    }
}

template <typename T, int V>
__global__ void __launch_bounds__(128) mingru_scan_kernel(const T* __restrict__ zxg, const float* __restrict__ z_bias,
                                                          const float* __restrict__ x_bias, int width,
                                                          const int32_t* __restrict__ seq_start,
                                                          const int32_t* __restrict__ seq_len,
                                                          const int32_t* __restrict__ seq_slot, float* __restrict__ state,
                                                          T* __restrict__ y) {
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    const int s = blockIdx.y;
    if (c >= width) return;
    const int n = seq_len[s];
    if (n <= 0) return;
    const int64_t r0 = seq_start[s];
    float zb[V], xb[V], S[V], o[V];
    mingru_biases<V>(z_bias, x_bias, c, zb, xb);
    float* sp = state + (int64_t)seq_slot[s] * width + c;
#pragma unroll
    for (int i = 0; i < V; ++i) S[i] = sp[i];
#pragma unroll 4
    for (int t = 0; t < n; ++t) {
        const MinGruStep<T, V> st(zxg + (r0 + t) * 3 * width, width, c, zb, xb);
#pragma unroll
        for (int i = 0; i < V; ++i) {
            S[i] = st.a[i] * S[i] + st.b[i];
            o[i] = S[i] * st.gate[i];
        }
        MinGruVec<T, V>::store(y + (r0 + t) * width + c, o);
    }
#pragma unroll
    for (int i = 0; i < V; ++i) sp[i] = S[i];
}

// Chunked scan for long portions.  A portion is cut into chunks of `chunk` tokens (chunk list built by the host:
// chunk -> (first row, length, portion, index within portion)).  Pass 1: every (chunk, channel) folds its tokens into
// the pair (A, B) with S_out = A * S_in + B.  Pass 2: per (portion, channel) the chunk pairs are chained in order from
// the state slot, leaving each chunk's S_in in place of its A and the new state in the slot.  Pass 3: every chunk
// replays its tokens from S_in and writes the outputs.
template <typename T, int V>
__global__ void __launch_bounds__(128) mingru_chunk_fold_kernel(const T* __restrict__ zxg, const float* __restrict__ z_bias,
                                                                const float* __restrict__ x_bias, int width,
                                                                const int32_t* __restrict__ chunk_start,
                                                                const int32_t* __restrict__ chunk_len,
                                                                float* __restrict__ AB) {
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    const int k = blockIdx.y;
    if (c >= width) return;
    const int n = chunk_len[k];
    const int64_t r0 = chunk_start[k];
    float zb[V], xb[V], A[V], B[V];
    mingru_biases<V>(z_bias, x_bias, c, zb, xb);
#pragma unroll
    for (int i = 0; i < V; ++i) { A[i] = 1.f; B[i] = 0.f; }
#pragma unroll 8
    for (int t = 0; t < n; ++t) {
        const MinGruStep<T, V> st(zxg + (r0 + t) * 3 * width, width, c, zb, xb);
#pragma unroll
        for (int i = 0; i < V; ++i) {
            A[i] *= st.a[i];
            B[i] = st.a[i] * B[i] + st.b[i];
        }
    }
#pragma unroll
    for (int i = 0; i < V; ++i) {
        AB[((int64_t)k * 2) * width + c + i] = A[i];
        AB[((int64_t)k * 2 + 1) * width + c + i] = B[i];
    }
}

__global__ void __launch_bounds__(128) mingru_chunk_chain_kernel(float* __restrict__ AB, int width,
                                                                 const int32_t* __restrict__ seq_chunk0,
                                                                 const int32_t* __restrict__ seq_nchunks,
                                                                 const int32_t* __restrict__ seq_slot,
                                                                 float* __restrict__ state) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int s = blockIdx.y;
    if (c >= width) return;
    const int n = seq_nchunks[s];
    if (n <= 0) return;
    const int k0 = seq_chunk0[s];
    float* sp = state + (int64_t)seq_slot[s] * width + c;
    float S = *sp;
    // the pairs of 8 chunks are read before any incoming state is written over them: the loads do not wait on the chain
    constexpr int U = 8;
    for (int k = k0; k < k0 + n; k += U) {
        float A[U], B[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const bool ok = k + u < k0 + n;
            A[u] = ok ? AB[((int64_t)(k + u) * 2) * width + c] : 1.f;
            B[u] = ok ? AB[((int64_t)(k + u) * 2 + 1) * width + c] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (k + u < k0 + n) AB[((int64_t)(k + u) * 2) * width + c] = S;  // the chunk's incoming state
            S = A[u] * S + B[u];
        }
    }
    *sp = S;
}

template <typename T, int V>
__global__ void __launch_bounds__(128) mingru_chunk_apply_kernel(const T* __restrict__ zxg, const float* __restrict__ z_bias,
                                                                 const float* __restrict__ x_bias, int width,
                                                                 const int32_t* __restrict__ chunk_start,
                                                                 const int32_t* __restrict__ chunk_len,
                                                                 const float* __restrict__ AB, T* __restrict__ y) {
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    const int k = blockIdx.y;
    if (c >= width) return;
    const int n = chunk_len[k];
    const int64_t r0 = chunk_start[k];
    float zb[V], xb[V], S[V], o[V];
    mingru_biases<V>(z_bias, x_bias, c, zb, xb);
#pragma unroll
    for (int i = 0; i < V; ++i) S[i] = AB[((int64_t)k * 2) * width + c + i];
#pragma unroll 8
    for (int t = 0; t < n; ++t) {
        const MinGruStep<T, V> st(zxg + (r0 + t) * 3 * width, width, c, zb, xb);
#pragma unroll
        for (int i = 0; i < V; ++i) {
            S[i] = st.a[i] * S[i] + st.b[i];
            o[i] = S[i] * st.gate[i];
        }
        MinGruVec<T, V>::store(y + (r0 + t) * width + c, o);
    }
}

// ---- activations ----------------------------------------------------------------------------------------------------
template <typename T>
__global__ void gelu_kernel(T* __restrict__ x, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = from_f32<T>(gelu_erf_f32(to_f32<T>(x[i])));
}

// gu rows are [gate (ff) | up (ff)]; out[r, j] = act(gate_j) * up_j, act: 0 = silu, 1 = relu, 2 = tanh-form gelu
__device__ __forceinline__ float glu_act(float g, int act) {
    if (act == 1) return fmaxf(g, 0.f);
    if (act == 2) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    return silu_f32(g);
}

template <typename T>
__global__ void act_mul_kernel(const T* __restrict__ gu, int64_t rows, int ff, int act, T* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * ff) return;
    const int64_t r = i / ff;
    const int j = (int)(i % ff);
    const float g = to_f32<T>(gu[r * 2 * ff + j]), u = to_f32<T>(gu[r * 2 * ff + ff + j]);
    out[i] = from_f32<T>(glu_act(g, act) * u);
}

// the same on bfloat16 rows whose halves start on 16-byte boundaries: eight outputs per thread
__global__ void act_mul_bf16x8_kernel(const bf16_t* __restrict__ gu, int64_t rows, int ff, int act, bf16_t* __restrict__ out) {
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= rows * ff) return;
    const int64_t r = i / ff;
    const int j = (int)(i % ff);
    float g[8], u[8], o[8];
    bf16x8_unpack(*reinterpret_cast<const uint4*>(gu + r * 2 * ff + j), g);
    bf16x8_unpack(*reinterpret_cast<const uint4*>(gu + r * 2 * ff + ff + j), u);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = glu_act(g[k], act) * u[k];
    *reinterpret_cast<uint4*>(out + i) = bf16x8_pack(o);
}

template <typename T>
__global__ void residual_combine_kernel(float* __restrict__ x, int64_t rows, int width, float mult,
                                        const T* __restrict__ mix, const T* __restrict__ dense,
                                        const float* __restrict__ routed, int top, const T* __restrict__ shared,
                                        const float* __restrict__ shared_gate) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * width) return;
    const int64_t r = i / width;
    const int j = (int)(i % width);
    float s = 0.f;
    if (mix) s += to_f32<T>(mix[i]);
    if (dense) s += to_f32<T>(dense[i]);
    if (routed) {
        float e = 0.f;
        for (int k = 0; k < top; ++k) e += routed[(r * top + k) * width + j];
        s += e;
    }
    if (shared) s += (shared_gate ? shared_gate[r] : 1.0f) * to_f32<T>(shared[i]);
    x[i] = x[i] + mult * s;
}

// One CTA per row: s = y (activation type, optional) + sum_k w[r, k] * routed[(r, k)] (float pairs, optional);
// x[r] += s / sqrt(mean(s^2) + eps) * gain; the new row is also left in `next` (activation type) when asked for.
template <typename T>
__global__ void __launch_bounds__(256) residual_add_norm_kernel(float* __restrict__ x, int width, float eps,
                                                                const float* __restrict__ gain, const T* __restrict__ y,
                                                                const float* __restrict__ routed,
                                                                const float* __restrict__ sel_w, int top,
                                                                T* __restrict__ next) {
    extern __shared__ float row[];                    // [width]
    __shared__ float sm[32];
    const int64_t r = blockIdx.x;
    float ss = 0.f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        float s = y ? to_f32<T>(y[r * width + j]) : 0.f;
        if (routed)
            for (int k = 0; k < top; ++k) s = fmaf(sel_w ? sel_w[r * top + k] : 1.0f, routed[(r * top + k) * width + j], s);
        row[j] = s;
        ss = fmaf(s, s, ss);
    }
    ss = block_sum(ss, sm);
    const float rn = 1.0f / sqrtf(ss / (float)width + eps);
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        const float v = x[r * width + j] + row[j] * rn * gain[j];
        x[r * width + j] = v;
        if (next) next[r * width + j] = from_f32<T>(v);
    }
}

// One CTA per row.  Every addend is optional; `next` (with `gain`) is left out after the last sublayer.
template <typename T>
__global__ void __launch_bounds__(256) residual_add_prenorm_kernel(float* __restrict__ x, int width, const T* __restrict__ y,
                                                                   float y_scale, const T* __restrict__ y2, float y2_scale,
                                                                   const float* __restrict__ routed,
                                                                   const float* __restrict__ sel_w, int top,
                                                                   const T* __restrict__ shared, const float* __restrict__ bias,
                                                                   float eps, const float* __restrict__ gain,
                                                                   T* __restrict__ next) {
    extern __shared__ float row[];                    // [width]
    __shared__ float sm[32];
    const int64_t r = blockIdx.x;
    float ss = 0.f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        float s = 0.f;
        if (y) s = y_scale * to_f32<T>(y[r * width + j]);
        if (y2) s = fmaf(y2_scale, to_f32<T>(y2[r * width + j]), s);
        if (routed)
            for (int k = 0; k < top; ++k) s = fmaf(sel_w ? sel_w[r * top + k] : 1.0f, routed[(r * top + k) * width + j], s);
        if (shared) s += to_f32<T>(shared[r * width + j]);
        if (bias) s += bias[j];
        const float v = x[r * width + j] + s;
        x[r * width + j] = v;
        row[j] = v;
        ss = fmaf(v, v, ss);
    }
    if (!next) return;
    ss = block_sum(ss, sm);
    const float rn = 1.0f / sqrtf(ss / (float)width + eps);
    for (int j = threadIdx.x; j < width; j += blockDim.x) next[r * width + j] = from_f32<T>(row[j] * rn * gain[j]);
}

// One CTA per row.  s = y + y2 (activation type, optional) + sum_k w[r, k] * e_k, where e_k is the float row
// routed[(r, k)] of a real expert (sel_id < experts) or the row ident[r] itself (an identity expert); x[r] += s; then
// next1 = x / rms(x) * gain1 and next2 = x / rms(x) * gain2 (each optional) in the activation type.
template <typename T>
__global__ void __launch_bounds__(256) residual_add_norm2_kernel(float* __restrict__ x, int width, const T* __restrict__ y,
                                                                 const T* __restrict__ y2, const float* __restrict__ routed,
                                                                 const float* __restrict__ sel_w,
                                                                 const int32_t* __restrict__ sel_id, int top, int experts,
                                                                 const T* __restrict__ ident, float eps,
                                                                 const float* __restrict__ gain1, T* __restrict__ next1,
                                                                 const float* __restrict__ gain2, T* __restrict__ next2) {
    extern __shared__ float row[];                    // [width]
    __shared__ float sm[32];
    const int64_t r = blockIdx.x;
    float ss = 0.f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        float s = 0.f;
        if (y) s = to_f32<T>(y[r * width + j]);
        if (y2) s += to_f32<T>(y2[r * width + j]);
        if (routed) {
            float e = 0.f;
            for (int k = 0; k < top; ++k) {
                const bool same = sel_id && sel_id[r * top + k] >= experts;
                const float v = same ? to_f32<T>(ident[r * width + j]) : routed[(r * top + k) * width + j];
                e = fmaf(sel_w ? sel_w[r * top + k] : 1.0f, v, e);
            }
            s += e;
        }
        const float v = x[r * width + j] + s;
        x[r * width + j] = v;
        row[j] = v;
        ss = fmaf(v, v, ss);
    }
    if (!next1 && !next2) return;
    ss = block_sum(ss, sm);
    const float rn = 1.0f / sqrtf(ss / (float)width + eps);
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        const float v = row[j] * rn;
        if (next1) next1[r * width + j] = from_f32<T>(v * gain1[j]);
        if (next2) next2[r * width + j] = from_f32<T>(v * gain2[j]);
    }
}

// One CTA per row of `ff` values: the mean squares of z, z^2 and z^3 in one pass, then the weighted sum.
template <typename T>
__global__ void __launch_bounds__(256) poly_norm_kernel(const T* __restrict__ z, int ff, const float* __restrict__ coef,
                                                        float eps, T* __restrict__ out) {
    __shared__ float sm[32];
    const int64_t r = blockIdx.x;
    const T* zr = z + r * ff;
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    for (int j = threadIdx.x; j < ff; j += blockDim.x) {
        const float v = to_f32<T>(zr[j]), v2 = v * v;
        s1 += v2;
        s2 = fmaf(v2, v2, s2);
        s3 = fmaf(v2 * v, v2 * v, s3);
    }
    s1 = block_sum(s1, sm);
    s2 = block_sum(s2, sm);
    s3 = block_sum(s3, sm);
    const float n = (float)ff;
    const float a = coef[0] / sqrtf(s1 / n + eps), b = coef[1] / sqrtf(s2 / n + eps), c = coef[2] / sqrtf(s3 / n + eps);
    const float e = coef[3];
    for (int j = threadIdx.x; j < ff; j += blockDim.x) {
        const float v = to_f32<T>(zr[j]), v2 = v * v;
        out[r * ff + j] = from_f32<T>(a * v + b * v2 + c * (v2 * v) + e);
    }
}

__global__ void logit_softcap_kernel(float* __restrict__ z, int64_t n, float scale, float cap) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = z[i] * scale;
    z[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
}

template <typename T>
__global__ void concat_rows_kernel(const float* __restrict__ a, const float* __restrict__ b, int64_t rows, int width,
                                   T* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * 2 * width) return;
    const int64_t r = i / (2 * width);
    const int j = (int)(i % (2 * width));
    out[i] = from_f32<T>(j < width ? a[r * width + j] : b[r * width + j - width]);
}

template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ x, int64_t n, T* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_f32<T>(x[i]);
}

template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ src, const int32_t* __restrict__ rows, int n, int width,
                                   T* __restrict__ dst) {
    const int r = blockIdx.x;
    const T* s = src + (int64_t)rows[r] * width;
    for (int j = threadIdx.x; j < width; j += blockDim.x) dst[(int64_t)r * width + j] = s[j];
}

}  // namespace pa

using namespace pa;

PA_API int pa_embedding_rows_scaled(const void* d_table, int elem, const int32_t* d_ids, int rows, int width, int vocab,
                                    float scale, float* d_out, pa_stream_t stream) {
    PA_CHECK_ARG(d_table && d_ids && d_out && rows >= 0 && width > 0 && vocab > 0);
    if (rows == 0) return PA_OK;
    PA_DISPATCH_ELEM(elem, embedding_rows_kernel<T><<<rows, 256, 0, as_stream(stream)>>>(
                               static_cast<const T*>(d_table), d_ids, rows, width, vocab, scale, d_out));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_embedding_rows(const void* d_table, int elem, const int32_t* d_ids, int rows, int width, int vocab,
                             float* d_out, pa_stream_t stream) {
    return pa_embedding_rows_scaled(d_table, elem, d_ids, rows, width, vocab, 1.0f, d_out, stream);
}

PA_API int pa_rms_norm_shift(const float* d_x, int rows, int width, float eps, float gain, const float* d_gain_vec,
                             const float* d_shift, const int32_t* d_row_prev, const int32_t* d_row_slot,
                             const float* d_state, void* d_out, void* d_out_shifted, int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_x && rows >= 0 && width > 0 && (d_out || d_out_shifted));
    PA_CHECK_ARG(!(d_shift && d_out_shifted) || (d_row_prev && d_row_slot && d_state));
    if (rows == 0) return PA_OK;
    PA_DISPATCH_ELEM(elem, rms_shift_kernel<T><<<rows, 256, 0, as_stream(stream)>>>(
                               d_x, width, eps, gain, d_gain_vec, d_shift, d_row_prev, d_row_slot, d_state,
                               static_cast<T*>(d_out), static_cast<T*>(d_out_shifted)));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_rms_norm_state_store(const float* d_x, int width, float eps, float gain, const float* d_gain_vec,
                                   const int32_t* d_seq_start, const int32_t* d_seq_len, const int32_t* d_seq_slot,
                                   int num_seqs, float* d_state, pa_stream_t stream) {
    PA_CHECK_ARG(d_x && width > 0 && d_seq_start && d_seq_len && d_seq_slot && d_state && num_seqs >= 0);
    if (num_seqs == 0) return PA_OK;
    rms_state_store_kernel<<<num_seqs, 256, 0, as_stream(stream)>>>(d_x, width, eps, gain, d_gain_vec, d_seq_start,
                                                                   d_seq_len, d_seq_slot, d_state);
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_mingru_scan(const void* d_zxg, const float* d_z_bias, const float* d_x_bias, int width,
                          const int32_t* d_seq_start, const int32_t* d_seq_len, const int32_t* d_seq_slot, int num_seqs,
                          float* d_state, void* d_y, int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_zxg && width > 0 && d_seq_start && d_seq_len && d_seq_slot && d_state && d_y && num_seqs >= 0);
    if (num_seqs == 0) return PA_OK;
    // two channels per thread where every row, field and state pointer stays aligned for the paired loads
    const bool pair = width % 2 == 0 && (uintptr_t)d_zxg % 8 == 0 && (uintptr_t)d_y % 8 == 0;
    if (pair) {
        dim3 grid((unsigned)((width / 2 + 127) / 128), (unsigned)num_seqs);
        PA_DISPATCH_ELEM(elem, (mingru_scan_kernel<T, 2><<<grid, 128, 0, as_stream(stream)>>>(
                                   static_cast<const T*>(d_zxg), d_z_bias, d_x_bias, width, d_seq_start, d_seq_len,
                                   d_seq_slot, d_state, static_cast<T*>(d_y))));
    } else {
        dim3 grid((unsigned)((width + 127) / 128), (unsigned)num_seqs);
        PA_DISPATCH_ELEM(elem, (mingru_scan_kernel<T, 1><<<grid, 128, 0, as_stream(stream)>>>(
                                   static_cast<const T*>(d_zxg), d_z_bias, d_x_bias, width, d_seq_start, d_seq_len,
                                   d_seq_slot, d_state, static_cast<T*>(d_y))));
    }
    PA_RETURN_LAUNCH_STATUS();
}

PA_API size_t pa_mingru_chunked_workspace_bytes(int num_chunks, int width) {
    return num_chunks > 0 && width > 0 ? (size_t)num_chunks * 2 * width * sizeof(float) : 0;
}

PA_API int pa_mingru_scan_chunked(const void* d_zxg, const float* d_z_bias, const float* d_x_bias, int width,
                                  const int32_t* d_chunk_start, const int32_t* d_chunk_len, int num_chunks,
                                  const int32_t* d_seq_chunk0, const int32_t* d_seq_nchunks, const int32_t* d_seq_slot,
                                  int num_seqs, float* d_state, void* d_y, int elem, void* d_workspace,
                                  size_t workspace_bytes, pa_stream_t stream) {
    PA_CHECK_ARG(d_zxg && width > 0 && d_chunk_start && d_chunk_len && d_seq_chunk0 && d_seq_nchunks && d_seq_slot);
    PA_CHECK_ARG(d_state && d_y && num_seqs >= 0 && num_chunks >= 0);
    if (num_seqs == 0 || num_chunks == 0) return PA_OK;
    if (!d_workspace || workspace_bytes < pa_mingru_chunked_workspace_bytes(num_chunks, width)) return PA_ERR_WORKSPACE;
    float* AB = static_cast<float*>(d_workspace);
    const unsigned gx = (unsigned)((width + 127) / 128);
    cudaStream_t st = as_stream(stream);
    const bool pair = width % 2 == 0 && (uintptr_t)d_zxg % 8 == 0 && (uintptr_t)d_y % 8 == 0;
    const unsigned gv = pair ? (unsigned)((width / 2 + 127) / 128) : gx;
#define PA_MINGRU_CHUNKED(V)                                                                                           \
    PA_DISPATCH_ELEM(elem, {                                                                                           \
        mingru_chunk_fold_kernel<T, V><<<dim3(gv, (unsigned)num_chunks), 128, 0, st>>>(                                \
            static_cast<const T*>(d_zxg), d_z_bias, d_x_bias, width, d_chunk_start, d_chunk_len, AB);                  \
        mingru_chunk_chain_kernel<<<dim3(gx, (unsigned)num_seqs), 128, 0, st>>>(AB, width, d_seq_chunk0, d_seq_nchunks, \
                                                                               d_seq_slot, d_state);                   \
        mingru_chunk_apply_kernel<T, V><<<dim3(gv, (unsigned)num_chunks), 128, 0, st>>>(                               \
            static_cast<const T*>(d_zxg), d_z_bias, d_x_bias, width, d_chunk_start, d_chunk_len, AB,                   \
            static_cast<T*>(d_y));                                                                                     \
    })
    if (pair) PA_MINGRU_CHUNKED(2);
    else PA_MINGRU_CHUNKED(1);
#undef PA_MINGRU_CHUNKED
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_gelu_inplace(void* d_x, int64_t n, int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_x && n >= 0);
    if (n == 0) return PA_OK;
    PA_DISPATCH_ELEM(elem, gelu_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>(static_cast<T*>(d_x), n));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_act_mul(const void* d_gate_up, int64_t rows, int ff, int act, void* d_out, int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_gate_up && d_out && rows >= 0 && ff > 0 && act >= 0 && act <= 2);
    if (rows == 0) return PA_OK;
    const int64_t n = rows * ff;
    if (elem == 2 && ff % 8 == 0 && (uintptr_t)d_gate_up % 16 == 0 && (uintptr_t)d_out % 16 == 0) {
        act_mul_bf16x8_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, as_stream(stream)>>>(
            static_cast<const bf16_t*>(d_gate_up), rows, ff, act, static_cast<bf16_t*>(d_out));
        PA_RETURN_LAUNCH_STATUS();
    }
    PA_DISPATCH_ELEM(elem, act_mul_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>(
                               static_cast<const T*>(d_gate_up), rows, ff, act, static_cast<T*>(d_out)));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_silu_mul(const void* d_gate_up, int64_t rows, int ff, void* d_out, int elem, pa_stream_t stream) {
    return pa_act_mul(d_gate_up, rows, ff, 0, d_out, elem, stream);
}

PA_API int pa_residual_add_norm(float* d_x, int64_t rows, int width, float eps, const float* d_gain, const void* d_y,
                                const float* d_routed, const float* d_sel_w, int top, void* d_next, int elem,
                                pa_stream_t stream) {
    PA_CHECK_ARG(d_x && d_gain && rows >= 0 && width > 0 && (d_y || d_routed) && (!d_routed || top > 0));
    if (rows == 0) return PA_OK;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 48 * 1024) return PA_ERR_UNSUPPORTED;
    PA_DISPATCH_ELEM(elem, residual_add_norm_kernel<T><<<(unsigned)rows, 256, smem, as_stream(stream)>>>(
                               d_x, width, eps, d_gain, static_cast<const T*>(d_y), d_routed, d_sel_w, top,
                               static_cast<T*>(d_next)));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_residual_add_prenorm(float* d_x, int64_t rows, int width, const void* d_y, float y_scale, const void* d_y2,
                                   float y2_scale, const float* d_routed, const float* d_sel_w, int top,
                                   const void* d_shared, const float* d_bias, float eps, const float* d_gain, void* d_next,
                                   int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_x && rows >= 0 && width > 0 && (!d_routed || top > 0) && (!d_next || d_gain));
    if (rows == 0) return PA_OK;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 48 * 1024) return PA_ERR_UNSUPPORTED;
    PA_DISPATCH_ELEM(elem, residual_add_prenorm_kernel<T><<<(unsigned)rows, 256, smem, as_stream(stream)>>>(
                               d_x, width, static_cast<const T*>(d_y), y_scale, static_cast<const T*>(d_y2), y2_scale,
                               d_routed, d_sel_w, top, static_cast<const T*>(d_shared), d_bias, eps, d_gain,
                               static_cast<T*>(d_next)));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_residual_add_norm2(float* d_x, int64_t rows, int width, const void* d_y, const void* d_y2,
                                 const float* d_routed, const float* d_sel_w, const int32_t* d_sel_id, int top,
                                 int experts, const void* d_ident, float eps, const float* d_gain1, void* d_next1,
                                 const float* d_gain2, void* d_next2, int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_x && rows >= 0 && width > 0 && (!d_routed || top > 0) && (!d_next1 || d_gain1) && (!d_next2 || d_gain2));
    PA_CHECK_ARG(!d_sel_id || (d_routed && d_ident && experts >= 0));
    if (rows == 0) return PA_OK;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 48 * 1024) return PA_ERR_UNSUPPORTED;
    PA_DISPATCH_ELEM(elem, residual_add_norm2_kernel<T><<<(unsigned)rows, 256, smem, as_stream(stream)>>>(
                               d_x, width, static_cast<const T*>(d_y), static_cast<const T*>(d_y2), d_routed, d_sel_w,
                               d_sel_id, top, experts, static_cast<const T*>(d_ident), eps, d_gain1,
                               static_cast<T*>(d_next1), d_gain2, static_cast<T*>(d_next2)));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_poly_norm(const void* d_z, int64_t rows, int ff, const float* d_coef, float eps, void* d_out, int elem,
                        pa_stream_t stream) {
    PA_CHECK_ARG(d_z && d_coef && d_out && rows >= 0 && ff > 0);
    if (rows == 0) return PA_OK;
    PA_DISPATCH_ELEM(elem, poly_norm_kernel<T><<<(unsigned)rows, 256, 0, as_stream(stream)>>>(
                               static_cast<const T*>(d_z), ff, d_coef, eps, static_cast<T*>(d_out)));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_logit_softcap(float* d_logits, int64_t n, float scale, float cap, pa_stream_t stream) {
    PA_CHECK_ARG(d_logits && n >= 0 && cap >= 0.f);
    if (n == 0) return PA_OK;
    logit_softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>(d_logits, n, scale, cap);
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_concat_rows(const float* d_a, const float* d_b, int64_t rows, int width, void* d_out, int elem,
                          pa_stream_t stream) {
    PA_CHECK_ARG(d_a && d_b && d_out && rows >= 0 && width > 0);
    if (rows == 0) return PA_OK;
    const int64_t n = rows * 2 * width;
    PA_DISPATCH_ELEM(elem, concat_rows_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>(
                               d_a, d_b, rows, width, static_cast<T*>(d_out)));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_cast_rows(const float* d_x, int64_t n, void* d_out, int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_x && d_out && n >= 0);
    if (n == 0) return PA_OK;
    PA_DISPATCH_ELEM(elem, cast_rows_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>(
                               d_x, n, static_cast<T*>(d_out)));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_residual_combine(float* d_x, int64_t rows, int width, float mult, const void* d_mix, const void* d_dense,
                               const float* d_routed, int top, const void* d_shared, const float* d_shared_gate,
                               int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_x && rows >= 0 && width > 0 && (!d_routed || top > 0));
    if (rows == 0) return PA_OK;
    const int64_t n = rows * width;
    PA_DISPATCH_ELEM(elem, residual_combine_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>(
                               d_x, rows, width, mult, static_cast<const T*>(d_mix), static_cast<const T*>(d_dense),
                               d_routed, top, static_cast<const T*>(d_shared), d_shared_gate));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_gather_rows_f32(const float* d_src, const int32_t* d_rows, int n, int width, float* d_dst,
                              pa_stream_t stream) {
    PA_CHECK_ARG(d_src && d_rows && d_dst && n >= 0 && width > 0);
    if (n == 0) return PA_OK;
    gather_rows_kernel<float><<<n, 256, 0, as_stream(stream)>>>(d_src, d_rows, n, width, d_dst);
    PA_RETURN_LAUNCH_STATUS();
}
