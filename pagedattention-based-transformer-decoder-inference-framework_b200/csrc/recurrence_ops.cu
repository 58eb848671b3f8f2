// recurrence_ops.cu -- matrix-state recurrences over a RAGGED batch (see seq_ops.cu for the batch description) and the
// small ops around them.
//
//   causal_conv_kernel        per-channel causal convolution over the tokens of a sequence (taps from the config, the
//                             last column of the weight is the current token's) + bias + silu; inputs before a portion's
//                             first token come from the sequence's state slot, which holds its last taps - 1 inputs
//   conv_state_kernel         state slot <- the last taps - 1 inputs of a portion (older ones slide out)
//   decay_scan_kernel         S_t = a_t S_{t-1} + k_t (s_t v_t)^T,  o_t = S_t^T q_t + skip * v_t   per head, S is dim x vdim,
//                             float, one slot per sequence.  The decay is a constant of the head (linear attention with
//                             decay), or a_t = exp(-exp(A_log) dt_t) with dt_t = softplus(raw_t + bias) and s_t = dt_t
//                             (selective state space); q / k may be shared by the heads of a group; q, k, v may pass silu
//   decay_chunk_* kernels     the same recurrence for long portions as a three-pass chunked scan (fold every chunk from a
//                             zero state, chain the chunks from the state slot, replay every chunk from its incoming state)
//   gated_norm_kernel         RMS norm in equal groups of a float row with a per-channel weight and a gate from another
//                             buffer: silu(gate) multiplied in BEFORE the norm, or sigmoid(gate) AFTER it
//
// States, decays and their logarithms, softplus, step sizes and the norms are float whatever the activation type.
#include "seq_common.cuh"

namespace pa {

// ---- causal convolution -----------------------------------------------------------------------------------------------
// chunks: [n][4] = first row, tokens, slot, offset of the first token within its portion.  A thread owns one channel of
// one chunk and slides a window of kMaxTaps inputs along it.
constexpr int kMaxTaps = 8;

template <typename T>
__global__ void __launch_bounds__(128) causal_conv_kernel(const T* __restrict__ in, int64_t in_stride, int in_off, int channels,
                                                          int taps, const float* __restrict__ w, const float* __restrict__ bias,
                                                          const float* __restrict__ state, const int32_t* __restrict__ chunks,
                                                          T* __restrict__ out, int64_t out_stride, int act) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int* ch = chunks + 4 * blockIdx.y;
    const int row0 = ch[0], n = ch[1], slot = ch[2], off = ch[3];
    float wt[kMaxTaps], win[kMaxTaps];
#pragma unroll
    for (int i = 0; i < kMaxTaps; ++i) wt[i] = i < taps ? w[(int64_t)c * taps + (taps - 1 - i)] : 0.f;   // wt[i]: i tokens back
    const float b = bias ? bias[c] : 0.f;
    const float* st = state + (int64_t)slot * (taps - 1) * channels;
    // win[i] = input i + 1 tokens before the chunk's first token
#pragma unroll
    for (int i = 0; i < kMaxTaps - 1; ++i) {
        float v = 0.f;
        if (i < taps - 1) {
            const int t = off - 1 - i;                 // offset within the portion
            v = t >= 0 ? to_f32<T>(in[(int64_t)(row0 - 1 - i) * in_stride + in_off + c]) : st[(int64_t)(taps - 1 + t) * channels + c];
        }
        win[i + 1] = v;
    }
    for (int t = 0; t < n; ++t) {
        win[0] = to_f32<T>(in[(int64_t)(row0 + t) * in_stride + in_off + c]);
        float acc = b;
#pragma unroll
        for (int i = 0; i < kMaxTaps; ++i) acc = fmaf(wt[i], win[i], acc);
        out[(int64_t)(row0 + t) * out_stride + c] = from_f32<T>(act ? silu_f32(acc) : acc);
#pragma unroll
        for (int i = kMaxTaps - 1; i > 0; --i) win[i] = win[i - 1];
    }
}

template <typename T>
__global__ void __launch_bounds__(128) conv_state_kernel(const T* __restrict__ in, int64_t in_stride, int in_off, int channels,
                                                         int taps, const int32_t* __restrict__ seq_start,
                                                         const int32_t* __restrict__ seq_len, const int32_t* __restrict__ seq_slot,
                                                         float* __restrict__ state) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int s = blockIdx.y, n = seq_len[s], r0 = seq_start[s];
    if (n <= 0) return;
    float* st = state + (int64_t)seq_slot[s] * (taps - 1) * channels;
    float nv[kMaxTaps];
#pragma unroll
    for (int i = 0; i < kMaxTaps - 1; ++i) {
        nv[i] = 0.f;
        if (i < taps - 1) {
            const int t = n - (taps - 1) + i;          // offset within the portion of the input that lands in place i
            nv[i] = t >= 0 ? to_f32<T>(in[(int64_t)(r0 + t) * in_stride + in_off + c]) : st[(int64_t)(taps - 1 + t) * channels + c];
        }
    }
#pragma unroll
    for (int i = 0; i < kMaxTaps - 1; ++i)
        if (i < taps - 1) st[(int64_t)i * channels + c] = nv[i];
}

// ---- the recurrence ---------------------------------------------------------------------------------------------------
struct DecayScanParams {
    const void* q; int64_t q_stride; int q_off;       // q of head h: q_off + (h / heads_per_group) * dim
    const void* k; int64_t k_stride; int k_off;
    const void* v; int64_t v_stride; int v_off;       // v of head h: v_off + h * vdim
    int heads, groups, dim, vdim;
    int act;                                          // 1: q, k and v pass silu as they are read
    const float* decay;                               // [heads] constant decays (dt == nullptr)
    const void* dt; int64_t dt_stride; int dt_off;    // raw step size of head h at dt_off + h
    const float* dt_bias; const float* a_log; const float* skip;   // [heads] each (dt != nullptr); skip may be null
    float* state;                                     // [slots][heads][dim][vdim]
    float* out; int64_t out_stride;                   // float rows [heads * vdim]
    // work items: [n][4] = first row, tokens, slot, kind-specific; mode 0: a portion from / to its state slot;
    // mode 1: fold a chunk from a zero state into part[item]; mode 2: replay a chunk from part[item] (no state written)
    const int32_t* items;
    int mode;
    int vec;                                          // every staged piece of q, k and v starts on a 16-byte boundary
    float* part;                                      // [items][heads][dim * vdim + 1]: state, then the chunk's total decay
};

constexpr int kDsTokens = 16;                         // tokens staged per step
constexpr int kDsMaxThreads = 128;

__device__ __forceinline__ float softplus_f32(float z) { return z > 20.f ? z : log1pf(expf(z)); }

template <typename T>
__device__ __forceinline__ void ds_load16(const T* __restrict__ p, float (&f)[16 / sizeof(T)]) {
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

// A thread keeps a DPT x CPT block of the state in registers: lane = (column group) * NSL + (row slice), so the NSL
// threads that share a column group cover NSL * DPT >= dim rows and their partial outputs meet in a shuffle reduction.
// q, k, v, the decays and the input scales of kDsTokens tokens are staged in shared memory per step (one 16-byte read of
// q and of k feeds 4 x CPT updates and as many output terms).  MODE 0: a portion from / to its state slot; 1: fold a
// chunk from a zero state into part[item] (no outputs); 2: replay a chunk from part[item] (no state written).
template <typename T, int DPT, int MODE, int CPT>
__global__ void __launch_bounds__(kDsMaxThreads) decay_scan_kernel(const DecayScanParams p, int NSL) {
    extern __shared__ __align__(16) float ds_smem[];
    const int dpad = NSL * DPT;
    const int ccols = blockDim.x / NSL * CPT;       // value columns of this CTA
    float* Qs = ds_smem;                               // [kDsTokens][dpad]
    float* Ks = Qs + kDsTokens * dpad;                 // [kDsTokens][dpad]
    float* Vs = Ks + kDsTokens * dpad;                 // [kDsTokens][ccols]
    float* As = Vs + kDsTokens * ccols;                // [kDsTokens] decay
    float* Ss = As + kDsTokens;                        // [kDsTokens] input scale
    const int slice = threadIdx.x % NSL, cgrp = threadIdx.x / NSL;
    const int h = blockIdx.y, cl = cgrp * CPT, c = blockIdx.z * ccols + cl;
    const int g = h / (p.heads / p.groups);
    const int* it = p.items + 4 * blockIdx.x;
    const int row0 = it[0], n = it[1], slot = it[2];
    const int d0 = slice * DPT;
    const int64_t sz = (int64_t)p.dim * p.vdim;

    float S[DPT][CPT];
    const float* src = MODE == 0 ? p.state + ((int64_t)slot * p.heads + h) * sz
                     : MODE == 2 ? p.part + ((int64_t)blockIdx.x * p.heads + h) * (sz + 1) : nullptr;
#pragma unroll
    for (int i = 0; i < DPT; ++i)
#pragma unroll
        for (int j = 0; j < CPT; ++j)
            S[i][j] = (MODE != 1 && d0 + i < p.dim && c + j < p.vdim) ? src[(int64_t)(d0 + i) * p.vdim + c + j] : 0.f;
    float total = 1.f;                                 // product of the decays (MODE 1)
    const float hd = p.dt ? 0.f : p.decay[h];
    const float a_rate = p.dt ? -expf(p.a_log[h]) : 0.f, dtb = p.dt ? p.dt_bias[h] : 0.f;
    const float skip = p.skip ? p.skip[h] : 0.f;
    const T* qb = static_cast<const T*>(p.q) + p.q_off + (int64_t)g * p.dim;
    const T* kb = static_cast<const T*>(p.k) + p.k_off + (int64_t)g * p.dim;
    const T* vb = static_cast<const T*>(p.v) + p.v_off + (int64_t)h * p.vdim + (int64_t)blockIdx.z * ccols;
    const int vcols = min(ccols, p.vdim - blockIdx.z * ccols);

    // rows whose pieces start on 16-byte boundaries are staged with 16-byte loads (`vec`, checked by the host); the columns
    // past dim / past this CTA's share of vdim are zeroed once and never written again
    constexpr int VN = 16 / sizeof(T);
    if (p.vec) {
        for (int idx = threadIdx.x; idx < kDsTokens * dpad; idx += blockDim.x) Qs[idx] = Ks[idx] = 0.f;
        for (int idx = threadIdx.x; idx < kDsTokens * ccols; idx += blockDim.x) Vs[idx] = 0.f;
    }
    for (int t0 = 0; t0 < n; t0 += kDsTokens) {
        const int nt = min(kDsTokens, n - t0);
        __syncthreads();
        if (p.vec) {
            const int kvecs = p.dim / VN, vvecs = vcols / VN;
            for (int idx = threadIdx.x; idx < nt * kvecs; idx += blockDim.x) {
                const int t = idx / kvecs, d = (idx % kvecs) * VN;
                float kf[VN], qf[VN];
                ds_load16<T>(kb + (int64_t)(row0 + t0 + t) * p.k_stride + d, kf);
                if (MODE != 1) ds_load16<T>(qb + (int64_t)(row0 + t0 + t) * p.q_stride + d, qf);
#pragma unroll
                for (int i = 0; i < VN; ++i) {
                    if (MODE == 1) qf[i] = 0.f;
                    if (p.act) { qf[i] = silu_f32(qf[i]); kf[i] = silu_f32(kf[i]); }
                }
#pragma unroll
                for (int i = 0; i < VN; i += 4) {
                    *reinterpret_cast<float4*>(Ks + t * dpad + d + i) = make_float4(kf[i], kf[i + 1], kf[i + 2], kf[i + 3]);
                    *reinterpret_cast<float4*>(Qs + t * dpad + d + i) = make_float4(qf[i], qf[i + 1], qf[i + 2], qf[i + 3]);
                }
            }
            for (int idx = threadIdx.x; idx < nt * vvecs; idx += blockDim.x) {
                const int t = idx / vvecs, cc = (idx % vvecs) * VN;
                float xf[VN];
                ds_load16<T>(vb + (int64_t)(row0 + t0 + t) * p.v_stride + cc, xf);
#pragma unroll
                for (int i = 0; i < VN; ++i)
                    if (p.act) xf[i] = silu_f32(xf[i]);
#pragma unroll
                for (int i = 0; i < VN; i += 4)
                    *reinterpret_cast<float4*>(Vs + t * ccols + cc + i) = make_float4(xf[i], xf[i + 1], xf[i + 2], xf[i + 3]);
            }
        } else {
        for (int idx = threadIdx.x; idx < nt * dpad; idx += blockDim.x) {
            const int t = idx / dpad, d = idx % dpad;
            float qv = 0.f, kv = 0.f;
            if (d < p.dim) {
                kv = to_f32<T>(kb[(int64_t)(row0 + t0 + t) * p.k_stride + d]);
                if (MODE != 1) qv = to_f32<T>(qb[(int64_t)(row0 + t0 + t) * p.q_stride + d]);
                if (p.act) { qv = silu_f32(qv); kv = silu_f32(kv); }
            }
            Qs[idx] = qv;
            Ks[idx] = kv;
        }
        for (int idx = threadIdx.x; idx < nt * ccols; idx += blockDim.x) {
            const int t = idx / ccols, cc = idx % ccols;
            float x = cc < vcols ? to_f32<T>(vb[(int64_t)(row0 + t0 + t) * p.v_stride + cc]) : 0.f;
            if (p.act) x = silu_f32(x);
            Vs[idx] = x;
        }
        }
        if (threadIdx.x < nt) {
            float a = hd, sc = 1.f;
            if (p.dt) {
                const float raw = to_f32<T>(static_cast<const T*>(p.dt)[(int64_t)(row0 + t0 + threadIdx.x) * p.dt_stride + p.dt_off + h]);
                sc = softplus_f32(raw + dtb);
                a = expf(a_rate * sc);
            }
            As[threadIdx.x] = a;
            Ss[threadIdx.x] = sc;
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float a = As[t], sc = Ss[t];
            float x[CPT];
            if (CPT == 4) {
                const float4 x4 = *reinterpret_cast<const float4*>(Vs + t * ccols + cl);
                x[0] = x4.x; x[1] = x4.y; x[CPT - 2] = x4.z; x[CPT - 1] = x4.w;
            } else {
                const float2 x2 = *reinterpret_cast<const float2*>(Vs + t * ccols + cl);
                x[0] = x2.x; x[1] = x2.y;
            }
            float xv[CPT], o[CPT];
#pragma unroll
            for (int j = 0; j < CPT; ++j) { xv[j] = x[j] * sc; o[j] = 0.f; }
            const float* kt = Ks + t * dpad + d0;
            const float* qt = Qs + t * dpad + d0;
#pragma unroll
            for (int i = 0; i < DPT; i += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(kt + i);
                const float kk[4] = {k4.x, k4.y, k4.z, k4.w};
                float qq[4] = {0.f, 0.f, 0.f, 0.f};
                if (MODE != 1) {
                    const float4 q4 = *reinterpret_cast<const float4*>(qt + i);
                    qq[0] = q4.x; qq[1] = q4.y; qq[2] = q4.z; qq[3] = q4.w;
                }
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int j = 0; j < CPT; ++j) {
                        S[i + u][j] = fmaf(a, S[i + u][j], kk[u] * xv[j]);
                        if (MODE != 1) o[j] = fmaf(S[i + u][j], qq[u], o[j]);
                    }
            }
            total *= a;
            if (MODE != 1) {
                for (int w = 1; w < NSL; w <<= 1)
#pragma unroll
                    for (int j = 0; j < CPT; ++j) o[j] += __shfl_xor_sync(0xffffffffu, o[j], w);
                if (slice == 0) {
                    float* dst = p.out + (int64_t)(row0 + t0 + t) * p.out_stride + (int64_t)h * p.vdim + c;
#pragma unroll
                    for (int j = 0; j < CPT; ++j)
                        if (c + j < p.vdim) dst[j] = fmaf(skip, x[j], o[j]);
                }
            }
        }
    }
    if (MODE == 2) return;
    float* dst = MODE == 0 ? p.state + ((int64_t)slot * p.heads + h) * sz : p.part + ((int64_t)blockIdx.x * p.heads + h) * (sz + 1);
#pragma unroll
    for (int i = 0; i < DPT; ++i)
#pragma unroll
        for (int j = 0; j < CPT; ++j)
            if (d0 + i < p.dim && c + j < p.vdim) dst[(int64_t)(d0 + i) * p.vdim + c + j] = S[i][j];
    if (MODE == 1 && threadIdx.x == 0 && blockIdx.z == 0) dst[sz] = total;
}

// Chain pass of the chunked scan: per (portion, head, state element) walk the portion's chunks in order from the state
// slot; every chunk's folded state is replaced by its INCOMING state, and the slot gets the state after the last chunk.
__global__ void __launch_bounds__(256) decay_chunk_chain_kernel(float* __restrict__ part, int heads, int64_t sz,
                                                                const int32_t* __restrict__ seq_chunk0,
                                                                const int32_t* __restrict__ seq_nchunks,
                                                                const int32_t* __restrict__ seq_slot, float* __restrict__ state) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int h = blockIdx.y, s = blockIdx.z;
    if (e >= sz) return;
    const int n = seq_nchunks[s], k0 = seq_chunk0[s];
    if (n <= 0) return;
    float* sp = state + ((int64_t)seq_slot[s] * heads + h) * sz + e;
    float S = *sp;
    // the folded values of 8 chunks are read before any incoming state is written over them: the loads do not wait on
    // the chain
    constexpr int U = 8;
    for (int k = k0; k < k0 + n; k += U) {
        float A[U], B[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const bool ok = k + u < k0 + n;
            const float* pk = part + ((int64_t)(ok ? k + u : k) * heads + h) * (sz + 1);
            A[u] = ok ? pk[sz] : 1.f;
            B[u] = ok ? pk[e] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (k + u < k0 + n) part[((int64_t)(k + u) * heads + h) * (sz + 1) + e] = S;
            S = fmaf(A[u], S, B[u]);
        }
    }
    *sp = S;
}

// ---- gated group norm ---------------------------------------------------------------------------------------------------
// One warp per (row, group).  gate_mode 0: none; 1: y <- y * silu(gate) before the norm; 2: out <- norm(y) * sigmoid(gate).
template <typename T>
__global__ void __launch_bounds__(256) gated_norm_kernel(const float* __restrict__ y, int64_t rows, int inner, int groups,
                                                         const T* __restrict__ gate, int64_t gate_stride, int gate_off,
                                                         int gate_mode, const float* __restrict__ weight, float eps,
                                                         T* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (w >= rows * groups) return;
    const int64_t r = w / groups;
    const int gsz = inner / groups, c0 = (int)(w % groups) * gsz;
    const float* yr = y + r * inner + c0;
    const T* gr = gate ? gate + r * gate_stride + gate_off + c0 : nullptr;
    float ss = 0.f;
    for (int j = lane; j < gsz; j += 32) {
        float v = yr[j];
        if (gate_mode == 1) v *= silu_f32(to_f32<T>(gr[j]));
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float rn = 1.0f / sqrtf(ss / (float)gsz + eps);
    for (int j = lane; j < gsz; j += 32) {
        float v = yr[j];
        if (gate_mode == 1) v *= silu_f32(to_f32<T>(gr[j]));
        v = v * rn * weight[c0 + j];
        if (gate_mode == 2) v *= sigmoid_f32(to_f32<T>(gr[j]));
        out[r * inner + c0 + j] = from_f32<T>(v);
    }
}

// the same with one CTA per (row, group): groups of many values, or few rows
template <typename T>
__global__ void __launch_bounds__(256) gated_norm_block_kernel(const float* __restrict__ y, int inner, int groups,
                                                               const T* __restrict__ gate, int64_t gate_stride, int gate_off,
                                                               int gate_mode, const float* __restrict__ weight, float eps,
                                                               T* __restrict__ out) {
    __shared__ float sm[32];
    const int64_t r = blockIdx.x / groups;
    const int gsz = inner / groups, c0 = (int)(blockIdx.x % groups) * gsz;
    const float* yr = y + r * inner + c0;
    const T* gr = gate ? gate + r * gate_stride + gate_off + c0 : nullptr;
    float ss = 0.f;
    for (int j = threadIdx.x; j < gsz; j += blockDim.x) {
        float v = yr[j];
        if (gate_mode == 1) v *= silu_f32(to_f32<T>(gr[j]));
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, sm);
    const float rn = 1.0f / sqrtf(ss / (float)gsz + eps);
    for (int j = threadIdx.x; j < gsz; j += blockDim.x) {
        float v = yr[j];
        if (gate_mode == 1) v *= silu_f32(to_f32<T>(gr[j]));
        v = v * rn * weight[c0 + j];
        if (gate_mode == 2) v *= sigmoid_f32(to_f32<T>(gr[j]));
        out[r * inner + c0 + j] = from_f32<T>(v);
    }
}

template <typename T, int DPT, int MODE, int CPT>
static int ds_launch(const DecayScanParams& p, int nitems, int NSL, cudaStream_t st) {
    // threads: enough column groups for vdim, whole warps, at most kDsMaxThreads
    int threads = (p.vdim + CPT - 1) / CPT * NSL;
    threads = (threads + 31) / 32 * 32;
    if (threads > kDsMaxThreads) threads = kDsMaxThreads;
    const int ccols = threads / NSL * CPT;
    DecayScanParams q = p;
    {   // 16-byte staging: pointers, row strides, column offsets, dim, vdim and a CTA's share of the columns all whole vectors
        const int VN = 16 / (int)sizeof(T);
        auto al = [&](const void* ptr, int64_t stride, int off) {
            return (uintptr_t)ptr % 16 == 0 && stride % VN == 0 && off % VN == 0;
        };
        q.vec = p.dim % VN == 0 && p.vdim % VN == 0 && ccols % VN == 0 && al(p.q, p.q_stride, p.q_off) &&
                al(p.k, p.k_stride, p.k_off) && al(p.v, p.v_stride, p.v_off);
    }
    const size_t smem = ((size_t)2 * kDsTokens * NSL * DPT + (size_t)kDsTokens * ccols + 2 * kDsTokens) * sizeof(float);
    if (smem > 200 * 1024) return PA_ERR_UNSUPPORTED;
    auto kern = decay_scan_kernel<T, DPT, MODE, CPT>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid((unsigned)nitems, (unsigned)p.heads, (unsigned)((p.vdim + ccols - 1) / ccols));
    kern<<<grid, threads, smem, st>>>(q, NSL);
    PA_RETURN_LAUNCH_STATUS();
}

// A thread's block of the state is DPT rows x CPT columns.  States of up to 64 rows: 16 x 4 (64 state registers, about
// twice the resident warps of 32 x 4; measured 1.3x faster at 64 rows).  Larger ones: 32 x 4.  Measured at 128 rows x 64
// columns: 16 x 4 (eight row slices, a three-round shuffle reduction) the same time, 32 x 2 (twice the warps, but twice
// the shared-memory operand reads per update) 1.6x slower -- the kernel is bound by those reads and the shuffles, so the
// block that feeds the most updates per read wins.
template <typename T, int MODE>
static int ds_dispatch(const DecayScanParams& p, int nitems, cudaStream_t st) {
    if (p.dim <= 8) return ds_launch<T, 8, MODE, 4>(p, nitems, 1, st);
    if (p.dim <= 64) return ds_launch<T, 16, MODE, 4>(p, nitems, p.dim <= 16 ? 1 : p.dim <= 32 ? 2 : 4, st);
    int NSL = 4;
    while (NSL * 32 < p.dim) NSL <<= 1;
    if (NSL > 32) return PA_ERR_UNSUPPORTED;
    return ds_launch<T, 32, MODE, 4>(p, nitems, NSL, st);
}

}  // namespace pa

using namespace pa;

PA_API int pa_causal_conv_silu(const void* d_in, int64_t in_stride, int in_off, int channels, int taps, const float* d_weight,
                               const float* d_bias, const float* d_state, const int32_t* d_chunks, int num_chunks,
                               void* d_out, int64_t out_stride, int elem, pa_stream_t stream) {
    return pa_causal_conv(d_in, in_stride, in_off, channels, taps, d_weight, d_bias, 1, d_state, d_chunks, num_chunks, d_out,
                          out_stride, elem, stream);
}

PA_API int pa_causal_conv(const void* d_in, int64_t in_stride, int in_off, int channels, int taps, const float* d_weight,
                          const float* d_bias, int act, const float* d_state, const int32_t* d_chunks, int num_chunks,
                          void* d_out, int64_t out_stride, int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_in && d_weight && (d_state || taps == 1) && d_chunks && d_out && channels > 0 && num_chunks >= 0);
    PA_CHECK_ARG(taps >= 1 && taps <= kMaxTaps && (act == 0 || act == 1));
    if (num_chunks == 0) return PA_OK;
    dim3 grid((unsigned)((channels + 127) / 128), (unsigned)num_chunks);
    PA_DISPATCH_ELEM(elem, causal_conv_kernel<T><<<grid, 128, 0, as_stream(stream)>>>(
                               static_cast<const T*>(d_in), in_stride, in_off, channels, taps, d_weight, d_bias, d_state,
                               d_chunks, static_cast<T*>(d_out), out_stride, act));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_conv_state_update(const void* d_in, int64_t in_stride, int in_off, int channels, int taps,
                                const int32_t* d_seq_start, const int32_t* d_seq_len, const int32_t* d_seq_slot, int num_seqs,
                                float* d_state, int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_in && d_seq_start && d_seq_len && d_seq_slot && d_state && channels > 0 && num_seqs >= 0);
    PA_CHECK_ARG(taps >= 1 && taps <= kMaxTaps);
    if (num_seqs == 0 || taps == 1) return PA_OK;
    dim3 grid((unsigned)((channels + 127) / 128), (unsigned)num_seqs);
    PA_DISPATCH_ELEM(elem, conv_state_kernel<T><<<grid, 128, 0, as_stream(stream)>>>(
                               static_cast<const T*>(d_in), in_stride, in_off, channels, taps, d_seq_start, d_seq_len,
                               d_seq_slot, d_state));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API size_t pa_decay_scan_workspace_bytes(int num_chunks, int heads, int dim, int vdim) {
    if (num_chunks <= 0 || heads <= 0 || dim <= 0 || vdim <= 0) return 0;
    return (size_t)num_chunks * heads * ((size_t)dim * vdim + 1) * sizeof(float);
}

PA_API int pa_decay_scan(const void* d_q, int64_t q_stride, int q_off, const void* d_k, int64_t k_stride, int k_off,
                         const void* d_v, int64_t v_stride, int v_off, int heads, int groups, int dim, int vdim, int act,
                         const float* d_decay, const void* d_dt, int64_t dt_stride, int dt_off, const float* d_dt_bias,
                         const float* d_a_log, const float* d_skip, float* d_state, float* d_out, int64_t out_stride,
                         const int32_t* d_items, int num_items, const int32_t* d_seq_chunk0, const int32_t* d_seq_nchunks,
                         const int32_t* d_seq_slot, int num_seqs, int chunked, void* d_workspace, size_t workspace_bytes,
                         int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_q && d_k && d_v && d_state && d_out && d_items && num_items >= 0);
    PA_CHECK_ARG(heads > 0 && groups > 0 && heads % groups == 0 && dim > 0 && vdim > 0);
    PA_CHECK_ARG(d_dt ? (d_dt_bias && d_a_log) : d_decay != nullptr);
    if (num_items == 0) return PA_OK;
    if (elem != 4 && elem != 2) return PA_ERR_UNSUPPORTED;
    DecayScanParams p;
    p.q = d_q; p.q_stride = q_stride; p.q_off = q_off; p.k = d_k; p.k_stride = k_stride; p.k_off = k_off;
    p.v = d_v; p.v_stride = v_stride; p.v_off = v_off; p.heads = heads; p.groups = groups; p.dim = dim; p.vdim = vdim;
    p.act = act; p.decay = d_decay; p.dt = d_dt; p.dt_stride = dt_stride; p.dt_off = dt_off; p.dt_bias = d_dt_bias;
    p.a_log = d_a_log; p.skip = d_skip; p.state = d_state; p.out = d_out; p.out_stride = out_stride; p.items = d_items;
    p.part = static_cast<float*>(d_workspace);
    cudaStream_t st = as_stream(stream);
#define PA_DS(MODE)                                                                                \
    do {                                                                                           \
        p.mode = MODE;                                                                             \
        const int rc = elem == 4 ? ds_dispatch<float, MODE>(p, num_items, st) : ds_dispatch<bf16_t, MODE>(p, num_items, st); \
        if (rc != PA_OK) return rc;                                                                \
    } while (0)
    if (!chunked) {
        PA_DS(0);
        return PA_OK;
    }
    PA_CHECK_ARG(d_seq_chunk0 && d_seq_nchunks && d_seq_slot && num_seqs > 0);
    if (!d_workspace || workspace_bytes < pa_decay_scan_workspace_bytes(num_items, heads, dim, vdim)) return PA_ERR_WORKSPACE;
    PA_DS(1);
    const int64_t sz = (int64_t)dim * vdim;
    dim3 grid((unsigned)((sz + 255) / 256), (unsigned)heads, (unsigned)num_seqs);
    decay_chunk_chain_kernel<<<grid, 256, 0, st>>>(p.part, heads, sz, d_seq_chunk0, d_seq_nchunks, d_seq_slot, d_state);
    PA_DS(2);
#undef PA_DS
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_gated_rms_norm(const float* d_y, int64_t rows, int inner, int groups, const void* d_gate, int64_t gate_stride,
                             int gate_off, int gate_mode, const float* d_weight, float eps, void* d_out, int elem,
                             pa_stream_t stream) {
    PA_CHECK_ARG(d_y && d_weight && d_out && rows >= 0 && inner > 0 && groups > 0 && inner % groups == 0);
    PA_CHECK_ARG(gate_mode >= 0 && gate_mode <= 2 && (gate_mode == 0 || d_gate));
    if (rows == 0) return PA_OK;
    if (inner / groups >= 512 && rows * groups < (1 << 30)) {
        PA_DISPATCH_ELEM(elem, gated_norm_block_kernel<T><<<(unsigned)(rows * groups), 256, 0, as_stream(stream)>>>(
                                   d_y, inner, groups, static_cast<const T*>(d_gate), gate_stride, gate_off, gate_mode, d_weight,
                                   eps, static_cast<T*>(d_out)));
        PA_RETURN_LAUNCH_STATUS();
    }
    const int64_t threads = rows * groups * 32;
    PA_DISPATCH_ELEM(elem, gated_norm_kernel<T><<<(unsigned)((threads + 255) / 256), 256, 0, as_stream(stream)>>>(
                               d_y, rows, inner, groups, static_cast<const T*>(d_gate), gate_stride, gate_off, gate_mode,
                               d_weight, eps, static_cast<T*>(d_out)));
    PA_RETURN_LAUNCH_STATUS();
}
