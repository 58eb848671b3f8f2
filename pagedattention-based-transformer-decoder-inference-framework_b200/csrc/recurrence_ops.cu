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
                                                          T* __restrict__ out, int64_t out_stride) {
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
        out[(int64_t)(row0 + t) * out_stride + c] = from_f32<T>(silu_f32(acc));
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
    float* part;                                      // [items][heads][dim * vdim + 1]: state, then the chunk's total decay
};

constexpr int kDsTokens = 16;                         // tokens staged per step
constexpr int kDsCols = 64;                           // value columns per CTA

__device__ __forceinline__ float softplus_f32(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// CTA = kDsCols value columns x NS slices of the state's rows: thread (column, slice) keeps DPT rows of its column in
// registers.  q, k, the decays and the input scales of kDsTokens tokens are staged in shared memory per step; a thread
// reads its own v.  With NS > 1 the slices' partial outputs are summed through shared memory once per step.
template <typename T, int DPT>
__global__ void __launch_bounds__(256) decay_scan_kernel(const DecayScanParams p) {
    extern __shared__ __align__(16) float ds_smem[];
    const int NS = blockDim.x / kDsCols;
    const int dpad = NS * DPT;
    float* Qs = ds_smem;                               // [kDsTokens][dpad]
    float* Ks = Qs + kDsTokens * dpad;                 // [kDsTokens][dpad]
    float* As = Ks + kDsTokens * dpad;                 // [kDsTokens] decay
    float* Ss = As + kDsTokens;                        // [kDsTokens] input scale
    float* Ps = Ss + kDsTokens;                        // [kDsTokens][NS][kDsCols] partial outputs (NS > 1)
    const int col = threadIdx.x % kDsCols, slice = threadIdx.x / kDsCols;
    const int h = blockIdx.y, c = blockIdx.z * kDsCols + col;
    const int g = h / (p.heads / p.groups);
    const int* it = p.items + 4 * blockIdx.x;
    const int row0 = it[0], n = it[1], slot = it[2];
    const bool live = c < p.vdim;
    const int d0 = slice * DPT;
    const int64_t sz = (int64_t)p.dim * p.vdim;

    float S[DPT];
    const float* src = p.mode == 0 ? p.state + ((int64_t)slot * p.heads + h) * sz
                     : p.mode == 2 ? p.part + ((int64_t)blockIdx.x * p.heads + h) * (sz + 1) : nullptr;
#pragma unroll
    for (int i = 0; i < DPT; ++i) S[i] = (src && live && d0 + i < p.dim) ? src[(int64_t)(d0 + i) * p.vdim + c] : 0.f;
    float total = 1.f;                                 // product of the decays (mode 1)
    const float hd = p.dt ? 0.f : p.decay[h];
    const float a_rate = p.dt ? -expf(p.a_log[h]) : 0.f, dtb = p.dt ? p.dt_bias[h] : 0.f;
    const float skip = p.skip ? p.skip[h] : 0.f;
    const T* qb = static_cast<const T*>(p.q) + p.q_off + (int64_t)g * p.dim;
    const T* kb = static_cast<const T*>(p.k) + p.k_off + (int64_t)g * p.dim;
    const T* vb = static_cast<const T*>(p.v) + p.v_off + (int64_t)h * p.vdim;

    for (int t0 = 0; t0 < n; t0 += kDsTokens) {
        const int nt = min(kDsTokens, n - t0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * dpad; idx += blockDim.x) {
            const int t = idx / dpad, d = idx % dpad;
            float qv = 0.f, kv = 0.f;
            if (d < p.dim) {
                qv = to_f32<T>(qb[(int64_t)(row0 + t0 + t) * p.q_stride + d]);
                kv = to_f32<T>(kb[(int64_t)(row0 + t0 + t) * p.k_stride + d]);
                if (p.act) { qv = silu_f32(qv); kv = silu_f32(kv); }
            }
            Qs[idx] = qv;
            Ks[idx] = kv;
        }
        if (threadIdx.x < nt) {
            float a = hd, s = 1.f;
            if (p.dt) {
                const float raw = to_f32<T>(static_cast<const T*>(p.dt)[(int64_t)(row0 + t0 + threadIdx.x) * p.dt_stride + p.dt_off + h]);
                s = softplus_f32(raw + dtb);
                a = expf(a_rate * s);
            }
            As[threadIdx.x] = a;
            Ss[threadIdx.x] = s;
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            float x = live ? to_f32<T>(vb[(int64_t)(row0 + t0 + t) * p.v_stride + c]) : 0.f;
            if (p.act) x = silu_f32(x);
            const float a = As[t], xv = x * Ss[t];
            const float* kt = Ks + t * dpad + d0;
            const float* qt = Qs + t * dpad + d0;
            float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
            for (int i = 0; i < DPT; i += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(kt + i);
                const float4 q4 = *reinterpret_cast<const float4*>(qt + i);
                S[i] = fmaf(a, S[i], k4.x * xv);
                S[i + 1] = fmaf(a, S[i + 1], k4.y * xv);
                S[i + 2] = fmaf(a, S[i + 2], k4.z * xv);
                S[i + 3] = fmaf(a, S[i + 3], k4.w * xv);
                o0 = fmaf(S[i], q4.x, o0);
                o1 = fmaf(S[i + 1], q4.y, o1);
                o2 = fmaf(S[i + 2], q4.z, o2);
                o3 = fmaf(S[i + 3], q4.w, o3);
            }
            total *= a;
            if (p.mode != 1) {
                const float o = (o0 + o1) + (o2 + o3);
                if (NS == 1) {
                    if (live) p.out[(int64_t)(row0 + t0 + t) * p.out_stride + (int64_t)h * p.vdim + c] = fmaf(skip, x, o);
                } else {
                    Ps[(t * NS + slice) * kDsCols + col] = slice == 0 ? fmaf(skip, x, o) : o;
                }
            }
        }
        if (NS > 1 && p.mode != 1) {
            __syncthreads();
            for (int idx = threadIdx.x; idx < nt * kDsCols; idx += blockDim.x) {
                const int t = idx / kDsCols, cc = idx % kDsCols;
                if (blockIdx.z * kDsCols + cc >= p.vdim) continue;
                float o = 0.f;
                for (int s = 0; s < NS; ++s) o += Ps[(t * NS + s) * kDsCols + cc];
                p.out[(int64_t)(row0 + t0 + t) * p.out_stride + (int64_t)h * p.vdim + blockIdx.z * kDsCols + cc] = o;
            }
        }
    }
    if (p.mode == 2) return;
    float* dst = p.mode == 0 ? p.state + ((int64_t)slot * p.heads + h) * sz : p.part + ((int64_t)blockIdx.x * p.heads + h) * (sz + 1);
    if (live)
#pragma unroll
        for (int i = 0; i < DPT; ++i)
            if (d0 + i < p.dim) dst[(int64_t)(d0 + i) * p.vdim + c] = S[i];
    if (p.mode == 1 && threadIdx.x == 0 && blockIdx.z == 0) dst[sz] = total;
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
    for (int k = k0; k < k0 + n; ++k) {
        float* pk = part + ((int64_t)k * heads + h) * (sz + 1);
        const float B = pk[e], A = pk[sz];
        pk[e] = S;
        S = fmaf(A, S, B);
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

template <typename T, int DPT>
static int ds_launch(const DecayScanParams& p, int nitems, int NS, cudaStream_t st) {
    const size_t smem = ((size_t)2 * kDsTokens * NS * DPT + 2 * kDsTokens + (NS > 1 ? (size_t)kDsTokens * NS * kDsCols : 0)) * sizeof(float);
    dim3 grid((unsigned)nitems, (unsigned)p.heads, (unsigned)((p.vdim + kDsCols - 1) / kDsCols));
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(decay_scan_kernel<T, DPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    decay_scan_kernel<T, DPT><<<grid, kDsCols * NS, smem, st>>>(p);
    PA_RETURN_LAUNCH_STATUS();
}

template <typename T>
static int ds_dispatch(const DecayScanParams& p, int nitems, cudaStream_t st) {
    if (p.dim <= 16) return ds_launch<T, 16>(p, nitems, 1, st);
    if (p.dim <= 32) return ds_launch<T, 32>(p, nitems, 1, st);
    if (p.dim <= 64) return ds_launch<T, 64>(p, nitems, 1, st);
    const int NS = (p.dim + 127) / 128;
    if (NS > 4) return PA_ERR_UNSUPPORTED;
    return ds_launch<T, 128>(p, nitems, NS, st);
}

}  // namespace pa

using namespace pa;

PA_API int pa_causal_conv_silu(const void* d_in, int64_t in_stride, int in_off, int channels, int taps, const float* d_weight,
                               const float* d_bias, const float* d_state, const int32_t* d_chunks, int num_chunks,
                               void* d_out, int64_t out_stride, int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_in && d_weight && d_state && d_chunks && d_out && channels > 0 && num_chunks >= 0);
    PA_CHECK_ARG(taps >= 1 && taps <= kMaxTaps);
    if (num_chunks == 0) return PA_OK;
    dim3 grid((unsigned)((channels + 127) / 128), (unsigned)num_chunks);
    PA_DISPATCH_ELEM(elem, causal_conv_kernel<T><<<grid, 128, 0, as_stream(stream)>>>(
                               static_cast<const T*>(d_in), in_stride, in_off, channels, taps, d_weight, d_bias, d_state,
                               d_chunks, static_cast<T*>(d_out), out_stride));
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
        const int rc = elem == 4 ? ds_dispatch<float>(p, num_items, st) : ds_dispatch<bf16_t>(p, num_items, st); \
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
    const int64_t threads = rows * groups * 32;
    PA_DISPATCH_ELEM(elem, gated_norm_kernel<T><<<(unsigned)((threads + 255) / 256), 256, 0, as_stream(stream)>>>(
                               d_y, rows, inner, groups, static_cast<const T*>(d_gate), gate_stride, gate_off, gate_mode,
                               d_weight, eps, static_cast<T*>(d_out)));
    PA_RETURN_LAUNCH_STATUS();
}
