"""HybridDecoder -- a config-driven decoder stack over a ragged batch: every layer is one MIXER (picked by the layer's
`type` from MIXERS) plus an optional FEED-FORWARD (picked by `mlp.kind` from FEED_FORWARDS); the residual stream is
float.  A DESIGN (config "architecture", table DESIGNS) fixes how a layer is wired and with which constants the
mechanisms are built.  Four designs are served.

`Megusun` (wiring 'parallel': mixer and feed-forward both read the same pre-norm output):

    x      = embed[token]                                         (float residual)
    h      = x / sqrt(mean(x^2) + eps) * g_l                      (one number g_l per layer)
    hs     = h + (h_prev - h) * shift_l                           (token shift; h_prev carried per sequence)
    x     += m * (mixer_l(hs) + ff_l(h))                          (m = residual_mult)
    logits = head . (x / sqrt(mean(x^2) + eps) * g_final)

  mixer 'mingru'     z = sigmoid(W_z hs + b_z), u = W_x hs + b_x, c = u + 1/2 (u >= 0) | sigmoid(u),
                     S_t = (1 - z) S_{t-1} + z c,  out = W_o (S_t * silu(W_g hs))          state S per sequence, float
  mixer 'attention'  differential attention over the paged K/V pools (csrc/diff_attention.cu), no rotation, a
                     position-dependent query temperature, lambda = exp(lq1.lk1) - exp(lq2.lk2) + diff
  ff 'dense'         W_down gelu_erf(W_up h)
  ff 'moe'           sigmoid router, top-k by score, the score scales the expert's INPUT, experts W_down(silu(W_gate a) *
                     W_up a), plus a shared expert gated by sigmoid(w_sg . h)

`Domilix` (wiring 'post_norm': the sublayers read x itself, one after the other, and the norm is on their OUTPUT):

    x      = embed[token] * s_embed
    x     += N(mixer_l(x); w1_l),  then  x += N(ff_l(x); w2_l)         N(y; w) = y / sqrt(mean(y^2) + eps) * w  (per channel)
    logits = head . N(x; w_final)

  mixer 'latent_attention'   queries through a normed latent (q = W_uq N(W_dq x)), ONE cached row per token
                     [c = N(first kv_rank rows of W_dkv x) | kr = rotated last rot_dim rows] shared by all heads; keys and
                     values of head h are W_uk_h c and W_uv_h c, applied to the QUERY (ql_h = W_uk_h^T q_h) and to the
                     weighted sum of c instead of to the cache (csrc/latent_attention.cu); interleaved-pair rotation of
                     the rot_dim part of q and k; causal softmax; per-head output gate sigmoid(W_g x)_h; a layer with
                     `kv_from: j` has no W_dkv and reads layer j's pool
  ff 'dense'         W_down (relu(W_gate h) * (W_up h))
  ff 'moe'           logits W_r h + b, the `top` largest, weights = softmax over the chosen logits, applied to the
                     expert's OUTPUT; experts W_down relu(W_up h)^2

`Dubarax` (wiring 'pre_norm': x += mixer(N1(x)), then x += ff(N2(x)), N(x; w) = x / sqrt(mean(x^2) + eps) * (1 + w)); a
  block of layers [loop.start, loop.stop) may run loop.times times in a row with the same weights and a cache / state of
  its own per pass, each pass entered through x <- W_in [x | x0] + step_t (x0: the scaled embedding):

  mixer 'attention'  softmax attention with grouped key/value heads, biased projections, no rotation, tanh soft cap of the
                     scores, a learned bias over logarithmic distance buckets, and a sliding window (csrc/masked_attention.cu)
  mixer 'parallel'   two mixers on the same input, a_l * left + a_r * right: left = the same attention kernel with a
                     per-head linear distance penalty and visibility inside fixed chunks of positions; right = linear
                     attention with a per-head decay, S_t = d S_{t-1} + k_t v_t^T, o_t = S_t^T q_t on silu(q, k, v), normed
                     over all heads, gated by sigmoid(W_g h) (csrc/recurrence_ops.cu)
  mixer 'mamba2'     selective state space layer: one input product [z | x | B | C | dt], causal convolution + silu over
                     [x | B | C], S_t = exp(-exp(A) dt) S_{t-1} + dt B_t x_t^T, y_t = S_t^T C_t + D x_t, y * silu(z), RMS norm
                     in groups, output product (same scan kernel as the linear attention)
  ff 'moe'           softmax router over all experts, experts in groups of neighbours of which only the best `keep`
                     groups (by their largest score) can be chosen, the `top` largest scores un-renormalised on the
                     experts' OUTPUT, silu-gated experts, plus an always-on shared expert

`Gunulorn` (wiring 'parallel_two_norms': x += mixer(N(x; w1)) + ff(N(x; w2)), N(x; w) = x / sqrt(mean(x^2) + eps) * w, both
  sublayers read the same x); logits = cap * tanh(s * head . N(x; w_final) / cap) with s = logit_scale, cap = logit_softcap:

  mixer 'attention'  causal softmax attention with grouped key/value heads, no biases, no rotation; q, k and v pass a short
                     causal convolution over time right after their projections (its last taps - 1 inputs are state);
                     scores (q . k) * scale * temp[h]; a learned sink logit per head joins the softmax denominator; a layer
                     with `kv_from: j` has only a query projection and reads layer j's pool
  mixer 'attention_2'  a sliding window that also keeps the sequence's first mask.keep_first positions; interleaved-pair
                     rotation of the first rot.dims dimensions of q and k; values cached turned by their own position over
                     all of vdim and each head's output turned back by the query's position; one added to the denominator
  ff 'dense'         W_down P(W_up h + b_up) + b_down, P(z) = a N(z) + b N(z^2) + c N(z^3) + e (N over the token's ff values)
  ff 'moe'           softmax router over experts + identity outputs, the `top` largest of score + correction, weights = the
                     chosen scores over their sum, on the OUTPUT of silu-gated experts; an identity output returns h itself

Every size and constant comes from config.json (or a tensor's shape); the constants a design fixes are the arguments
the mechanisms are constructed with.  Two precisions: 'bfloat16' (matrix products and their activations in bfloat16
with float accumulation; norms, shift, recurrence, softmax, routers and the residual in float) and 'float32'
(everything in IEEE float: the fp32 FMA linear kernels, no reduced-precision matrix mode).

All compute is in libpa_b200.so kernels, except the plain bfloat16 matrix products, which go to the vendor GEMM
(cuBLASLt through torch.nn.functional.linear).  Weight names: '<layer>.mix.*', '<layer>.mlp.*', '<layer>.norm1',
'<layer>.shift', 'embed', 'final.norm', 'head' (linear weights [out, in])."""
import copy
import json
import math
import os

import torch

from . import _cabi
from .safetensors_io import load_file

_ELEM = {torch.float32: 4, torch.bfloat16: 2}
_KV = {torch.float32: "f32", torch.bfloat16: "bf16"}
SCAN_CHUNK = 64           # tokens per chunk of the chunked recurrent scan
SCAN_CHUNKED_FROM = 256   # portions at least this long use it
MMA_FROM = 16             # portions at least this long run their attention on the tensor cores (bfloat16)


def _chk(st, what):
    _cabi.check(st, what)


class _Ctx:
    """What a layer needs from the model during one step."""

    def __init__(self, model, batch):
        self.model, self.batch, self.lib = model, batch, model._lib
        self.dt, self.elem, self.dev = model.act_dtype, _ELEM[model.act_dtype], model.device
        self.R = batch.rows

        self._rope = {}

    def empty(self, *shape, dtype=None):
        return torch.empty(shape, dtype=dtype or self.dt, device=self.dev)

    def rope_table(self, dims, base):
        """[rows][dims / 2][cos, sin] of this step's rows (float), computed once per step and rotation."""
        key = (dims, base)
        if key not in self._rope:
            t = None
            if dims > 0:
                t = self.empty(self.R, dims // 2, 2, dtype=torch.float32)
                _chk(self.lib.pa_rope_table(self.batch.row_pos.data_ptr(), self.R, dims, base, t.data_ptr(), _cabi.stream()),
                     "pa_rope_table")
            self._rope[key] = t
        return self._rope[key]


# ---------------------------------------------------------------------------------------------------------------- mixers
class MinGRUMixer:
    """minGRU: gates read only the current token, so the three projections are one matrix product over the whole
    batch and the recurrence is an elementwise scan (pa_mingru_scan / _chunked) over each portion from the state slot."""
    kind = "mingru"

    def __init__(self, model, prefix, cfg, W):
        self.width = int(cfg["width"])
        self.w_zxg = model._weight(torch.cat([W[prefix + "z"], W[prefix + "x"], W[prefix + "g"]], 0))
        self.z_bias = model._f32(W[prefix + "z.b"])
        self.x_bias = model._f32(W[prefix + "x.b"])
        self.w_o = model._weight(W[prefix + "o"])
        self.state = model.states.add_state(self.width)

    def forward(self, c, hs):
        b, lib, s = c.batch, c.lib, _cabi.stream()
        zxg = c.model._linear(hs, self.w_zxg)
        y = c.empty(c.R, self.width)
        longest = max(p[1] for p in b.portions)
        if longest >= SCAN_CHUNKED_FROM:
            cs, cl, s0, sn, nch = b.scan_chunks(SCAN_CHUNK)
            ws = c.empty(lib.pa_mingru_chunked_workspace_bytes(nch, self.width), dtype=torch.uint8)
            _chk(lib.pa_mingru_scan_chunked(zxg.data_ptr(), self.z_bias.data_ptr(), self.x_bias.data_ptr(), self.width,
                                            cs.data_ptr(), cl.data_ptr(), nch, s0.data_ptr(), sn.data_ptr(),
                                            b.seq_slot.data_ptr(), b.num_seqs, self.state.data_ptr(), y.data_ptr(),
                                            c.elem, ws.data_ptr(), ws.numel(), s), "pa_mingru_scan_chunked")
        else:
            _chk(lib.pa_mingru_scan(zxg.data_ptr(), self.z_bias.data_ptr(), self.x_bias.data_ptr(), self.width,
                                    b.seq_start.data_ptr(), b.seq_len.data_ptr(), b.seq_slot.data_ptr(), b.num_seqs,
                                    self.state.data_ptr(), y.data_ptr(), c.elem, s), "pa_mingru_scan")
        return c.model._linear(y, self.w_o)


class DiffAttentionMixer:
    """Differential attention with grouped key/value heads over a paged pool of its own (KVTileCache with key rows
    of 2 * dim and value rows of vdim)."""
    kind = "attention"

    def __init__(self, model, prefix, cfg, W):
        self.heads, self.kv_heads = int(cfg["heads"]), int(cfg["kv_heads"])
        self.dim, self.vdim = int(cfg["dim"]), int(cfg["vdim"])
        if self.heads % self.kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        self.scale = float(cfg["scale"])
        self.diff = float(cfg["diff"])
        qt = cfg.get("q_temp") or {}
        self.temp_coef, self.temp_every = float(qt.get("coef", 0.0)), int(qt.get("every", 1))
        f = lambda n: W[prefix + n].to(torch.float32)  # noqa: E731
        self.lam = float(torch.exp((f("lq1") * f("lk1")).sum()) - torch.exp((f("lq2") * f("lk2")).sum())) + self.diff
        self.w_qkv = model._weight(torch.cat([W[prefix + "q"], W[prefix + "k"], W[prefix + "v"]], 0))
        self.w_o = model._weight(W[prefix + "o"])
        self.q_cols = self.heads * 2 * self.dim
        self.k_cols = self.kv_heads * 2 * self.dim
        self.kv = model.states.add_kv_layer(self.kv_heads, 2 * self.dim, self.vdim, _KV[model.act_dtype])
        self.tile_tokens = model._lib.pa_diff_attention_tile_tokens(self.heads, self.kv_heads)
        # portions of MMA_FROM tokens and more: the tensor-core kernel, where it serves the shape (0 = it does not)
        self.mma_tokens = model._lib.pa_diff_attention_mma_tile_tokens(self.dim, self.vdim, _ELEM[model.act_dtype])
        # decoded tokens of a batch with at least one (token, kv head) pair per SM: the same kernel, heads as rows
        self.mma_head_rows = bool(model._lib.pa_diff_attention_mma_head_rows(self.heads, self.kv_heads, self.dim, self.vdim,
                                                                               _ELEM[model.act_dtype]))

    def forward(self, c, hs):
        b, lib, kv, s = c.batch, c.lib, self.kv, _cabi.stream()
        qkv = c.model._linear(hs, self.w_qkv)
        kv.append_rows(qkv, self.q_cols, self.q_cols + self.k_cols, b.row_slot, b.row_pos)
        out = c.empty(c.R, self.heads * self.vdim)
        pt = kv.page_table_
        table = pt.device_data()
        sms = c.model.sm_count
        for kind, group in b.query_tiles(self.tile_tokens, self.mma_tokens, MMA_FROM).items():
            if group is None:
                continue
            tiles, ntiles, longest = group
            # too few CTAs for the chip over a long context: cut the keys (at least 256 per part)
            ctas = ntiles * self.kv_heads * max(1, math.ceil(self.heads // self.kv_heads / 32))
            nsplit = 1
            if kind == 1 and self.mma_head_rows and ntiles * self.kv_heads >= sms:
                kind = 3
            if kind < 2 and ctas < 4 * sms and longest > 512:
                nsplit = max(1, min(math.ceil(4 * sms / ctas), longest // 256, 64))
            ws = None
            if nsplit > 1:
                ws = c.empty(lib.pa_diff_attention_workspace_bytes(ntiles, self.heads, self.kv_heads, self.vdim, nsplit),
                             dtype=torch.uint8)
            _chk(lib.pa_diff_attention(qkv.data_ptr(), qkv.stride(0), 0, kv.key_buffer_.data_ptr(),
                                       kv.value_buffer_.data_ptr(), table.data_ptr(), pt.num_beams_, pt.num_heads_,
                                       pt.num_tiles_, kv.total_pages_, kv.tile_size_, tiles.data_ptr(), ntiles, self.heads,
                                       self.dim, self.vdim, self.scale, self.temp_coef, self.temp_every, self.lam,
                                       1.0 - self.diff, c.model.eps, out.data_ptr(), c.elem, nsplit, kind, _cabi.ptr(ws),
                                       ws.numel() if ws is not None else 0, s), "pa_diff_attention")
        return c.model._linear(out, self.w_o)


def latent_key_splits(ctas, longest, sms):
    """Too few CTAs for the chip over a long context: cut the keys into parts (at least 256 keys each), as many as still
    make ONE wave of CTAs -- the kernels hold most of an SM's shared memory, so a second, partial wave costs a whole one."""
    if ctas >= sms or longest <= 512:
        return 1
    return max(1, min(sms // ctas, longest // 256, 64))


class LatentAttentionMixer:
    """Attention through a low-rank latent over a paged pool with ONE row per token (KVTileCache with one key/value head
    and no value pool: row = [c | kr]).  The per-head key and value maps are applied on the query side and after the
    weighted sum (pa_head_linear), so a step reads kv_rank + rot_dim values per cached token whatever the head count."""
    kind = "latent_attention"

    def __init__(self, model, prefix, cfg, W):
        H, self.dim, self.rot_dim, self.vdim = int(cfg["heads"]), int(cfg["dim"]), int(cfg["rot_dim"]), int(cfg["vdim"])
        self.heads, self.kv_rank, self.q_rank = H, int(cfg["kv_rank"]), int(cfg["q_rank"])
        rot = cfg.get("rot") or {}
        self.rot_dims, self.rot_base = int(rot.get("dims", self.rot_dim)), float(rot.get("base", 10000.0))
        if self.rot_dims > self.rot_dim or self.rot_dims % 2:
            raise ValueError("rot.dims must be even and at most rot_dim")
        self.scale = float(cfg["scale"])
        self.kv_from = cfg.get("kv_from")
        self.own_kv = self.kv_from is None
        qd, kd = self.dim + self.rot_dim, self.kv_rank + self.rot_dim
        self.qd, self.kd = qd, kd
        for name, shape in (("dq", (self.q_rank, model.width)), ("uq", (H * qd, self.q_rank)), ("uk", (H * self.dim, self.kv_rank)),
                            ("uv", (H * self.vdim, self.kv_rank)), ("g", (H, model.width)), ("o", (model.width, H * self.vdim))):
            if tuple(W[prefix + name].shape) != shape:
                raise ValueError(f"{prefix}{name}: shape {tuple(W[prefix + name].shape)} does not match the config {shape}")
        # one product for everything that reads the layer's input: [dq | dkv (own pool only) | g]
        parts = [W[prefix + "dq"]] + ([W[prefix + "dkv"]] if self.own_kv else []) + [W[prefix + "g"]]
        self.w_in = model._weight(torch.cat(parts, 0))
        self.c_off = self.q_rank
        self.g_off = self.q_rank + (kd if self.own_kv else 0)
        self.dq_gain = model._f32(W[prefix + "dq.norm"])
        self.w_uq = model._weight(W[prefix + "uq"])
        self.w_uk = model._weight_raw(W[prefix + "uk"].reshape(H, self.dim, self.kv_rank))                    # [H][dim][kv_rank]
        self.w_uv = model._weight_raw(W[prefix + "uv"].reshape(H, self.vdim, self.kv_rank).transpose(1, 2))   # [H][kv_rank][vdim]
        self.w_o = model._weight(W[prefix + "o"])
        if self.own_kv:
            if tuple(W[prefix + "dkv"].shape) != (kd, model.width):
                raise ValueError(f"{prefix}dkv: shape does not match kv_rank + rot_dim")
            self.dkv_gain = model._f32(W[prefix + "dkv.norm"])
            self.kv = model.states.add_kv_layer(1, kd, 0, _KV[model.act_dtype])
        else:
            j = int(self.kv_from)
            src = model.layers[j].mixer if 0 <= j < len(model.layers) else None
            if not isinstance(src, LatentAttentionMixer) or not src.own_kv:
                raise ValueError(f"{prefix}: kv_from must name an earlier latent-attention layer with a pool of its own")
            if (src.kv_rank, src.rot_dim, src.rot_dims, src.rot_base) != (self.kv_rank, self.rot_dim, self.rot_dims, self.rot_base):
                raise ValueError(f"{prefix}: kv_rank, rot_dim and rotation must equal those of layer {j}")
            self.kv = src.kv
        self.tile_tokens = model._lib.pa_latent_attention_tile_tokens(H)
        # bfloat16 with 16-byte aligned query parts: every tile (portions and decoded tokens) runs on the tensor cores
        self.mma_tokens = 0
        if self.dim % 8 == 0 and qd % 8 == 0:
            self.mma_tokens = model._lib.pa_latent_attention_mma_tile_tokens(H, self.kv_rank, self.rot_dim, _ELEM[model.act_dtype])

    def _head_linear(self, c, x, x_rs, x_hs, w, K, N):
        """out[h, r, :] = x[r, h, :K] . w[h] for every head: [H, R, N] (row stride N, head stride R * N).  bfloat16: the
        vendor's batched product on the strided view; float32: the IEEE FMA kernel."""
        H, R = self.heads, c.R
        if c.elem == 2:
            return torch.bmm(torch.as_strided(x, (H, R, K), (x_hs, x_rs, 1)), w)
        out = c.empty(H, R, N)
        _chk(c.lib.pa_head_linear(x.data_ptr(), x_rs, x_hs, w.data_ptr(), H, K, N, R, out.data_ptr(), N, R * N, c.elem,
                                  _cabi.stream()), "pa_head_linear")
        return out

    def _attend(self, c, q, ql, lat, mma):
        """Launch the attention kernels over this step's tiles (prompt portions, then single decoded tokens).  Returns
        False when the tensor-core kernel refuses the operands (nothing was written that the float kernel does not
        write again)."""
        b, lib, kv, s, R, H, kvr = c.batch, c.lib, self.kv, _cabi.stream(), c.R, self.heads, self.kv_rank
        pt = kv.page_table_
        table = pt.device_data()
        rows_per_cta = 64 if mma else 32
        for kind, group in b.query_tiles(self.mma_tokens if mma else self.tile_tokens).items():
            if group is None:
                continue
            tiles, ntiles, longest = group
            ws = None
            nsplit = latent_key_splits(ntiles * math.ceil(H / rows_per_cta), longest, c.model.sm_count)
            if nsplit > 1:
                ws = c.empty(lib.pa_latent_attention_workspace_bytes(ntiles, H, kvr, nsplit), dtype=torch.uint8)
            st = lib.pa_latent_attention(ql.data_ptr(), kvr, R * kvr, q.data_ptr() + self.dim * c.elem, q.stride(0), self.qd,
                                         kv.key_buffer_.data_ptr(), table.data_ptr(), pt.num_beams_, pt.num_tiles_,
                                         kv.total_pages_, kv.tile_size_, tiles.data_ptr(), ntiles, H, kvr, self.rot_dim,
                                         self.scale, lat.data_ptr(), kvr, R * kvr, c.elem, nsplit,
                                         (3 if kind == 1 else 2) if mma else 0, _cabi.ptr(ws),
                                         ws.numel() if ws is not None else 0, s)
            if mma and st == _cabi.PA_ERR_UNSUPPORTED:
                return False
            _chk(st, "pa_latent_attention")
        return True

    def forward(self, c, h):
        b, lib, kv, s, R, H = c.batch, c.lib, self.kv, _cabi.stream(), c.R, self.heads
        proj = c.model._linear(h, self.w_in)
        cq = c.empty(R, self.q_rank)
        _chk(lib.pa_rms_norm_rows(proj.data_ptr(), proj.stride(0), 0, self.q_rank, c.model.eps, self.dq_gain.data_ptr(),
                                  cq.data_ptr(), self.q_rank, R, c.elem, s), "pa_rms_norm_rows")
        q = c.model._linear(cq, self.w_uq)
        rope = c.rope_table(self.rot_dims, self.rot_base)
        _chk(lib.pa_rope_rows(q.data_ptr(), q.stride(0), self.dim, self.qd, H, self.rot_dims, _cabi.ptr(rope), R, c.elem, s),
             "pa_rope_rows")
        pt = kv.page_table_
        table = pt.device_data()
        if self.own_kv:
            _chk(lib.pa_latent_kv_append(kv.key_buffer_.data_ptr(), table.data_ptr(), pt.num_beams_, pt.num_tiles_,
                                         kv.total_pages_, kv.tile_size_, self.kv_rank, self.rot_dim, self.rot_dims,
                                         proj.data_ptr(), proj.stride(0), self.c_off, self.dkv_gain.data_ptr(), c.model.eps,
                                         _cabi.ptr(rope), b.row_slot.data_ptr(), b.row_pos.data_ptr(), R, c.elem, s),
                 "pa_latent_kv_append")
        kvr = self.kv_rank
        ql = self._head_linear(c, q, q.stride(0), self.qd, self.w_uk, self.dim, kvr)          # [H, R, kv_rank]
        lat = c.empty(H, R, kvr)
        if self.mma_tokens > 0 and not self._attend(c, q, ql, lat, True):
            self.mma_tokens = 0         # a stride or an alignment the tensor-core kernel does not take: the float kernel
        if self.mma_tokens == 0:
            self._attend(c, q, ql, lat, False)
        ov = self._head_linear(c, lat, kvr, R * kvr, self.w_uv, kvr, self.vdim)               # [H, R, vdim]
        og = c.empty(R, H * self.vdim)
        _chk(lib.pa_head_gate(ov.data_ptr(), self.vdim, R * self.vdim, proj.data_ptr() + self.g_off * c.elem, proj.stride(0),
                              H, self.vdim, R, og.data_ptr(), c.elem, s), "pa_head_gate")
        return c.model._linear(og, self.w_o)


MASK_KIND = {"causal": 0, "window": 1, "chunk": 2}
CONV_CHUNK = 64           # tokens per work item of the causal convolution
DECAY_CHUNK = 64          # tokens per chunk of the chunked matrix-state scan
DECAY_CHUNKED_FROM = 256  # portions at least this long use it


def log_distance_bucket(n, buckets, far):
    """Bucket of distance n >= 0: exact below buckets // 2, then logarithmic steps that reach the last bucket at `far`."""
    half = buckets // 2
    if n < half:
        return n
    return min(buckets - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (buckets - half))))


class MaskedAttention:
    """Softmax attention with grouped key/value heads over a paged pool of its own; the design picks the visibility rule
    (`mask`: 'causal', 'window' or 'chunk' of cfg mask.size; a window also keeps the first cfg mask.keep_first positions),
    the distance bias (`bias`: None, 'slope' -- minus 2^(-slope_exp (h + 1) / heads) per step of distance -- or 'bucket' --
    a learned table '<prefix>rel' [buckets, heads] over log_distance_bucket(distance, buckets, cfg bias_max)), whether cfg
    'softcap' caps the scores, and

      proj_bias    whether the four projections have biases ('<name>.b')
      conv         a short causal convolution (cfg 'conv' taps, weights '<name>.conv' [channels, taps], no bias, no
                   activation) on q, k and v right after the projection; the last taps - 1 projected rows are state
      rot          interleaved-pair rotation of the first cfg rot.dims dimensions of every q and k head (cfg rot.base)
      rot_values   values cached turned by their own position over all of vdim (same pairs, angles p * base^(-2m / vdim));
                   every head's output is turned back by the query's position inside the attention kernels
      head_temp    a learned factor per query head on the scaled dot products ('<prefix>temp')
      sink         'learned': a logit per head ('<prefix>sink') in the softmax denominator, without key or value;
                   'zero': the same with logit 0 (one added to the denominator)

    A layer whose cfg has `kv_from: j` owns no key / value projections (nor their convolutions): it reads the pool of
    layer j (keys and values as cached there) with its own queries.  The mixer reads its q | k | v from a projection
    buffer at a column offset, so a mixer can fuse its input product with others."""

    def __init__(self, model, prefix, cfg, W, mask="causal", bias=None, softcap=False, slope_exp=8.0, proj_bias=True,
                 conv=False, rot=False, rot_values=False, head_temp=False, sink=None):
        self.heads, self.kv_heads = int(cfg["heads"]), int(cfg["kv_heads"])
        self.dim, self.vdim = int(cfg["dim"]), int(cfg["vdim"])
        if self.heads % self.kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        self.scale = float(cfg["scale"])
        self.softcap = float(cfg["softcap"]) if softcap else 0.0
        self.mask_kind = MASK_KIND[mask]
        self.mask_size = int(cfg["mask"]["size"]) if mask != "causal" else 0
        self.mask_keep = int(cfg["mask"].get("keep_first", 0)) if mask == "window" else 0
        self.kv_from = cfg.get("kv_from")
        self.own_kv = self.kv_from is None
        H = self.heads
        shapes = (("q", H * self.dim),) + ((("k", self.kv_heads * self.dim), ("v", self.kv_heads * self.vdim)) if self.own_kv else ())
        for name, rows in shapes:
            if tuple(W[prefix + name].shape) != (rows, model.width) or (proj_bias and tuple(W[prefix + name + ".b"].shape) != (rows,)):
                raise ValueError(f"{prefix}{name}: shape does not match the config")
        if tuple(W[prefix + "o"].shape) != (model.width, H * self.vdim):
            raise ValueError(f"{prefix}o: shape does not match the config")
        self.in_weight = torch.cat([W[prefix + n] for n, _ in shapes], 0)
        self.in_bias = torch.cat([W[prefix + n + ".b"] for n, _ in shapes], 0) if proj_bias else None
        self.q_cols, self.k_cols = H * self.dim, self.kv_heads * self.dim
        self.in_cols = int(self.in_weight.shape[0])
        self.w_o, self.b_o = model._weight(W[prefix + "o"]), model._bias(W[prefix + "o.b"]) if proj_bias else None
        self.taps, self.conv_w = 0, None
        if conv:
            self.taps = int(W[prefix + "q.conv"].shape[-1])     # the tensors' shape gives the taps; cfg 'conv' must agree
            if int(cfg.get("conv", self.taps)) != self.taps:
                raise ValueError(f"{prefix}q.conv: shape does not match the config")
            if not 1 <= self.taps <= 8:
                raise ValueError(f"{prefix}: 1 to 8 convolution taps are served")
            for name, rows in shapes:
                if tuple(W[prefix + name + ".conv"].shape) != (rows, self.taps):
                    raise ValueError(f"{prefix}{name}.conv: shape does not match the config")
            self.conv_w = model._f32(torch.cat([W[prefix + n + ".conv"] for n, _ in shapes], 0))
        self.rot_dims, self.rot_base, self.rot_values = 0, 0.0, bool(rot_values)
        if rot or rot_values:
            self.rot_base = float(cfg["rot"]["base"])
        if rot:
            self.rot_dims = int(cfg["rot"]["dims"])
            if self.rot_dims % 2 or self.rot_dims > self.dim:
                raise ValueError(f"{prefix}: rot.dims must be even and at most dim")
        if self.rot_values and self.vdim % 2:
            raise ValueError(f"{prefix}: turned values need an even vdim")
        self.head_scale = None
        if head_temp:
            if tuple(W[prefix + "temp"].shape) != (H,):
                raise ValueError(f"{prefix}temp: one number per head expected")
            self.head_scale = model._f32(W[prefix + "temp"])
        self.sink = None
        if sink == "learned":
            if tuple(W[prefix + "sink"].shape) != (H,):
                raise ValueError(f"{prefix}sink: one number per head expected")
            self.sink = model._f32(W[prefix + "sink"])
        elif sink == "zero":
            self.sink = model._f32(torch.zeros(H))
        elif sink is not None:
            raise ValueError(f"unknown sink {sink!r}")
        self._src = None
        if not self.own_kv:
            j = int(self.kv_from)
            src = model.layers[j].mixer if 0 <= j < len(model.layers) else None
            src = getattr(src, "core", None)
            if not isinstance(src, MaskedAttention) or not src.own_kv:
                raise ValueError(f"{prefix}: kv_from must name an earlier attention layer with a pool of its own")
            mine = (self.kv_heads, self.dim, self.vdim, self.rot_dims, self.rot_base, self.rot_values)
            if (src.kv_heads, src.dim, src.vdim, src.rot_dims, src.rot_base, src.rot_values) != mine:
                raise ValueError(f"{prefix}: key/value heads, sizes and rotation must equal those of layer {j}")
            self._src = src
        self.bias_kind, self.bias_len, self.bias = 0, 0, None
        if bias == "slope":
            self.bias_kind = 1
            self.bias = model._f32(torch.tensor([2.0 ** (-slope_exp * (h + 1) / H) for h in range(H)], dtype=torch.float64))
        elif bias == "bucket":
            rel = W[prefix + "rel"].to(torch.float64)
            if rel.dim() != 2 or rel.shape[1] != H:
                raise ValueError(f"{prefix}rel: one column per head expected")
            B, far = int(rel.shape[0]), float(cfg["bias_max"])
            # every distance from `far` on falls into the last bucket, and a window never looks further than its size
            n = int(math.ceil(far)) + 1
            if self.mask_kind == 1:
                n = min(n, self.mask_size)
            idx = torch.tensor([log_distance_bucket(d, B, far) for d in range(max(n, 1))])
            self.bias_kind, self.bias_len, self.bias = 2, int(idx.numel()), model._f32(rel[idx])
        elif bias is not None:
            raise ValueError(f"unknown distance bias {bias!r}")
        self.tile_tokens = model._lib.pa_masked_attention_tile_tokens(self.heads, self.kv_heads)
        self.mma_tokens = model._lib.pa_masked_attention_mma_tile_tokens(self.dim, self.vdim, _ELEM[model.act_dtype])
        self.alloc_state(model)

    def alloc_state(self, model):
        if self.own_kv:
            self.kv = model.states.add_kv_layer(self.kv_heads, self.dim, self.vdim, _KV[model.act_dtype])
        else:
            if getattr(self, "kv", None) is not None:
                raise ValueError("a layer that borrows keys and values cannot run in a looped block")
            self.kv = self._src.kv
        self.conv_state = model.states.add_state((self.taps - 1) * self.in_cols) if self.taps > 1 else None

    def _prepare(self, c, proj, off):
        """Convolution and rotation of this step's q | k | v rows, then the new keys and values go to the pool.  Returns
        the buffer and column offset the attention kernels read the queries from."""
        b, lib, s, R = c.batch, c.lib, _cabi.stream(), c.R
        if self.taps:
            chunks, nch, _s0, _sn = b.chunk_items(CONV_CHUNK)
            y = c.empty(R, self.in_cols)
            _chk(lib.pa_causal_conv(proj.data_ptr(), proj.stride(0), off, self.in_cols, self.taps, self.conv_w.data_ptr(),
                                    None, 0, _cabi.ptr(self.conv_state), chunks.data_ptr(), nch, y.data_ptr(), self.in_cols,
                                    c.elem, s), "pa_causal_conv")
            if self.taps > 1:
                _chk(lib.pa_conv_state_update(proj.data_ptr(), proj.stride(0), off, self.in_cols, self.taps,
                                              b.seq_start.data_ptr(), b.seq_len.data_ptr(), b.seq_slot.data_ptr(),
                                              b.num_seqs, self.conv_state.data_ptr(), c.elem, s), "pa_conv_state_update")
            proj, off = y, 0
        k_off, v_off = off + self.q_cols, off + self.q_cols + self.k_cols
        kv = self.kv
        if self.rot_dims or self.rot_values:    # q in place; k rotated and v turned on their way into the pool: one launch
            pt = kv.page_table_
            own = self.own_kv
            _chk(lib.pa_rope_kv_append(proj.data_ptr(), proj.stride(0), off, k_off, v_off, self.heads, self.kv_heads, self.dim,
                                       self.vdim, self.rot_dims, _cabi.ptr(c.rope_table(self.rot_dims, self.rot_base)),
                                       _cabi.ptr(c.rope_table(self.vdim, self.rot_base)) if self.rot_values else None,
                                       kv.key_buffer_.data_ptr() if own else None,
                                       kv.value_buffer_.data_ptr() if own else None, pt.device_data().data_ptr(),
                                       pt.num_beams_, pt.num_tiles_, kv.total_pages_, kv.tile_size_, b.row_slot.data_ptr(),
                                       b.row_pos.data_ptr(), R, c.elem, s), "pa_rope_kv_append")
        elif self.own_kv:
            kv.append_rows(proj, k_off, v_off, b.row_slot, b.row_pos)
        return proj, off

    def attend(self, c, proj, off):
        """proj [R, stride] holds q | k | v of this step's rows from column `off`; appends k / v to the pool and
        returns the heads' outputs [R, heads * vdim]."""
        proj, off = self._prepare(c, proj, off)
        out = c.empty(c.R, self.heads * self.vdim)
        if not self._attend_tiles(c, proj, off, out, self.mma_tokens):
            self.mma_tokens = 0     # a stride or an alignment the tensor-core kernel refuses: the float kernels
            self._attend_tiles(c, proj, off, out, 0)
        return out

    def _attend_tiles(self, c, proj, off, out, mma_tokens):
        b, lib, kv, s = c.batch, c.lib, self.kv, _cabi.stream()
        pt = kv.page_table_
        table = pt.device_data()
        out_rot = c.rope_table(self.vdim, self.rot_base) if self.rot_values else None
        for kind, group in b.query_tiles(self.tile_tokens, mma_tokens, MMA_FROM).items():
            if group is None:
                continue
            tiles, ntiles, _longest = group
            st = lib.pa_masked_attention_sink(proj.data_ptr(), proj.stride(0), off, kv.key_buffer_.data_ptr(),
                                              kv.value_buffer_.data_ptr(), table.data_ptr(), pt.num_beams_, pt.num_heads_,
                                              pt.num_tiles_, kv.total_pages_, kv.tile_size_, tiles.data_ptr(), ntiles,
                                              self.heads, self.dim, self.vdim, self.scale, self.softcap, self.mask_kind,
                                              self.mask_size, self.mask_keep, self.bias_kind, _cabi.ptr(self.bias),
                                              self.bias_len, _cabi.ptr(self.head_scale), _cabi.ptr(self.sink),
                                              _cabi.ptr(out_rot), out.data_ptr(), c.elem, kind, s)
            if kind == 2 and st == _cabi.PA_ERR_UNSUPPORTED:
                return False
            _chk(st, "pa_masked_attention_sink")
        return True

    def project_out(self, c, heads_out):
        return c.model._linear(heads_out, self.w_o, bias=self.b_o)


def decay_scan(c, state, out, heads, groups, dim, vdim, q, k, v, act=0, decay=None, dt=None, dt_bias=None, a_log=None,
               skip=None):
    """The matrix-state recurrence of csrc/recurrence_ops.cu over this step's portions: q, k, v and dt are (buffer,
    column offset) pairs; long portions take the chunked three-pass form."""
    b, lib = c.batch, c.lib
    chunked = max(p[1] for p in b.portions) >= DECAY_CHUNKED_FROM
    items, n, s0, sn = b.chunk_items(DECAY_CHUNK if chunked else 0)
    ws = None
    if chunked:
        ws = c.empty(lib.pa_decay_scan_workspace_bytes(n, heads, dim, vdim), dtype=torch.uint8)
    _chk(lib.pa_decay_scan(q[0].data_ptr(), q[0].stride(0), q[1], k[0].data_ptr(), k[0].stride(0), k[1], v[0].data_ptr(),
                           v[0].stride(0), v[1], heads, groups, dim, vdim, act, _cabi.ptr(decay),
                           dt[0].data_ptr() if dt else None, dt[0].stride(0) if dt else 0, dt[1] if dt else 0,
                           _cabi.ptr(dt_bias), _cabi.ptr(a_log), _cabi.ptr(skip), state.data_ptr(), out.data_ptr(),
                           out.stride(0), items.data_ptr(), n, s0.data_ptr(), sn.data_ptr(), b.seq_slot.data_ptr(),
                           b.num_seqs, 1 if chunked else 0, _cabi.ptr(ws), ws.numel() if ws is not None else 0, c.elem,
                           _cabi.stream()), "pa_decay_scan")


class DecayLinearAttention:
    """Linear attention with a constant decay per head (cfg 'decay', one number per head): q, k, v = silu of their
    projections, the matrix state per head and sequence in a float state slot, the heads' outputs normed together
    (plain weight '<prefix>norm'), gated by sigmoid(W_g h), then the output product.  Reads q | k | v | g from a
    projection buffer at a column offset."""

    def __init__(self, model, prefix, cfg, W):
        self.heads, self.dim, self.vdim = int(cfg["heads"]), int(cfg["dim"]), int(cfg["vdim"])
        H = self.heads
        if len(cfg["decay"]) != H:
            raise ValueError(f"{prefix}: one decay per head expected")
        shapes = (("q", H * self.dim), ("k", H * self.dim), ("v", H * self.vdim), ("g", H * self.vdim))
        for name, rows in shapes:
            if tuple(W[prefix + name].shape) != (rows, model.width):
                raise ValueError(f"{prefix}{name}: shape does not match the config")
        self.in_weight = torch.cat([W[prefix + n] for n, _ in shapes], 0)
        self.in_bias = torch.zeros(self.in_weight.shape[0], dtype=self.in_weight.dtype, device=self.in_weight.device)
        self.in_cols = int(self.in_weight.shape[0])
        self.decay = model._f32(torch.tensor([float(d) for d in cfg["decay"]], dtype=torch.float64))
        self.norm = model._f32(W[prefix + "norm"])
        self.w_o = model._weight(W[prefix + "o"])
        self.alloc_state(model)

    def alloc_state(self, model):
        self.state = model.states.add_state(self.heads * self.dim * self.vdim)

    def forward(self, c, proj, off):
        H, d, vd = self.heads, self.dim, self.vdim
        o = c.empty(c.R, H * vd, dtype=torch.float32)
        decay_scan(c, self.state, o, H, H, d, vd, (proj, off), (proj, off + H * d), (proj, off + 2 * H * d), act=1,
                   decay=self.decay)
        on = c.empty(c.R, H * vd)
        _chk(c.lib.pa_gated_rms_norm(o.data_ptr(), c.R, H * vd, 1, proj.data_ptr(), proj.stride(0), off + 2 * H * d + H * vd, 2,
                                     self.norm.data_ptr(), c.model.eps, on.data_ptr(), c.elem, _cabi.stream()),
             "pa_gated_rms_norm")
        return c.model._linear(on, self.w_o)


class SoftmaxAttentionMixer:
    """A MaskedAttention as a layer's only mixer: one fused q | k | v product, attention, output product."""
    kind = "attention"

    def __init__(self, model, prefix, cfg, W, **constants):
        self.core = MaskedAttention(model, prefix, cfg, W, **constants)
        self.w_in, self.b_in = model._weight(self.core.in_weight), model._bias(self.core.in_bias)

    def new_pass(self, model):
        m = copy.copy(self)
        m.core = copy.copy(self.core)
        m.core.alloc_state(model)
        return m

    def forward(self, c, h):
        proj = c.model._linear(h, self.w_in, bias=self.b_in)
        return self.core.project_out(c, self.core.attend(c, proj, 0))


class ParallelMixer:
    """Two mixers side by side on the same input, left_scale * left + right_scale * right: a MaskedAttention (cfg 'left')
    and a DecayLinearAttention (cfg 'right').  Everything that reads the input is ONE product."""
    kind = "parallel"

    def __init__(self, model, prefix, cfg, W, left=None, right=None):
        self.left = MaskedAttention(model, prefix + "left.", cfg["left"], W, **(left or {}))
        self.right = DecayLinearAttention(model, prefix + "right.", cfg["right"], W, **(right or {}))
        self.left_scale, self.right_scale = float(cfg["left_scale"]), float(cfg["right_scale"])
        self.w_in = model._weight(torch.cat([self.left.in_weight, self.right.in_weight], 0))
        self.b_in = model._bias(torch.cat([self.left.in_bias, self.right.in_bias], 0))

    def new_pass(self, model):
        m = copy.copy(self)
        m.left, m.right = copy.copy(self.left), copy.copy(self.right)
        m.left.alloc_state(model)
        m.right.alloc_state(model)
        return m

    def forward(self, c, h):
        proj = c.model._linear(h, self.w_in, bias=self.b_in)
        left = self.left.project_out(c, self.left.attend(c, proj, 0))
        right = self.right.forward(c, proj, self.left.in_cols)
        return dict(y=left, y_scale=self.left_scale, y2=right, y2_scale=self.right_scale)


class Mamba2Mixer:
    """Selective state space layer with scalar decay per head (state-space duality form): W_in h = [z | x | B | C | dt]
    (inner = heads * vdim, B and C of `groups` x `state`), causal convolution + silu over [x | B | C] whose last taps - 1
    inputs are carried per sequence, dt = softplus(dt + dt_bias), the matrix state per head in a float slot, y * silu(z),
    RMS norm in norm_groups parts, output product."""
    kind = "mamba2"

    def __init__(self, model, prefix, cfg, W):
        self.heads, self.vdim, self.state_dim = int(cfg["heads"]), int(cfg["vdim"]), int(cfg["state"])
        self.groups, self.taps, self.norm_groups = int(cfg["groups"]), int(cfg["conv"]), int(cfg["norm_groups"])
        H, P, N, G = self.heads, self.vdim, self.state_dim, self.groups
        self.inner = H * P
        self.channels = self.inner + 2 * G * N
        if H % G or self.inner % self.norm_groups:
            raise ValueError(f"{prefix}: heads must be a multiple of groups and heads * vdim of norm_groups")
        if not 1 <= self.taps <= 8:
            raise ValueError(f"{prefix}: 1 to 8 convolution taps are served")
        want = {"in": (2 * self.inner + 2 * G * N + H, model.width), "conv": (self.channels, self.taps),
                "conv.b": (self.channels,), "dt_bias": (H,), "A_log": (H,), "D": (H,), "norm": (self.inner,),
                "o": (model.width, self.inner)}
        for name, shape in want.items():
            if tuple(W[prefix + name].shape) != shape:
                raise ValueError(f"{prefix}{name}: shape {tuple(W[prefix + name].shape)} does not match the config {shape}")
        self.w_in = model._weight(W[prefix + "in"])
        self.conv_w, self.conv_b = model._f32(W[prefix + "conv"]), model._f32(W[prefix + "conv.b"])
        self.dt_bias, self.a_log, self.skip = (model._f32(W[prefix + n]) for n in ("dt_bias", "A_log", "D"))
        self.norm = model._f32(W[prefix + "norm"])
        self.w_o = model._weight(W[prefix + "o"])
        self.alloc_state(model)

    def alloc_state(self, model):
        self.state = model.states.add_state(self.heads * self.state_dim * self.vdim)
        self.conv_state = model.states.add_state(max(1, (self.taps - 1) * self.channels))

    def new_pass(self, model):
        m = copy.copy(self)
        m.alloc_state(model)
        return m

    def forward(self, c, h):
        b, lib, s, R = c.batch, c.lib, _cabi.stream(), c.R
        H, P, N, G, inner, C = self.heads, self.vdim, self.state_dim, self.groups, self.inner, self.channels
        proj = c.model._linear(h, self.w_in)
        chunks, nch, _s0, _sn = b.chunk_items(CONV_CHUNK)
        xbc = c.empty(R, C)
        _chk(lib.pa_causal_conv_silu(proj.data_ptr(), proj.stride(0), inner, C, self.taps, self.conv_w.data_ptr(),
                                     self.conv_b.data_ptr(), self.conv_state.data_ptr(), chunks.data_ptr(), nch,
                                     xbc.data_ptr(), C, c.elem, s), "pa_causal_conv_silu")
        _chk(lib.pa_conv_state_update(proj.data_ptr(), proj.stride(0), inner, C, self.taps, b.seq_start.data_ptr(),
                                      b.seq_len.data_ptr(), b.seq_slot.data_ptr(), b.num_seqs, self.conv_state.data_ptr(),
                                      c.elem, s), "pa_conv_state_update")
        y = c.empty(R, inner, dtype=torch.float32)
        decay_scan(c, self.state, y, H, G, N, P, (xbc, inner + G * N), (xbc, inner), (xbc, 0), act=0,
                   dt=(proj, 2 * inner + 2 * G * N), dt_bias=self.dt_bias, a_log=self.a_log, skip=self.skip)
        yn = c.empty(R, inner)
        _chk(lib.pa_gated_rms_norm(y.data_ptr(), R, inner, self.norm_groups, proj.data_ptr(), proj.stride(0), 0, 1,
                                   self.norm.data_ptr(), c.model.eps, yn.data_ptr(), c.elem, s), "pa_gated_rms_norm")
        return c.model._linear(yn, self.w_o)


MIXERS = {"mingru": MinGRUMixer, "attention": DiffAttentionMixer, "latent_attention": LatentAttentionMixer}


# --------------------------------------------------------------------------------------------------------- feed-forwards
_GLU_ACT = {"silu": 0, "relu": 1, "gelu_tanh": 2}
_EXPERT_ACT = {"silu": 0, "relu": 1, "relu2": 2}


class DenseFF:
    """W_down act(W_up h) (gated=False; act 'gelu_erf', or 'poly_norm': a N(z) + b N(z^2) + c N(z^3) + e with the four
    numbers of '<prefix>act', N = division by the root mean square over the token's ff values), or the gated form
    W_down (act(W_gate h) * (W_up h)).  bias=True: both products have biases ('<name>.b')."""
    kind = "dense"

    def __init__(self, model, prefix, cfg, W, act="gelu_erf", gated=False, bias=False):
        self.gated, self.act = bool(gated), act
        if (self.gated and act not in _GLU_ACT) or (not self.gated and act not in ("gelu_erf", "poly_norm")):
            raise ValueError(f"dense feed-forward: activation {act!r} is not served")
        self.ff = int(W[prefix + "up"].shape[0])
        if "ff" in cfg and int(cfg["ff"]) != self.ff:
            raise ValueError(f"{prefix}up: shape does not match the config")
        self.w_up = model._weight(torch.cat([W[prefix + "gate"], W[prefix + "up"]], 0) if self.gated else W[prefix + "up"])
        self.w_down = model._weight(W[prefix + "down"])
        self.b_up = self.b_down = self.coef = None
        if bias:
            names = ("gate.b", "up.b") if self.gated else ("up.b",)
            self.b_up = model._bias(torch.cat([W[prefix + n] for n in names], 0))
            self.b_down = model._bias(W[prefix + "down.b"])
        if act == "poly_norm":
            if tuple(W[prefix + "act"].shape) != (4,):
                raise ValueError(f"{prefix}act: four numbers expected")
            self.coef = model._f32(W[prefix + "act"])

    def forward(self, c, h):
        a = c.model._linear(h, self.w_up, bias=self.b_up)
        if self.gated:
            gu, a = a, c.empty(c.R, self.ff)
            _chk(c.lib.pa_act_mul(gu.data_ptr(), c.R, self.ff, _GLU_ACT[self.act], a.data_ptr(), c.elem, _cabi.stream()),
                 "pa_act_mul")
        elif self.act == "poly_norm":
            z, a = a, c.empty(c.R, self.ff)
            _chk(c.lib.pa_poly_norm(z.data_ptr(), c.R, self.ff, self.coef.data_ptr(), c.model.eps, a.data_ptr(), c.elem,
                                    _cabi.stream()), "pa_poly_norm")
        else:
            _chk(c.lib.pa_gelu_inplace(a.data_ptr(), a.numel(), c.elem, _cabi.stream()), "pa_gelu_inplace")
        return dict(dense=c.model._linear(a, self.w_down, bias=self.b_down))


_SCORE_FN = {"sigmoid": 0, "softmax": 1, "softmax_chosen": 2}


class MoEFF:
    """Routed experts over the pairs sorted by expert (grouped matrix products, csrc/moe_ops.cu).  Constants of a design:
    score ('sigmoid' / 'softmax' over all experts, the `top` largest scores, or 'softmax_chosen': the `top` largest
    logits, softmax over those only), an optional router bias ('<prefix>router.b'), weight_on ('input': the score scales
    the expert's input row; 'output': the weighted sum of the experts' outputs), gated experts W_down(act(W_gate a) *
    W_up a) or plain ones W_down act(W_up a), and an optional shared expert (gated per token where '<prefix>shared.sg'
    exists).  cfg router.groups {count, keep}: experts in `count` equal groups of neighbours, only the `keep` groups with
    the largest maxima can be chosen.  correction=True: '<prefix>correction' (one number per router output) is added to
    the scores for the CHOICE only; renorm=True: the chosen scores are divided by their sum.  cfg router.identity = n: the
    router has n more outputs than there are experts, and a token that chooses one of those gets its own input row back
    from it (weight_on 'output'); such experts have no tensors."""
    kind = "moe"

    def __init__(self, model, prefix, cfg, W, score="sigmoid", weight_on="input", act="silu", gated=True, correction=False,
                 renorm=False):
        self.experts, self.top = int(cfg["router"]["experts"]), int(cfg["router"]["top"])
        self.identity = int(cfg["router"].get("identity", 0))
        self.outputs = self.experts + self.identity
        self.ff = int((cfg.get("expert") or {}).get("ff", W[prefix + "e0.up"].shape[0] if self.experts else 0))
        grp = cfg["router"].get("groups") or {}
        self.ngroups, self.keep = int(grp.get("count", 1)), int(grp.get("keep", grp.get("count", 1)))
        if self.outputs % self.ngroups or not 1 <= self.keep <= self.ngroups or self.keep * (self.outputs // self.ngroups) < self.top:
            raise ValueError("routed feed-forward: expert groups do not fit experts / top")
        self.score_fn, self.weight_on, self.act, self.gated = _SCORE_FN[score], weight_on, _EXPERT_ACT[act], bool(gated)
        self.renorm = 1 if renorm else 0
        if weight_on not in ("input", "output") or not 0 < self.top <= self.outputs or self.identity < 0:
            raise ValueError("routed feed-forward: bad constants")
        if self.identity and weight_on != "output":
            raise ValueError("routed feed-forward: identity experts need the weight on the output")
        if tuple(W[prefix + "router"].shape) != (self.outputs, model.width):
            raise ValueError(f"{prefix}router: shape does not match experts + identity")
        self.choice_bias = None
        if correction:
            if tuple(W[prefix + "correction"].shape) != (self.outputs,):
                raise ValueError(f"{prefix}correction: one number per router output expected")
            self.choice_bias = model._f32(W[prefix + "correction"])
        ex = lambda n: [W[f"{prefix}e{e}.{n}"] for e in range(self.experts)]  # noqa: E731
        if self.gated:
            self.w_gate_up = model._weight_raw(torch.stack([torch.cat([g, u], 0) for g, u in zip(ex("gate"), ex("up"))]))
        else:
            self.w_gate_up = model._weight_raw(torch.stack(ex("up")))
        self.w_down = model._weight_raw(torch.stack(ex("down")))
        self.w_router = model._f32(W[prefix + "router"])
        self.b_router = model._f32(W[prefix + "router.b"]) if prefix + "router.b" in W else None
        self.shared = None
        if cfg.get("shared"):
            sp = prefix + "shared."
            self.shared = dict(w_gate_up=model._weight(torch.cat([W[sp + "gate"], W[sp + "up"]], 0)),
                               w_down=model._weight(W[sp + "down"]), ff=int(cfg["shared"]["ff"]),
                               w_sg=model._f32(W[sp + "sg"].reshape(-1)) if sp + "sg" in W else None)

    def forward(self, c, h):
        lib, R, s, wdt = c.lib, c.R, _cabi.stream(), c.model.width
        i32, f32 = dict(dtype=torch.int32), dict(dtype=torch.float32)
        pairs = R * self.top
        sel_id, sel_w = c.empty(pairs, **i32), c.empty(pairs, **f32)
        sh = self.shared
        sgate = c.empty(R, **f32) if sh and sh["w_sg"] is not None else None
        _chk(lib.pa_router_topk_biased(h.data_ptr(), self.w_router.data_ptr(), _cabi.ptr(self.b_router),
                                       _cabi.ptr(sh["w_sg"]) if sgate is not None else None, R, wdt, self.outputs,
                                       self.top, self.score_fn, self.renorm, self.ngroups, self.keep,
                                       _cabi.ptr(self.choice_bias), sel_id.data_ptr(), sel_w.data_ptr(), _cabi.ptr(sgate),
                                       c.elem, s), "pa_router_topk_biased")
        order = c.empty(pairs, **i32)
        meta = c.empty(lib.pa_moe_meta_ints(pairs, self.experts), **i32)
        _chk(lib.pa_moe_sort(sel_id.data_ptr(), pairs, self.experts, order.data_ptr(), meta.data_ptr(), s), "pa_moe_sort")
        act = c.empty(pairs, self.ff)
        in_w = sel_w.data_ptr() if self.weight_on == "input" else None
        _chk((lib.pa_moe_gate_up_act if self.gated else lib.pa_moe_up)(
            h.data_ptr(), h.stride(0), self.w_gate_up.data_ptr(), wdt, self.ff, self.experts, order.data_ptr(), in_w,
            self.top, meta.data_ptr(), pairs, self.act, act.data_ptr(), c.elem, s), "pa_moe_gate_up_act / pa_moe_up")
        routed = c.empty(pairs, wdt, **f32)
        _chk(lib.pa_moe_down(act.data_ptr(), self.w_down.data_ptr(), self.ff, wdt, self.experts, order.data_ptr(),
                             meta.data_ptr(), pairs, routed.data_ptr(), c.elem, s), "pa_moe_down")
        out = dict(routed=routed, top=self.top, sel_w=sel_w if self.weight_on == "output" else None)
        if self.identity:       # ids from `experts` on were left out by the sort: the residual kernel reads h for them
            out.update(sel_id=sel_id, experts=self.experts, ident=h)
        if sh:
            gu = c.model._linear(h, sh["w_gate_up"])
            a = c.empty(R, sh["ff"])
            _chk(lib.pa_silu_mul(gu.data_ptr(), R, sh["ff"], a.data_ptr(), c.elem, s), "pa_silu_mul")
            out.update(shared=c.model._linear(a, sh["w_down"]), shared_gate=sgate)
        return out


FEED_FORWARDS = {"dense": DenseFF, "moe": MoEFF}

# What a design fixes: the wiring of a layer, and the constants its feed-forwards are built with (its mixers take
# theirs from the layer's config).
DESIGNS = {
    "Megusun": dict(wiring="parallel", ff={"dense": dict(act="gelu_erf", gated=False),
                                            "moe": dict(score="sigmoid", weight_on="input", act="silu", gated=True)}),
    "Domilix": dict(wiring="post_norm", ff={"dense": dict(act="relu", gated=True),
                                            "moe": dict(score="softmax_chosen", weight_on="output", act="relu2", gated=False)}),
    "Dubarax": dict(wiring="pre_norm",
                    mixers={"attention": (SoftmaxAttentionMixer, dict(mask="window", bias="bucket", softcap=True)),
                            "parallel": (ParallelMixer, dict(left=dict(mask="chunk", bias="slope", slope_exp=8.0))),
                            "mamba2": (Mamba2Mixer, {})},
                    ff={"moe": dict(score="softmax", weight_on="output", act="silu", gated=True)}),
    "Gunulorn": dict(wiring="parallel_two_norms",
                     mixers={"attention": (SoftmaxAttentionMixer, dict(mask="causal", proj_bias=False, conv=True,
                                                                       head_temp=True, sink="learned")),
                             "attention_2": (SoftmaxAttentionMixer, dict(mask="window", proj_bias=False, rot=True,
                                                                         rot_values=True, sink="zero"))},
                     ff={"dense": dict(act="poly_norm", gated=False, bias=True),
                         "moe": dict(score="softmax", weight_on="output", act="silu", gated=True, correction=True,
                                     renorm=True)}),
}


class _Layer:
    pass


class HybridDecoder:
    ARCHITECTURES = tuple(DESIGNS)

    def __init__(self, config, weights, dtype="bfloat16", *, max_tokens=4096, max_seqs=4, tile_size=16, device=None):
        from .seq_state import SequenceStateCache
        self.act_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[str(dtype).replace("torch.", "")]
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self._lib = _cabi.lib()
        self.sm_count = _cabi.device_info()[0]
        self.config = config
        self.width, self.vocab = int(config["width"]), int(config["vocab"])
        self.eps = float(config["norm"]["eps"])
        self.design = DESIGNS[config.get("architecture", "Megusun")]
        self.wiring = self.design["wiring"]
        self.mult = float(config.get("residual_mult", 1.0))
        self.embed_scale = float((config.get("embedding") or {}).get("scale", 1.0))
        self.states = SequenceStateCache(max_seqs, max_tokens, tile_size, self.device)
        self._ws = None
        W = weights
        if tuple(W["embed"].shape) != (self.vocab, self.width):
            raise ValueError("embed does not match config vocab / width")
        self.embed = W["embed"].to(self.device, self.act_dtype).contiguous()
        self.head = self._weight(W["head"])
        post, pre, par2 = self.wiring == "post_norm", self.wiring == "pre_norm", self.wiring == "parallel_two_norms"
        self.final_gain = 1.0 if post or pre or par2 else float(W["final.norm"].to(torch.float32))
        self.final_gain_vec = (self._f32(W["final.norm"].reshape(-1)) if post or par2 else
                               self._gain1p(W["final.norm"]) if pre else None)
        if self.final_gain_vec is not None and self.final_gain_vec.numel() != self.width:
            raise ValueError("final.norm does not match width")
        ls, lc_ = config.get("logit_scale"), config.get("logit_softcap")      # absent or null: no scaling / no cap
        self.logit_scale, self.logit_softcap = 1.0 if ls is None else float(ls), 0.0 if lc_ is None else float(lc_)
        mixers = self.design.get("mixers") or {k: (v, {}) for k, v in MIXERS.items()}
        self.layers = []
        for i, lc in enumerate(config["layers"]):
            L = _Layer()
            p = f"l{i}."
            if post or par2:    # per-channel gains: post-norm on the two sublayers' outputs; two norms of the same x in front of them
                L.gain1 = self._f32(W[p + "norm1"].reshape(-1))
                L.gain2 = self._f32(W[p + "norm2"].reshape(-1)) if lc.get("mlp") else None
                L.shift = L.prev = None
            elif pre:   # per-channel gains of the norms in front of the two sublayers, stored around zero
                L.gain1 = self._gain1p(W[p + "norm1"])
                L.gain2 = self._gain1p(W[p + "norm2"]) if lc.get("mlp") else None
                L.shift = L.prev = None
            else:
                L.gain = float(W[p + "norm1"].to(torch.float32))
                L.shift = self._f32(W[p + "shift"]) if p + "shift" in W else None
                L.prev = self.states.add_state(self.width) if L.shift is not None else None
            if lc["type"] not in mixers:
                raise ValueError(f"unknown mixer type {lc['type']!r}")
            mixer_cls, constants = mixers[lc["type"]]
            L.mixer = mixer_cls(self, p + "mix.", lc.get("mixer") or {}, W, **constants)
            mc = lc.get("mlp")
            L.ff = None
            if mc:
                if mc["kind"] not in FEED_FORWARDS:
                    raise ValueError(f"unknown feed-forward kind {mc['kind']!r}")
                if mc["kind"] not in self.design["ff"]:
                    raise ValueError(f"feed-forward kind {mc['kind']!r} is not part of this design")
                L.ff = FEED_FORWARDS[mc["kind"]](self, p + "mlp.", mc, W, **self.design["ff"][mc["kind"]])
            self.layers.append(L)
        self._build_runs(config.get("loop"), W)

    def _build_runs(self, loop, W):
        """The order in which layers RUN: (layer, mixer, pass number or None).  A looped block [start, stop) runs `times`
        times in a row with the same weights; every pass after the first gets mixers with a cache / state of their own
        (new_pass), and its first run carries the pass number: the block input x <- W_in [x | x0] + step[t] comes first."""
        n = len(self.layers)
        self.loop_in = self.loop_step = None
        if not loop or int(loop.get("times", 0)) < 1 or int(loop["stop"]) <= int(loop["start"]):
            self.runs = [(L, L.mixer, None) for L in self.layers]
            return
        if self.wiring != "pre_norm":
            raise ValueError("looped blocks are served in the pre-norm wiring")
        a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
        if not 0 <= a < b <= n:
            raise ValueError("loop: start / stop outside the layer list")
        if tuple(W["loop.in"].shape) != (self.width, 2 * self.width) or tuple(W["loop.step"].shape) != (times, self.width):
            raise ValueError("loop.in / loop.step do not match width / times")
        self.loop_in = self._weight(W["loop.in"])
        self.loop_step = self._f32(W["loop.step"])
        self.runs = [(L, L.mixer, None) for L in self.layers[:a]]
        for t in range(times):
            for i in range(a, b):
                L = self.layers[i]
                if t and not hasattr(L.mixer, "new_pass"):
                    raise ValueError(f"mixer {L.mixer.kind!r} cannot run in a looped block")
                self.runs.append((L, L.mixer if t == 0 else L.mixer.new_pass(self), t if i == a else None))
        self.runs += [(L, L.mixer, None) for L in self.layers[b:]]

    @classmethod
    def from_pretrained(cls, path, dtype="bfloat16", **kw):
        with open(os.path.join(path, "config.json")) as f:
            config = json.load(f)
        return cls(config, load_file(os.path.join(path, "model.safetensors")), dtype, **kw)

    # ---- weights ----------------------------------------------------------------------------------------------------
    def _f32(self, t):
        return t.to(torch.float32).to(self.device).contiguous()

    def _gain1p(self, t):
        """1 + w of a norm weight stored around zero (float)."""
        return (1.0 + t.reshape(-1).to(torch.float32)).to(self.device).contiguous()

    def _bias(self, t):
        """A linear layer's bias for _linear: the activation type for the vendor GEMM's epilogue, float for the fp32 kernel."""
        return None if t is None else t.to(self.act_dtype).to(self.device).contiguous()

    def _weight_raw(self, t):
        """[.., out, in] in the activation type (the grouped kernels read the stored orientation)."""
        return t.to(self.act_dtype).to(self.device).contiguous()

    def _weight(self, t):
        """A linear layer's weight for _linear: bfloat16 keeps [out, in] (vendor GEMM, transposed operand); float32
        is stored [in, out], the layout of the fp32 linear kernels."""
        if self.act_dtype == torch.float32:
            return t.to(torch.float32).t().contiguous().to(self.device)
        return self._weight_raw(t)

    def _linear(self, x, w, out_dtype=None, bias=None):
        R = x.shape[0]
        if self.act_dtype == torch.float32:
            K, N = w.shape
            out = torch.empty((R, N), dtype=torch.float32, device=self.device)
            need = self._lib.pa_linear_workspace_bytes(R, K, N)
            if need and (self._ws is None or self._ws.numel() < need):
                self._ws = torch.empty(need, dtype=torch.uint8, device=self.device)
            _chk(self._lib.pa_linear_f32_exact(x.data_ptr(), w.data_ptr(), _cabi.ptr(bias), R, K, N, 0, out.data_ptr(),
                                               _cabi.ptr(self._ws) if need else None, self._ws.numel() if need else 0,
                                               _cabi.stream()), "pa_linear_f32_exact")
            return out
        if out_dtype == torch.float32:
            if bias is not None:
                raise ValueError("_linear: no bias with a float result of bfloat16 operands")
            return torch.mm(x, w.t(), out_dtype=torch.float32)
        return torch.nn.functional.linear(x, w, bias)

    # ---- the step ---------------------------------------------------------------------------------------------------
    def forward(self, batch, want_rows=None):
        """Run the rows of `batch` through the stack from the cache / state earlier steps left (and leave theirs).
        want_rows: int32 device tensor of rows whose logits are wanted (None: all).  Returns float logits
        [len(want_rows), vocab]."""
        c = _Ctx(self, batch)
        lib, R, W, s = self._lib, batch.rows, self.width, _cabi.stream()
        x = torch.empty((R, W), dtype=torch.float32, device=self.device)
        _chk(lib.pa_embedding_rows_scaled(self.embed.data_ptr(), c.elem, batch.ids.data_ptr(), R, W, self.vocab,
                                          self.embed_scale, x.data_ptr(), s), "pa_embedding_rows_scaled")
        if self.wiring == "post_norm":
            self._post_norm_layers(c, x)
        elif self.wiring == "pre_norm":
            x = self._pre_norm_layers(c, x)
        elif self.wiring == "parallel_two_norms":
            self._parallel_two_norm_layers(c, x)
        for L in self.layers if self.wiring == "parallel" else ():
            h = c.empty(R, W)
            hs = c.empty(R, W) if L.shift is not None else None
            _chk(lib.pa_rms_norm_shift(x.data_ptr(), R, W, self.eps, L.gain, None, _cabi.ptr(L.shift),
                                       batch.row_prev.data_ptr(), batch.row_slot.data_ptr(), _cabi.ptr(L.prev),
                                       h.data_ptr(), _cabi.ptr(hs), c.elem, s), "pa_rms_norm_shift")
            if L.shift is not None:
                _chk(lib.pa_rms_norm_state_store(x.data_ptr(), W, self.eps, L.gain, None, batch.seq_start.data_ptr(),
                                                 batch.seq_len.data_ptr(), batch.seq_slot.data_ptr(), batch.num_seqs,
                                                 L.prev.data_ptr(), s), "pa_rms_norm_state_store")
            mix = L.mixer.forward(c, hs if hs is not None else h)
            ff = L.ff.forward(c, h) if L.ff is not None else {}
            _chk(lib.pa_residual_combine(x.data_ptr(), R, W, self.mult, mix.data_ptr(), _cabi.ptr(ff.get("dense")),
                                         _cabi.ptr(ff.get("routed")), ff.get("top", 1), _cabi.ptr(ff.get("shared")),
                                         _cabi.ptr(ff.get("shared_gate")), c.elem, s), "pa_residual_combine")
            if self.layer_hook is not None:
                self.layer_hook(x)
        if want_rows is not None and want_rows.numel() == 0:
            return torch.empty((0, self.vocab), dtype=torch.float32, device=self.device)
        if want_rows is not None:
            n = want_rows.numel()
            xs = torch.empty((n, W), dtype=torch.float32, device=self.device)
            _chk(lib.pa_gather_rows_f32(x.data_ptr(), want_rows.data_ptr(), n, W, xs.data_ptr(), s), "pa_gather_rows_f32")
        else:
            n, xs = R, x
        hf = torch.empty((n, W), dtype=self.act_dtype, device=self.device)
        _chk(lib.pa_rms_norm_shift(xs.data_ptr(), n, W, self.eps, self.final_gain, _cabi.ptr(self.final_gain_vec), None, None,
                                   None, None, hf.data_ptr(), None, c.elem, s), "pa_rms_norm_shift")
        logits = self._linear(hf, self.head, out_dtype=torch.float32)
        if self.logit_scale != 1.0 or self.logit_softcap > 0.0:
            _chk(lib.pa_logit_softcap(logits.data_ptr(), logits.numel(), self.logit_scale, self.logit_softcap, s),
                 "pa_logit_softcap")
        return logits

    def _parallel_two_norm_layers(self, c, x):
        """x += mixer(N(x; w1)) + ff(N(x; w2)): both sublayers read the same x through norms that differ only in their
        gains.  pa_residual_add_norm2 adds a layer's outputs to the float residual and leaves BOTH operands of the next
        layer (one mean square) in the activation type."""
        lib, R, W, s = self._lib, c.R, self.width, _cabi.stream()

        def add_norm(add, nxt):
            if add.get("shared") is not None:
                raise ValueError("a shared expert is not served in the two-norm parallel wiring")
            h1 = c.empty(R, W) if nxt is not None else None
            h2 = c.empty(R, W) if nxt is not None and nxt.gain2 is not None else None
            _chk(lib.pa_residual_add_norm2(x.data_ptr(), R, W, _cabi.ptr(add.get("y")), _cabi.ptr(add.get("dense")),
                                           _cabi.ptr(add.get("routed")), _cabi.ptr(add.get("sel_w")),
                                           _cabi.ptr(add.get("sel_id")), add.get("top", 0), add.get("experts", 0),
                                           _cabi.ptr(add.get("ident")), self.eps,
                                           _cabi.ptr(nxt.gain1) if nxt is not None else None, _cabi.ptr(h1),
                                           _cabi.ptr(nxt.gain2) if h2 is not None else None, _cabi.ptr(h2), c.elem, s),
                 "pa_residual_add_norm2")
            return h1, h2

        layers = self.layers
        h1, h2 = add_norm({}, layers[0]) if layers else (None, None)
        for i, L in enumerate(layers):
            add = dict(y=L.mixer.forward(c, h1))
            if L.ff is not None:
                add.update(L.ff.forward(c, h2))
            h1, h2 = add_norm(add, layers[i + 1] if i + 1 < len(layers) else None)
            if self.layer_hook is not None:
                self.layer_hook(x)

    def _post_norm_layers(self, c, x):
        """x += N(mixer(x)), then x += N(ff(x)): the sublayers read the residual itself (rounded to the activation type
        for the products in bfloat16; the float rows themselves in float32), the norm is on their output, and the
        residual sum stays float.  pa_residual_add_norm leaves the next sublayer's operand as it updates x."""
        lib, R, W, s = self._lib, c.R, self.width, _cabi.stream()
        f32 = self.act_dtype == torch.float32
        h = x
        if not f32:
            h = c.empty(R, W)
            _chk(lib.pa_cast_rows(x.data_ptr(), R * W, h.data_ptr(), c.elem, s), "pa_cast_rows")
        for L in self.layers:
            mix = L.mixer.forward(c, h)
            nxt = None if f32 else c.empty(R, W)
            _chk(lib.pa_residual_add_norm(x.data_ptr(), R, W, self.eps, L.gain1.data_ptr(), mix.data_ptr(), None, None, 0,
                                          _cabi.ptr(nxt), c.elem, s), "pa_residual_add_norm")
            h = x if f32 else nxt
            if L.ff is not None:
                ff = L.ff.forward(c, h)
                nxt = None if f32 else c.empty(R, W)
                _chk(lib.pa_residual_add_norm(x.data_ptr(), R, W, self.eps, L.gain2.data_ptr(), _cabi.ptr(ff.get("dense")),
                                              _cabi.ptr(ff.get("routed")), _cabi.ptr(ff.get("sel_w")), ff.get("top", 0),
                                              _cabi.ptr(nxt), c.elem, s), "pa_residual_add_norm")
                h = x if f32 else nxt
            if self.layer_hook is not None:
                self.layer_hook(x)

    def _pre_norm_layers(self, c, x):
        """x += mixer(N1(x)), then x += ff(N2(x)), over self.runs.  The residual sum stays float; every add to x is fused
        with the norm in front of the NEXT sublayer (pa_residual_add_prenorm), which leaves that sublayer's operand in the
        activation type.  Returns the residual (a looped block's input product makes a new tensor)."""
        lib, R, W, s = self._lib, c.R, self.width, _cabi.stream()
        x0 = x.clone() if self.loop_in is not None else None

        def add_norm(x, add, gain):
            """x += the addends of `add`; returns N(x) * gain in the activation type (None without a gain)."""
            if not add and gain is None:
                return None
            h = c.empty(R, W) if gain is not None else None
            if add.get("shared_gate") is not None:
                raise ValueError("a gated shared expert is not served in the pre-norm wiring")
            y = add.get("y", add.get("dense"))
            _chk(lib.pa_residual_add_prenorm(x.data_ptr(), R, W, _cabi.ptr(y), add.get("y_scale", 1.0), _cabi.ptr(add.get("y2")),
                                             add.get("y2_scale", 1.0), _cabi.ptr(add.get("routed")), _cabi.ptr(add.get("sel_w")),
                                             add.get("top", 0), _cabi.ptr(add.get("shared")), _cabi.ptr(add.get("bias")),
                                             self.eps, _cabi.ptr(gain), _cabi.ptr(h), c.elem, s), "pa_residual_add_prenorm")
            return h

        pending = {}
        for L, mixer, pass_t in self.runs:
            if pass_t is not None:
                add_norm(x, pending, None)
                cat = c.empty(R, 2 * W)
                _chk(lib.pa_concat_rows(x.data_ptr(), x0.data_ptr(), R, W, cat.data_ptr(), c.elem, s), "pa_concat_rows")
                x = self._linear(cat, self.loop_in, out_dtype=torch.float32)
                pending = dict(bias=self.loop_step[pass_t])
            h = add_norm(x, pending, L.gain1)
            mix = mixer.forward(c, h)
            pending = mix if isinstance(mix, dict) else dict(y=mix)
            if L.ff is not None:
                h = add_norm(x, pending, L.gain2)
                pending = L.ff.forward(c, h)
            if self.layer_hook is not None:
                add_norm(x, pending, None)
                pending = {}
                self.layer_hook(x)
        add_norm(x, pending, None)
        return x

    layer_hook = None   # debugging aid: called with the float residual after every layer
