"""TEST INFRASTRUCTURE ONLY -- plain float64 restatement of the `Dubarax` design, one function per mechanism, written
from the equations; shares no code with the product path (llm_decoder.hybrid and the CUDA kernels).  Slow on purpose:
attention is a loop over queries and keys, the recurrences walk token by token, every sequence is recomputed from its
first token.

Notation: a sequence is a matrix X [tokens, width]; position i counts from 0.

    norm(x; w)      = x / sqrt(mean(x^2) + eps) * (1 + w)
    layer           X <- X + mixer(norm(X; w1));  X <- X + ff(norm(X; w2))
    looped block    layers [a, b) run `times` times; pass t starts with X <- [X | X0] W_in^T + step_t, X0 = scaled embedding
"""
import math

import torch

F = torch.float64


# ------------------------------------------------------------------------------------------------------- small functions
def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm1p(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def silu(z):
    return z / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.where(z > 40.0, z, torch.log1p(torch.exp(torch.clamp(z, max=40.0))))


def distance_bucket(n, buckets, far):
    """Distances below buckets // 2 get a bucket each; beyond, buckets widen geometrically and end at `far`."""
    half = buckets // 2
    if n < half:
        return n
    return min(buckets - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (buckets - half))))


def sees_window(i, j, size):
    return 0 <= i - j < size


def sees_chunk(i, j, size):
    return j <= i and i // size == j // size


def head_slope(h, heads, exponent=8.0):
    return 2.0 ** (-exponent * (h + 1) / heads)


# ------------------------------------------------------------------------------------------------------------ mechanisms
def softmax_attention(q, k, v, heads, kv_heads, dim, vdim, score, sees):
    """q [T, heads * dim], k [T, kv_heads * dim], v [T, kv_heads * vdim]; score(h, i, j, dot) -> float, sees(i, j) -> bool.
    One query, one key at a time."""
    T = q.shape[0]
    out = torch.zeros(T, heads * vdim, dtype=F)
    per = heads // kv_heads
    for h in range(heads):
        g = h // per
        for i in range(T):
            js = [j for j in range(T) if sees(i, j)]
            s = torch.stack([score(h, i, j, q[i, h * dim:(h + 1) * dim] @ k[j, g * dim:(g + 1) * dim]) for j in js])
            p = torch.exp(s - s.max())
            p = p / p.sum()
            out[i, h * vdim:(h + 1) * vdim] = sum(p[n] * v[j, g * vdim:(g + 1) * vdim] for n, j in enumerate(js))
    return out


def softmax_attention_matrix(q, k, v, heads, kv_heads, dim, vdim, score, sees):
    """The same numbers with one score matrix per head (for long sequences); `score` and `sees` are called per entry only
    through small tables, so a test compares this form with the loop above."""
    T = q.shape[0]
    out = torch.zeros(T, heads * vdim, dtype=F)
    per = heads // kv_heads
    vis = torch.tensor([[bool(sees(i, j)) for j in range(T)] for i in range(T)])
    for h in range(heads):
        g = h // per
        dots = q[:, h * dim:(h + 1) * dim] @ k[:, g * dim:(g + 1) * dim].T
        # the score of (h, i, j, dot) is (dot-dependent part) + (distance-dependent part): both read off the scalar form
        s = torch.stack([torch.stack([score(h, i, j, dots[i, j]) if vis[i, j] else torch.tensor(-math.inf, dtype=F)
                                      for j in range(T)]) for i in range(T)]) if T <= 8 else _score_rows(score, h, dots, vis)
        p = torch.softmax(s, -1)
        out[:, h * vdim:(h + 1) * vdim] = p @ v[:, g * vdim:(g + 1) * vdim]
    return out


def _score_rows(score, h, dots, vis):
    """score() applied to whole diagonals: all entries of one distance share the distance-dependent part."""
    T = dots.shape[0]
    s = torch.full((T, T), -math.inf, dtype=F)
    for dist in range(T):
        i = torch.arange(dist, T)
        j = i - dist
        s[i, j] = score(h, dist, 0, dots[i, j])          # (i, j) enter the score only through i - j
    return s.masked_fill(~vis, -math.inf)


ATTENTION = {"loop": softmax_attention, "matrix": softmax_attention_matrix}
FORM = "matrix"


def qkv_biased(h, W, p):
    return tuple(h @ W[p + n].T + W[p + n + ".b"] for n in ("q", "k", "v"))


def window_attention(h, W, p, c):
    """Soft-capped scores plus a learned bias per distance bucket and head, inside a sliding window."""
    q, k, v = qkv_biased(h, W, p)
    rel, cap = W[p + "rel"], c["softcap"]

    def score(hd, i, j, dot):
        s = cap * torch.tanh(dot * c["scale"] / cap)
        return s + rel[distance_bucket(i - j, rel.shape[0], c["bias_max"]), hd]
    o = ATTENTION[FORM](q, k, v, c["heads"], c["kv_heads"], c["dim"], c["vdim"], score,
                        lambda i, j: sees_window(i, j, c["mask"]["size"]))
    return o @ W[p + "o"].T + W[p + "o.b"]


def chunk_attention(h, W, p, c):
    """Scores minus slope_h * distance, visibility inside fixed chunks of positions."""
    q, k, v = qkv_biased(h, W, p)
    o = ATTENTION[FORM](q, k, v, c["heads"], c["kv_heads"], c["dim"], c["vdim"],
                        lambda hd, i, j, dot: dot * c["scale"] - head_slope(hd, c["heads"]) * (i - j),
                        lambda i, j: sees_chunk(i, j, c["mask"]["size"]))
    return o @ W[p + "o"].T + W[p + "o.b"]


def decayed_linear_attention(h, W, p, c, eps):
    H, d, vd = c["heads"], c["dim"], c["vdim"]
    q, k, v = silu(h @ W[p + "q"].T), silu(h @ W[p + "k"].T), silu(h @ W[p + "v"].T)
    T = h.shape[0]
    o = torch.zeros(T, H * vd, dtype=F)
    for hd in range(H):
        S = torch.zeros(d, vd, dtype=F)
        for t in range(T):
            S = c["decay"][hd] * S + torch.outer(k[t, hd * d:(hd + 1) * d], v[t, hd * vd:(hd + 1) * vd])
            o[t, hd * vd:(hd + 1) * vd] = q[t, hd * d:(hd + 1) * d] @ S
    o = rms(o, eps) * W[p + "norm"]
    return (o * torch.sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


def parallel_mixer(h, W, p, c, eps):
    return c["left_scale"] * chunk_attention(h, W, p + "left.", c["left"]) + \
        c["right_scale"] * decayed_linear_attention(h, W, p + "right.", c["right"], eps)


def causal_conv(x, w, b):
    """x [T, C], w [C, taps] (last column: the current token), zeros before the first token."""
    T, taps = x.shape[0], w.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        acc = b.clone()
        for i in range(taps):
            s = t - (taps - 1 - i)
            if s >= 0:
                acc = acc + w[:, i] * x[s]
        out[t] = acc
    return out


def state_space_mixer(h, W, p, c, eps):
    H, P, N, G = c["heads"], c["vdim"], c["state"], c["groups"]
    inner = H * P
    u = h @ W[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x, B, C = xbc[:, :inner], xbc[:, inner:inner + G * N], xbc[:, inner + G * N:]
    dt = softplus(dt + W[p + "dt_bias"])
    T = h.shape[0]
    y = torch.zeros(T, inner, dtype=F)
    for hd in range(H):
        g = hd // (H // G)
        rate = torch.exp(W[p + "A_log"][hd])
        S = torch.zeros(N, P, dtype=F)
        for t in range(T):
            xt = x[t, hd * P:(hd + 1) * P]
            S = torch.exp(-rate * dt[t, hd]) * S + dt[t, hd] * torch.outer(B[t, g * N:(g + 1) * N], xt)
            y[t, hd * P:(hd + 1) * P] = C[t, g * N:(g + 1) * N] @ S + W[p + "D"][hd] * xt
    y = y * silu(z)
    parts = c["norm_groups"]
    y = rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * W[p + "norm"]
    return y @ W[p + "o"].T


def gated_expert(h, W, p):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(scores, top, count, keep):
    """The chosen experts of one token: only experts of the `keep` groups whose best score is largest are eligible."""
    E = scores.numel()
    per = E // count
    best = sorted(range(count), key=lambda g: (-float(scores[g * per:(g + 1) * per].max()), g))[:keep]
    eligible = [e for e in range(E) if e // per in best]
    return sorted(eligible, key=lambda e: (-float(scores[e]), e))[:top]


def moe_ff(h, W, p, c):
    r = c["router"]
    grp = r.get("groups") or {"count": 1, "keep": 1}
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        s = torch.softmax(W[p + "router"] @ h[t], 0)
        for e in route(s, r["top"], grp["count"], grp["keep"]):
            out[t] = out[t] + s[e] * gated_expert(h[t], W, f"{p}e{e}.")
    if c.get("shared"):
        out = out + gated_expert(h, W, p + "shared.")
    return out


# ----------------------------------------------------------------------------------------------------------------- model
def layer(config, W, i, X):
    lc, p, eps = config["layers"][i], f"l{i}.", config["norm"]["eps"]
    h = norm1p(X, W[p + "norm1"], eps)
    kind = lc["type"]
    if kind == "attention":
        m = window_attention(h, W, p + "mix.", lc["mixer"])
    elif kind == "parallel":
        m = parallel_mixer(h, W, p + "mix.", lc["mixer"], eps)
    elif kind == "mamba2":
        m = state_space_mixer(h, W, p + "mix.", lc["mixer"], eps)
    else:
        raise ValueError(kind)
    X = X + m
    if lc.get("mlp"):
        X = X + moe_ff(norm1p(X, W[p + "norm2"], eps), W, p + "mlp.", lc["mlp"])
    return X


def forward(config, weights, tokens):
    """Returns (logits [T, vocab], residual after every layer run [runs, T, width]), float64."""
    W = {k: v.to(F) for k, v in weights.items()}
    X0 = W["embed"][torch.tensor(list(tokens))] * config["embedding"]["scale"]
    X, after = X0, []
    n = len(config["layers"])
    lp = config.get("loop")
    a, b, times = (lp["start"], lp["stop"], lp["times"]) if lp else (0, 0, 0)
    for i in range(a):
        X = layer(config, W, i, X)
        after.append(X)
    for t in range(times):
        X = torch.cat([X, X0], 1) @ W["loop.in"].T + W["loop.step"][t]
        for i in range(a, b):
            X = layer(config, W, i, X)
            after.append(X)
    for i in range(b, n):
        X = layer(config, W, i, X)
        after.append(X)
    logits = norm1p(X, W["final.norm"], config["norm"]["eps"]) @ W["head"].T
    return logits, torch.stack(after)


# --------------------------------------------------------------------------------------------- configurations and weights
def moe_mlp(experts=6, top=2, ff=16, count=1, keep=1, shared_ff=24):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}},
            "shared": {"ff": shared_ff} if shared_ff else None}


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=16, window=24, buckets=8, bias_max=40, softcap=20.0, scale=None, mlp=None):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window},
                      "bias_max": bias_max, "softcap": softcap, "scale": scale if scale is not None else dim ** -0.5,
                      "buckets": buckets}}


def parallel_layer(heads=4, kv_heads=1, dim=16, vdim=8, chunk=20, scale=None, lin_heads=2, lin_dim=8, lin_vdim=16,
                   decay=(0.7, 0.98), left_scale=0.9, right_scale=1.2, mlp=None):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": chunk},
                               "scale": scale if scale is not None else dim ** -0.5},
                      "right": {"heads": lin_heads, "dim": lin_dim, "vdim": lin_vdim, "decay": list(decay)},
                      "left_scale": left_scale, "right_scale": right_scale}}


def mamba_layer(heads=4, vdim=8, state=16, groups=2, conv=4, norm_groups=2, mlp=None):
    return {"type": "mamba2", "mlp": mlp,
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}}


def make_config(layers, width=64, vocab=80, eps=1e-6, embed_scale=4.0, loop=None):
    cfg = {"architecture": "Dubarax", "embedding": {"scale": embed_scale}, "layers": layers, "norm": {"eps": eps},
           "vocab": vocab, "width": width}
    if loop:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


def random_weights(config, seed=0):
    """bfloat16 tensors under the names the loader reads."""
    g = torch.Generator().manual_seed(seed)
    Wd, width = {}, config["width"]

    def lin(name, out, inp, gain=1.0):
        Wd[name] = (torch.randn(out, inp, generator=g) * gain / math.sqrt(inp)).to(torch.bfloat16)

    def vec(name, n, std=0.1, mean=0.0):
        Wd[name] = (torch.randn(n, generator=g) * std + mean).to(torch.bfloat16)

    Wd["embed"] = (torch.randn(config["vocab"], width, generator=g) * 0.5).to(torch.bfloat16)
    lin("head", config["vocab"], width)
    vec("final.norm", width)
    if config.get("loop"):
        lin("loop.in", width, 2 * width)
        Wd["loop.step"] = (torch.randn(config["loop"]["times"], width, generator=g) * 0.3).to(torch.bfloat16)

    def attn(p, c, rel):
        H, G, d, vd = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
        for n, rows in (("q", H * d), ("k", G * d), ("v", G * vd)):
            lin(p + n, rows, width, 2.0 if n != "v" else 1.0)
            vec(p + n + ".b", rows, 0.2)
        lin(p + "o", width, H * vd)
        vec(p + "o.b", width, 0.1)
        if rel:
            Wd[p + "rel"] = torch.randn(c.pop("buckets"), H, generator=g).to(torch.bfloat16)

    for i, lc in enumerate(config["layers"]):
        p, c = f"l{i}.mix.", lc["mixer"]
        vec(f"l{i}.norm1", width)
        if lc["type"] == "attention":
            attn(p, c, True)
        elif lc["type"] == "parallel":
            attn(p + "left.", c["left"], False)
            r = c["right"]
            H, d, vd = r["heads"], r["dim"], r["vdim"]
            for n, rows in (("q", H * d), ("k", H * d), ("v", H * vd), ("g", H * vd)):
                lin(p + "right." + n, rows, width, 1.5)
            lin(p + "right.o", width, H * vd)
            vec(p + "right.norm", H * vd, 0.2, 1.0)
        else:
            H, P, N, G = c["heads"], c["vdim"], c["state"], c["groups"]
            inner, ch = H * P, H * P + 2 * G * N
            lin(p + "in", 2 * inner + 2 * G * N + H, width, 1.5)
            Wd[p + "conv"] = (torch.randn(ch, c["conv"], generator=g) * 0.5).to(torch.bfloat16)
            vec(p + "conv.b", ch, 0.2)
            vec(p + "dt_bias", H, 0.7, -0.5)
            vec(p + "A_log", H, 0.7, -0.5)
            vec(p + "D", H, 0.3, 1.0)
            vec(p + "norm", inner, 0.2, 1.0)
            lin(p + "o", width, inner)
        m = lc.get("mlp")
        if m:
            q = f"l{i}.mlp."
            vec(f"l{i}.norm2", width)
            lin(q + "router", m["router"]["experts"], width, 1.0)
            names = [f"e{e}." for e in range(m["router"]["experts"])] + (["shared."] if m.get("shared") else [])
            for nm in names:
                ff = m["shared"]["ff"] if nm == "shared." else m["expert"]["ff"]
                lin(q + nm + "gate", ff, width, 1.5)
                lin(q + nm + "up", ff, width, 1.5)
                lin(q + nm + "down", width, ff)
    return Wd
