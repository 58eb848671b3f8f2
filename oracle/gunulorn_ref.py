"""TEST INFRASTRUCTURE ONLY -- plain float64 restatement of the `Gunulorn` design, one function per mechanism, written
from the equations; shares no code with the product path (llm_decoder.hybrid and the CUDA kernels).  Slow on purpose:
attention is a loop over queries and keys, every sequence is recomputed from its first token.

Notation: a sequence is a matrix X [tokens, width]; position i counts from 0.

    norm(x; w)   = x / sqrt(mean(x^2) + eps) * w
    layer        X <- X + mixer(norm(X; w1)) + ff(norm(X; w2))         (both sublayers read the same X)
    logits       cap * tanh(s * (norm(X; w_final) head^T) / cap)
"""
import math

import torch

F = torch.float64


# ------------------------------------------------------------------------------------------------------- small functions
def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z / (1.0 + torch.exp(-z))


def sees_causal(i, j):
    return j <= i


def sees_window_keep(i, j, size, keep):
    """A sliding window of `size` positions that also keeps the first `keep` positions of the sequence."""
    return j <= i and (i - j < size or j < keep)


def turn_pairs(x, pos, dims, base, sign=1.0):
    """Turns the neighbouring pairs (2m, 2m + 1), m < dims / 2, of the vector x by sign * pos * base^(-2m / dims); what
    lies beyond `dims` passes."""
    y = x.clone()
    for m in range(dims // 2):
        a = sign * pos * base ** (-2.0 * m / dims)
        u, v = x[2 * m], x[2 * m + 1]
        y[2 * m] = u * math.cos(a) - v * math.sin(a)
        y[2 * m + 1] = v * math.cos(a) + u * math.sin(a)
    return y


def short_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the first token."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def sink_attention(q, k, v, heads, kv_heads, dim, vdim, scale, sees, sink):
    """q [T, heads * dim], k [T, kv_heads * dim], v [T, kv_heads * vdim]; scale[h] multiplies head h's dot products;
    sink[h] is a logit that joins the denominator of head h's softmax and carries no value.  One query and one key at a
    time."""
    T = q.shape[0]
    out = torch.zeros(T, heads * vdim, dtype=F)
    per = heads // kv_heads
    for h in range(heads):
        g = h // per
        for i in range(T):
            js = [j for j in range(T) if sees(i, j)]
            s = torch.stack([(q[i, h * dim:(h + 1) * dim] @ k[j, g * dim:(g + 1) * dim]) * scale[h] for j in js])
            m = max(float(s.max()), float(sink[h]))
            p = torch.exp(s - m)
            p = p / (p.sum() + math.exp(float(sink[h]) - m))
            out[i, h * vdim:(h + 1) * vdim] = sum(p[n] * v[j, g * vdim:(g + 1) * vdim] for n, j in enumerate(js))
    return out


def sink_attention_matrix(q, k, v, heads, kv_heads, dim, vdim, scale, sees, sink):
    """The same numbers with one score matrix per head (for long sequences)."""
    T = q.shape[0]
    out = torch.zeros(T, heads * vdim, dtype=F)
    per = heads // kv_heads
    vis = torch.tensor([[bool(sees(i, j)) for j in range(T)] for i in range(T)])
    for h in range(heads):
        g = h // per
        s = (q[:, h * dim:(h + 1) * dim] @ k[:, g * dim:(g + 1) * dim].T) * scale[h]
        s = s.masked_fill(~vis, -math.inf)
        s = torch.cat([s, torch.full((T, 1), float(sink[h]), dtype=F)], 1)
        p = torch.softmax(s, -1)[:, :T]
        out[:, h * vdim:(h + 1) * vdim] = p @ v[:, g * vdim:(g + 1) * vdim]
    return out


ATTENTION = {"loop": sink_attention, "matrix": sink_attention_matrix}
FORM = "matrix"


# ----------------------------------------------------------------------------------------------------------------- mixers
def conv_sink_keys_values(h, W, p):
    """Keys and values of a convolved-projection attention layer as its cache holds them."""
    return short_conv(h @ W[p + "k"].T, W[p + "k.conv"]), short_conv(h @ W[p + "v"].T, W[p + "v.conv"])


def conv_sink_attention(h, W, p, c, kv=None):
    """Causal attention on projections that pass a short causal convolution; a temperature per head on the scores and a
    learned sink logit per head.  kv: keys and values of the layer this one borrows them from."""
    H = c["heads"]
    q = short_conv(h @ W[p + "q"].T, W[p + "q.conv"])
    k, v = kv if kv is not None else conv_sink_keys_values(h, W, p)
    scale = [c["scale"] * float(W[p + "temp"][hd]) for hd in range(H)]
    o = ATTENTION[FORM](q, k, v, H, c["kv_heads"], c["dim"], c["vdim"], scale, sees_causal, W[p + "sink"])
    return o @ W[p + "o"].T


def turned_window_attention(h, W, p, c):
    """Attention inside a sliding window that keeps the first positions: q and k turned over their first rot.dims
    dimensions, the VALUES turned by their own position over all of vdim and each head's output turned back by the query's
    position; the softmax denominator holds an extra 1."""
    H, G, d, vd = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    rd, base = c["rot"]["dims"], c["rot"]["base"]
    T = h.shape[0]
    q, k, v = (h @ W[p + n].T for n in ("q", "k", "v"))
    q, k, v = q.clone(), k.clone(), v.clone()
    for t in range(T):
        for hd in range(H):
            q[t, hd * d:(hd + 1) * d] = turn_pairs(q[t, hd * d:(hd + 1) * d], t, rd, base)
        for g in range(G):
            k[t, g * d:(g + 1) * d] = turn_pairs(k[t, g * d:(g + 1) * d], t, rd, base)
            v[t, g * vd:(g + 1) * vd] = turn_pairs(v[t, g * vd:(g + 1) * vd], t, vd, base)
    size, keep = c["mask"]["size"], c["mask"]["keep_first"]
    o = ATTENTION[FORM](q, k, v, H, G, d, vd, [c["scale"]] * H, lambda i, j: sees_window_keep(i, j, size, keep),
                        torch.zeros(H, dtype=F))
    for t in range(T):
        for hd in range(H):
            o[t, hd * vd:(hd + 1) * vd] = turn_pairs(o[t, hd * vd:(hd + 1) * vd], t, vd, base, sign=-1.0)
    return o @ W[p + "o"].T


# --------------------------------------------------------------------------------------------------------- feed-forwards
def poly_norm(z, coef, eps):
    """a N(z) + b N(z^2) + c N(z^3) + e with N = division by the root mean square over a token's values."""
    a, b, c, e = (float(t) for t in coef)
    return a * rms(z, eps) + b * rms(z * z, eps) + c * rms(z * z * z, eps) + e


def dense_ff(h, W, p, eps):
    z = h @ W[p + "up"].T + W[p + "up.b"]
    return poly_norm(z, W[p + "act"], eps) @ W[p + "down"].T + W[p + "down.b"]


def gated_expert(h, W, p):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(h, W, p, top):
    """Softmax over all router outputs; the `top` largest of score + correction are chosen; the weights are the chosen
    scores (without the correction) over their sum.  Returns per token a list of (expert, weight)."""
    s = torch.softmax(h @ W[p + "router"].T, -1)
    pick = s + W[p + "correction"]
    out = []
    for t in range(h.shape[0]):
        ids = sorted(range(s.shape[1]), key=lambda e: (-float(pick[t, e]), e))[:top]
        tot = sum(float(s[t, e]) for e in ids) + 1e-20
        out.append([(e, float(s[t, e]) / tot) for e in ids])
    return out


def moe_ff(h, W, p, c):
    """Routed experts; the last router.identity router outputs stand for experts that return their input."""
    E = c["router"]["experts"]
    out = torch.zeros_like(h)
    for t, chosen in enumerate(route(h, W, p, c["router"]["top"])):
        for e, w in chosen:
            out[t] += w * (gated_expert(h[t:t + 1], W, f"{p}e{e}.")[0] if e < E else h[t])
    return out


# ------------------------------------------------------------------------------------------------------------------ model
def layer(config, W, i, X, kv_cache):
    lc, eps, p = config["layers"][i], config["norm"]["eps"], f"l{i}."
    h1 = rms(X, eps) * W[p + "norm1"]
    c = lc["mixer"]
    if lc["type"] == "attention":
        if c.get("kv_from") is None:
            kv_cache[i] = conv_sink_keys_values(h1, W, p + "mix.")
            mix = conv_sink_attention(h1, W, p + "mix.", c, kv_cache[i])
        else:
            mix = conv_sink_attention(h1, W, p + "mix.", c, kv_cache[int(c["kv_from"])])
    elif lc["type"] == "attention_2":
        mix = turned_window_attention(h1, W, p + "mix.", c)
    else:
        raise ValueError(lc["type"])
    mc = lc.get("mlp")
    if not mc:
        return X + mix
    h2 = rms(X, eps) * W[p + "norm2"]
    ff = dense_ff(h2, W, p + "mlp.", eps) if mc["kind"] == "dense" else moe_ff(h2, W, p + "mlp.", mc)
    return X + (mix + ff)


def forward(config, weights, tokens, layers_out=None):
    """Logits [T, vocab] (float64) of one sequence from its first token; layers_out collects the residual after every layer."""
    W = {k: (v.to(F) if v.is_floating_point() else v) for k, v in weights.items()}
    X = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kv_cache = {}
    for i in range(len(config["layers"])):
        X = layer(config, W, i, X, kv_cache)
        if layers_out is not None:
            layers_out.append(X.clone())
    z = (rms(X, config["norm"]["eps"]) * W["final.norm"]) @ W["head"].T * config["logit_scale"]
    cap = config["logit_softcap"]
    return cap * torch.tanh(z / cap)


# ------------------------------------------------------------------------------------------- configurations and weights
def moe_mlp(experts=6, identity=1, top=2, ff=16):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, identity=identity, top=top))


def dense_mlp(ff=48):
    return dict(kind="dense", ff=ff)


def conv_layer(heads=4, kv_heads=2, dim=16, vdim=8, conv=3, scale=None, kv_from=None, mlp=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, scale=scale or dim ** -0.5)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="attention", mixer=m, mlp=mlp)


def window_layer(heads=4, kv_heads=2, dim=16, vdim=16, size=24, keep=3, rot_dims=8, base=10000.0, scale=None, mlp=None):
    return dict(type="attention_2", mlp=mlp,
                mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale or dim ** -0.5,
                           mask=dict(size=size, keep_first=keep), rot=dict(dims=rot_dims, base=base)))


def make_config(layers, width=64, vocab=80, eps=1e-6, logit_scale=0.5, logit_softcap=20.0):
    return dict(architecture="Gunulorn", width=width, vocab=vocab, norm=dict(eps=eps), logit_scale=logit_scale,
                logit_softcap=logit_softcap, layers=layers)


def random_weights(config, seed=0, sharp=1.0):
    """bfloat16 weights (as a model folder holds them).  sharp scales q and k: larger values make the softmax pick few keys."""
    g = torch.Generator().manual_seed(seed)
    width, W = config["width"], {}

    def lin(o, i, s=1.0):
        return torch.randn(o, i, generator=g) * (s / math.sqrt(i))

    def vec(n, mean=0.0, std=1.0):
        return mean + std * torch.randn(n, generator=g)

    W["embed"] = torch.randn(config["vocab"], width, generator=g)
    for i, lc in enumerate(config["layers"]):
        p, c = f"l{i}.mix.", lc["mixer"]
        W[f"l{i}.norm1"] = vec(width, 1.0, 0.2)
        H, G, d, vd = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
        own = c.get("kv_from") is None
        W[p + "q"] = lin(H * d, width, sharp)
        if own:
            W[p + "k"], W[p + "v"] = lin(G * d, width, sharp), lin(G * vd, width)
        W[p + "o"] = lin(width, H * vd)
        if lc["type"] == "attention":
            for n, rows in (("q", H * d), ("k", G * d), ("v", G * vd)):
                if n == "q" or own:
                    W[p + n + ".conv"] = torch.randn(rows, c["conv"], generator=g) * 0.5 + (torch.arange(c["conv"]) == c["conv"] - 1) * 0.5
            W[p + "temp"] = vec(H, 1.0, 0.3).abs() + 0.2
            W[p + "sink"] = vec(H, 0.0, 1.5)
        mc = lc.get("mlp")
        if not mc:
            continue
        W[f"l{i}.norm2"] = vec(width, 1.0, 0.2)
        p = f"l{i}.mlp."
        if mc["kind"] == "dense":
            W[p + "up"], W[p + "up.b"] = lin(mc["ff"], width), vec(mc["ff"], 0.0, 0.3)
            W[p + "down"], W[p + "down.b"] = lin(width, mc["ff"]), vec(width, 0.0, 0.1)
            W[p + "act"] = torch.tensor([0.9, 0.5, 0.3, 0.1]) + 0.1 * torch.randn(4, generator=g)
        else:
            E, I, ff = mc["router"]["experts"], mc["router"].get("identity", 0), mc["expert"]["ff"]
            for e in range(E):
                W[f"{p}e{e}.gate"], W[f"{p}e{e}.up"], W[f"{p}e{e}.down"] = lin(ff, width), lin(ff, width), lin(width, ff)
            W[p + "router"] = lin(E + I, width, 2.0)
            W[p + "correction"] = vec(E + I, 0.0, 0.05)
    W["final.norm"] = vec(width, 1.0, 0.2)
    W["head"] = lin(config["vocab"], width)
    return {k: v.to(torch.bfloat16) for k, v in W.items()}
