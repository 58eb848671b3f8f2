#!/usr/bin/env python
"""Throughput of the `Dubarax` design (llm_decoder.hybrid: pre-norm wiring, a looped block, windowed / chunked softmax
attention with distance biases, decayed linear attention, a selective state-space mixer, group-limited routed experts) at
layer sizes that resemble a real model, next to the framework's closest existing model -- the same config-driven stack
serving `Megusun` (recurrent + attention mixers, routed experts) -- at equal width, layer count, vocabulary, batch and
context; random weights, synthetic tokens.  `python bench.py --dubarax` prints its JSON line.

Per size: prefill tokens/s (PREFILL_SEQS prompts of PREFILL_LEN tokens in one step) and decode tokens/s (DECODE_SEQS
sequences at DECODE_CTX tokens of context, one token each per step), CUDA events around back-to-back steps after
warm-up.  `kernels` times the design's own kernels alone at the largest size against their roofline (algorithmic bytes
over the measured copy bandwidth, FLOPs over the measured bf16 GEMM rate; MEASURED_PEAKS.json)."""
import json
import math
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "pagedattention-based-transformer-decoder-inference-framework_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)

from benchmarks import hybrid as hy  # noqa: E402

PREFILL_SEQS, PREFILL_LEN = hy.PREFILL_SEQS, hy.PREFILL_LEN
DECODE_SEQS, DECODE_CTX = hy.DECODE_SEQS, hy.DECODE_CTX
VOCAB = hy.VOCAB
SIZES = {
    "w1024": dict(width=1024, heads=8, kv_heads=2, dim=64, vdim=128, window=1024, chunk=512, lin_heads=8, lin_dim=64, lin_vdim=128,
                  ssm_heads=32, ssm_vdim=64, ssm_state=128, ssm_groups=2, experts=8, top=2, eff=512, sff=1024),
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=64, vdim=128, window=1024, chunk=512, lin_heads=16, lin_dim=64, lin_vdim=128,
                  ssm_heads=64, ssm_vdim=64, ssm_state=128, ssm_groups=2, experts=8, top=2, eff=1024, sff=2048),
}
timed, peaks = hy.timed, hy.peaks


def dubarax_config(s):
    moe = {"kind": "moe", "expert": {"ff": s["eff"]}, "shared": {"ff": s["sff"]},
           "router": {"experts": s["experts"], "top": s["top"], "groups": {"count": 4, "keep": 2}}}
    soft = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"], "scale": s["dim"] ** -0.5}
    att = {"type": "attention", "mlp": moe, "mixer": dict(soft, mask={"size": s["window"]}, bias_max=2 * s["window"], softcap=30.0)}
    par = {"type": "parallel", "mlp": moe,
           "mixer": {"left": dict(soft, mask={"size": s["chunk"]}), "left_scale": 0.8, "right_scale": 1.1,
                     "right": {"heads": s["lin_heads"], "dim": s["lin_dim"], "vdim": s["lin_vdim"],
                               "decay": [1.0 - 2.0 ** (-2 - 6 * h / s["lin_heads"]) for h in range(s["lin_heads"])]}}}
    ssm = {"type": "mamba2", "mlp": moe,
           "mixer": {"heads": s["ssm_heads"], "vdim": s["ssm_vdim"], "state": s["ssm_state"], "groups": s["ssm_groups"], "conv": 4,
                     "norm_groups": 2}}
    return {"architecture": "Dubarax", "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5}, "vocab": VOCAB, "width": s["width"],
            "layers": [att, ssm, par, att], "loop": {"start": 1, "stop": 3, "times": 1}}


def dubarax_weights(config, dev, buckets=32):
    g = torch.Generator(device=dev).manual_seed(0)
    Wd = config["width"]
    mat = lambda o, i: (torch.randn(o, i, device=dev, generator=g) / math.sqrt(i)).to(torch.bfloat16)  # noqa: E731
    vec = lambda n, std=0.02, mean=0.0: (torch.randn(n, device=dev, generator=g) * std + mean).to(torch.bfloat16)  # noqa: E731
    W = {"embed": torch.randn(config["vocab"], Wd, device=dev, generator=g).to(torch.bfloat16), "head": mat(config["vocab"], Wd),
         "final.norm": vec(Wd), "loop.in": mat(Wd, 2 * Wd), "loop.step": vec(config["loop"]["times"] * Wd).reshape(-1, Wd)}

    def soft(p, c, rel):
        H, G, D, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
        for n, rows in (("q", H * D), ("k", G * D), ("v", G * V)):
            W[p + n], W[p + n + ".b"] = mat(rows, Wd), vec(rows)
        W[p + "o"], W[p + "o.b"] = mat(Wd, H * V), vec(Wd)
        if rel:
            W[p + "rel"] = torch.randn(buckets, H, device=dev, generator=g).to(torch.bfloat16)

    for i, lc in enumerate(config["layers"]):
        p, c = f"l{i}.", lc["mixer"]
        W[p + "norm1"], W[p + "norm2"] = vec(Wd), vec(Wd)
        if lc["type"] == "attention":
            soft(p + "mix.", c, True)
        elif lc["type"] == "parallel":
            soft(p + "mix.left.", c["left"], False)
            r = c["right"]
            H, D, V = r["heads"], r["dim"], r["vdim"]
            q = p + "mix.right."
            W[q + "q"], W[q + "k"], W[q + "v"], W[q + "g"] = mat(H * D, Wd), mat(H * D, Wd), mat(H * V, Wd), mat(H * V, Wd)
            W[q + "o"], W[q + "norm"] = mat(Wd, H * V), vec(H * V, 0.02, 1.0)
        else:
            H, P, N, G = c["heads"], c["vdim"], c["state"], c["groups"]
            inner, ch = H * P, H * P + 2 * G * N
            q = p + "mix."
            W[q + "in"], W[q + "o"] = mat(2 * inner + 2 * G * N + H, Wd), mat(Wd, inner)
            W[q + "conv"], W[q + "conv.b"] = (torch.randn(ch, c["conv"], device=dev, generator=g) * 0.5).to(torch.bfloat16), vec(ch)
            W[q + "dt_bias"], W[q + "A_log"], W[q + "D"] = vec(H, 0.5, -2.0), vec(H, 0.5, 0.0), vec(H, 0.1, 1.0)
            W[q + "norm"] = vec(inner, 0.02, 1.0)
        ml = lc["mlp"]
        f, E = ml["expert"]["ff"], ml["router"]["experts"]
        for nm, ff in [(f"e{e}.", f) for e in range(E)] + [("shared.", ml["shared"]["ff"])]:
            W[f"{p}mlp.{nm}gate"], W[f"{p}mlp.{nm}up"], W[f"{p}mlp.{nm}down"] = mat(ff, Wd), mat(ff, Wd), mat(Wd, ff)
        W[p + "mlp.router"] = mat(E, Wd)
    return W


def bench_model(s, dtype, dev):
    import llm_decoder as ld
    config = dubarax_config(s)
    cap = DECODE_SEQS * (DECODE_CTX + 64)
    model = ld.HybridDecoder(config, dubarax_weights(config, dev), dtype, max_tokens=cap, max_seqs=DECODE_SEQS, tile_size=16)
    eng = ld.Engine(model)
    g = torch.Generator().manual_seed(1)
    toks = lambda n: torch.randint(0, VOCAB, (n,), generator=g).tolist()  # noqa: E731
    prompts = [toks(PREFILL_LEN) for _ in range(PREFILL_SEQS)]

    def prefill():
        out = eng.step([(f"p{i}", p, [PREFILL_LEN - 1]) for i, p in enumerate(prompts)])
        for i in range(PREFILL_SEQS):
            eng.finish(f"p{i}")
        return out
    t_pre = timed(prefill, 2, 4)
    for lo in range(0, DECODE_SEQS, 8):
        eng.step([(f"d{i}", toks(DECODE_CTX), []) for i in range(lo, lo + 8)])
    nxt = [toks(1) for _ in range(DECODE_SEQS)]
    t_dec = timed(lambda: eng.step([(f"d{i}", nxt[i], [0]) for i in range(DECODE_SEQS)]), 3, 10)
    for i in range(DECODE_SEQS):
        eng.finish(f"d{i}")
    del model, eng
    torch.cuda.empty_cache()
    return dict(prefill_tok_s=PREFILL_SEQS * PREFILL_LEN / t_pre, prefill_ms=t_pre * 1e3,
                decode_tok_s=DECODE_SEQS / t_dec, decode_ms=t_dec * 1e3)


def bench_kernels(s, dev):
    """The design's own kernels alone (bfloat16 activations) at the prefill and decode shapes of size `s`."""
    from llm_decoder import _cabi
    from llm_decoder.hybrid import DECAY_CHUNK, DECAY_CHUNKED_FROM, MMA_FROM, log_distance_bucket
    from llm_decoder.seq_state import SequenceStateCache
    lib, st = _cabi.lib(), _cabi.stream
    hbm, tfl, how = peaks()
    out = {}
    bf, i32 = torch.bfloat16, torch.int32
    W, H, G, D, V = s["width"], s["heads"], s["kv_heads"], s["dim"], s["vdim"]

    def rec(name, secs, bytes_=None, flops=None):
        e = dict(us=secs * 1e6)
        if bytes_ is not None:
            e.update(gbs=bytes_ / secs / 1e9, frac_of_hbm=bytes_ / secs / 1e9 / hbm)
        if flops is not None:
            e.update(tflops=flops / secs / 1e12, frac_of_bf16_gemm=flops / secs / 1e12 / tfl)
        if bytes_ is not None and flops is not None:
            e["frac_of_roofline"] = max(bytes_ / (hbm * 1e9), flops / (tfl * 1e12)) / secs
        out[name] = e

    for tag, nseq, plen, ctx0 in (("prefill", PREFILL_SEQS, PREFILL_LEN, 0), ("decode", DECODE_SEQS, 1, DECODE_CTX)):
        R = nseq * plen
        states = SequenceStateCache(nseq, nseq * (ctx0 + plen + 16), 16, dev)
        kv = states.add_kv_layer(G, D, V, "bf16")
        LH, LD, LV = s["lin_heads"], s["lin_dim"], s["lin_vdim"]
        SH, SP, SN, SG = s["ssm_heads"], s["ssm_vdim"], s["ssm_state"], s["ssm_groups"]
        inner, ch = SH * SP, SH * SP + 2 * SG * SN
        lin_state, ssm_state, conv_state = states.add_state(LH * LD * LV), states.add_state(SH * SN * SP), states.add_state(3 * ch)
        slots = [states.alloc() for _ in range(nseq)]
        if ctx0:
            for sl in slots:
                states.extend(sl, ctx0)
        b = states.make_batch([(sl, [1] * plen) for sl in slots])
        pt = kv.page_table_
        table = pt.device_data()
        kv.key_buffer_.normal_()
        kv.value_buffer_.normal_()
        # ---- softmax attention: window + bucket table + soft cap, and chunks + slopes
        qkv = torch.randn(R, H * D + G * D + G * V, device=dev).to(bf)
        o = torch.empty(R, H * V, device=dev, dtype=bf)
        tt, mt = lib.pa_masked_attention_tile_tokens(H, G), lib.pa_masked_attention_mma_tile_tokens(D, V, 2)
        for name, mask_kind, size, bias_kind in (("window", 1, s["window"], 2), ("chunk", 2, s["chunk"], 1)):
            if bias_kind == 2:
                idx = torch.tensor([log_distance_bucket(d, 32, 2.0 * size) for d in range(size)])
                bias = torch.randn(32, H)[idx].contiguous().to(dev)
            else:
                bias = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], device=dev)
            for kind, group in b.query_tiles(tt, mt, MMA_FROM).items():
                if group is None:
                    continue
                tiles, ntiles, _longest = group
                fn = lambda: lib.pa_masked_attention(qkv.data_ptr(), qkv.stride(0), 0, kv.key_buffer_.data_ptr(),  # noqa: E731
                                                     kv.value_buffer_.data_ptr(), table.data_ptr(), pt.num_beams_, pt.num_heads_,
                                                     pt.num_tiles_, kv.total_pages_, kv.tile_size_, tiles.data_ptr(), ntiles, H, D,
                                                     V, D ** -0.5, 30.0 if bias_kind == 2 else 0.0, mask_kind, size, bias_kind,
                                                     bias.data_ptr(), int(bias.shape[0]), o.data_ptr(), 2, kind, st())
                assert fn() == 0
                if plen > 1:     # visible (query, key) pairs
                    if mask_kind == 1:
                        pairs = sum(min(i + 1, size) for i in range(plen))
                    else:
                        pairs = sum(i % size + 1 for i in range(plen))
                    rec(f"masked_attention_{name}/{tag}", timed(fn, 2, 4), flops=nseq * H * pairs * (2 * D + 2 * V))
                else:
                    seen = min(ctx0 + 1, size) if mask_kind == 1 else ctx0 % size + 1
                    rec(f"masked_attention_{name}/{tag}", timed(fn), bytes_=nseq * seen * G * (D + V) * 2)
        # ---- matrix-state scans
        chunked = plen >= DECAY_CHUNKED_FROM
        items, n, s0, sn = b.chunk_items(DECAY_CHUNK if chunked else 0)
        lin = torch.randn(R, 2 * LH * LD + 2 * LH * LV, device=dev).to(bf)
        lo = torch.empty(R, LH * LV, device=dev)
        decay = torch.full((LH,), 0.97, device=dev)
        wsb = lib.pa_decay_scan_workspace_bytes(n, max(LH, SH), max(LD, SN), max(LV, SP)) if chunked else 0
        ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=dev)
        fn = lambda: lib.pa_decay_scan(lin.data_ptr(), lin.stride(0), 0, lin.data_ptr(), lin.stride(0), LH * LD, lin.data_ptr(),  # noqa: E731
                                       lin.stride(0), 2 * LH * LD, LH, LH, LD, LV, 1, decay.data_ptr(), None, 0, 0, None, None, None,
                                       lin_state.data_ptr(), lo.data_ptr(), LH * LV, items.data_ptr(), n, s0.data_ptr(),
                                       sn.data_ptr(), b.seq_slot.data_ptr(), nseq, 1 if chunked else 0, ws.data_ptr(), wsb, 2, st())
        assert fn() == 0
        if plen > 1:
            rec(f"decay_scan_linear_attention/{tag}", timed(fn, 2, 4), flops=R * LH * LD * LV * 4.0,
                bytes_=R * (2 * LH * LD + LH * LV) * 2 + R * LH * LV * 4)
        else:
            rec(f"decay_scan_linear_attention/{tag}", timed(fn), bytes_=nseq * LH * LD * LV * 8)
        proj = torch.randn(R, 2 * inner + 2 * SG * SN + SH, device=dev).to(bf)
        xbc = torch.empty(R, ch, device=dev, dtype=bf)
        cw, cb = torch.randn(ch, 4, device=dev), torch.zeros(ch, device=dev)
        chunks, nch, _a, _b = b.chunk_items(64)
        rec(f"causal_conv_silu/{tag}", timed(lambda: lib.pa_causal_conv_silu(proj.data_ptr(), proj.stride(0), inner, ch, 4, cw.data_ptr(),
                                                                             cb.data_ptr(), conv_state.data_ptr(), chunks.data_ptr(), nch,
                                                                             xbc.data_ptr(), ch, 2, st())), bytes_=R * ch * 4)
        dtb, alog, skip = torch.full((SH,), -2.0, device=dev), torch.zeros(SH, device=dev), torch.ones(SH, device=dev)
        y = torch.empty(R, inner, device=dev)
        fn = lambda: lib.pa_decay_scan(xbc.data_ptr(), ch, inner + SG * SN, xbc.data_ptr(), ch, inner, xbc.data_ptr(), ch, 0, SH, SG,  # noqa: E731
                                       SN, SP, 0, None, proj.data_ptr(), proj.stride(0), 2 * inner + 2 * SG * SN, dtb.data_ptr(),
                                       alog.data_ptr(), skip.data_ptr(), ssm_state.data_ptr(), y.data_ptr(), inner, items.data_ptr(), n,
                                       s0.data_ptr(), sn.data_ptr(), b.seq_slot.data_ptr(), nseq, 1 if chunked else 0, ws.data_ptr(),
                                       wsb, 2, st())
        assert fn() == 0
        if plen > 1:
            rec(f"decay_scan_state_space/{tag}", timed(fn, 2, 4), flops=R * SH * SN * SP * 4.0, bytes_=R * ch * 2 + R * inner * 4)
        else:
            rec(f"decay_scan_state_space/{tag}", timed(fn), bytes_=nseq * SH * SN * SP * 8)
        yn, nw = torch.empty(R, inner, device=dev, dtype=bf), torch.ones(inner, device=dev)
        rec(f"gated_rms_norm/{tag}", timed(lambda: lib.pa_gated_rms_norm(y.data_ptr(), R, inner, 2, proj.data_ptr(), proj.stride(0), 0, 1,
                                                                         nw.data_ptr(), 1e-5, yn.data_ptr(), 2, st())),
            bytes_=R * inner * (4 + 2 + 2))
        # ---- pre-norm residual, router
        E, top = s["experts"], s["top"]
        pairs = R * top
        hb = torch.randn(R, W, device=dev).to(bf)
        wr = torch.randn(E, W, device=dev) / math.sqrt(W)
        sel_id, sel_w = torch.empty(pairs, device=dev, dtype=i32), torch.empty(pairs, device=dev)
        rec(f"router_topk_grouped/{tag}", timed(lambda: lib.pa_router_topk_grouped(hb.data_ptr(), wr.data_ptr(), None, None, R, W, E, top,
                                                                                   1, 0, 4, 2, sel_id.data_ptr(), sel_w.data_ptr(), None,
                                                                                   2, st())), bytes_=R * W * 2)
        x, nxt, g1 = torch.randn(R, W, device=dev), torch.empty(R, W, device=dev, dtype=bf), torch.ones(W, device=dev)
        routed = torch.randn(pairs, W, device=dev)
        rec(f"residual_add_prenorm_routed/{tag}", timed(lambda: lib.pa_residual_add_prenorm(
            x.data_ptr(), R, W, None, 1.0, None, 1.0, routed.data_ptr(), sel_w.data_ptr(), top, hb.data_ptr(), None, 1e-5,
            g1.data_ptr(), nxt.data_ptr(), 2, st())), bytes_=R * W * (8 + 2 + 2 + 4 * top))
        rec(f"residual_add_prenorm/{tag}", timed(lambda: lib.pa_residual_add_prenorm(
            x.data_ptr(), R, W, hb.data_ptr(), 0.8, hb.data_ptr(), 1.1, None, None, 0, None, None, 1e-5, g1.data_ptr(),
            nxt.data_ptr(), 2, st())), bytes_=R * W * (8 + 2 + 2 + 2))
        del states, kv
        torch.cuda.empty_cache()
    out["_denominators"] = dict(hbm_gbs=hbm, bf16_tflops=tfl, source=how)
    return out


def run(sizes=None, kernels=True):
    assert torch.cuda.is_available(), "needs a GPU"
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    res = {"workload": dict(prefill=f"{PREFILL_SEQS} x {PREFILL_LEN} tokens in one step",
                            decode=f"{DECODE_SEQS} sequences at {DECODE_CTX} tokens, one token each per step",
                            layers="window attention+moe, [state space+moe, parallel(chunk attention | linear attention)+moe] as a "
                                   "looped block of one pass, window attention+moe", vocab=VOCAB,
                            data="synthetic tokens, random-init weights"), "sizes": {}}
    for name in sizes or SIZES:
        s = SIZES[name]
        res["sizes"][name] = dict(shape=s, dubarax_bf16=bench_model(s, "bfloat16", dev), dubarax_f32=bench_model(s, "float32", dev),
                                  megusun_bf16=hy.bench_hybrid(hy.SIZES[name], "bfloat16", dev))
    if kernels:
        res["kernels_w2048_bf16"] = bench_kernels(SIZES["w2048"], dev)
    return res


if __name__ == "__main__":
    if len(sys.argv) == 3 and sys.argv[1] == "--kernels":     # the kernels alone at one size (a small case for a profiler)
        torch.cuda.set_device(0)
        print(json.dumps({"kernels_" + sys.argv[2]: bench_kernels(SIZES[sys.argv[2]], torch.device("cuda", 0))}, default=float))
    else:
        print(json.dumps(run(), default=float))
