#!/usr/bin/env python
"""Throughput of the `Gunulorn` design (llm_decoder.hybrid: two-norm parallel wiring; causal attention on convolved
projections with a temperature and a sink per head; windowed attention that keeps the first positions, with rotated
queries / keys and turned values; PolyNorm dense layers; routed experts with a choice correction and identity outputs) at
layer sizes that resemble a real model, next to the framework's closest existing model -- the same config-driven stack
serving `Dubarax` (windowed / chunked softmax attention through the same attention kernels, routed experts) -- at equal
width, layer count, vocabulary, batch and context; random weights, synthetic tokens.  `python bench.py --gunulorn` prints
its JSON line.

Per size: prefill tokens/s (PREFILL_SEQS prompts of PREFILL_LEN tokens in one step) and decode tokens/s (DECODE_SEQS
sequences at DECODE_CTX tokens of context, one token each per step), CUDA events around back-to-back steps after
warm-up.  `kernels` times the design's own kernels alone at the largest size, each next to the like kernel of the other
design, against their roofline (algorithmic bytes over the measured copy bandwidth, FLOPs over the measured bf16 GEMM
rate; MEASURED_PEAKS.json)."""
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

from benchmarks import dubarax as du  # noqa: E402
from benchmarks import hybrid as hy  # noqa: E402

PREFILL_SEQS, PREFILL_LEN = hy.PREFILL_SEQS, hy.PREFILL_LEN
DECODE_SEQS, DECODE_CTX = hy.DECODE_SEQS, hy.DECODE_CTX
VOCAB = hy.VOCAB
SIZES = {
    "w1024": dict(width=1024, heads=8, kv_heads=2, dim=64, vdim=128, window=1024, keep=8, rot_dims=32, conv=4, ff=4096,
                  experts=8, identity=2, top=2, eff=512),
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=64, vdim=128, window=1024, keep=8, rot_dims=32, conv=4, ff=8192,
                  experts=8, identity=2, top=2, eff=1024),
}
timed, peaks = hy.timed, hy.peaks


def gunulorn_config(s):
    moe = {"kind": "moe", "expert": {"ff": s["eff"]}, "router": {"experts": s["experts"], "identity": s["identity"], "top": s["top"]}}
    soft = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"], "scale": s["dim"] ** -0.5}
    conv = lambda mlp, src=None: {"type": "attention", "mlp": mlp,  # noqa: E731
                                  "mixer": dict(soft, conv=s["conv"], **({} if src is None else {"kv_from": src}))}
    win = {"type": "attention_2", "mlp": moe,
           "mixer": dict(soft, mask={"size": s["window"], "keep_first": s["keep"]}, rot={"dims": s["rot_dims"], "base": 500000.0})}
    return {"architecture": "Gunulorn", "norm": {"eps": 1e-5}, "vocab": VOCAB, "width": s["width"], "logit_scale": 0.5,
            "logit_softcap": 30.0, "layers": [conv({"kind": "dense", "ff": s["ff"]}), win, conv(moe, 0), win]}


def gunulorn_weights(config, dev):
    g = torch.Generator(device=dev).manual_seed(0)
    Wd = config["width"]
    mat = lambda o, i: (torch.randn(o, i, device=dev, generator=g) / math.sqrt(i)).to(torch.bfloat16)  # noqa: E731
    vec = lambda n, std=0.02, mean=0.0: (torch.randn(n, device=dev, generator=g) * std + mean).to(torch.bfloat16)  # noqa: E731
    W = {"embed": torch.randn(config["vocab"], Wd, device=dev, generator=g).to(torch.bfloat16), "head": mat(config["vocab"], Wd),
         "final.norm": vec(Wd, 0.02, 1.0)}
    for i, lc in enumerate(config["layers"]):
        p, c = f"l{i}.", lc["mixer"]
        W[p + "norm1"], W[p + "norm2"] = vec(Wd, 0.02, 1.0), vec(Wd, 0.02, 1.0)
        H, G, D, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
        names = (("q", H * D),) + ((("k", G * D), ("v", G * V)) if "kv_from" not in c else ())
        for n, rows in names:
            W[p + "mix." + n] = mat(rows, Wd)
            if lc["type"] == "attention":
                W[p + "mix." + n + ".conv"] = (torch.randn(rows, c["conv"], device=dev, generator=g) * 0.5).to(torch.bfloat16)
        W[p + "mix.o"] = mat(Wd, H * V)
        if lc["type"] == "attention":
            W[p + "mix.temp"], W[p + "mix.sink"] = vec(H, 0.1, 1.0), vec(H, 1.0, 0.0)
        ml = lc["mlp"]
        if ml["kind"] == "dense":
            W[p + "mlp.up"], W[p + "mlp.up.b"] = mat(ml["ff"], Wd), vec(ml["ff"])
            W[p + "mlp.down"], W[p + "mlp.down.b"] = mat(Wd, ml["ff"]), vec(Wd)
            W[p + "mlp.act"] = torch.tensor([0.9, 0.4, 0.2, 0.05], device=dev).to(torch.bfloat16)
        else:
            f, E, I = ml["expert"]["ff"], ml["router"]["experts"], ml["router"]["identity"]
            for e in range(E):
                W[f"{p}mlp.e{e}.gate"], W[f"{p}mlp.e{e}.up"], W[f"{p}mlp.e{e}.down"] = mat(f, Wd), mat(f, Wd), mat(Wd, f)
            W[p + "mlp.router"], W[p + "mlp.correction"] = mat(E + I, Wd), vec(E + I)
    return W


def bench_model(s, dtype, dev):
    import llm_decoder as ld
    config = gunulorn_config(s)
    cap = DECODE_SEQS * (DECODE_CTX + 64)
    model = ld.HybridDecoder(config, gunulorn_weights(config, dev), dtype, max_tokens=cap, max_seqs=DECODE_SEQS, tile_size=16)
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
    """The design's own kernels alone (bfloat16 activations) at the prefill and decode shapes of size `s`, each followed by
    the like kernel of the `Dubarax` design on the same operands (names ending in `~`)."""
    from llm_decoder import _cabi
    from llm_decoder.hybrid import MMA_FROM
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
        out[name] = e

    for tag, nseq, plen, ctx0 in (("prefill", PREFILL_SEQS, PREFILL_LEN, 0), ("decode", DECODE_SEQS, 1, DECODE_CTX)):
        R = nseq * plen
        states = SequenceStateCache(nseq, nseq * (ctx0 + plen + 16), 16, dev)
        kv = states.add_kv_layer(G, D, V, "bf16")
        cols = H * D + G * D + G * V
        conv_state = states.add_state((s["conv"] - 1) * cols)
        slots = [states.alloc() for _ in range(nseq)]
        if ctx0:
            for sl in slots:
                states.extend(sl, ctx0)
        b = states.make_batch([(sl, [1] * plen) for sl in slots])
        pt = kv.page_table_
        table = pt.device_data()
        kv.key_buffer_.normal_()
        kv.value_buffer_.normal_()
        qkv = torch.randn(R, cols, device=dev).to(bf)
        o = torch.empty(R, H * V, device=dev, dtype=bf)
        tt, mt = lib.pa_masked_attention_tile_tokens(H, G), lib.pa_masked_attention_mma_tile_tokens(D, V, 2)
        temp, sink, zero = torch.rand(H, device=dev) + 0.5, torch.randn(H, device=dev), torch.zeros(H, device=dev)
        rope, vrot = torch.empty(R, s["rot_dims"] // 2, 2, device=dev), torch.empty(R, V // 2, 2, device=dev)
        assert lib.pa_rope_table(b.row_pos.data_ptr(), R, s["rot_dims"], 500000.0, rope.data_ptr(), st()) == 0
        assert lib.pa_rope_table(b.row_pos.data_ptr(), R, V, 500000.0, vrot.data_ptr(), st()) == 0
        # ---- attention: causal + temperature + sink; window + kept prefix + one in the denominator + output turned back; and
        # the other design's forms through the same kernels (causal plain; window + bucket table + soft cap)
        size, keep = s["window"], s["keep"]
        bucket = torch.randn(size, H, device=dev)
        forms = (("causal_temp_sink", 0, 0, 0, temp, sink, None, 0.0, 0, None), ("causal_plain~", 0, 0, 0, None, None, None, 0.0, 0, None),
                 ("window_keep_turned", 1, size, keep, None, zero, vrot, 0.0, 0, None),
                 ("window_bucket_cap~", 1, size, 0, None, None, None, 30.0, 2, bucket))
        for name, mask_kind, msize, mkeep, hs, sk, orot, cap, bias_kind, bias in forms:
            for kind, group in b.query_tiles(tt, mt, MMA_FROM).items():
                if group is None:
                    continue
                tiles, ntiles, _longest = group
                fn = lambda: lib.pa_masked_attention_sink(  # noqa: E731
                    qkv.data_ptr(), qkv.stride(0), 0, kv.key_buffer_.data_ptr(), kv.value_buffer_.data_ptr(), table.data_ptr(),
                    pt.num_beams_, pt.num_heads_, pt.num_tiles_, kv.total_pages_, kv.tile_size_, tiles.data_ptr(), ntiles, H, D, V,
                    D ** -0.5, cap, mask_kind, msize, mkeep, bias_kind, _cabi.ptr(bias), int(bias.shape[0]) if bias is not None else 0,
                    _cabi.ptr(hs), _cabi.ptr(sk), _cabi.ptr(orot), o.data_ptr(), 2, kind, st())
                assert fn() == 0
                if plen > 1:     # visible (query, key) pairs
                    pairs = sum(min(i + 1, msize) + max(0, min(mkeep, i + 1 - msize)) if mask_kind else i + 1 for i in range(plen))
                    rec(f"attention_{name}/{tag}", timed(fn, 2, 4), flops=nseq * H * pairs * (2 * D + 2 * V))
                else:
                    seen = min(ctx0 + 1, msize) + max(0, min(mkeep, ctx0 + 1 - msize)) if mask_kind else ctx0 + 1
                    rec(f"attention_{name}/{tag}", timed(fn), bytes_=nseq * seen * G * (D + V) * 2)
        # ---- convolution of q | k | v (no activation) and the other design's (silu, bias); rotation fused with the append
        chunks, nch, _a, _b = b.chunk_items(64)
        y = torch.empty(R, cols, device=dev, dtype=bf)
        cw, cb = torch.randn(cols, s["conv"], device=dev), torch.zeros(cols, device=dev)
        rec(f"causal_conv/{tag}", timed(lambda: lib.pa_causal_conv(qkv.data_ptr(), cols, 0, cols, s["conv"], cw.data_ptr(), None, 0,
                                                                   conv_state.data_ptr(), chunks.data_ptr(), nch, y.data_ptr(), cols, 2,
                                                                   st())), bytes_=R * cols * 4)
        rec(f"causal_conv_silu~/{tag}", timed(lambda: lib.pa_causal_conv_silu(qkv.data_ptr(), cols, 0, cols, s["conv"], cw.data_ptr(),
                                                                              cb.data_ptr(), conv_state.data_ptr(), chunks.data_ptr(), nch,
                                                                              y.data_ptr(), cols, 2, st())), bytes_=R * cols * 4)
        rec(f"rope_kv_append/{tag}", timed(lambda: lib.pa_rope_kv_append(
            qkv.data_ptr(), cols, 0, H * D, H * D + G * D, H, G, D, V, s["rot_dims"], rope.data_ptr(), vrot.data_ptr(),
            kv.key_buffer_.data_ptr(), kv.value_buffer_.data_ptr(), table.data_ptr(), pt.num_beams_, pt.num_tiles_, kv.total_pages_,
            kv.tile_size_, b.row_slot.data_ptr(), b.row_pos.data_ptr(), R, 2, st())),
            bytes_=R * (2 * H * s["rot_dims"] * 2 + 2 * G * (D + V) * 2 + (s["rot_dims"] + V) * 4))
        rec(f"kv_append_rows~/{tag}", timed(lambda: kv.append_rows(qkv, H * D, H * D + G * D, b.row_slot, b.row_pos)),
            bytes_=R * 2 * G * (D + V) * 2)
        # ---- router with correction, the two-norm residual step, PolyNorm; and the other design's router and residual step
        E, I, top = s["experts"], s["identity"], s["top"]
        pairs = R * top
        hb = torch.randn(R, W, device=dev).to(bf)
        wr, corr = torch.randn(E + I, W, device=dev) / math.sqrt(W), torch.randn(E + I, device=dev) * 0.02
        sel_id, sel_w = torch.empty(pairs, device=dev, dtype=i32), torch.empty(pairs, device=dev)
        rec(f"router_topk_biased/{tag}", timed(lambda: lib.pa_router_topk_biased(hb.data_ptr(), wr.data_ptr(), None, None, R, W, E + I,
                                                                                 top, 1, 1, 1, 1, corr.data_ptr(), sel_id.data_ptr(),
                                                                                 sel_w.data_ptr(), None, 2, st())), bytes_=R * W * 2)
        rec(f"router_topk_grouped~/{tag}", timed(lambda: lib.pa_router_topk_grouped(hb.data_ptr(), wr.data_ptr(), None, None, R, W, E, top,
                                                                                    1, 0, 4, 2, sel_id.data_ptr(), sel_w.data_ptr(), None,
                                                                                    2, st())), bytes_=R * W * 2)
        assert lib.pa_router_topk_biased(hb.data_ptr(), wr.data_ptr(), None, None, R, W, E + I, top, 1, 1, 1, 1, corr.data_ptr(),
                                         sel_id.data_ptr(), sel_w.data_ptr(), None, 2, st()) == 0
        x, g1 = torch.randn(R, W, device=dev), torch.ones(W, device=dev)
        n1, n2 = torch.empty(R, W, device=dev, dtype=bf), torch.empty(R, W, device=dev, dtype=bf)
        routed = torch.randn(pairs, W, device=dev)
        rec(f"residual_add_norm2_routed/{tag}", timed(lambda: lib.pa_residual_add_norm2(
            x.data_ptr(), R, W, hb.data_ptr(), None, routed.data_ptr(), sel_w.data_ptr(), sel_id.data_ptr(), top, E, hb.data_ptr(), 1e-5,
            g1.data_ptr(), n1.data_ptr(), g1.data_ptr(), n2.data_ptr(), 2, st())), bytes_=R * W * (8 + 2 + 2 + 2 + 4 * top))
        rec(f"residual_add_prenorm_routed~/{tag}", timed(lambda: lib.pa_residual_add_prenorm(
            x.data_ptr(), R, W, None, 1.0, None, 1.0, routed.data_ptr(), sel_w.data_ptr(), top, hb.data_ptr(), None, 1e-5,
            g1.data_ptr(), n1.data_ptr(), 2, st())), bytes_=R * W * (8 + 2 + 2 + 4 * top))
        ff = s["ff"]
        z, za, coef = torch.randn(R, ff, device=dev).to(bf), torch.empty(R, ff, device=dev, dtype=bf), torch.rand(4, device=dev)
        rec(f"poly_norm/{tag}", timed(lambda: lib.pa_poly_norm(z.data_ptr(), R, ff, coef.data_ptr(), 1e-5, za.data_ptr(), 2, st())),
            bytes_=R * ff * 4)
        rec(f"gelu_inplace~/{tag}", timed(lambda: lib.pa_gelu_inplace(z.data_ptr(), z.numel(), 2, st())), bytes_=R * ff * 4)
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
                            layers="convolved causal attention+dense, windowed attention+moe, convolved causal attention on layer 0's "
                                   "pool+moe, windowed attention+moe", vocab=VOCAB, data="synthetic tokens, random-init weights"),
           "sizes": {}}
    for name in sizes or SIZES:
        s = SIZES[name]
        res["sizes"][name] = dict(shape=s, gunulorn_bf16=bench_model(s, "bfloat16", dev), gunulorn_f32=bench_model(s, "float32", dev),
                                  dubarax_bf16=du.bench_model(du.SIZES[name], "bfloat16", dev))
    if kernels:
        res["kernels_w2048_bf16"] = bench_kernels(SIZES["w2048"], dev)
    return res


if __name__ == "__main__":
    if len(sys.argv) == 3 and sys.argv[1] == "--kernels":     # the kernels alone at one size (a small case for a profiler)
        torch.cuda.set_device(0)
        print(json.dumps({"kernels_" + sys.argv[2]: bench_kernels(SIZES[sys.argv[2]], torch.device("cuda", 0))}, default=float))
    else:
        print(json.dumps(run(), default=float))
