"""The `Gunulorn` design in the config-driven stack (llm_decoder.hybrid: two-norm parallel wiring, MaskedAttention with
convolved projections / a temperature per head / a sink / a window that keeps the first positions / rotated queries and
keys / turned values, PolyNorm dense layer, router with a choice correction and identity experts;
csrc/masked_attention.cu, recurrence_ops.cu, seq_ops.cu, moe_ops.cu) against the plain float64 oracle
(oracle/gunulorn_ref.py), on small random models of its own making.

The engine's logits at a position must equal the oracle's full recomputation whatever the cut into steps, the batch
around it, and the pages / slots in use."""
import json
import math
import os
import random
import subprocess

import pytest
import torch

from oracle import gunulorn_ref as R

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F32_TOL = 5e-4      # max abs error of float32 logits (magnitude of a few units)
BF16_TOL = 0.08     # relative rms error of bfloat16 logits


def _model(config, weights, dtype="float32", max_tokens=1024, max_seqs=4, tile_size=16):
    import llm_decoder as ld
    return ld.HybridDecoder(config, weights, dtype, max_tokens=max_tokens, max_seqs=max_seqs, tile_size=tile_size)


def _tokens(n, vocab, seed):
    rnd = random.Random(seed)
    return [rnd.randrange(vocab) for _ in range(n)]


_ORACLE = {}


def _oracle(key, config, weights, tokens):
    k = (key, tuple(tokens))
    if k not in _ORACLE:
        _ORACLE[k] = R.forward(config, weights, tokens)
    return _ORACLE[k]


def _close(got, want, dtype="float32", tol=F32_TOL, bf16_tol=BF16_TOL):
    got, want = got.double().cpu(), want.double()
    if dtype == "float32":
        err = (got - want).abs().max().item()
        assert err < tol * max(1.0, want.abs().max().item() / 4), f"max abs error {err}"
    else:
        # per position; a router decision that bfloat16 rounding flips moves a position by much more than rounding does, so
        # the bound is on the median position (float32 carries the exact comparison)
        got, want = got.reshape(-1, got.shape[-1]), want.reshape(-1, want.shape[-1])
        assert torch.isfinite(got).all()
        rel = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt()
        q = rel.median().item()
        assert q < bf16_tol, f"relative rms error {q} (median of the positions)"


def _feed(engine, rid, tokens, cuts):
    """Feed `tokens` of one request in portions ending at `cuts`; returns logits of ALL positions."""
    outs, lo = [], 0
    for hi in list(cuts) + [len(tokens)]:
        if hi > lo:
            outs.append(engine.step([(rid, tokens[lo:hi], list(range(hi - lo)))]))
            lo = hi
    return torch.cat(outs, 0)


# ---- configurations: sizes and constants unlike each other -- one, two and three key/value heads, key and value sizes that
# differ and are no multiples of 8 or 32, windows that are no multiples of a page or a key step, no kept position, one and
# many, one tap and many, rotation over a part and over all of a head, top = 1 and top = all outputs, no identity output and
# several, a layer without feed-forward -----------------------------------------------------------------------------------
def cfg_conv():
    return R.make_config([R.conv_layer(heads=4, kv_heads=2, dim=16, vdim=24, conv=3)], width=64)


def cfg_borrow():
    return R.make_config([R.conv_layer(heads=3, kv_heads=1, dim=12, vdim=20, conv=2),
                          R.window_layer(heads=2, kv_heads=2, dim=8, vdim=8, size=11, keep=0, rot_dims=8),
                          R.conv_layer(heads=3, kv_heads=1, dim=12, vdim=20, conv=5, kv_from=0, scale=0.4)], width=48)


def cfg_window():
    return R.make_config([R.window_layer(heads=4, kv_heads=2, dim=16, vdim=24, size=21, keep=3, rot_dims=6, base=500.0)], width=64)


def cfg_dense():
    return R.make_config([R.conv_layer(heads=2, kv_heads=2, dim=8, vdim=8, conv=1, mlp=R.dense_mlp(52))], width=40)


def cfg_moe():
    return R.make_config([R.window_layer(heads=2, kv_heads=1, dim=8, vdim=8, size=9, keep=1, rot_dims=4,
                                         mlp=R.moe_mlp(experts=7, identity=3, top=3, ff=24))], width=40)


def cfg_full():
    layers = [R.conv_layer(heads=6, kv_heads=3, dim=24, vdim=16, conv=4, mlp=R.dense_mlp(80)),
              R.window_layer(heads=6, kv_heads=2, dim=16, vdim=40, size=37, keep=5, rot_dims=12, base=10000.0,
                             mlp=R.moe_mlp(experts=8, identity=2, top=2, ff=16)),
              R.conv_layer(heads=6, kv_heads=3, dim=24, vdim=16, conv=2, kv_from=0, mlp=R.moe_mlp(experts=5, identity=0, top=1, ff=24)),
              R.window_layer(heads=2, kv_heads=2, dim=40, vdim=8, size=64, keep=1, rot_dims=40, base=300.0, mlp=None),
              R.conv_layer(heads=2, kv_heads=1, dim=8, vdim=40, conv=6, mlp=R.moe_mlp(experts=3, identity=1, top=4, ff=8))]
    return R.make_config(layers, width=72, vocab=97, eps=1e-5, logit_scale=0.7, logit_softcap=9.0)


def cfg_wide():
    """40 query heads on one key/value head (two head chunks of a CTA's rows), value rows of 130, a window shorter than its
    kept prefix."""
    layers = [R.conv_layer(heads=40, kv_heads=1, dim=4, vdim=6, conv=3),
              R.window_layer(heads=2, kv_heads=2, dim=8, vdim=130, size=33, keep=2, rot_dims=2),
              R.window_layer(heads=9, kv_heads=1, dim=16, vdim=32, size=6, keep=19, rot_dims=16)]
    return R.make_config(layers, width=50, vocab=61, logit_scale=1.0, logit_softcap=50.0)


CONFIGS = {"conv": cfg_conv, "borrow": cfg_borrow, "window": cfg_window, "dense": cfg_dense, "moe": cfg_moe, "full": cfg_full,
           "wide": cfg_wide}


def _case(name, seed=0):
    config = CONFIGS[name]()
    return config, R.random_weights(config, seed)


# ------------------------------------------------------------------------------------------------------------ CPU tests
def test_oracle_attention_loop_equals_matrix_form():
    config, W = _case("full")
    toks = _tokens(41, config["vocab"], 1)
    try:
        R.FORM = "loop"
        a = R.forward(config, W, toks)
    finally:
        R.FORM = "matrix"
    assert (a - R.forward(config, W, toks)).abs().max() < 1e-9


def test_oracle_prefix_property():
    config, W = _case("full")
    toks = _tokens(50, config["vocab"], 2)
    full = R.forward(config, W, toks)
    assert (R.forward(config, W, toks[:17]) - full[:17]).abs().max() < 1e-9


def test_oracle_small_functions():
    assert [j for j in range(12) if R.sees_window_keep(9, j, 4, 0)] == [6, 7, 8, 9]
    assert [j for j in range(12) if R.sees_window_keep(9, j, 4, 2)] == [0, 1, 6, 7, 8, 9]
    assert [j for j in range(12) if R.sees_window_keep(3, j, 4, 2)] == [0, 1, 2, 3]
    assert [j for j in range(12) if R.sees_window_keep(1, j, 1, 5)] == [0, 1]
    x = torch.arange(1.0, 9.0, dtype=torch.float64)
    y = R.turn_pairs(x, 5, 6, 100.0)
    assert torch.equal(y[6:], x[6:]) and abs(float(y[:2].norm() - x[:2].norm())) < 1e-12
    assert (R.turn_pairs(y, 5, 6, 100.0, sign=-1.0) - x).abs().max() < 1e-12
    assert abs(float(y[0]) - (1 * math.cos(5.0) - 2 * math.sin(5.0))) < 1e-12      # pair 0 turns by the position itself
    assert abs(float(y[3]) - (4 * math.cos(5 * 100 ** (-1 / 3)) + 3 * math.sin(5 * 100 ** (-1 / 3)))) < 1e-12
    u = torch.tensor([[1.0, 0.0], [2.0, 1.0], [3.0, 1.0]], dtype=torch.float64)
    w = torch.tensor([[0.5, 2.0], [1.0, 1.0]], dtype=torch.float64)
    assert torch.equal(R.short_conv(u, w), torch.tensor([[2.0, 0.0], [4.5, 1.0], [7.0, 2.0]], dtype=torch.float64))
    z = torch.tensor([[1.0, -2.0, 3.0]], dtype=torch.float64)
    p = R.poly_norm(z, torch.tensor([2.0, 0.0, 0.0, 0.5]), 0.0)
    assert (p - (2.0 * z / math.sqrt(14 / 3) + 0.5)).abs().max() < 1e-12
    p = R.poly_norm(z, torch.tensor([0.0, 1.0, 1.0, 0.0]), 0.0)
    assert (p - (z ** 2 / math.sqrt(98 / 3) + z ** 3 / math.sqrt((1 + 64 + 729) / 3))).abs().max() < 1e-12


def test_oracle_router_correction_and_identity():
    W = {"r.router": torch.eye(4, dtype=torch.float64) * 2.0, "r.correction": torch.tensor([0.0, 0.0, 0.5, 0.0], dtype=torch.float64)}
    h = torch.tensor([[1.0, 0.8, 0.1, 0.0]], dtype=torch.float64)
    s = torch.softmax(h[0] * 2.0, 0)
    chosen = R.route(h, W, "r.", 2)[0]
    assert [e for e, _w in chosen] == [2, 0]                # the correction lifts output 2 over 0 and 1 ...
    assert abs(chosen[0][1] - float(s[2] / (s[2] + s[0]))) < 1e-12     # ... but the weights are the plain scores
    W["e0.gate"] = W["e0.up"] = W["e0.down"] = torch.zeros(4, 4, dtype=torch.float64)
    W["e1.gate"] = W["e1.up"] = W["e1.down"] = torch.zeros(4, 4, dtype=torch.float64)
    W["router"], W["correction"] = W.pop("r.router"), W.pop("r.correction")
    out = R.moe_ff(h, W, "", dict(router=dict(experts=2, identity=2, top=2)))
    assert (out - chosen[0][1] * h).abs().max() < 1e-12     # output 2 is an identity expert, expert 0 returns zero here


def test_registry_names_the_design():
    from llm_decoder.hybrid import DESIGNS, FEED_FORWARDS
    from llm_decoder.registry import MODEL_REGISTRY
    assert "Gunulorn" in MODEL_REGISTRY and DESIGNS["Gunulorn"]["wiring"] == "parallel_two_norms"
    assert set(DESIGNS["Gunulorn"]["mixers"]) == {"attention", "attention_2"}
    assert set(DESIGNS["Gunulorn"]["ff"]) <= set(FEED_FORWARDS)


# ------------------------------------------------------------------------------------------------------------ GPU tests
@pytest.mark.gpu
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_each_mechanism(name, dtype):
    import llm_decoder as ld
    config, W = _case(name)
    toks = _tokens(85, config["vocab"], 3)
    eng = ld.Engine(_model(config, W, dtype))
    _close(_feed(eng, "a", toks, []), _oracle(name, config, W, toks), dtype)


@pytest.mark.gpu
def test_residual_after_every_layer():
    import llm_decoder as ld
    config, W = _case("full")
    toks = _tokens(45, config["vocab"], 6)
    model = _model(config, W)
    seen = []
    model.layer_hook = lambda x: seen.append(x.double().cpu())
    ld.Engine(model).step([("a", toks, [])])
    want = []
    R.forward(config, W, toks, want)
    assert len(seen) == len(want) == 5
    for i, x in enumerate(seen):
        assert (x - want[i]).abs().max() < 3e-4, f"layer {i}"


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["sink", "temp", "correction", "conv_k", "value_turn", "keep"])
def test_every_constant_shows_in_the_logits(name):
    """Changing one tensor or constant of the model moves the oracle's logits AND the engine follows: none of them is
    left out on the way."""
    import llm_decoder as ld
    config, W = _case("full", seed=3)
    toks = _tokens(60, config["vocab"], 16)
    base = R.forward(config, W, toks)
    W2, config2 = dict(W), json.loads(json.dumps(config))
    if name == "sink":
        W2["l0.mix.sink"] = (W["l0.mix.sink"].float() + 2.0).to(torch.bfloat16)
    elif name == "temp":
        W2["l4.mix.temp"] = (W["l4.mix.temp"].float() * 1.7).to(torch.bfloat16)
    elif name == "correction":
        W2["l1.mlp.correction"] = (W["l1.mlp.correction"].float() + torch.tensor([0.0] * 8 + [0.4, 0.4])).to(torch.bfloat16)
    elif name == "conv_k":
        W2["l0.mix.k.conv"] = W["l0.mix.k.conv"].flip(1).contiguous()
    elif name == "value_turn":
        config2["layers"][1]["mixer"]["rot"]["base"] = 50.0
    else:
        config2["layers"][1]["mixer"]["mask"]["keep_first"] = 0
    want = R.forward(config2, W2, toks)
    assert (want - base).abs().max() > 0.02
    _close(_feed(ld.Engine(_model(config2, W2)), "a", toks, [33]), want)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["full", "conv", "borrow", "window", "wide"])
def test_prefill_equals_token_by_token(name):
    import llm_decoder as ld
    config, W = _case(name)
    toks = _tokens(70, config["vocab"], 4)
    eng = ld.Engine(_model(config, W))
    _close(_feed(eng, "a", toks, range(1, 70)), _oracle(name, config, W, toks))      # every token a step of its own


@pytest.mark.gpu
@pytest.mark.parametrize("cuts", [[2, 4, 6, 9, 40], [15, 16, 17, 31, 33, 48, 64, 66], [1, 80], [63], [4, 5, 6, 41, 42, 43, 78],
                                  [36, 37, 38, 74, 75]])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_many_sizes(cuts, dtype):
    """Cuts at, before and after page borders (16 tokens), key steps (32, 64), the kept prefix (5) and window lengths (37),
    down to two tokens and fewer than the convolutions' taps."""
    import llm_decoder as ld
    config, W = _case("full")
    toks = _tokens(90, config["vocab"], 5)
    eng = ld.Engine(_model(config, W, dtype))
    _close(_feed(eng, "a", toks, cuts), _oracle("full", config, W, toks), dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_of_unequal_requests(dtype):
    """Four requests of unequal length advance together: portions next to single tokens, one sitting out a step."""
    import llm_decoder as ld
    config, W = _case("full")
    reqs = {r: _tokens(n, config["vocab"], 10 + i) for i, (r, n) in enumerate([("a", 70), ("b", 33), ("c", 5), ("d", 51)])}
    plan = [[("a", 40), ("b", 2)], [("a", 1), ("b", 17), ("c", 5)], [("a", 1), ("d", 30)], [("a", 1), ("b", 1), ("d", 1)],
            [("b", 13), ("d", 20), ("a", 27)]]
    eng = ld.Engine(_model(config, W, dtype))
    at = {r: 0 for r in reqs}
    got = {r: [] for r in reqs}
    for step in plan:
        entries = []
        for r, n in step:
            entries.append((r, reqs[r][at[r]:at[r] + n], list(range(n))))
            at[r] += n
        out = eng.step(entries)
        o = 0
        for r, n in step:
            got[r].append(out[o:o + n])
            o += n
    for r in reqs:
        assert at[r] == len(reqs[r])
        _close(torch.cat(got[r], 0), _oracle("full", config, W, reqs[r]), dtype)


@pytest.mark.gpu
def test_slots_and_pages_are_used_again():
    """A pool of 160 tokens and two slots serves six requests one after another and interleaved: freed pages and slots
    come back (dirty) and the next request must not see the keys or convolution inputs they held."""
    import llm_decoder as ld
    config, W = _case("full")
    model = _model(config, W, max_tokens=160, max_seqs=2)
    assert len(model.states._kv) == 4                       # layer 2 reads layer 0's pool
    eng = ld.Engine(model)
    seqs = [_tokens(n, config["vocab"], 20 + i) for i, n in enumerate([90, 60, 33, 100, 17, 59])]
    out = eng.step([("r0", seqs[0][:50], list(range(50))), ("r1", seqs[1][:10], list(range(10)))])
    g0, g1 = [out[:50]], [out[50:]]
    out = eng.step([("r1", seqs[1][10:], list(range(50))), ("r0", seqs[0][50:], list(range(40)))])
    g1.append(out[:50])
    g0.append(out[50:])
    _close(torch.cat(g0), _oracle("full", config, W, seqs[0]))
    _close(torch.cat(g1), _oracle("full", config, W, seqs[1]))
    assert model.states.free_slots() == 0 and model.states.free_tokens() == 0
    with pytest.raises(RuntimeError):
        eng.step([("r2", [1], [0])])                 # no slot left
    eng.finish("r0")
    eng.finish("r1")
    assert model.states.free_slots() == 2 and model.states.free_tokens() == 160
    for i in (2, 3, 4, 5):
        _close(_feed(eng, f"r{i}", seqs[i], [len(seqs[i]) // 2]), _oracle("full", config, W, seqs[i]))
        eng.finish(f"r{i}")


@pytest.mark.gpu
@pytest.mark.parametrize("tile_size", [16, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_edges_and_far_keys_sharp_attention(tile_size, dtype):
    """300 tokens, peaked attention (queries and keys scaled up): causal attention over everything, a window of 70 that
    keeps 6 positions, and a layer that borrows the first one's pool; prompts cut around page borders, the kept prefix and
    the window, then 40 decoded tokens that slide the window over decoded tokens."""
    import llm_decoder as ld
    config = R.make_config([R.conv_layer(heads=4, kv_heads=2, dim=16, vdim=32, conv=3),
                            R.window_layer(heads=4, kv_heads=1, dim=16, vdim=16, size=70, keep=6, rot_dims=8),
                            R.conv_layer(heads=4, kv_heads=2, dim=16, vdim=32, conv=2, kv_from=0)], width=64, vocab=80)
    W = R.random_weights(config, 7, sharp=4.0)
    toks = _tokens(300, config["vocab"], 8)
    want = R.forward(config, W, toks)
    eng = ld.Engine(_model(config, W, dtype, tile_size=tile_size))
    cuts = [5, 6, 7, 69, 70, 71, 75, 76, 77, 127, 129, 135, 192, 255, 256] + list(range(260, 300))
    _close(_feed(eng, "a", toks, cuts), want, dtype)
    eng.finish("a")
    eng = ld.Engine(_model(config, W, dtype, tile_size=tile_size))
    _close(_feed(eng, "b", toks, [5, 290]), want, dtype)


def _needle_model(kind, size=0, keep=0):
    """One attention layer of one head whose key map got a rank-one term: the needle token's key lands on the probe
    token's query, so the needle takes almost all the weight of the probe -- where the probe sees it.  'window': the
    rank-one term lives in the dimensions the rotation leaves alone; 'causal': the convolutions of q and k pass their
    input through (one tap of 1), that of v mixes as drawn, and the sink stays well below the needle's score."""
    if kind == "window":
        config = R.make_config([R.window_layer(heads=1, kv_heads=1, dim=12, vdim=16, size=size, keep=keep, rot_dims=4, scale=1.0)],
                               width=32, vocab=40)
    else:
        config = R.make_config([R.conv_layer(heads=1, kv_heads=1, dim=12, vdim=16, conv=3, scale=1.0)], width=32, vocab=40)
    p = "l0.mix."
    W = R.random_weights(config, 9)
    needle, probe = 7, 11
    D = {k: v.double() for k, v in W.items()}
    if kind == "causal":
        for n in ("q", "k"):
            W[p + n + ".conv"] = torch.tensor([[0.0, 0.0, 1.0]]).repeat(12, 1).to(torch.bfloat16)
        W[p + "temp"] = torch.ones(1, dtype=torch.bfloat16)
        W[p + "sink"] = torch.full((1,), 3.0, dtype=torch.bfloat16)
    h = R.rms(D["embed"][[needle, probe]], 1e-6) * D["l0.norm1"]
    q = D[p + "q"] @ h[1]
    if kind == "window":
        q[:4] = 0.0
    W[p + "k"] = (D[p + "k"] * 0.1 + 16.0 * torch.outer(q / (q @ q), h[0] / (h[0] @ h[0]))).to(torch.bfloat16)
    return config, W, needle, probe


@pytest.mark.gpu
@pytest.mark.parametrize("size,keep", [(48, 0), (17, 3), (33, 16), (5, 1)])
def test_single_key_at_the_window_edge_and_the_kept_prefix(size, keep):
    """The needle sits at the last position the probe still sees or at the first it does not -- at the window's far edge,
    and at the end of the kept prefix; the probe comes at the end of a prompt portion, or decoded alone.  The test first
    proves that the placements give different logits."""
    import llm_decoder as ld
    config, W, needle, probe = _needle_model("window", size, keep)
    others = [t for t in range(40) if t not in (needle, probe)]
    rnd = random.Random(3)
    n = 3 * size + 5 + keep                                # the probe's position
    pairs = [(n - size + 1, n - size)] + ([(keep - 1, keep)] if keep else [])
    for inside, outside in pairs:
        results = {}
        for where in (inside, outside):
            toks = [rnd.choice(others) for _ in range(n)] + [probe]
            toks[where] = needle
            want = R.forward(config, W, toks)
            results[where] = want[-1]
            for cuts in ([n], [n - 7], [where, where + 1, n - 1, n]):
                eng = ld.Engine(_model(config, W))
                got = _feed(eng, "a", toks, cuts)
                _close(got[-1], want[-1])
                _close(got[:-1], want[:-1])
        assert (results[inside] - results[outside]).abs().max() > 0.3


@pytest.mark.gpu
@pytest.mark.parametrize("where", [0, 15, 16, 17, 31, 32, 140])
def test_single_far_key_among_hundreds(where):
    """Causal attention over 400 tokens: one key, far back, takes the probe's weight; without it the logits differ."""
    import llm_decoder as ld
    config, W, needle, probe = _needle_model("causal")
    others = [t for t in range(40) if t not in (needle, probe)]
    rnd = random.Random(where)
    toks = [rnd.choice(others) for _ in range(400)] + [probe]
    without = R.forward(config, W, toks)[-1]
    toks[where] = needle
    want = R.forward(config, W, toks)
    assert (want[-1] - without).abs().max() > 0.3
    for cuts in ([400], [390], [where + 1, 399, 400]):
        got = _feed(ld.Engine(_model(config, W)), "a", toks, cuts)
        _close(got[-1], want[-1])
        _close(got[:-1], want[:-1])


@pytest.mark.gpu
def test_first_tokens():
    import llm_decoder as ld
    config, W = _case("full")
    for n in (1, 2, 3):
        toks = _tokens(n, config["vocab"], 30 + n)
        eng = ld.Engine(_model(config, W))
        _close(_feed(eng, "a", toks, []), _oracle("full", config, W, toks))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_portion_and_long_decoding(dtype):
    """A 560-token portion followed by 150 decoded tokens; the same request again cut at 300."""
    import llm_decoder as ld
    config, W = _case("full")
    toks = _tokens(710, config["vocab"], 40)
    want = _oracle("full", config, W, toks)
    eng = ld.Engine(_model(config, W, dtype))
    _close(_feed(eng, "a", toks, [560] + list(range(561, 710))), want, dtype, tol=1.5e-3)
    eng.finish("a")
    _close(_feed(eng, "b", toks, [300, 301, 700]), want, dtype, tol=1.5e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(dtype):
    """Scheduler: five prompts of unequal length on four slots with a small token budget (chunked prompts, continuous
    batching, slot reuse); greedy tokens equal the oracle's argmax at every step (float32), and the teacher-forced
    logits stay close (bfloat16)."""
    import llm_decoder as ld
    config, W = _case("full")
    prompts = [_tokens(n, config["vocab"], 50 + i) for i, n in enumerate([37, 5, 64, 18, 2])]
    model = _model(config, W, dtype, max_tokens=512, max_seqs=4)
    outs = ld.generate(model, prompts, 12, max_batch_tokens=48)
    for p, o in zip(prompts, outs):
        assert o[:len(p)] == p and len(o) == len(p) + 12
        logits = R.forward(config, W, o[:-1])
        if dtype == "float32":
            for t in range(len(p) - 1, len(o) - 1):
                top2 = logits[t].topk(2).values
                if float(top2[0] - top2[1]) > 1e-3:                 # no test on a near tie
                    assert int(logits[t].argmax()) == o[t + 1]
        else:
            chosen = torch.tensor([logits[t, o[t + 1]] for t in range(len(p) - 1, len(o) - 1)])
            best = logits[len(p) - 1:len(o) - 1].max(-1).values
            assert float((best - chosen).median()) < 0.1 and float((best - chosen).max()) < 1.5


def _random_config(rnd):
    """Layer count and order, which layers borrow whose pool, every size and constant drawn at random."""
    def mlp():
        x = rnd.random()
        if x < 0.2:
            return None
        if x < 0.45:
            return R.dense_mlp(rnd.choice([8, 30, 64, 100]))
        experts, identity = rnd.randint(1, 9), rnd.randint(0, 3)
        return R.moe_mlp(experts=experts, identity=identity, top=rnd.randint(1, experts + identity), ff=rnd.choice([8, 16, 24, 30]))
    layers, owners = [], []
    for i in range(rnd.randint(2, 6)):
        kv = rnd.choice([1, 2, 3])
        if rnd.random() < 0.5:
            if owners and rnd.random() < 0.4:
                j = rnd.choice(owners)
                m = layers[j]["mixer"]
                layers.append(R.conv_layer(heads=m["kv_heads"] * rnd.randint(1, 4), kv_heads=m["kv_heads"], dim=m["dim"],
                                           vdim=m["vdim"], conv=rnd.randint(1, 6), scale=rnd.uniform(0.1, 0.4), kv_from=j, mlp=mlp()))
            else:
                owners.append(i)
                layers.append(R.conv_layer(heads=kv * rnd.randint(1, 4), kv_heads=kv, dim=rnd.choice([8, 12, 16, 24, 20]),
                                           vdim=rnd.choice([8, 16, 40, 20, 6]), conv=rnd.randint(1, 6), scale=rnd.uniform(0.1, 0.4),
                                           mlp=mlp()))
        else:
            dim = rnd.choice([8, 12, 16, 24, 20])
            layers.append(R.window_layer(heads=kv * rnd.randint(1, 4), kv_heads=kv, dim=dim, vdim=rnd.choice([8, 16, 40, 20, 6]),
                                         size=rnd.randint(1, 90), keep=rnd.choice([0, 0, 1, 2, 7, 20]),
                                         rot_dims=rnd.randrange(2, dim + 1, 2), base=rnd.choice([50.0, 10000.0, 500000.0]),
                                         scale=rnd.uniform(0.1, 0.4), mlp=mlp()))
    return R.make_config(layers, width=rnd.choice([40, 64, 72, 96, 50, 128]), vocab=rnd.choice([61, 97, 128]),
                         eps=rnd.choice([1e-5, 1e-6]), logit_scale=rnd.uniform(0.2, 1.5), logit_softcap=rnd.choice([5.0, 30.0]))


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(8))
def test_random_configurations_in_random_schedules(seed):
    """Three requests of a randomly drawn model advance in random portions (1 to 100 tokens, some sitting out) through
    one engine; float32 against the oracle at every position, bfloat16 at the median position."""
    import llm_decoder as ld
    rnd = random.Random(seed)
    config = _random_config(rnd)
    W = R.random_weights(config, seed)
    reqs = {r: _tokens(n, config["vocab"], 100 * seed + i)
            for i, (r, n) in enumerate((("a", rnd.randint(120, 300)), ("b", rnd.randint(2, 90)), ("c", rnd.randint(1, 40))))}
    plan, at = [], {r: 0 for r in reqs}
    while any(at[r] < len(reqs[r]) for r in reqs):
        step = []
        for r in reqs:
            left = len(reqs[r]) - at[r]
            if left and rnd.random() < 0.8:
                n = min(left, rnd.choice([1, 1, 2, 3, 17, 64, 100]))
                step.append((r, at[r], n))
                at[r] += n
        if step:
            plan.append(step)
    outs = {}
    for dtype in ("float32", "bfloat16"):
        eng = ld.Engine(_model(config, W, dtype, max_tokens=640, max_seqs=3))
        got = {r: [] for r in reqs}
        for step in plan:
            out = eng.step([(r, reqs[r][lo:lo + n], list(range(n))) for r, lo, n in step])
            o = 0
            for r, _lo, n in step:
                got[r].append(out[o:o + n])
                o += n
        outs[dtype] = {r: torch.cat(got[r], 0) for r in reqs}
    for r in reqs:
        want = R.forward(config, W, reqs[r])
        _close(outs["float32"][r], want, tol=1e-3)
        _close(outs["bfloat16"][r], want, "bfloat16", bf16_tol=0.2)


# ---- kernels alone -----------------------------------------------------------------------------------------------------
def _turn_back_rows(o, first, vdim, base):
    """R.turn_pairs(., position, vdim, base, sign=-1) for the rows of o at positions first, first + 1, ... at once."""
    m = torch.arange(vdim // 2, dtype=torch.float64)
    a = torch.arange(first, first + o.shape[0], dtype=torch.float64)[:, None] * base ** (-2.0 * m / vdim)
    u, v = o[:, 0::2], o[:, 1::2]
    out = torch.empty_like(o)
    out[:, 0::2] = u * torch.cos(a) + v * torch.sin(a)
    out[:, 1::2] = v * torch.cos(a) - u * torch.sin(a)
    return out


def test_turn_back_rows_equals_the_oracle():
    o = torch.randn(5, 10, dtype=torch.float64, generator=torch.Generator().manual_seed(0))
    want = torch.stack([R.turn_pairs(o[t], 30 + t, 10, 700.0, sign=-1.0) for t in range(5)])
    assert (_turn_back_rows(o, 30, 10, 700.0) - want).abs().max() < 1e-12


@pytest.mark.gpu
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 16, 24), (6, 1, 96, 96), (8, 2, 64, 128), (3, 3, 40, 8), (2, 1, 128, 64),
                                                     (5, 1, 24, 32), (2, 2, 8, 70)])
@pytest.mark.parametrize("mask,size,keep,sink,temp,turn", [("window", 37, 4, "zero", False, True), ("window", 200, 0, "zero", False, True),
                                                           ("causal", 0, 0, "learned", True, False), ("window", 5, 70, None, True, True),
                                                           ("window", 9, 33, "learned", False, False)])
def test_attention_kernels_alone(heads, kv_heads, dim, vdim, mask, size, keep, sink, temp, turn):
    """The float tile kernel, the streaming single-token kernel and the tensor-core kernel over the same paged pool
    (pages handed out in a scattered order) against attention written out in float64, with a sink, a temperature per head,
    kept first positions and the output turned back: a 150-token portion that starts at position 70 of its sequence, a first
    token, a two-token portion at positions 63 and 64, and a single token at position 219 of three others."""
    from llm_decoder import _cabi
    from llm_decoder.hybrid import MASK_KIND
    from llm_decoder.seq_state import SequenceStateCache
    lib, dev = _cabi.lib(), torch.device("cuda")
    g = torch.Generator().manual_seed(heads * 7 + dim)
    per = heads // kv_heads
    scale, base = dim ** -0.5 * 2.0, 700.0
    ctx = [70, 0, 63, 219]                                  # tokens already cached per sequence
    new = [150, 1, 2, 1]                                    # tokens of this step
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 2e-2)):
        states = SequenceStateCache(4, 1024, 16, dev)
        kv = states.add_kv_layer(kv_heads, dim, vdim, "f32" if dtype == torch.float32 else "bf16")
        slots = [states.alloc() for _ in range(4)]
        for rnd_ in range(14):                              # interleave the sequences' growth so that their pages interleave
            for i in [2, 0, 3, 1]:
                n = min(16, ctx[i] - rnd_ * 16)
                if n > 0:
                    states.extend(slots[i], n)
        K = [torch.randn(ctx[i] + new[i], kv_heads * dim, generator=g).to(dtype) for i in range(4)]
        V = [torch.randn(ctx[i] + new[i], kv_heads * vdim, generator=g).to(dtype) for i in range(4)]
        Q = [torch.randn(new[i], heads * dim, generator=g).to(dtype) for i in range(4)]
        temps = (torch.rand(heads, generator=g) + 0.5) if temp else None
        sinks = torch.randn(heads, generator=g) * 2 if sink == "learned" else torch.zeros(heads) if sink == "zero" else None
        pt = kv.page_table_
        for i in range(4):
            if ctx[i]:
                rows = torch.cat([K[i][:ctx[i]], V[i][:ctx[i]]], 1).to(dev)
                kv.append_rows(rows, 0, kv_heads * dim, torch.full((ctx[i],), slots[i], dtype=torch.int32, device=dev),
                               torch.arange(ctx[i], dtype=torch.int32, device=dev))
        batch = states.make_batch([(slots[i], [0] * new[i]) for i in range(4)])
        proj = torch.cat([torch.cat([Q[i], K[i][ctx[i]:], V[i][ctx[i]:]], 1) for i in range(4)], 0).to(dev)
        kv.append_rows(proj, heads * dim, heads * dim + kv_heads * dim, batch.row_slot, batch.row_pos)
        rot = None
        if turn:
            rot = torch.empty(sum(new), vdim // 2, 2, dtype=torch.float32, device=dev)
            assert lib.pa_rope_table(batch.row_pos.data_ptr(), sum(new), vdim, base, rot.data_ptr(), _cabi.stream()) == 0
        want = []
        for i in range(4):
            q, k, v = Q[i].double(), K[i].double(), V[i].double()
            out = torch.zeros(new[i], heads * vdim, dtype=torch.float64)
            pos = torch.arange(ctx[i], ctx[i] + new[i])[:, None]
            j = torch.arange(ctx[i] + new[i])[None, :]
            vis = pos - j >= 0
            if mask == "window":
                vis &= (pos - j < size) | (j < keep)
            for h in range(heads):
                gi = h // per
                sc = q[:, h * dim:(h + 1) * dim] @ k[:, gi * dim:(gi + 1) * dim].T * scale * (float(temps[h]) if temp else 1.0)
                sc = sc.masked_fill(~vis, -float("inf"))
                if sinks is not None:
                    sc = torch.cat([sc, torch.full((new[i], 1), float(sinks[h]), dtype=torch.float64)], 1)
                o = torch.softmax(sc, -1)[:, :ctx[i] + new[i]] @ v[:, gi * vdim:(gi + 1) * vdim]
                if turn:
                    o = _turn_back_rows(o, ctx[i], vdim, base)
                out[:, h * vdim:(h + 1) * vdim] = o
            want.append(out)
        want = torch.cat(want, 0)
        tt = lib.pa_masked_attention_tile_tokens(heads, kv_heads)
        mt = lib.pa_masked_attention_mma_tile_tokens(dim, vdim, proj.element_size())
        table_dev = pt.device_data()
        td, sd = (temps.to(dev) if temp else None), (sinks.to(dev) if sinks is not None else None)
        for use_mma, use_stream in ((0, 0), (mt, 1)):
            out = torch.zeros(sum(new), heads * vdim, dtype=dtype, device=dev)
            for kind, group in batch.query_tiles(tt, use_mma, 16).items():
                if group is None:
                    continue
                tiles, ntiles, _longest = group
                rc = lib.pa_masked_attention_sink(proj.data_ptr(), proj.stride(0), 0, kv.key_buffer_.data_ptr(),
                                                  kv.value_buffer_.data_ptr(), table_dev.data_ptr(), pt.num_beams_, pt.num_heads_,
                                                  pt.num_tiles_, kv.total_pages_, kv.tile_size_, tiles.data_ptr(), ntiles, heads, dim,
                                                  vdim, scale, 0.0, MASK_KIND[mask], size, keep if mask == "window" else 0, 0, None, 0,
                                                  _cabi.ptr(td), _cabi.ptr(sd), _cabi.ptr(rot), out.data_ptr(), proj.element_size(),
                                                  kind if (use_stream or kind != 1) else 0, _cabi.stream())
                assert rc == 0, (kind, rc)
            err = (out.double().cpu() - want).abs().max().item()
            assert err < tol * max(1.0, want.abs().max().item()), (dtype, use_mma, err)


@pytest.mark.gpu
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rot_dims", [(4, 2, 16, 24, 6), (3, 1, 7, 10, 4), (2, 2, 64, 64, 64), (5, 5, 8, 6, 0)])
def test_rotation_fused_with_the_append(heads, kv_heads, dim, vdim, rot_dims):
    """pa_rope_kv_append against the rotation written out: queries in place, keys and values as they land in the pool
    (read back through the page table), rows of three sequences at positions around a page border; and a layer without a
    pool, whose keys and values must stay untouched."""
    from llm_decoder import _cabi
    from llm_decoder.seq_state import SequenceStateCache
    lib, dev, base = _cabi.lib(), torch.device("cuda"), 300.0
    g = torch.Generator().manual_seed(dim)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
        states = SequenceStateCache(3, 256, 16, dev)
        kv = states.add_kv_layer(kv_heads, dim, vdim, "f32" if dtype == torch.float32 else "bf16")
        slots = [states.alloc() for _ in range(3)]
        ctx, new = [14, 0, 37], [5, 1, 20]
        for s, n in zip(slots, ctx):
            if n:
                states.extend(s, n)
        batch = states.make_batch([(s, [0] * n) for s, n in zip(slots, new)])
        cols = heads * dim + kv_heads * (dim + vdim)
        src = torch.randn(sum(new), cols + 3, generator=g).to(dtype)
        rows, pos = sum(new), torch.cat([torch.arange(c, c + n) for c, n in zip(ctx, new)])
        tabs = {}
        for dims in {rot_dims, vdim}:
            if dims:
                t = torch.empty(rows, dims // 2, 2, dtype=torch.float32, device=dev)
                assert lib.pa_rope_table(batch.row_pos.data_ptr(), rows, dims, base, t.data_ptr(), _cabi.stream()) == 0
                tabs[dims] = t
        pt = kv.page_table_
        for own in (True, False):
            x = src.to(dev).clone()
            kv.key_buffer_.zero_()
            kv.value_buffer_.zero_()
            rc = lib.pa_rope_kv_append(x.data_ptr(), x.stride(0), 2, 2 + heads * dim, 2 + heads * dim + kv_heads * dim, heads, kv_heads,
                                       dim, vdim, rot_dims, _cabi.ptr(tabs.get(rot_dims)), tabs[vdim].data_ptr(),
                                       kv.key_buffer_.data_ptr() if own else None, kv.value_buffer_.data_ptr() if own else None,
                                       pt.device_data().data_ptr(), pt.num_beams_, pt.num_tiles_, kv.total_pages_, kv.tile_size_,
                                       batch.row_slot.data_ptr(), batch.row_pos.data_ptr(), rows, src.element_size(), _cabi.stream())
            assert rc == 0
            got = x.double().cpu()
            assert torch.equal(got[:, :2], src[:, :2].double()) and torch.equal(got[:, 2 + heads * dim:], src[:, 2 + heads * dim:].double())
            table = pt.device_data().cpu().reshape(pt.num_beams_, kv_heads, pt.num_tiles_)
            kb = kv.key_buffer_.double().cpu().reshape(-1, kv.tile_size_, dim)
            vb = kv.value_buffer_.double().cpu().reshape(-1, kv.tile_size_, vdim)
            r = 0
            for s, c0, n in zip(slots, ctx, new):
                for t in range(c0, c0 + n):
                    row = src[r].double()
                    for h in range(heads):
                        a = 2 + h * dim
                        assert (got[r, a:a + dim] - R.turn_pairs(row[a:a + dim], t, rot_dims, base)).abs().max() < tol * 4
                    for gi in range(kv_heads):
                        page = int(table[s, gi, t // 16])
                        a = 2 + heads * dim + gi * dim
                        b = 2 + heads * dim + kv_heads * dim + gi * vdim
                        if own:
                            assert (kb[page, t % 16] - R.turn_pairs(row[a:a + dim], t, rot_dims, base)).abs().max() < tol * 4
                            assert (vb[page, t % 16] - R.turn_pairs(row[b:b + vdim], t, vdim, base)).abs().max() < tol * 4
                    r += 1
            if not own:
                assert float(kv.key_buffer_.abs().max()) == 0.0 and float(kv.value_buffer_.abs().max()) == 0.0


@pytest.mark.gpu
def test_router_with_correction_kernel_alone():
    from llm_decoder import _cabi
    lib, dev = _cabi.lib(), torch.device("cuda")
    g = torch.Generator().manual_seed(5)
    for outputs, top, width in ((12, 4, 64), (5, 1, 40), (10, 10, 33), (18, 3, 24)):
        h = torch.randn(50, width, generator=g)
        W = {"router": torch.randn(outputs, width, generator=g).double() * 0.3, "correction": torch.randn(outputs, generator=g).double() * 0.2}
        sel_id = torch.empty(50 * top, dtype=torch.int32, device=dev)
        sel_w = torch.empty(50 * top, dtype=torch.float32, device=dev)
        hd, wd, cd = h.to(dev), W["router"].float().to(dev), W["correction"].float().to(dev)
        assert lib.pa_router_topk_biased(hd.data_ptr(), wd.data_ptr(), None, None, 50, width, outputs, top, 1, 1, 1, 1, cd.data_ptr(),
                                         sel_id.data_ptr(), sel_w.data_ptr(), None, 4, _cabi.stream()) == 0
        ids, ws = sel_id.cpu().reshape(50, top), sel_w.cpu().reshape(50, top)
        want = R.route(h.double(), W, "", top)
        for r in range(50):
            assert ids[r].tolist() == [e for e, _w in want[r]]
            assert (ws[r].double() - torch.tensor([w for _e, w in want[r]])).abs().max() < 1e-6


@pytest.mark.gpu
def test_small_kernels_alone():
    """PolyNorm rows, the two-norm residual step with identity experts, capped logits, the convolution without
    activation."""
    from llm_decoder import _cabi
    from llm_decoder.seq_state import SequenceStateCache
    lib, dev, s = _cabi.lib(), torch.device("cuda"), _cabi.stream()
    g = torch.Generator().manual_seed(11)
    for ff in (7, 64, 300, 1100):
        z, coef = torch.randn(9, ff, generator=g) * 2, torch.randn(4, generator=g)
        want = R.poly_norm(z.double(), coef.double(), 1e-5)
        for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 2e-2)):
            zd, out = z.to(dtype).to(dev), torch.empty(9, ff, dtype=dtype, device=dev)
            assert lib.pa_poly_norm(zd.data_ptr(), 9, ff, coef.to(dev).data_ptr(), 1e-5, out.data_ptr(), zd.element_size(), s) == 0
            ref = R.poly_norm(zd.double().cpu(), coef.double(), 1e-5)
            assert (out.double().cpu() - ref).abs().max() < tol * max(1.0, float(want.abs().max()))
    for width, top, experts in ((40, 3, 4), (72, 1, 2), (130, 2, 0)):
        rows = 6
        x, y, y2 = torch.randn(rows, width, generator=g), torch.randn(rows, width, generator=g), torch.randn(rows, width, generator=g)
        routed, sel_w = torch.randn(rows * top, width, generator=g), torch.rand(rows * top, generator=g)
        sel_id = torch.randint(0, experts + 2, (rows * top,), generator=g, dtype=torch.int32)
        ident, g1, g2 = torch.randn(rows, width, generator=g), torch.randn(width, generator=g), torch.randn(width, generator=g)
        e = torch.where((sel_id >= experts)[:, None], ident.double().repeat_interleave(top, 0), routed.double())
        xn = x.double() + y.double() + y2.double() + (sel_w.double()[:, None] * e).reshape(rows, top, width).sum(1)
        xd, n1, n2 = x.to(dev), torch.empty(rows, width, device=dev), torch.empty(rows, width, device=dev)
        assert lib.pa_residual_add_norm2(xd.data_ptr(), rows, width, y.to(dev).data_ptr(), y2.to(dev).data_ptr(), routed.to(dev).data_ptr(),
                                         sel_w.to(dev).data_ptr(), sel_id.to(dev).data_ptr(), top, experts, ident.to(dev).data_ptr(), 1e-6,
                                         g1.to(dev).data_ptr(), n1.data_ptr(), g2.to(dev).data_ptr(), n2.data_ptr(), 4, s) == 0
        assert (xd.double().cpu() - xn).abs().max() < 1e-5
        assert (n1.double().cpu() - R.rms(xn, 1e-6) * g1.double()).abs().max() < 1e-5
        assert (n2.double().cpu() - R.rms(xn, 1e-6) * g2.double()).abs().max() < 1e-5
    z = torch.randn(5, 33, generator=g) * 40
    zd = z.to(dev)
    assert lib.pa_logit_softcap(zd.data_ptr(), z.numel(), 0.3, 7.0, s) == 0
    assert (zd.double().cpu() - 7.0 * torch.tanh(z.double() * 0.3 / 7.0)).abs().max() < 1e-5
    for taps in (1, 2, 5):
        C, lens, slots = 21, [1, 2, taps, 70], [3, 1, 0, 2]
        w, x = torch.randn(C, taps, generator=g), torch.randn(sum(lens), C + 4, generator=g)
        states = SequenceStateCache(4, 256, 16, dev)
        st = states.add_state(max(1, (taps - 1) * C))
        for _ in slots:
            states.alloc()
        carried = torch.randn(4, max(1, (taps - 1) * C), generator=g)
        st.copy_(carried)
        batch = states.make_batch([(sl, [0] * n) for sl, n in zip(slots, lens)])
        chunks, n, _s0, _sn = batch.chunk_items(64)
        xd, out = x.to(dev), torch.empty(sum(lens), C, device=dev)
        assert lib.pa_causal_conv(xd.data_ptr(), C + 4, 2, C, taps, w.to(dev).data_ptr(), None, 0, st.data_ptr(), chunks.data_ptr(), n,
                                  out.data_ptr(), C, 4, s) == 0
        r0 = 0
        for sl, m in zip(slots, lens):
            hist = carried[sl].double().reshape(taps - 1, C) if taps > 1 else torch.zeros(0, C, dtype=torch.float64)
            full = torch.cat([hist, x[r0:r0 + m, 2:2 + C].double()], 0)
            want = R.short_conv(full, w.double())[taps - 1:]
            assert (out[r0:r0 + m].double().cpu() - want).abs().max() < 1e-5
            r0 += m


@pytest.mark.gpu
def test_configuration_errors():
    config, W = _case("borrow")
    bad = json.loads(json.dumps(config))
    bad["layers"][2]["mixer"]["kv_from"] = 1                # a layer of another kind
    with pytest.raises(ValueError):
        _model(bad, W)
    bad = json.loads(json.dumps(config))
    bad["layers"][2]["mixer"]["vdim"] = 8                   # sizes unlike the owner's
    with pytest.raises(ValueError):
        _model(bad, W)
    config, W = _case("moe")
    bad = json.loads(json.dumps(config))
    bad["layers"][0]["mlp"]["router"]["identity"] = 1       # the router has other rows
    with pytest.raises(ValueError):
        _model(bad, W)
    config, W = _case("conv")
    bad = json.loads(json.dumps(config))
    bad["layers"][0]["mixer"]["conv"] += 1                  # taps unlike the tensors'
    with pytest.raises(ValueError):
        _model(bad, W)
    bare = json.loads(json.dumps(config))
    del bare["layers"][0]["mixer"]["conv"]                  # the tensors' shape alone gives the taps
    toks = _tokens(20, config["vocab"], 5)
    _close(ld_step(_model(bare, W), toks), _oracle("conv0", config, W, toks))


def ld_step(model, tokens):
    import llm_decoder as ld
    return ld.Engine(model).step([("a", tokens, list(range(len(tokens))))])


# ---- the command-line programs -------------------------------------------------------------------------------------------
@pytest.mark.gpu
def test_trace_runner_and_generate_programs(tmp_path):
    from llm_decoder.safetensors_io import save_file
    config, W = _case("full")
    mdir = tmp_path / "model"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(config))
    save_file(W, str(mdir / "model.safetensors"))
    a, b = _tokens(40, config["vocab"], 60), _tokens(9, config["vocab"], 61)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}, {"id": "b", "tokens": b[:2], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": b[2:], "want": [6]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[30:], "want": [9]}], "end": ["a"]}]
    out = tmp_path / "out"
    p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", str(mdir), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True,
                       text=True, timeout=600)
    assert p.returncode == 0, p.stderr
    assert [ln for ln in p.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    import numpy as np
    wa, wb = R.forward(config, W, a), R.forward(config, W, b)
    _close(torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)), wa[[0, 29]])
    _close(torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1)), wb[[8]])
    _close(torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(1, -1)), wa[[39]])
    p = subprocess.run([os.path.join(ROOT, "bin", "generate"), "--model", str(mdir), "--dtype", "float32", "--prompt",
                        ",".join(map(str, a[:12])), "--max-new-tokens", "5"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr
    toks = [int(t) for t in p.stdout.strip().splitlines()[-1].split(",")]
    assert toks[:12] == a[:12] and len(toks) == 17
    logits = R.forward(config, W, toks[:-1])
    for t in range(11, 16):
        top2 = logits[t].topk(2).values
        if float(top2[0] - top2[1]) > 1e-3:
            assert int(logits[t].argmax()) == toks[t + 1]
