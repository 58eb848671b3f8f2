"""The `Dubarax` design in the config-driven stack (llm_decoder.hybrid: pre-norm wiring, looped blocks, MaskedAttention,
DecayLinearAttention, Mamba2Mixer, group-limited router; csrc/masked_attention.cu, recurrence_ops.cu, seq_ops.cu,
moe_ops.cu) against the plain float64 oracle (oracle/dubarax_ref.py), on small random models of its own making.

The engine's logits at a position must equal the oracle's full recomputation whatever the cut into steps, the batch
around it, and the pages / slots in use."""
import json
import os
import random
import subprocess

import pytest
import torch

from oracle import dubarax_ref as R

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
        _ORACLE[k] = R.forward(config, weights, tokens)[0]
    return _ORACLE[k]


def _close(got, want, dtype="float32", tol=F32_TOL, bf16_tol=BF16_TOL):
    got, want = got.double().cpu(), want.double()
    if dtype == "float32":
        err = (got - want).abs().max().item()
        assert err < tol * max(1.0, want.abs().max().item() / 4), f"max abs error {err}"
    else:
        # per position; a router decision that bfloat16 rounding flips moves a position by much more than rounding does,
        # and every later layer run (up to eleven here) carries the difference on, so the bound is on the median position
        # (float32 carries the exact comparison)
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


# ---- configurations: sizes and constants unlike each other -- several key/value heads, key and value sizes that differ
# and are no multiples of 8 or 32, windows and chunks that are no multiples of a page or a key step, one and many taps,
# one norm group, top = 1 and top = experts, all groups kept, no shared expert, a layer without feed-forward -------------
def cfg_window():
    return R.make_config([R.attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, window=21, buckets=10, bias_max=30)], width=64)


def cfg_parallel():
    return R.make_config([R.parallel_layer(heads=3, kv_heads=3, dim=12, vdim=20, chunk=19, lin_heads=3, lin_dim=10, lin_vdim=36,
                                           decay=(0.5, 0.9, 0.995))], width=48)


def cfg_mamba():
    return R.make_config([R.mamba_layer(heads=6, vdim=12, state=24, groups=3, conv=3, norm_groups=4)], width=40)


def cfg_moe():
    return R.make_config([R.attention_layer(heads=2, kv_heads=1, dim=8, vdim=8, window=9, buckets=6, bias_max=20,
                                            mlp=R.moe_mlp(12, 3, 24, count=4, keep=2, shared_ff=40))], width=40)


def cfg_full():
    """Five layers; layers 1 to 3 run three times (a cache and state per pass), layers 0 and 4 once."""
    layers = [R.attention_layer(heads=6, kv_heads=2, dim=24, vdim=16, window=37, buckets=12, bias_max=100, softcap=8.0,
                                mlp=R.moe_mlp(8, 2, 16, count=4, keep=3, shared_ff=24)),
              R.mamba_layer(heads=4, vdim=20, state=12, groups=1, conv=5, norm_groups=1, mlp=R.moe_mlp(5, 5, 24, shared_ff=0)),
              R.parallel_layer(heads=4, kv_heads=2, dim=8, vdim=24, chunk=26, lin_heads=2, lin_dim=40, lin_vdim=24,
                               decay=(0.8, 0.99), mlp=None),
              R.attention_layer(heads=2, kv_heads=2, dim=40, vdim=8, window=64, buckets=5, bias_max=50, softcap=50.0,
                                mlp=R.moe_mlp(9, 1, 16, count=3, keep=1, shared_ff=8)),
              R.mamba_layer(heads=2, vdim=40, state=72, groups=2, conv=1, norm_groups=5, mlp=R.moe_mlp(6, 4, 8, count=2, keep=2))]
    return R.make_config(layers, width=72, vocab=97, eps=1e-5, embed_scale=3.0, loop=(1, 4, 3))


def cfg_loop_tail():
    """The looped block reaches the last layer and runs once; no layer follows it."""
    layers = [R.mamba_layer(heads=2, vdim=8, state=8, groups=2, conv=2, norm_groups=2, mlp=R.moe_mlp(4, 2, 8)),
              R.parallel_layer(heads=2, kv_heads=1, dim=16, vdim=16, chunk=8, lin_heads=1, lin_dim=16, lin_vdim=8, decay=(0.9,),
                               mlp=R.moe_mlp(4, 1, 8, count=2, keep=1))]
    return R.make_config(layers, width=32, vocab=50, loop=(1, 2, 1))


def cfg_wide():
    """32 query heads per key/value head and more (two head chunks of a CTA's rows), value rows of 130, a matrix state
    with 160 rows (two register slices) and 70 columns (two column blocks)."""
    layers = [R.attention_layer(heads=40, kv_heads=1, dim=4, vdim=6, window=50, buckets=8, bias_max=60, mlp=None),
              R.attention_layer(heads=2, kv_heads=2, dim=8, vdim=130, window=33, buckets=8, bias_max=60, mlp=None),
              R.parallel_layer(heads=2, kv_heads=1, dim=8, vdim=8, chunk=30, lin_heads=1, lin_dim=160, lin_vdim=70, decay=(0.97,))]
    return R.make_config(layers, width=50, vocab=61, embed_scale=1.0)


CONFIGS = {"window": cfg_window, "parallel": cfg_parallel, "mamba": cfg_mamba, "moe": cfg_moe, "full": cfg_full,
           "loop_tail": cfg_loop_tail, "wide": cfg_wide}


def _case(name, seed=0):
    config = CONFIGS[name]()
    return config, R.random_weights(config, seed)


# ------------------------------------------------------------------------------------------------------------ CPU tests
def test_oracle_attention_loop_equals_matrix_form():
    config, W = _case("full")
    toks = _tokens(41, config["vocab"], 1)
    try:
        R.FORM = "loop"
        a, la = R.forward(config, W, toks)
    finally:
        R.FORM = "matrix"
    b, lb = R.forward(config, W, toks)
    assert (a - b).abs().max() < 1e-9 and (la - lb).abs().max() < 1e-9
    assert la.shape[0] == 1 + 3 * 3 + 1                    # layer runs: one, three passes of three, one


def test_oracle_prefix_property():
    config, W = _case("full")
    toks = _tokens(50, config["vocab"], 2)
    full = R.forward(config, W, toks)[0]
    assert (R.forward(config, W, toks[:17])[0] - full[:17]).abs().max() < 1e-9


def test_oracle_masks_and_buckets():
    assert [j for j in range(12) if R.sees_window(9, j, 4)] == [6, 7, 8, 9]
    assert [j for j in range(12) if R.sees_chunk(9, j, 4)] == [8, 9]
    assert [j for j in range(12) if R.sees_chunk(8, j, 4)] == [8]
    assert [j for j in range(12) if R.sees_chunk(7, j, 4)] == [4, 5, 6, 7]
    b = [R.distance_bucket(n, 8, 32) for n in range(40)]
    assert b[:4] == [0, 1, 2, 3] and b[4] == 4 and b[7] == 5 and b[8] == 5 and b[31] == 7 and b[39] == 7
    assert all(x <= y for x, y in zip(b, b[1:]))
    assert abs(R.head_slope(3, 4) - 2.0 ** -8) < 1e-12 and abs(R.head_slope(0, 4) - 0.25) < 1e-12


def test_oracle_router_groups():
    s = torch.tensor([0.05, 0.30, 0.02, 0.03, 0.25, 0.20, 0.10, 0.05], dtype=torch.float64)
    assert R.route(s, 3, 1, 1) == [1, 4, 5]
    assert R.route(s, 3, 4, 2) == [1, 4, 5]                 # groups (0,1) (2,3) (4,5) (6,7): best two are 0 and 2
    assert R.route(s, 2, 4, 1) == [1, 0]                    # only group 0 is eligible
    assert R.route(s, 3, 2, 1) == [1, 0, 3]                 # halves: the first one wins with 0.30


def test_oracle_state_space_equals_convolution_free_recurrence():
    """taps = 1 reduces the convolution to a per-channel scale + bias."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(7, 5, generator=g, dtype=torch.float64)
    w, b = torch.randn(5, 1, generator=g, dtype=torch.float64), torch.randn(5, generator=g, dtype=torch.float64)
    assert torch.allclose(R.causal_conv(x, w, b), x * w[:, 0] + b)
    w3 = torch.randn(5, 3, generator=g, dtype=torch.float64)
    y = R.causal_conv(x, w3, b)
    assert torch.allclose(y[0], b + w3[:, 2] * x[0]) and torch.allclose(y[2], b + w3[:, 0] * x[0] + w3[:, 1] * x[1] + w3[:, 2] * x[2])


def test_registry_names_the_design():
    from llm_decoder.hybrid import DESIGNS, FEED_FORWARDS
    from llm_decoder.registry import MODEL_REGISTRY
    assert "Dubarax" in MODEL_REGISTRY and DESIGNS["Dubarax"]["wiring"] == "pre_norm"
    assert set(DESIGNS["Dubarax"]["mixers"]) == {"attention", "parallel", "mamba2"}
    assert set(DESIGNS["Dubarax"]["ff"]) <= set(FEED_FORWARDS)


def test_bucket_table_matches_oracle():
    from llm_decoder.hybrid import log_distance_bucket
    for B, far in ((8, 32), (16, 200), (5, 50), (12, 100), (32, 128), (7, 9)):
        assert [log_distance_bucket(n, B, far) for n in range(300)] == [R.distance_bucket(n, B, far) for n in range(300)]


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
def test_residual_after_every_layer_run():
    import llm_decoder as ld
    config, W = _case("full")
    toks = _tokens(45, config["vocab"], 6)
    model = _model(config, W)
    seen = []
    model.layer_hook = lambda x: seen.append(x.double().cpu())
    ld.Engine(model).step([("a", toks, [])])
    want = R.forward(config, W, toks)[1]
    assert len(seen) == want.shape[0] == 11
    for i, x in enumerate(seen):
        assert (x - want[i]).abs().max() < 3e-4, f"layer run {i}"


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["full", "window", "parallel", "mamba", "loop_tail", "wide"])
def test_prefill_equals_token_by_token(name):
    import llm_decoder as ld
    config, W = _case(name)
    toks = _tokens(70, config["vocab"], 4)
    eng = ld.Engine(_model(config, W))
    _close(_feed(eng, "a", toks, range(1, 70)), _oracle(name, config, W, toks))      # every token a step of its own


@pytest.mark.gpu
@pytest.mark.parametrize("cuts", [[2, 4, 6, 9, 40], [15, 16, 17, 31, 33, 48, 64, 66], [1, 80], [63], [25, 26, 27, 51, 52, 53, 78],
                                  [36, 37, 38, 74, 75]])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_many_sizes(cuts, dtype):
    """Cuts at, before and after page borders (16 tokens), key steps (32, 64), chunk borders (26) and window lengths (37),
    down to two tokens and fewer than the convolution's taps."""
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
    come back (dirty) and the next request must not see the keys, matrix states or convolution inputs they held."""
    import llm_decoder as ld
    config, W = _case("full")
    model = _model(config, W, max_tokens=160, max_seqs=2)
    assert len(model.states._kv) == 1 + 3 * 2               # one pool per attention run: layer 0, and layers 2 and 3 per pass
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


def _sharp(W, factor=4.0):
    """Queries scaled up: the softmax concentrates on its best key, so one wrong, missing or extra key moves the output
    by O(1) instead of O(1/n)."""
    W = dict(W)
    for k in list(W):
        if k.endswith("mix.q") or k.endswith("left.q"):
            W[k] = (W[k].float() * factor).to(torch.bfloat16)
    return W


@pytest.mark.gpu
@pytest.mark.parametrize("tile_size", [16, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_and_chunk_edges_sharp_attention(tile_size, dtype):
    """300 tokens, peaked attention with a window of 70 and chunks of 45: prompts cut around page borders, windows and
    chunk borders, then 40 decoded tokens that cross a chunk border and slide the window over decoded tokens."""
    import llm_decoder as ld
    config = R.make_config([R.attention_layer(heads=4, kv_heads=2, dim=16, vdim=32, window=70, buckets=16, bias_max=90, softcap=40.0),
                            R.parallel_layer(heads=4, kv_heads=1, dim=16, vdim=16, chunk=45, lin_heads=2, lin_dim=8, lin_vdim=8)],
                           width=64, vocab=80)
    W = _sharp(R.random_weights(config, 7))
    toks = _tokens(300, config["vocab"], 8)
    want = R.forward(config, W, toks)[0]
    eng = ld.Engine(_model(config, W, dtype, tile_size=tile_size))
    cuts = [44, 45, 46, 69, 70, 71, 127, 129, 135, 192, 255, 256] + list(range(260, 300))
    _close(_feed(eng, "a", toks, cuts), want, dtype)
    eng.finish("a")
    eng = ld.Engine(_model(config, W, dtype, tile_size=tile_size))
    _close(_feed(eng, "b", toks, [5, 290]), want, dtype)


def _needle_model(kind, size):
    """One attention layer of one head whose key map got a rank-one term: the needle token's key lands on the probe
    token's query, so the needle takes almost all the weight of the probe -- where the probe sees it."""
    if kind == "window":
        config = R.make_config([R.attention_layer(heads=1, kv_heads=1, dim=8, vdim=16, window=size, buckets=8, bias_max=2 * size,
                                                  softcap=30.0, scale=1.0)], width=32, vocab=40, embed_scale=1.5)
        p = "l0.mix."
    else:
        config = R.make_config([R.parallel_layer(heads=1, kv_heads=1, dim=8, vdim=16, chunk=size, scale=1.0, lin_heads=1,
                                                 lin_dim=4, lin_vdim=4, decay=(0.5,), right_scale=0.05)],
                               width=32, vocab=40, embed_scale=1.5)
        p = "l0.mix.left."
    W = R.random_weights(config, 9)
    needle, probe = 7, 11
    D = {k: v.double() for k, v in W.items()}
    h = R.norm1p(D["embed"][[needle, probe]] * 1.5, D["l0.norm1"], 1e-6)
    q = D[p + "q"] @ h[1] + D[p + "q.b"]
    W[p + "k"] = (D[p + "k"] * 0.1 + 16.0 * torch.outer(q / (q @ q), h[0] / (h[0] @ h[0]))).to(torch.bfloat16)
    if kind == "window":
        W[p + "rel"] = (D[p + "rel"] * 0.2).to(torch.bfloat16)
    return config, W, needle, probe


@pytest.mark.gpu
@pytest.mark.parametrize("kind,size", [("window", 48), ("window", 17), ("chunk", 40), ("chunk", 16)])
def test_single_key_just_inside_and_just_outside(kind, size):
    """The needle sits at the last position the probe still sees, or at the first it does not; the probe comes at the end
    of a prompt portion, or decoded alone.  The test first proves that the two placements give different logits."""
    import llm_decoder as ld
    config, W, needle, probe = _needle_model(kind, size)
    others = [t for t in range(40) if t not in (needle, probe)]
    rnd = random.Random(3)
    n = 3 * size + 5                                       # the probe's position
    inside = n - size + 1 if kind == "window" else n // size * size
    outside = inside - 1
    results = {}
    for where in (inside, outside):
        toks = [rnd.choice(others) for _ in range(n)] + [probe]
        toks[where] = needle
        want = R.forward(config, W, toks)[0]
        results[where] = want[-1]
        for cuts in ([n], [n - 7], [where, where + 1, n - 1, n]):
            eng = ld.Engine(_model(config, W))
            got = _feed(eng, "a", toks, cuts)
            _close(got[-1], want[-1])
            _close(got[:-1], want[:-1])
    assert (results[inside] - results[outside]).abs().max() > 0.3


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
    """A 560-token portion (chunked matrix-state scan: fold, chain, replay) followed by 150 decoded tokens; the same
    request again cut at 300 (two chunked portions chained through the state slot)."""
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
def test_long_portion_beside_short_ones(dtype):
    """One step holds a 300-token portion (which switches the matrix-state scan of the WHOLE batch to its chunked form), a
    decoded token of a running request, a 2-token portion and a 70-token portion that continues a request."""
    import llm_decoder as ld
    config, W = _case("full")
    reqs = {r: _tokens(n, config["vocab"], 70 + i) for i, (r, n) in enumerate([("a", 330), ("b", 41), ("c", 2), ("d", 100)])}
    plan = [[("b", 40), ("d", 30)], [("a", 300), ("b", 1), ("c", 2), ("d", 70)], [("a", 30)]]
    eng = ld.Engine(_model(config, W, dtype))
    at, got = {r: 0 for r in reqs}, {r: [] for r in reqs}
    for step in plan:
        out = eng.step([(r, reqs[r][at[r]:at[r] + n], list(range(n))) for r, n in step])
        o = 0
        for r, n in step:
            got[r].append(out[o:o + n])
            at[r] += n
            o += n
    for r in reqs:
        assert at[r] == len(reqs[r])
        _close(torch.cat(got[r], 0), _oracle("full", config, W, reqs[r]), dtype, tol=1.5e-3)


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
        logits = R.forward(config, W, o[:-1])[0]
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
    """Layer count and order, the looped block, every size and constant drawn at random."""
    def mlp():
        if rnd.random() < 0.25:
            return None
        count = rnd.choice([1, 2, 3, 4])
        per = rnd.randint(1, 4)
        keep = rnd.randint(1, count)
        return R.moe_mlp(count * per, rnd.randint(1, keep * per), rnd.choice([8, 16, 24, 30]), count=count, keep=keep,
                         shared_ff=rnd.choice([0, 8, 40]))
    layers = []
    for _ in range(rnd.randint(2, 5)):
        kind = rnd.choice(["attention", "parallel", "mamba2"])
        kv = rnd.choice([1, 2, 3])
        if kind == "attention":
            layers.append(R.attention_layer(heads=kv * rnd.randint(1, 4), kv_heads=kv, dim=rnd.choice([8, 12, 16, 24, 20]),
                                            vdim=rnd.choice([8, 16, 40, 20]), window=rnd.randint(3, 90), buckets=rnd.randint(4, 20),
                                            bias_max=rnd.randint(30, 200), softcap=rnd.uniform(5.0, 50.0),
                                            scale=rnd.uniform(0.1, 0.4), mlp=mlp()))
        elif kind == "parallel":
            lh = rnd.randint(1, 3)
            layers.append(R.parallel_layer(heads=kv * rnd.randint(1, 3), kv_heads=kv, dim=rnd.choice([8, 16, 24, 12]),
                                           vdim=rnd.choice([8, 16, 40, 20]), chunk=rnd.randint(2, 80), scale=rnd.uniform(0.1, 0.4),
                                           lin_heads=lh, lin_dim=rnd.choice([4, 8, 16, 33, 72]), lin_vdim=rnd.choice([8, 16, 40, 66]),
                                           decay=tuple(rnd.uniform(0.3, 0.999) for _ in range(lh)),
                                           left_scale=rnd.uniform(0.5, 1.5), right_scale=rnd.uniform(0.5, 1.5), mlp=mlp()))
        else:
            groups = rnd.choice([1, 2, 3])
            heads, vdim, ng = groups * rnd.randint(1, 3), rnd.choice([8, 12, 16, 24]), rnd.choice([1, 2, 4])
            layers.append(R.mamba_layer(heads=heads, vdim=vdim, state=rnd.choice([4, 8, 16, 24, 40]), groups=groups,
                                        conv=rnd.randint(1, 6), norm_groups=ng, mlp=mlp()))
    loop = None
    if rnd.random() < 0.7:
        a = rnd.randrange(len(layers))
        loop = (a, rnd.randint(a + 1, len(layers)), rnd.randint(1, 3))
    return R.make_config(layers, width=rnd.choice([40, 64, 72, 96, 50, 128]), vocab=rnd.choice([61, 97, 128]),
                         eps=rnd.choice([1e-5, 1e-6]), embed_scale=rnd.uniform(0.5, 3.0), loop=loop)


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(8))
def test_random_configurations_in_random_schedules(seed):
    """Three requests of a randomly drawn model advance in random portions (1 to 100 tokens, some sitting out) through
    one engine; float32 against the oracle at every position, bfloat16 finite and equal to its own whole-prompt run up
    to rounding."""
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
        want = R.forward(config, W, reqs[r])[0]
        # a group norm over values that nearly cancel multiplies float rounding by 1 / sqrt(eps): hundreds of times
        _close(outs["float32"][r], want, tol=4e-3)
        # up to fifteen layer runs with top-1 routers: rounding differences grow from run to run
        _close(outs["bfloat16"][r], want, "bfloat16", bf16_tol=0.25)


# ---- kernels alone -----------------------------------------------------------------------------------------------------
def _scan_case(heads, groups, dim, vdim, lens, selective, act, seed, dtype=torch.float32):
    """Random operands of pa_decay_scan for portions of the given lengths, and the float64 recurrence token by token."""
    g = torch.Generator().manual_seed(seed)
    R_ = sum(lens)
    q = torch.randn(R_, groups * dim, generator=g).to(dtype)
    k = (torch.randn(R_, groups * dim, generator=g) * 0.5).to(dtype)
    v = torch.randn(R_, heads * vdim, generator=g).to(dtype)
    dt = torch.randn(R_, heads, generator=g).to(dtype)
    decay = torch.rand(heads, generator=g) * 0.6 + 0.39
    dt_bias, a_log, skip = torch.randn(heads, generator=g) * 0.5, torch.randn(heads, generator=g) * 0.5, torch.randn(heads, generator=g)
    state0 = torch.randn(len(lens), heads, dim, vdim, generator=g)
    f = (lambda z: z / (1 + torch.exp(-z))) if act else (lambda z: z)
    qd, kd, vd, dtd = f(q.double()), f(k.double()), f(v.double()), dt.double()
    out = torch.zeros(R_, heads * vdim, dtype=torch.float64)
    state = state0.double().clone()
    r0 = 0
    for s, n in enumerate(lens):
        for h in range(heads):
            gi = h // (heads // groups)
            S = state[s, h]
            for t in range(r0, r0 + n):
                if selective:
                    step = R.softplus(dtd[t, h] + dt_bias[h].double())
                    a, scale = torch.exp(-torch.exp(a_log[h].double()) * step), step
                else:
                    a, scale = decay[h].double(), 1.0
                x = vd[t, h * vdim:(h + 1) * vdim]
                S = a * S + torch.outer(kd[t, gi * dim:(gi + 1) * dim], scale * x)
                out[t, h * vdim:(h + 1) * vdim] = qd[t, gi * dim:(gi + 1) * dim] @ S + (skip[h].double() * x if selective else 0)
            state[s, h] = S
        r0 += n
    return dict(q=q, k=k, v=v, dt=dt, decay=decay, dt_bias=dt_bias, a_log=a_log, skip=skip, state0=state0, out=out, state=state)


@pytest.mark.gpu
@pytest.mark.parametrize("heads,groups,dim,vdim", [(2, 2, 16, 8), (4, 2, 24, 40), (1, 1, 150, 70), (3, 1, 64, 64), (2, 1, 5, 3),
                                                    (1, 1, 300, 20)])
@pytest.mark.parametrize("selective", [False, True])
def test_decay_scan_kernel_alone(heads, groups, dim, vdim, selective):
    """Portions of 1, 3, 40 and 300 tokens from random states in slots 2, 0, 3, 1: the walk in order and the chunked
    three-pass form against the float64 recurrence, float and bfloat16 operands."""
    from llm_decoder import _cabi
    from llm_decoder.seq_state import SequenceStateCache
    lib = _cabi.lib()
    lens, slots = [1, 3, 40, 300], [2, 0, 3, 1]
    dev = torch.device("cuda")
    for dtype, tol in ((torch.float32, 2e-3), (torch.bfloat16, 2e-3)):
        c = _scan_case(heads, groups, dim, vdim, lens, selective, act=not selective, seed=heads * 100 + dim, dtype=dtype)
        for chunk in (0, 64):
            states = SequenceStateCache(4, 1024, 16, dev)
            st = states.add_state(heads * dim * vdim)
            for sl in slots:
                assert states.alloc() in range(4)
            batch = states.make_batch([(sl, [0] * n) for sl, n in zip(slots, lens)])
            for i, sl in enumerate(slots):
                st[sl] = c["state0"][i].reshape(-1).to(dev)
            items, n, s0, sn = batch.chunk_items(chunk)
            ws = torch.empty(lib.pa_decay_scan_workspace_bytes(n, heads, dim, vdim) if chunk else 1, dtype=torch.uint8, device=dev)
            out = torch.empty(sum(lens), heads * vdim, dtype=torch.float32, device=dev)
            d = {k_: c[k_].to(dev).contiguous() for k_ in ("q", "k", "v", "dt", "decay", "dt_bias", "a_log", "skip")}
            rc = lib.pa_decay_scan(d["q"].data_ptr(), groups * dim, 0, d["k"].data_ptr(), groups * dim, 0, d["v"].data_ptr(),
                                   heads * vdim, 0, heads, groups, dim, vdim, 0 if selective else 1,
                                   None if selective else d["decay"].data_ptr(), d["dt"].data_ptr() if selective else None, heads, 0,
                                   d["dt_bias"].data_ptr() if selective else None, d["a_log"].data_ptr() if selective else None,
                                   d["skip"].data_ptr() if selective else None, st.data_ptr(), out.data_ptr(), heads * vdim,
                                   items.data_ptr(), n, s0.data_ptr(), sn.data_ptr(), batch.seq_slot.data_ptr(), batch.num_seqs,
                                   1 if chunk else 0, ws.data_ptr(), ws.numel(), d["q"].element_size(), _cabi.stream())
            assert rc == 0
            scale = c["out"].abs().max().item()
            assert (out.double().cpu() - c["out"]).abs().max().item() < tol * max(1.0, scale), (dtype, chunk)
            for i, sl in enumerate(slots):
                got = st[sl].double().cpu().reshape(heads, dim, vdim)
                assert (got - c["state"][i]).abs().max().item() < tol * max(1.0, c["state"][i].abs().max().item())


@pytest.mark.gpu
@pytest.mark.parametrize("taps", [1, 2, 4, 8])
def test_causal_convolution_kernel_alone(taps):
    """Portions shorter than, equal to and longer than taps - 1 from a random carried state; then the state update."""
    from llm_decoder import _cabi
    from llm_decoder.seq_state import SequenceStateCache
    lib, dev, C = _cabi.lib(), torch.device("cuda"), 37
    g = torch.Generator().manual_seed(taps)
    lens, slots = [1, 2, taps, 70, 130], [4, 1, 0, 3, 2]
    w, b = torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    for dtype in (torch.float32, torch.bfloat16):
        x = torch.randn(sum(lens), C + 5, generator=g).to(dtype)
        states = SequenceStateCache(5, 1024, 16, dev)
        st = states.add_state(max(1, (taps - 1) * C))
        for _ in slots:
            states.alloc()
        carried = torch.randn(5, max(1, (taps - 1) * C), generator=g).to(dtype).float()
        st.copy_(carried)
        batch = states.make_batch([(sl, [0] * n) for sl, n in zip(slots, lens)])
        chunks, n, _s0, _sn = batch.chunk_items(64)
        xd, out = x.to(dev), torch.empty(sum(lens), C, dtype=dtype, device=dev)
        wd, bd = w.to(dev), b.to(dev)
        assert lib.pa_causal_conv_silu(xd.data_ptr(), C + 5, 3, C, taps, wd.data_ptr(), bd.data_ptr(), st.data_ptr(),
                                       chunks.data_ptr(), n, out.data_ptr(), C, x.element_size(), _cabi.stream()) == 0
        assert lib.pa_conv_state_update(xd.data_ptr(), C + 5, 3, C, taps, batch.seq_start.data_ptr(), batch.seq_len.data_ptr(),
                                        batch.seq_slot.data_ptr(), batch.num_seqs, st.data_ptr(), x.element_size(),
                                        _cabi.stream()) == 0
        r0 = 0
        for sl, m in zip(slots, lens):
            hist = carried[sl].double().reshape(taps - 1, C) if taps > 1 else torch.zeros(0, C, dtype=torch.float64)
            full = torch.cat([hist, x[r0:r0 + m, 3:3 + C].double()], 0)
            want = torch.stack([(full[t:t + taps].T * w.double()).sum(-1) + b.double() for t in range(m)])
            want = want / (1 + torch.exp(-want))
            tol = 1e-5 if dtype == torch.float32 else 2e-2
            assert (out[r0:r0 + m].double().cpu() - want).abs().max().item() < tol * max(1.0, want.abs().max().item())
            if taps > 1:
                assert torch.equal(st[sl].cpu().reshape(taps - 1, C), full[m:].float())
            r0 += m


@pytest.mark.gpu
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 16, 24), (6, 1, 96, 96), (8, 2, 64, 128), (3, 3, 40, 8), (2, 1, 128, 64)])
@pytest.mark.parametrize("mask,size,bias", [("window", 37, "bucket"), ("window", 200, "bucket"), ("chunk", 50, "slope"), ("chunk", 64, None),
                                            ("causal", 0, "bucket"), ("window", 5, "slope")])
def test_attention_kernels_alone(heads, kv_heads, dim, vdim, mask, size, bias):
    """The float tile kernel, the streaming single-token kernel and the tensor-core kernel over the same paged pool
    (pages handed out in a scattered order) against softmax attention written out in float64: a 150-token portion that
    starts at position 70 of its sequence, a first token, a two-token portion at positions 63 and 64, and a single token at
    position 219 of three others."""
    from llm_decoder import _cabi
    from llm_decoder.hybrid import MASK_KIND, log_distance_bucket
    from llm_decoder.seq_state import SequenceStateCache
    lib, dev = _cabi.lib(), torch.device("cuda")
    g = torch.Generator().manual_seed(heads * 7 + dim)
    per = heads // kv_heads
    scale, cap = dim ** -0.5 * 2.0, 6.0 if bias == "bucket" else 0.0
    ctx = [70, 0, 63, 219]                                  # tokens already cached per sequence
    new = [150, 1, 2, 1]                                    # tokens of this step
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 2e-2)):
        states = SequenceStateCache(4, 1024, 16, dev)
        kv = states.add_kv_layer(kv_heads, dim, vdim, "f32" if dtype == torch.float32 else "bf16")
        slots = [states.alloc() for _ in range(4)]
        order = [2, 0, 3, 1]
        for rnd_ in range(14):                              # interleave the sequences' growth so that their pages interleave
            for i in order:
                n = min(16, ctx[i] - rnd_ * 16)
                if n > 0:
                    states.extend(slots[i], n)
        K = [torch.randn(ctx[i] + new[i], kv_heads * dim, generator=g).to(dtype) for i in range(4)]
        V = [torch.randn(ctx[i] + new[i], kv_heads * vdim, generator=g).to(dtype) for i in range(4)]
        Q = [torch.randn(new[i], heads * dim, generator=g).to(dtype) for i in range(4)]
        # the cached part goes in through the same append call, as earlier steps would have left it
        pt = kv.page_table_
        for i in range(4):
            if ctx[i]:
                rows = torch.cat([K[i][:ctx[i]], V[i][:ctx[i]]], 1).to(dev)
                kv.append_rows(rows, 0, kv_heads * dim, torch.full((ctx[i],), slots[i], dtype=torch.int32, device=dev),
                               torch.arange(ctx[i], dtype=torch.int32, device=dev))
        batch = states.make_batch([(slots[i], [0] * new[i]) for i in range(4)])
        proj = torch.cat([torch.cat([Q[i], K[i][ctx[i]:], V[i][ctx[i]:]], 1) for i in range(4)], 0).to(dev)
        kv.append_rows(proj, heads * dim, heads * dim + kv_heads * dim, batch.row_slot, batch.row_pos)
        if bias == "bucket":
            rel = torch.randn(9, heads, generator=g)
            far = 120.0
            n = int(far) + 1 if mask != "window" else min(int(far) + 1, size)
            table = rel[torch.tensor([log_distance_bucket(d, 9, far) for d in range(n)])].contiguous()
            bias_kind, bias_t = 2, table.to(dev)
        elif bias == "slope":
            slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)])
            bias_kind, bias_t = 1, slopes.to(dev)
        else:
            bias_kind, bias_t = 0, None
        want = []
        for i in range(4):
            q, k, v = Q[i].double(), K[i].double(), V[i].double()
            out = torch.zeros(new[i], heads * vdim, dtype=torch.float64)
            pos = torch.arange(ctx[i], ctx[i] + new[i])[:, None]
            j = torch.arange(ctx[i] + new[i])[None, :]
            dist = pos - j
            vis = dist >= 0
            if mask == "window":
                vis &= dist < size
            elif mask == "chunk":
                vis &= (pos // size) == (j // size)
            for h in range(heads):
                gi = h // per
                sc = q[:, h * dim:(h + 1) * dim] @ k[:, gi * dim:(gi + 1) * dim].T * scale
                if cap:
                    sc = cap * torch.tanh(sc / cap)
                if bias == "bucket":
                    sc = sc + table.double()[dist.clamp(0, table.shape[0] - 1), h]
                elif bias == "slope":
                    sc = sc - float(slopes[h]) * dist
                out[:, h * vdim:(h + 1) * vdim] = torch.softmax(sc.masked_fill(~vis, -float("inf")), -1) @ v[:, gi * vdim:(gi + 1) * vdim]
            want.append(out)
        want = torch.cat(want, 0)
        tt = lib.pa_masked_attention_tile_tokens(heads, kv_heads)
        mt = lib.pa_masked_attention_mma_tile_tokens(dim, vdim, proj.element_size())
        table_dev = pt.device_data()
        for use_mma, use_stream in ((0, 0), (mt, 1)):
            out = torch.zeros(sum(new), heads * vdim, dtype=dtype, device=dev)
            for kind, group in batch.query_tiles(tt, use_mma, 16).items():
                if group is None:
                    continue
                tiles, ntiles, _longest = group
                rc = lib.pa_masked_attention(proj.data_ptr(), proj.stride(0), 0, kv.key_buffer_.data_ptr(), kv.value_buffer_.data_ptr(),
                                             table_dev.data_ptr(), pt.num_beams_, pt.num_heads_, pt.num_tiles_, kv.total_pages_,
                                             kv.tile_size_, tiles.data_ptr(), ntiles, heads, dim, vdim, scale, cap, MASK_KIND[mask],
                                             size, bias_kind, _cabi.ptr(bias_t), int(bias_t.shape[0]) if bias_kind == 2 else 0,
                                             out.data_ptr(), proj.element_size(), kind if (use_stream or kind != 1) else 0,
                                             _cabi.stream())
                assert rc == 0, (kind, rc)
            err = (out.double().cpu() - want).abs().max().item()
            assert err < tol * max(1.0, want.abs().max().item()), (dtype, use_mma, err)


@pytest.mark.gpu
def test_router_groups_kernel_alone():
    from llm_decoder import _cabi
    lib, dev = _cabi.lib(), torch.device("cuda")
    g = torch.Generator().manual_seed(5)
    for E, top, count, keep, width in ((12, 4, 4, 3, 64), (12, 3, 4, 1, 40), (10, 2, 5, 5, 33), (7, 7, 1, 1, 24), (64, 8, 64, 9, 48)):
        h = torch.randn(50, width, generator=g)
        wr = torch.randn(E, width, generator=g) * 0.3
        sel_id = torch.empty(50 * top, dtype=torch.int32, device=dev)
        sel_w = torch.empty(50 * top, dtype=torch.float32, device=dev)
        hd, wd = h.to(dev), wr.to(dev)
        assert lib.pa_router_topk_grouped(hd.data_ptr(), wd.data_ptr(), None, None, 50, width, E, top, 1, 0, count, keep,
                                          sel_id.data_ptr(), sel_w.data_ptr(), None, 4, _cabi.stream()) == 0
        ids, ws = sel_id.cpu().reshape(50, top), sel_w.cpu().reshape(50, top)
        for r in range(50):
            s = torch.softmax(wr.double() @ h[r].double(), 0)
            want = R.route(s, top, count, keep)
            assert ids[r].tolist() == want
            assert (ws[r].double() - s[want]).abs().max() < 1e-6


@pytest.mark.gpu
def test_gated_group_norm_kernel_alone():
    from llm_decoder import _cabi
    lib, dev = _cabi.lib(), torch.device("cuda")
    g = torch.Generator().manual_seed(6)
    for inner, groups in ((96, 2), (70, 1), (120, 5), (33, 3), (1100, 2), (2048, 1)):
        y, gate, w = torch.randn(9, inner, generator=g) * 3, torch.randn(9, inner + 7, generator=g), torch.randn(inner, generator=g)
        for mode in (0, 1, 2):
            out = torch.empty(9, inner, dtype=torch.float32, device=dev)
            yd, gd, wd = y.to(dev), gate.to(dev), w.to(dev)
            assert lib.pa_gated_rms_norm(yd.data_ptr(), 9, inner, groups, gd.data_ptr(), inner + 7, 4, mode, wd.data_ptr(), 1e-6,
                                         out.data_ptr(), 4, _cabi.stream()) == 0
            yy, gg = y.double(), gate[:, 4:4 + inner].double()
            if mode == 1:
                yy = yy * R.silu(gg)
            want = R.rms(yy.reshape(9, groups, inner // groups), 1e-6).reshape(9, inner) * w.double()
            if mode == 2:
                want = want * torch.sigmoid(gg)
            assert (out.double().cpu() - want).abs().max() < 2e-5


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
    wa, wb = R.forward(config, W, a)[0], R.forward(config, W, b)[0]
    g0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1))
    _close(g0, wa[[0, 29]])
    _close(torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1)), wb[[8]])
    _close(torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(1, -1)), wa[[39]])
    p = subprocess.run([os.path.join(ROOT, "bin", "generate"), "--model", str(mdir), "--dtype", "float32", "--prompt",
                        ",".join(map(str, a[:12])), "--max-new-tokens", "5"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr
    toks = [int(t) for t in p.stdout.strip().splitlines()[-1].split(",")]
    assert toks[:12] == a[:12] and len(toks) == 17
    logits = R.forward(config, W, toks[:-1])[0]
    for t in range(11, 16):
        top2 = logits[t].topk(2).values
        if float(top2[0] - top2[1]) > 1e-3:
            assert int(logits[t].argmax()) == toks[t + 1]
