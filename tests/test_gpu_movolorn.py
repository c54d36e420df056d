"""Movolorn through the engine against the plain CPU oracle (oracle/movolorn.py).

Every test makes its own small configuration and random weights.  The engine runs them through its runner
(`ModelRunner.run_step`, the paged cache, the native kernels); the oracle recomputes whole sequences without a
cache.  float32 runs are compared sharply (they show a key that is one position off), bfloat16 runs loosely."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0) if torch.cuda.is_available() else None


# ------------------------------------------------------------------------------------------------ configurations
def attn_cfg(heads=4, kv_heads=2, dim=24, vdim=24, chunk=12, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5}
    if chunk:
        m["mask"] = {"size": chunk}
    return m


def moe_cfg(ff=20, experts=6, identity=2, top=3, groups=4, keep=2, shared=28):
    m = {"kind": "moe", "expert": {"ff": ff},
         "router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": groups, "keep": keep}}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def config_a():
    """Two attention geometries, a dense and a routed feed-forward, a layer without feed-forward, a loop in the middle."""
    return {"architecture": "Movolorn", "vocab": 97, "width": 40, "embedding": {"scale": 1.7}, "norm": {"eps": 1e-5},
            "layers": [
                {"type": "attention", "mixer": attn_cfg(4, 2, 24, 16, 12), "mlp": {"kind": "dense", "ff": 56}},
                {"type": "attention", "mixer": attn_cfg(4, 2, 24, 16, 12), "mlp": moe_cfg()},
                {"type": "attention", "mixer": attn_cfg(6, 3, 8, 40, 7), "mlp": None},
                {"type": "attention", "mixer": attn_cfg(2, 2, 24, 16, 0), "mlp": moe_cfg(12, 4, 0, 1, 1, 1, 0)},
            ],
            "loop": {"start": 1, "stop": 3, "times": 2}}


def config_b(chunk=256, heads=2, kv_heads=1, dim=32):
    """One layer, a long chunk: far keys."""
    return {"architecture": "Movolorn", "vocab": 64, "width": 32, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "layers": [{"type": "attention", "mixer": attn_cfg(heads, kv_heads, dim, dim, chunk),
                        "mlp": {"kind": "dense", "ff": 48}}]}


def make_runner(cfg_json, dtype="float32", pages=24, page_size=16, max_seqs=4, seed=0, max_batched_tokens=None,
                device_allocator=False, eager=True):
    from compactor_vllm.config.engine_config import LLMConfig
    from compactor_vllm.config.model_config import MovolornConfig
    from compactor_vllm.core.model_runner import ModelRunner

    hf = MovolornConfig.from_json(cfg_json)
    cfg = LLMConfig(model="synthetic", hf_config=hf, dtype=dtype, max_num_seqs=max_seqs, kvcache_page_size=page_size,
                    max_model_len=pages * page_size, enforce_eager=eager)
    return ModelRunner(cfg, num_pages=pages, seed=seed, device_allocator=device_allocator,
                       max_batched_tokens=max_batched_tokens)


def oracle_model(model):
    """The engine model's parameters as the oracle's dict (fp32 copies on the CPU)."""
    cfg = model.config
    f = lambda p: p.detach().float().cpu()
    layers = []
    for i, layer in enumerate(model.layers):
        a = cfg.layers[i].mixer
        H, G, D, Dv = a.heads, a.kv_heads, a.dim, a.vdim
        w = f(layer.mixer.qkv_proj.weight)
        attn = {"q": w[:H * D], "k": w[H * D:(H + G) * D], "v": w[(H + G) * D:], "o": f(layer.mixer.o_proj.weight),
                "q_norm": f(layer.mixer.attn.q_norm_weight), "k_norm": f(layer.mixer.attn.k_norm_weight),
                "heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": a.scale, "chunk": a.chunk or None}
        entry = {"norm1": f(layer.norm1.weight), "norm1b": f(layer.norm1b.weight), "attn": attn, "mlp": None}
        mc = cfg.layers[i].mlp
        if mc is not None:
            entry["norm2"], entry["norm2b"] = f(layer.norm2.weight), f(layer.norm2b.weight)
            if mc.kind == "dense":
                gu = f(layer.mlp.gate_up_proj.weight)
                entry["mlp"] = {"kind": "dense", "gate": gu[:mc.ff], "up": gu[mc.ff:], "down": f(layer.mlp.down_proj.weight)}
            else:
                gu, dn = f(layer.mlp.gate_up), f(layer.mlp.down)
                shared = None
                if layer.mlp.shared is not None:
                    sg = f(layer.mlp.shared.gate_up_proj.weight)
                    shared = {"gate": sg[:mc.shared_ff], "up": sg[mc.shared_ff:], "down": f(layer.mlp.shared.down_proj.weight)}
                entry["mlp"] = {"kind": "moe", "router": f(layer.mlp.router), "correction": f(layer.mlp.correction),
                                "experts": [{"gate": gu[e, :mc.ff], "up": gu[e, mc.ff:], "down": dn[e]}
                                            for e in range(mc.experts)],
                                "top": mc.top, "groups": mc.groups, "keep": mc.keep, "identity": mc.identity, "shared": shared}
        layers.append(entry)
    return {"embed": f(model.embed_tokens.weight), "embed_scale": cfg.embedding_scale, "eps": cfg.rms_norm_eps,
            "final_norm": f(model.norm.weight), "head": f(model.lm_head.weight), "layers": layers, "loop": cfg.loop}


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def rel_err(got, want):
    """Per row: rms of the centred difference over the rms of the centred expectation."""
    d = got.double().cpu() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    return (d.pow(2).mean(-1).sqrt() / w.pow(2).mean().sqrt()).max().item()


def new_seq():
    from compactor_vllm.utils.sequence import Sequence

    return Sequence(prompt_token_ids=[])


def feed(runner, seq, toks, all_rows=True):
    seq.prompt_token_ids.extend(toks)
    return runner.run_step([(seq, toks)], rows=list(range(len(toks))) if all_rows else None)


def run_in_portions(runner, toks, sizes):
    """The request alone, cut into portions of the given sizes (cycled); logits of every position."""
    seq, out, at, k = new_seq(), [], 0, 0
    while at < len(toks):
        n = min(sizes[k % len(sizes)], len(toks) - at)
        out.append(feed(runner, seq, toks[at:at + n]))
        at, k = at + n, k + 1
    runner.release([seq])
    return torch.cat(out)


TOL = {"float32": 3e-5, "bfloat16": 6e-2}


def row_errs(got, want):
    d = got.double().cpu() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean().sqrt()


def close(got, want, dtype):
    """float32: every row within rounding.  bfloat16: rounding may flip a router's close call for a token, so the
    typical row has to be close and only a few rows may be further off."""
    e = row_errs(got, want).flatten()
    if dtype == "float32":
        return bool(e.max() < TOL[dtype])
    return bool(e.median() < 0.03 and (e > 0.1).double().mean() <= 0.1 and e.max() < 1.0)


# ------------------------------------------------------------------------------------------ mechanisms one by one
def test_sandwich_norm_against_oracle():
    from compactor_vllm.layers.layernorm import sandwich_norm
    from oracle import movolorn as O

    g = torch.Generator().manual_seed(1)
    for width in (40, 257, 1024):
        x = torch.randn(9, width, generator=g) * 3
        y = torch.randn(9, width, generator=g) * 0.2
        wa, wb = torch.rand(width, generator=g) + 0.5, torch.rand(width, generator=g) + 0.5
        for ydt in (torch.float32, torch.bfloat16):
            yq = y.to(ydt)
            want_x = x + O.rms_norm(yq.float(), wa, 1e-5)
            want_h = O.rms_norm(want_x, wb, 1e-5)
            xr = x.clone().to(DEV)
            h = sandwich_norm(xr, branch=yq.to(DEV), post_weight=wa.to(DEV), pre_weight=wb.to(DEV), eps=1e-5,
                              out_dtype=torch.float32)
            assert torch.allclose(xr.cpu(), want_x, rtol=1e-5, atol=1e-5)
            assert torch.allclose(h.cpu(), want_h, rtol=1e-5, atol=1e-5)
            # each half alone
            xr = x.clone().to(DEV)
            assert sandwich_norm(xr, branch=yq.to(DEV), post_weight=wa.to(DEV), eps=1e-5) is None
            assert torch.allclose(xr.cpu(), want_x, rtol=1e-5, atol=1e-5)
            h = sandwich_norm(xr, pre_weight=wb.to(DEV), eps=1e-5, out_dtype=torch.bfloat16)
            assert torch.allclose(h.float().cpu(), want_h, rtol=1e-2, atol=1e-2)
            assert torch.allclose(xr.cpu(), want_x, rtol=1e-5, atol=1e-5)  # the pre-norm leaves the residual alone


def test_gated_activations_against_oracle():
    from compactor_vllm.layers.moe import ACT_GELU_TANH, ACT_SILU, gated_act
    from oracle import movolorn as O

    g = torch.Generator().manual_seed(2)
    x = torch.randn(7, 2 * 33, generator=g) * 3
    for kind, act in ((ACT_SILU, O.silu), (ACT_GELU_TANH, O.gelu_tanh)):
        want = act(x[:, :33]) * x[:, 33:]
        assert torch.allclose(gated_act(x.to(DEV), kind).cpu(), want, rtol=1e-5, atol=1e-6)
        xb = x.to(torch.bfloat16)
        want_b = act(xb[:, :33].float()) * xb[:, 33:].float()
        assert torch.allclose(gated_act(xb.to(DEV), kind).float().cpu(), want_b, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("E,top,groups,keep", [(8, 3, 4, 2), (10, 3, 2, 1), (6, 1, 1, 1), (12, 4, 3, 3), (64, 6, 8, 3),
                                               (5, 5, 1, 1)])
def test_router_against_oracle(E, top, groups, keep):
    from compactor_vllm.layers.moe import route
    from oracle import movolorn as O

    g = torch.Generator().manual_seed(E * 100 + top)
    W = 16
    h = torch.randn(50, W, generator=g)
    m = {"router": torch.randn(E, W, generator=g), "correction": torch.randn(E, generator=g) * 0.3 - 0.2,
         "top": top, "groups": groups, "keep": keep}
    chosen, weights = O.route(h, m)
    logits = (h @ m["router"].T).to(DEV)
    idx, wts = route(logits, m["correction"].to(DEV), top, groups, keep)
    assert torch.equal(idx.cpu().long(), chosen)
    assert torch.allclose(wts.cpu(), weights, rtol=1e-5, atol=1e-7)
    # no correction: the choice follows the plain scores
    m["correction"] = None
    chosen, weights = O.route(h, m)
    idx, wts = route(logits, None, top, groups, keep)
    assert torch.equal(idx.cpu().long(), chosen)


def test_router_negative_choice_scores_stay_inside_kept_groups():
    """All choice scores negative: a struck group counts as minus infinity, not as zero."""
    from compactor_vllm.layers.moe import route

    logits = torch.zeros(1, 4, device=DEV)
    corr = torch.tensor([-5.0, -6.0, -1.0, -9.0], device=DEV)       # groups {0,1} and {2,3}; the second is best
    idx, wts = route(logits, corr, 2, 2, 1)
    assert sorted(idx[0].tolist()) == [2, 3]
    assert torch.allclose(wts.cpu(), torch.full((1, 2), 0.25))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_blocks_against_oracle(dtype):
    """The attention mixer and both feed-forwards as units, on the first portion of a sequence."""
    from oracle import movolorn as O

    r = make_runner(config_a(), dtype)
    om = oracle_model(r.model)
    toks = tokens(31, 97, 3)
    r.model.debug_residuals = []
    feed(r, new_seq(), toks)
    got = [x.cpu() for x in r.model.debug_residuals]
    r.model.debug_residuals = None
    want = []
    O.forward(om, toks, want)
    assert len(got) == len(want) == 6          # layers 0, (1, 2) x 2, 3
    for g_, w_ in zip(got, want):
        assert close(g_, w_, dtype)


def test_attention_first_tokens_and_sink():
    """A single token attends to itself and the sink: its output is v scaled by e^s / (1 + e^s), not v."""
    from oracle import movolorn as O

    r = make_runner(config_b(chunk=8), "float32")
    om = oracle_model(r.model)
    toks = tokens(3, 64, 4)
    got = run_in_portions(r, toks, [1])
    assert rel_err(got, O.forward(om, toks)) < TOL["float32"]
    # without the sink the lone token's output would be its value itself: the test can see the sink
    x = om["embed"][torch.tensor(toks[:1])] * om["embed_scale"]
    a = om["layers"][0]["attn"]
    h = O.rms_norm(x, om["layers"][0]["norm1"], om["eps"])
    v = (h @ a["v"].T)
    with_sink = O.attention_mixer(h, a, om["eps"])
    plain = v.repeat(1, a["heads"] // a["kv_heads"]) @ a["o"].T
    assert (with_sink - plain).abs().max() > 1e-3


# ------------------------------------------------------------------------------- whole prompts, portions, decoding
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_portions_and_token_by_token(dtype):
    from oracle import movolorn as O

    r = make_runner(config_a(), dtype)
    om = oracle_model(r.model)
    toks = tokens(75, 97, 5)
    want = O.forward(om, toks)
    whole = run_in_portions(r, toks, [len(toks)])
    assert close(whole, want, dtype)
    for sizes in ([1], [2], [3, 2, 17, 1, 1, 5], [64, 2], [7], [12], [13, 11]):
        got = run_in_portions(r, toks, sizes)
        assert close(got, want, dtype), sizes
        if dtype == "float32":      # the cut must not matter beyond rounding
            assert rel_err(got, whole.cpu()) < 1e-5, sizes


@pytest.mark.parametrize("eager", [True, False])
def test_long_decoding_over_pages_and_chunks(eager):
    """eager=False: single-token steps are CUDA-graph replays, the routed experts run without a host round trip."""
    from oracle import movolorn as O

    r = make_runner(config_a(), "float32", pages=16, page_size=16, eager=eager)
    om = oracle_model(r.model)
    toks = tokens(200, 97, 6)
    want = O.forward(om, toks)
    seq = new_seq()
    out = [feed(r, seq, toks[:5])]
    for t in toks[5:]:
        out.append(feed(r, seq, [t]))
    r.release([seq])
    assert rel_err(torch.cat(out), want) < TOL["float32"]
    assert (r.stats["graph_replays"] > 0) == (not eager)


@pytest.mark.parametrize("dtype,eager", [("float32", True), ("float32", False), ("bfloat16", True)])
def test_decoding_far_into_an_unchunked_sequence(dtype, eager):
    """No chunking: hundreds of keys per query, which the decode kernel cuts into several parts that are merged."""
    from oracle import movolorn as O

    r = make_runner(config_b(chunk=0, heads=4, kv_heads=2), dtype, pages=40, page_size=16, eager=eager)
    assert r.model.layers[0].mixer.attn.decode_splits(1, 600) > 1
    om = oracle_model(r.model)
    toks = tokens(540, 64, 8)
    want = O.forward(om, toks)
    seq = new_seq()
    out = [feed(r, seq, toks[:520])] + [feed(r, seq, [t]) for t in toks[520:]]
    r.release([seq])
    assert close(torch.cat(out), want, dtype)


def test_graph_decode_batches_with_padding_rows():
    """Three decoding requests (padded to four rows in the graph) of unequal lengths, one of which ends early."""
    from oracle import movolorn as O

    r = make_runner(config_a(), "float32", pages=20, page_size=16, eager=False)
    om = oracle_model(r.model)
    reqs = [tokens(n, 97, 40 + i) for i, n in enumerate((30, 12, 21))]
    want = [O.forward(om, t) for t in reqs]
    seqs = [new_seq() for _ in reqs]
    got = [[feed(r, s, t[:4])] for s, t in zip(seqs, reqs)]
    for k in range(4, 30):
        live = [i for i, t in enumerate(reqs) if k < len(t)]
        for i in live:
            seqs[i].prompt_token_ids.append(reqs[i][k])
        logits = r.run_step([(seqs[i], [reqs[i][k]]) for i in live])
        for j, i in enumerate(live):
            got[i].append(logits[j:j + 1])
        done = [i for i in live if k == len(reqs[i]) - 1]
        r.release([seqs[i] for i in done])
    assert r.stats["graph_replays"] == 26
    for i in range(3):
        assert rel_err(torch.cat(got[i]), want[i]) < TOL["float32"]


def _standout_runner(chunk, far, n):
    """One layer whose weights make ONE key stand out: token id 1 sits at position `far`, every other position holds
    token 0; the embedding of token 1 is made large along one direction that W_k and W_q both pass on."""
    r = make_runner(config_b(chunk=chunk, heads=2, kv_heads=1, dim=32), "float32", pages=40, page_size=16)
    m = r.model
    with torch.no_grad():
        m.embed_tokens.weight.mul_(0.05)
        m.embed_tokens.weight[1, :] = 0
        m.embed_tokens.weight[1, 0] = 40.0
        m.embed_tokens.weight[2, :] = 0
        m.embed_tokens.weight[2, 0] = 30.0
        m.embed_tokens.weight[2, 1] = 30.0
        D = 32                   # every query head projects like the key head, so that token 2's query meets token 1's key
        w = m.layers[0].mixer.qkv_proj.weight
        w[:D] = w[2 * D:3 * D]
        w[D:2 * D] = w[2 * D:3 * D]
    toks = [0] * n
    toks[far] = 1
    return r, toks


@pytest.mark.parametrize("chunk,far,query", [(256, 3, 250), (256, 0, 255), (256, 3, 256), (64, 63, 64), (64, 64, 127),
                                             (64, 64, 128), (48, 47, 48), (48, 48, 95)])
def test_standout_key_far_away_and_at_chunk_edges(chunk, far, query):
    """The query at `query` (token 2) sees the standout key at `far` only if both lie in one chunk: prompts in
    portions whose cuts fall elsewhere than the chunk edges, and the same while decoding."""
    from oracle import movolorn as O

    n = query + 2
    r, toks = _standout_runner(chunk, far, n)
    toks[query] = 2
    om = oracle_model(r.model)
    want = O.forward(om, toks)
    # the oracle itself must react to the far key at this place, else the case shows nothing
    alt = list(toks)
    alt[far] = 0
    moved = (O.forward(om, alt)[query] - want[query]).abs().max().item()
    same_chunk = far // chunk == query // chunk
    assert (moved > 1e-3) == same_chunk, (moved, same_chunk)
    for sizes in ([n], [50, 29], [query, 1, 1]):
        got = run_in_portions(r, toks, sizes)
        assert rel_err(got, want) < TOL["float32"], sizes
    seq = new_seq()
    out = [feed(r, seq, toks[:far + 1])] + [feed(r, seq, [t]) for t in toks[far + 1:]]
    r.release([seq])
    assert rel_err(torch.cat(out), want) < TOL["float32"]


# ---------------------------------------------------------------------------------- batches, pages and slots reused
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_equal_each_request_alone(dtype):
    from oracle import movolorn as O

    r = make_runner(config_a(), dtype, pages=20, page_size=16)
    om = oracle_model(r.model)
    reqs = [tokens(n, 97, 10 + i) for i, n in enumerate((70, 9, 33, 1))]
    want = [O.forward(om, t) for t in reqs]
    alone = [run_in_portions(r, t, [len(t)]).cpu() for t in reqs]
    # a schedule with portions beside single tokens; request 3 joins late, request 1 pauses for a step
    plan = [[(0, 20), (1, 2)], [(0, 1), (1, 3), (2, 30)], [(0, 13), (2, 1)], [(1, 1), (0, 30), (2, 1), (3, 1)],
            [(0, 6), (1, 3), (2, 1)]]
    seqs = [new_seq() for _ in reqs]
    at = [0] * len(reqs)
    got = [[] for _ in reqs]
    for step in plan:
        entries, spans, base = [], [], 0
        for i, n in step:
            part = reqs[i][at[i]:at[i] + n]
            assert len(part) == n
            seqs[i].prompt_token_ids.extend(part)
            entries.append((seqs[i], part))
            spans.append((i, base, n))
            at[i] += n
            base += n
        logits = r.run_step(entries, rows=list(range(base)))
        for i, b, n in spans:
            got[i].append(logits[b:b + n])
    r.release(seqs)
    for i, t in enumerate(reqs):
        assert at[i] == len(t)
        g_ = torch.cat(got[i])
        assert close(g_, want[i], dtype)
        if dtype == "float32":
            assert rel_err(g_, alone[i]) < 1e-5


@pytest.mark.parametrize("device_allocator", [False, True])
def test_pages_and_slots_are_reused(device_allocator):
    """A pool of 8 pages and 2 slots serves 6 requests of 3-4 pages each, two at a time: every page and slot is used
    again by a later request, whose logits must still be the oracle's."""
    from oracle import movolorn as O

    r = make_runner(config_a(), "float32", pages=8, page_size=16, max_seqs=2, device_allocator=device_allocator)
    om = oracle_model(r.model)
    assert r.kv.num_free_tokens == 8 * 16
    lens = (50, 60, 64, 33, 49, 17)
    for k in range(0, len(lens), 2):
        pair = [tokens(lens[k], 97, 20 + k), tokens(lens[k + 1], 97, 21 + k)]
        seqs = [new_seq(), new_seq()]
        outs = [[], []]
        at = [0, 0]
        while any(at[i] < len(pair[i]) for i in range(2)):
            entries, spans, base = [], [], 0
            for i in range(2):
                n = min(11 + 6 * i, len(pair[i]) - at[i])
                if n:
                    part = pair[i][at[i]:at[i] + n]
                    seqs[i].prompt_token_ids.extend(part)
                    entries.append((seqs[i], part))
                    spans.append((i, base, n))
                    at[i] += n
                    base += n
            logits = r.run_step(entries, rows=list(range(base)))
            for i, b, n in spans:
                outs[i].append(logits[b:b + n])
        assert r.kv.num_free_batches == 0
        r.release(seqs)
        assert r.kv.num_free_batches == 2 and r.kv.num_free_tokens == 8 * 16
        for i in range(2):
            assert rel_err(torch.cat(outs[i]), O.forward(om, pair[i])) < TOL["float32"]


def test_step_that_does_not_fit_is_refused():
    from compactor_vllm.core.model_runner import KVCacheExhausted

    r = make_runner(config_b(chunk=8), "float32", pages=2, page_size=16)
    seq = new_seq()
    feed(r, seq, tokens(30, 64, 1))
    with pytest.raises(KVCacheExhausted):
        feed(r, seq, tokens(5, 64, 2))


# --------------------------------------------------------------------------------------------- other sizes
@pytest.mark.parametrize("over", [
    dict(heads=1, kv_heads=1, dim=8, vdim=8, chunk=1),          # every size 1 where it can be; a chunk of one token
    dict(heads=8, kv_heads=8, dim=16, vdim=72, chunk=5),        # no grouping, values wider than keys
    dict(heads=6, kv_heads=2, dim=136, vdim=100, chunk=0),      # large odd sizes, no chunking
    dict(heads=3, kv_heads=1, dim=20, vdim=256, chunk=33),      # the widest values the kernels take
])
def test_other_attention_sizes(over):
    from oracle import movolorn as O

    cfg = {"architecture": "Movolorn", "vocab": 50, "width": 36, "embedding": {"scale": 0.5}, "norm": {"eps": 1e-6},
           "layers": [{"type": "attention", "mixer": attn_cfg(**over), "mlp": moe_cfg(10, 3, 1, 2, 2, 1, 12)}],
           "loop": {"start": 0, "stop": 1, "times": 3}}
    r = make_runner(cfg, "float32", pages=12, page_size=16)
    om = oracle_model(r.model)
    toks = tokens(70, 50, 7)
    want = O.forward(om, toks)
    assert rel_err(run_in_portions(r, toks, [70]), want) < TOL["float32"]
    assert rel_err(run_in_portions(r, toks, [37, 2, 1]), want) < TOL["float32"]
    assert rel_err(run_in_portions(r, toks[:40], [1]), want[:40]) < TOL["float32"]


def test_routed_experts_grouped_and_looped_products_agree():
    """bfloat16 with sizes that are multiples of 8 takes the grouped-GEMM path; the per-expert loop and the small-step
    kernel must give the same layer output, and all of them the oracle's."""
    from compactor_vllm.layers.moe import ACT_SILU, RoutedExperts
    from compactor_vllm.utils.context import reset_context, set_context
    from oracle import movolorn as O

    W, ff, E, ident = 48, 24, 6, 2
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(DEV):
            m = RoutedExperts(W, ff, E, ident, 3, 4, 2, 32, ACT_SILU, torch.bfloat16)
    finally:
        torch.set_default_dtype(prev)
    g = torch.Generator(device=DEV).manual_seed(3)
    with torch.no_grad():
        for name, p in m.named_parameters():
            p.copy_((torch.randn(p.shape, generator=g, device=DEV) * (0.1 if name == "correction" else p.shape[-1] ** -0.5)))
        x = torch.randn(200, W, generator=g, device=DEV).to(torch.bfloat16)
        f = lambda t: t.detach().float().cpu()
        gu, dn, sg = f(m.gate_up), f(m.down), f(m.shared.gate_up_proj.weight)
        om = {"kind": "moe", "router": f(m.router), "correction": f(m.correction), "top": 3, "groups": 4, "keep": 2,
              "identity": ident, "experts": [{"gate": gu[e, :ff], "up": gu[e, ff:], "down": dn[e]} for e in range(E)],
              "shared": {"gate": sg[:32], "up": sg[32:], "down": f(m.shared.down_proj.weight)}}
        want = O.moe_ff(x.float().cpu(), om)
        set_context(is_prefill=True)
        assert m.grouped_gemm
        grouped = m(x).cpu()
        m.grouped_gemm = False
        looped = m(x).cpu()
        set_context(is_prefill=False)
        small = m(x).cpu()
        reset_context()
    for got in (grouped, looped, small):
        e = row_errs(got, want)
        assert e.median() < 0.02 and e.max() < 0.2      # a flipped close call of the router may move single rows
    assert row_errs(grouped, looped).median() < 5e-3 and row_errs(small, looped).median() < 5e-3


@pytest.mark.parametrize("dim,vdim,chunk", [(32, 40, 50), (64, 64, 0), (80, 128, 33), (128, 24, 70), (16, 8, 5)])
def test_bfloat16_portions_on_tensor_cores(dim, vdim, chunk):
    """Head sizes the mma.sync portion kernel takes (key size a multiple of 16, value size of 8): against the oracle,
    and against the fp32 FMA kernel on the same bfloat16 inputs (they differ only by the rounding of P)."""
    from compactor_vllm import _native as N
    from oracle import movolorn as O

    cfg = {"architecture": "Movolorn", "vocab": 80, "width": 48, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
           "layers": [{"type": "attention", "mixer": attn_cfg(6, 2, dim, vdim, chunk), "mlp": {"kind": "dense", "ff": 64}},
                      {"type": "attention", "mixer": attn_cfg(2, 2, dim, vdim, chunk), "mlp": None}]}
    r = make_runner(cfg, "bfloat16", pages=24, page_size=16)
    om = oracle_model(r.model)
    reqs = [tokens(150, 80, 50), tokens(67, 80, 51)]
    want = [O.forward(om, t) for t in reqs]

    def run():
        seqs, got, at = [new_seq(), new_seq()], [[], []], [0, 0]
        for step in ([(0, 70), (1, 3)], [(0, 64), (1, 64)], [(0, 16)]):
            entries, spans, base = [], [], 0
            for i, n in step:
                part = reqs[i][at[i]:at[i] + n]
                seqs[i].prompt_token_ids.extend(part)
                entries.append((seqs[i], part))
                spans.append((i, base, len(part)))
                at[i] += len(part)
                base += len(part)
            logits = r.run_step(entries, rows=list(range(base)))
            for i, b_, n in spans:
                got[i].append(logits[b_:b_ + n])
        r.release(seqs)
        return [torch.cat(g_).float().cpu() for g_ in got]

    mma = run()
    N.set_test_option("bias_attn_fma", 1)
    try:
        fma = run()
    finally:
        N.set_test_option("bias_attn_fma", 0)
    for i in range(2):
        assert close(mma[i], want[i], "bfloat16") and close(fma[i], want[i], "bfloat16")
        assert rel_err(mma[i], fma[i]) < 0.05
        assert row_errs(mma[i], fma[i]).median() < 0.01


@pytest.mark.parametrize("chunk", [0, 128, 200, 37])
def test_bfloat16_portions_on_the_tcgen05_pipeline(chunk):
    """Key and value size 128, pages of 128 rows, two query heads per KV head: portions run on the tcgen05 kernel.
    Checked against the oracle and against the mma.sync and FMA kernels on the same inputs; the portions start and
    end off the 128-row tiles, and the chunk edges fall inside tiles."""
    from compactor_vllm import _native as N
    from oracle import movolorn as O

    cfg = {"architecture": "Movolorn", "vocab": 80, "width": 64, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
           "layers": [{"type": "attention", "mixer": attn_cfg(4, 2, 128, 128, chunk), "mlp": {"kind": "dense", "ff": 64}},
                      {"type": "attention", "mixer": attn_cfg(2, 1, 128, 128, chunk), "mlp": None}]}
    r = make_runner(cfg, "bfloat16", pages=8, page_size=128)
    om = oracle_model(r.model)
    reqs = [tokens(420, 80, 60), tokens(131, 80, 61)]
    want = [O.forward(om, t) for t in reqs]

    def run():
        seqs, got, at = [new_seq(), new_seq()], [[], []], [0, 0]
        for step in ([(0, 70), (1, 3)], [(0, 200), (1, 128)], [(0, 1)], [(0, 149)]):
            entries, spans, base = [], [], 0
            for i, n in step:
                part = reqs[i][at[i]:at[i] + n]
                seqs[i].prompt_token_ids.extend(part)
                entries.append((seqs[i], part))
                spans.append((i, base, len(part)))
                at[i] += len(part)
                base += len(part)
            logits = r.run_step(entries, rows=list(range(base)))
            for i, b_, n in spans:
                got[i].append(logits[b_:b_ + n])
        r.release(seqs)
        return [torch.cat(g_).float().cpu() for g_ in got]

    launches = N.lib().cvllm_launch_count()
    umma = run()
    assert N.lib().cvllm_launch_count() > launches
    outs = {}
    for option in (2, 1):
        N.set_test_option("bias_attn_fma", option)
        try:
            outs[option] = run()
        finally:
            N.set_test_option("bias_attn_fma", 0)
    for i in range(2):
        assert close(umma[i], want[i], "bfloat16"), i
        for option in (2, 1):
            assert close(outs[option][i], want[i], "bfloat16")
            assert row_errs(umma[i], outs[option][i]).median() < 0.01 and rel_err(umma[i], outs[option][i]) < 0.05


# ------------------------------------------------------------------------------ generation through the entry point
def test_greedy_generation_through_llm_generate():
    """`LLM.generate` with the step scheduler: prompts in portions of at most 16 tokens beside decoding requests, five
    requests on three slots.  Teacher forcing against the oracle: every generated token must be the oracle's argmax
    unless the oracle's two best logits are closer than the engine's rounding."""
    from compactor_vllm import LLM
    from compactor_vllm.api_types import SamplingParams
    from compactor_vllm.config.engine_config import LLMConfig
    from compactor_vllm.config.model_config import MovolornConfig
    from oracle import movolorn as O

    hf = MovolornConfig.from_json(config_a())
    cfg = LLMConfig(model="synthetic", hf_config=hf, dtype="float32", max_num_seqs=3, kvcache_page_size=16,
                    max_model_len=160)
    llm = LLM(cfg, num_pages=14, device_allocator=False, max_batched_tokens=16)
    om = oracle_model(llm.model_runner.model)
    prompts = [tokens(n, 97, 30 + i) for i, n in enumerate((40, 3, 25, 1, 18))]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=12))
    assert llm.model_runner.kv.num_free_batches == 3
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        logits = O.forward(om, p + o[:-1])[len(p) - 1:]
        for k, tok in enumerate(o):
            best = torch.topk(logits[k], 2)
            assert tok == int(best.indices[0]) or float(best.values[0] - best.values[1]) < 1e-3, (k, tok)
