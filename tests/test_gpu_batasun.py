"""Batasun through the engine against the plain CPU oracle (oracle/batasun.py).

Every test makes its own small configuration and random weights.  The engine runs them through its runner
(`ModelRunner.run_step`, the paged cache, the state pool, the native kernels); the oracle recomputes whole sequences
without a cache or a carried state.  float32 runs are compared sharply (they show a key that is one position off or a
state that was lost), bfloat16 runs loosely."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0) if torch.cuda.is_available() else None


# ------------------------------------------------------------------------------------------------ configurations
def latent(heads=3, dim=12, rot=8, vdim=10, kv_rank=20, q_rank=14, base=100.0, scale=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "rot": {"base": base, "dims": rot}, "scale": scale or 1.3 * (dim + rot) ** -0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def mamba(heads=4, vdim=6, state=10, groups=2, conv=3, norm_groups=2):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def moe(ff=12, limit=1.5, experts=5, top=2, shared=20, shared_limit=0.8):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared, "limit": shared_limit}
    return m


def model_cfg(layers, vocab=89, width=48, eps=1e-5):
    return {"architecture": "Batasun", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": [dict(mixer_layer, mlp=mlp) for mixer_layer, mlp in layers]}


def config_a():
    """Both mixers, a layer that borrows another's latent, layers without a feed-forward, odd sizes everywhere (key rows
    of 28 and 16 numbers: the kernels' scalar paths)."""
    return model_cfg([
        (latent(3, 12, 8, 10, 20, 14), moe()),
        (mamba(4, 6, 10, 2, 3, 2), None),
        (latent(2, 16, 8, 12, 20, 10, kv_from=0), moe(10, 2.5, 4, 1, 0)),
        (mamba(2, 16, 24, 1, 4, 1), moe(8, 0.7, 3, 3, 16, 2.0)),
        (latent(1, 8, 4, 8, 12, 6, base=7.0), None),
    ])


def config_b():
    """Sizes in multiples of 16: the vector and tensor-core paths of the attention kernels, a wider state."""
    return model_cfg([
        (mamba(4, 16, 40, 4, 2, 4), moe(16, 1.0, 8, 2, 32, 1.0)),
        (latent(4, 32, 16, 32, 48, 32, base=50000.0), moe(16, 3.0, 8, 3, 0)),
        (latent(2, 16, 16, 24, 48, 16, base=50000.0, kv_from=1), None),
    ], vocab=64, width=64, eps=1e-6)


def make_runner(cfg_json, dtype="float32", pages=24, page_size=16, max_seqs=4, seed=0, max_batched_tokens=None,
                device_allocator=False, eager=True):
    from compactor_vllm.config.engine_config import LLMConfig
    from compactor_vllm.config.model_config import BatasunConfig
    from compactor_vllm.core.model_runner import ModelRunner

    hf = BatasunConfig.from_json(cfg_json)
    cfg = LLMConfig(model="synthetic", hf_config=hf, dtype=dtype, max_num_seqs=max_seqs, kvcache_page_size=page_size,
                    max_model_len=pages * page_size, enforce_eager=eager)
    return ModelRunner(cfg, num_pages=pages, seed=seed, device_allocator=device_allocator,
                       max_batched_tokens=max_batched_tokens)


def oracle_model(model):
    """The engine model's parameters as the oracle's dict (fp32 copies on the CPU)."""
    from compactor_vllm.layers.latent_attention import LatentAttention

    cfg = model.config
    f = lambda p: p.detach().float().cpu()
    layers = []
    for i, layer in enumerate(model.layers):
        a, mx = cfg.layers[i].mixer, layer.mixer
        if isinstance(mx, LatentAttention):
            w = f(mx.in_proj.weight)
            m = {"type": "latent_attention", "heads": a.heads, "dim": a.dim, "rot_dim": a.rot_dim, "vdim": a.vdim,
                 "kv_rank": a.kv_rank, "q_rank": a.q_rank, "scale": a.scale, "rot_base": a.rot_base, "kv_from": a.kv_from,
                 "dq": w[:a.q_rank], "dq_norm": f(mx.q_norm), "uq": f(mx.uq_proj.weight),
                 "uk": f(mx.uk).reshape(a.heads * a.dim, a.kv_rank), "uv": f(mx.uv).reshape(a.heads * a.vdim, a.kv_rank),
                 "o": f(mx.o_proj.weight)}
            if a.kv_from is None:
                row = a.kv_rank + a.rot_dim
                m["dkv"], m["dkv_norm"], m["g"] = w[a.q_rank:a.q_rank + row], f(mx.kv_norm), w[a.q_rank + row:]
            else:
                m["g"] = w[a.q_rank:]
        else:
            m = {"type": "mamba2", "heads": a.heads, "vdim": a.vdim, "state": a.state, "groups": a.groups, "conv": a.conv,
                 "norm_groups": a.norm_groups, "in": f(mx.in_proj.weight), "conv_w": f(mx.conv_weight),
                 "conv_b": f(mx.conv_bias), "dt_bias": f(mx.dt_bias), "A_log": f(mx.A_log), "D": f(mx.D),
                 "norm": f(mx.norm_weight), "o": f(mx.o_proj.weight)}
        mlp, mc = None, cfg.layers[i].mlp
        if mc is not None:
            e = layer.mlp
            gu, dn, E = f(e.gate_up), f(e.down), mc.experts
            shared = None
            if e.shared is not None:
                sg = f(e.shared.gate_up_proj.weight)
                shared = {"gate": sg[:mc.shared_ff], "up": sg[mc.shared_ff:], "down": f(e.shared.down_proj.weight),
                          "sg": f(e.router)[E:], "limit": mc.shared_limit}
            mlp = {"experts": [{"gate": gu[k, :mc.ff], "up": gu[k, mc.ff:], "down": dn[k]} for k in range(E)],
                   "limit": mc.limit, "router": f(e.router)[:E], "router_b": f(e.router_bias)[:E], "top": mc.top,
                   "shared": shared}
        layers.append({"norm1": f(layer.norm1.weight), "norm2": f(layer.norm2.weight) if mc is not None else None,
                       "mixer": m, "mlp": mlp})
    return {"embed": f(model.embed_tokens.weight), "embed_norm": f(model.embed_norm.weight), "eps": cfg.rms_norm_eps,
            "final_norm": f(model.norm.weight), "head": f(model.lm_head.weight), "layers": layers}


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def row_errs(got, want):
    """Per row: rms of the centred difference over the rms of the centred expectation."""
    d = got.double().cpu() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean().sqrt()


def rel_err(got, want):
    return row_errs(got, want).max().item()


TOL = {"float32": 3e-5, "bfloat16": 6e-2}


def close(got, want, dtype):
    """float32: every row within rounding.  bfloat16: rounding may flip a router's close call for a token, so the
    typical row has to be close and only a few rows may be further off."""
    e = row_errs(got, want).flatten()
    if dtype == "float32":
        return bool(e.max() < TOL[dtype])
    return bool(e.median() < 0.03 and (e > 0.1).double().mean() <= 0.1 and e.max() < 1.0)


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


# ------------------------------------------------------------------------------------------ mechanisms one by one
def test_norm_with_gain_around_zero_assign_and_cast():
    from compactor_vllm.layers.layernorm import sandwich_norm
    from oracle import batasun as O

    g = torch.Generator().manual_seed(1)
    for width in (40, 257):
        x = torch.randn(7, width, generator=g) * 3
        y = (torch.randn(7, width, generator=g) * 0.2).to(torch.bfloat16)
        wa, wb = torch.randn(width, generator=g) * 0.2, torch.randn(width, generator=g) * 0.2
        want_x = x.double() + O.zero_centred_norm(y.float(), wa, 1e-5)
        xr = x.clone().to(DEV)
        h = sandwich_norm(xr, branch=y.to(DEV), post_weight=wa.to(DEV), eps=1e-5, out_dtype=torch.bfloat16,
                          gain_offset=1.0, cast_out=True)
        assert torch.allclose(xr.cpu().double(), want_x, rtol=1e-5, atol=1e-5)
        assert torch.equal(h.cpu(), xr.cpu().to(torch.bfloat16))        # the stream itself, rounded
        xr2 = torch.full_like(xr, 5.0)
        sandwich_norm(xr2, branch=y.to(DEV), post_weight=wa.to(DEV), eps=1e-5, gain_offset=1.0, assign=True)
        assert torch.allclose(xr2.cpu().double(), O.zero_centred_norm(y.float(), wa, 1e-5), rtol=1e-5, atol=1e-5)
        h = sandwich_norm(xr, pre_weight=wb.to(DEV), eps=1e-5, out_dtype=torch.float32, gain_offset=1.0)
        assert torch.allclose(h.cpu().double(), O.zero_centred_norm(want_x, wb, 1e-5), rtol=1e-5, atol=1e-5)


def test_clamped_gated_unit_at_and_beyond_its_limits():
    from compactor_vllm.layers.moe import ACT_CLAMPED_GLU, gated_act
    from oracle import batasun as O

    F, limit = 24, 1.25
    g = torch.Generator().manual_seed(2)
    x = torch.randn(11, 2 * F, generator=g) * 2.5          # many values beyond +-limit
    x[0, :4] = torch.tensor([limit, -limit, 2 * limit, -2 * limit])
    x[0, F:F + 4] = torch.tensor([limit, -limit, 2 * limit, -2 * limit])
    gate = torch.clamp(x[:, :F].double(), max=limit)
    up = torch.clamp(x[:, F:].double(), -limit, limit)
    want = gate * O.sigmoid(1.702 * gate) * (up + 1.0)
    got = gated_act(x.to(DEV), ACT_CLAMPED_GLU, limit=limit)
    assert torch.allclose(got.cpu().double(), want, rtol=1e-5, atol=1e-6)
    # the same unit inside the few-token expert product
    from compactor_vllm import _native as N
    E, K = 3, 20
    w = torch.randn(E, 2 * F, K, generator=g)
    xs = torch.randn(4, K, generator=g) * 2
    idx = torch.tensor([2, 0, 1, 1], dtype=torch.int32)
    out = torch.zeros(4, F, device=DEV)
    wd, xd, idd = w.to(DEV), xs.to(DEV), idx.to(DEV)
    N.check(N.lib().cvllm_expert_gemv(N.ptr(xd), 1, N.ptr(wd), N.ptr(idd), E, N.ptr(out), 4, F, K, ACT_CLAMPED_GLU, limit,
                                      N.CVLLM_F32, N.stream(DEV)), "gemv")
    for p in range(4):
        pre = w[idx[p]].double() @ xs[p].double()
        gg, uu = torch.clamp(pre[:F], max=limit), torch.clamp(pre[F:], -limit, limit)
        assert torch.allclose(out[p].cpu().double(), gg * O.sigmoid(1.702 * gg) * (uu + 1.0), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("E,top", [(5, 2), (12, 3), (7, 1), (4, 4), (40, 6), (1, 1)])
def test_router_takes_the_largest_logits_and_normalises_over_them(E, top):
    from compactor_vllm.layers.moe import ROUTE_TOP_LOGITS, route
    from oracle import batasun as O

    g = torch.Generator().manual_seed(E * 10 + top)
    z = torch.randn(33, E + 1, generator=g) * 2       # one more column than experts: it must not be chosen
    z[:, E] = 100.0
    if E > 2:
        z[0, 1] = z[0, 2] = z[0].max() + 1.0          # equal logits: the lower index first
    idx, wts = route(z.to(DEV), None, top, 1, 1, ROUTE_TOP_LOGITS, experts=E)
    for t in range(z.shape[0]):
        want_idx, want_w = O.route_top_logits(z[t, :E].double(), top)
        assert idx[t].tolist() == want_idx, t
        assert torch.allclose(wts[t].cpu().double(), want_w, rtol=1e-5, atol=1e-7)
        assert abs(float(wts[t].sum()) - 1.0) < 1e-5


def single_layer(mixer_layer, mlp, dtype, **kw):
    r = make_runner(model_cfg([(mixer_layer, mlp)], **kw), dtype, pages=12, page_size=16)
    r.model.debug_residuals = []
    return r


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["latent", "latent_wide", "mamba", "mamba_one_group", "moe", "moe_top1_no_shared"])
def test_each_mechanism_alone_against_oracle(dtype, which):
    """One layer with one mechanism; the residual stream after it (and the embedding norm before it) against the oracle."""
    from oracle import batasun as O

    layer = {"latent": (latent(), None), "latent_wide": (latent(2, 24, 16, 40, 64, 24, base=1e4), None),
             "mamba": (mamba(), None), "mamba_one_group": (mamba(3, 20, 33, 1, 2, 3), None),
             "moe": (mamba(1, 8, 4, 1, 1, 1), moe()), "moe_top1_no_shared": (mamba(1, 8, 4, 1, 1, 1), moe(9, 0.5, 6, 1, 0))}[which]
    r = single_layer(*layer, dtype)
    toks = tokens(37, 89, 5)
    seq = new_seq()
    logits = feed(r, seq, toks)
    want_res = []
    want = O.forward(oracle_model(r.model), toks, want_res)
    got_res = r.model.debug_residuals[0].cpu().double()
    scale = want_res[0].abs().max().item()
    tol = 2e-5 if dtype == "float32" else 4e-2
    bad = ((got_res - want_res[0]).abs().max(-1).values > tol * scale).double().mean().item()
    assert bad <= (0.0 if dtype == "float32" else 0.1), (which, bad)
    assert close(logits, want, dtype)


def test_rotation_angles_at_far_positions():
    """A one-layer model whose sequence starts far from position 0 only in the engine's eyes: the rotated parts at
    positions around 5000 against the oracle's 64-bit angles (the oracle runs the whole sequence; the engine is asked
    for the last rows only)."""
    from oracle import batasun as O

    r = make_runner(model_cfg([(latent(2, 8, 16, 8, 16, 8, base=3.0), None)]), "float32", pages=330, page_size=16)
    toks = tokens(5200, 89, 9)
    got = run_in_portions(r, toks, [1024])[-6:]
    # the oracle's forward is quadratic: its functions are applied to all keys but to the last six queries only
    om = oracle_model(r.model)
    m = om["layers"][0]["mixer"]
    x = O.zero_centred_norm(om["embed"].double()[torch.tensor(toks)], om["embed_norm"], om["eps"])
    c, kr = O.latent_kv(x, m, om["eps"])
    T = len(toks)
    cq = O.plain_norm(x[-6:] @ m["dq"].double().T, m["dq_norm"], om["eps"])
    q = (cq @ m["uq"].double().T).view(6, m["heads"], m["dim"] + m["rot_dim"])
    qr = O.rotate_half(q[..., m["dim"]:], torch.arange(T - 6, T), m["rot_base"])
    kp = (c @ m["uk"].double().T).view(T, m["heads"], m["dim"])
    v = (c @ m["uv"].double().T).view(T, m["heads"], m["vdim"])
    out = torch.zeros(6, m["heads"], m["vdim"], dtype=torch.float64)
    for i in range(6):
        n = T - 6 + i + 1
        for h in range(m["heads"]):
            s = (kp[:n, h] @ q[i, h, :m["dim"]] + kr[:n] @ qr[i, h]) * m["scale"]
            p = torch.softmax(s, 0)
            out[i, h] = p @ v[:n, h]
    y = (out.reshape(6, -1) * O.sigmoid(x[-6:] @ m["g"].double().T)) @ m["o"].double().T
    xx = x[-6:] + O.zero_centred_norm(y, om["layers"][0]["norm1"], om["eps"])
    want = O.zero_centred_norm(xx, om["final_norm"], om["eps"]) @ om["head"].double().T
    assert rel_err(got, want) < 1e-4


# ----------------------------------------------------------------------- prompts, portions, decoding, long decoding
# config_a in bfloat16 shows nothing: at its width a router's close call flips for many tokens and the comparison with
# the oracle drowns in that; it runs in float32, config_b in both
@pytest.mark.parametrize("dtype,cfg", [("float32", config_a), ("float32", config_b), ("bfloat16", config_b)])
def test_whole_prompt_portions_and_token_by_token(dtype, cfg):
    from oracle import batasun as O

    r = make_runner(cfg(), dtype, pages=30, page_size=16)
    toks = tokens(75, r.model.config.vocab_size, 3)
    want = O.forward(oracle_model(r.model), toks)
    whole = run_in_portions(r, toks, [len(toks)])
    assert close(whole, want, dtype)
    for sizes in ([2], [3, 2, 16, 1, 5], [17, 31], [64, 2, 2, 7], [1]):
        got = run_in_portions(r, toks, sizes)
        assert close(got, want, dtype), sizes
        if dtype == "float32":        # how a prompt is cut changes nothing beyond rounding
            assert rel_err(got, whole.cpu()) < TOL["float32"], sizes


def test_first_tokens_of_a_sequence():
    """Positions 0, 1, 2: no key but the token's own, a convolution window that is mostly zeros, a zero state; alone,
    as the start of a portion, and as single-token steps (eager and from the decode graph)."""
    from oracle import batasun as O

    for eager in (True, False):
        r = make_runner(config_a(), "float32", eager=eager)
        om = oracle_model(r.model)
        for n in (1, 2, 3, 5):
            toks = tokens(n, 89, 60 + n)
            want = O.forward(om, toks)
            assert rel_err(run_in_portions(r, toks, [n]), want) < TOL["float32"]
            assert rel_err(run_in_portions(r, toks, [1]), want) < TOL["float32"]


@pytest.mark.parametrize("eager", [True, False])
def test_long_decoding_over_pages(eager):
    """A short prompt, then 150 single-token steps over ten pages (eager kernels, and replays of the decode graph)."""
    from oracle import batasun as O

    r = make_runner(config_a(), "float32", pages=12, page_size=16, eager=eager)
    toks = tokens(160, 89, 11)
    want = O.forward(oracle_model(r.model), toks)
    seq = new_seq()
    out = [feed(r, seq, toks[:10])] + [feed(r, seq, [t]) for t in toks[10:]]
    r.release([seq])
    if not eager:
        assert r.stats["graph_replays"] == 150
    assert rel_err(torch.cat(out), want) < TOL["float32"]


def test_graph_decode_batches_with_padding_rows():
    """Three decoding requests (padded to four rows in the graph) of unequal lengths, one of which ends early."""
    from oracle import batasun as O

    r = make_runner(config_a(), "float32", pages=20, page_size=16, eager=False)
    om = oracle_model(r.model)
    reqs = [tokens(n, 89, 40 + i) for i, n in enumerate((30, 12, 21))]
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
        r.release([seqs[i] for i in live if k == len(reqs[i]) - 1])
    for i in range(3):
        assert rel_err(torch.cat(got[i]), want[i]) < TOL["float32"]


# ------------------------------------------------------------------------------ a key that stands out, far and at edges
def _standout(far, query, n, page_size=16):
    """One latent-attention layer whose weights make ONE key stand out for one query: token 1 sits at `far`, token 2 at
    `query`, token 0 everywhere else; head 0's unrotated query of token 2 is turned onto token 1's unrotated key."""
    from oracle import batasun as O

    r = make_runner(model_cfg([(latent(2, 16, 8, 16, 24, 12, base=20.0, scale=0.25), None)]), "float32", pages=40,
                    page_size=page_size)
    mx = r.model.layers[0].mixer
    om = oracle_model(r.model)
    m, eps = om["layers"][0]["mixer"], om["eps"]
    x = O.zero_centred_norm(om["embed"].double()[torch.tensor([0, 1, 2])], om["embed_norm"], eps)
    c, _ = O.latent_kv(x, m, eps)
    k1 = (c[1] @ m["uk"].double().T)[:16]                                  # head 0's key of token 1
    cq2 = O.plain_norm(x[2:3] @ m["dq"].double().T, m["dq_norm"], eps)[0]
    target = 60.0 * k1 / k1.norm() ** 2                                    # q . k1 = 60: score 15 above the rest
    uq = mx.uq_proj.weight.detach().double().cpu()
    cur = uq[:16] @ cq2
    uq[:16] += torch.outer(target - cur, cq2) / (cq2 @ cq2)
    with torch.no_grad():
        mx.uq_proj.weight.copy_(uq.to(mx.uq_proj.weight.dtype))
    toks = [0] * n
    toks[far], toks[query] = 1, 2
    return r, toks


@pytest.mark.parametrize("far,query", [(0, 255), (3, 250), (15, 16), (16, 17), (31, 32), (15, 31), (16, 300), (63, 64)])
def test_standout_key_far_away_and_at_page_borders(far, query):
    from oracle import batasun as O

    n = query + 2
    r, toks = _standout(far, query, n)
    om = oracle_model(r.model)
    want = O.forward(om, toks)
    alt = list(toks)
    alt[far] = 0         # the oracle itself must react to the far key, else the case shows nothing
    assert (O.forward(om, alt)[query] - want[query]).abs().max().item() > 1e-2
    for sizes in ([n], [50, 29], [query, 1, 1], [far + 1, 7]):
        assert rel_err(run_in_portions(r, toks, sizes), want) < TOL["float32"], sizes
    seq = new_seq()
    out = [feed(r, seq, toks[:far + 1])] + [feed(r, seq, [t]) for t in toks[far + 1:]]
    r.release([seq])
    assert rel_err(torch.cat(out), want) < TOL["float32"]


def test_state_far_back_reaches_the_last_token():
    """A state-space layer with almost no decay: the first token's input is still in the state 200 tokens later, through
    portions and decoding; swapping the first token must change the last logits in the oracle and the engine alike."""
    from oracle import batasun as O

    r = make_runner(model_cfg([(mamba(2, 8, 12, 1, 4, 1), None)]), "float32", pages=20, page_size=16)
    with torch.no_grad():
        r.model.layers[0].mixer.A_log.fill_(-9.0)
    om = oracle_model(r.model)
    toks = tokens(200, 89, 17)
    want = O.forward(om, toks)
    alt = [(toks[0] + 1) % 89] + toks[1:]
    assert (O.forward(om, alt)[-1] - want[-1]).abs().max().item() > 1e-3
    for sizes in ([200], [2], [16, 1, 33], [199, 1]):
        assert rel_err(run_in_portions(r, toks, sizes), want) < TOL["float32"], sizes


@pytest.mark.parametrize("seg", [16, 32, 48])
def test_long_portions_run_in_segments(seg):
    """Portions longer than a segment run their segments side by side (local states, a combine pass, a rerun); with short
    segments every cut of the test falls somewhere else: on a segment's edge, one token past it, inside it, and a batch
    of a long portion beside short ones and beside a sequence that continues from a carried state."""
    from compactor_vllm import _native as N
    from oracle import batasun as O

    N.set_test_option("ssm_segment", seg)
    try:
        r = make_runner(model_cfg([(mamba(3, 20, 33, 1, 3, 3), None), (mamba(4, 6, 10, 2, 4, 2), moe())]), "float32",
                        pages=40, page_size=16)
        om = oracle_model(r.model)
        toks = tokens(150, 89, 23)
        want = O.forward(om, toks)
        for sizes in ([150], [seg + 1, 2 * seg, 5], [3, 2 * seg + 1, seg], [seg, seg, seg + 7]):
            assert rel_err(run_in_portions(r, toks, sizes), want) < TOL["float32"], sizes
        reqs = [tokens(n, 89, 50 + i) for i, n in enumerate((140, 5, 70))]
        wants = [O.forward(om, t) for t in reqs]
        seqs = [new_seq() for _ in reqs]
        head = feed(r, seqs[2], reqs[2][:9])                       # request 2 carries a state into the big step
        for s_, t in zip(seqs[:2], reqs[:2]):
            s_.prompt_token_ids.extend(t)
        seqs[2].prompt_token_ids.extend(reqs[2][9:])
        logits = r.run_step([(seqs[0], reqs[0]), (seqs[1], reqs[1]), (seqs[2], reqs[2][9:])], rows=list(range(140 + 5 + 61)))
        r.release(seqs)
        assert rel_err(logits[:140], wants[0]) < TOL["float32"]
        assert rel_err(logits[140:145], wants[1]) < TOL["float32"]
        assert rel_err(torch.cat([head, logits[145:]]), wants[2]) < TOL["float32"]
    finally:
        N.set_test_option("ssm_segment", 0)


# ---------------------------------------------------------------------------------- batches, pages and slots reused
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_equal_each_request_alone(dtype):
    """Four requests of unequal lengths in one step after another: portions of some beside single tokens of others."""
    from oracle import batasun as O

    r = make_runner(config_a() if dtype == "float32" else config_b(), dtype, pages=30, page_size=16)
    om = oracle_model(r.model)
    reqs = [tokens(n, r.model.config.vocab_size, 70 + i) for i, n in enumerate((61, 9, 33, 2))]
    plan = [[5, 1, 1, 1, 20, 1, 1, 30, 1], [9], [1, 1, 16, 2, 13], [1, 1]]      # portion sizes per request, step by step
    seqs, at, outs = [new_seq() for _ in reqs], [0] * 4, [[] for _ in reqs]
    step = 0
    while any(at[i] < len(reqs[i]) for i in range(4)):
        entries, spans, base = [], [], 0
        for i in range(4):
            if step < len(plan[i]) and at[i] < len(reqs[i]):
                n = min(plan[i][step], len(reqs[i]) - at[i])
                part = reqs[i][at[i]:at[i] + n]
                seqs[i].prompt_token_ids.extend(part)
                entries.append((seqs[i], part))
                spans.append((i, base, n))
                at[i] += n
                base += n
        logits = r.run_step(entries, rows=list(range(base)))
        for i, b, n in spans:
            outs[i].append(logits[b:b + n])
        step += 1
    for i in range(4):
        assert close(torch.cat(outs[i]), O.forward(om, reqs[i]), dtype), i


@pytest.mark.parametrize("device_allocator", [False, True])
def test_pages_and_slots_are_reused(device_allocator):
    """A pool of 8 pages and 2 slots serves 6 requests, two at a time: every page and state slot is used again by a later
    request - also by a shorter one, whose first tokens must not see what the slot held before."""
    from oracle import batasun as O

    r = make_runner(config_a(), "float32", pages=8, page_size=16, max_seqs=2, device_allocator=device_allocator)
    om = oracle_model(r.model)
    lens = (50, 60, 64, 3, 1, 49)
    for k in range(0, len(lens), 2):
        pair = [tokens(lens[k], 89, 20 + k), tokens(lens[k + 1], 89, 21 + k)]
        seqs, outs, at = [new_seq(), new_seq()], [[], []], [0, 0]
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


def test_a_request_left_out_of_steps_goes_on_later():
    """Request A pauses while B runs through A's neighbouring slot; A's state and cache are as it left them."""
    from oracle import batasun as O

    r = make_runner(config_b(), "float32", pages=30, page_size=16)
    om = oracle_model(r.model)
    a, b = tokens(40, 64, 1), tokens(35, 64, 2)
    sa, sb = new_seq(), new_seq()
    out_a = [feed(r, sa, a[:13])]
    out_b = [feed(r, sb, b[:20]), feed(r, sb, b[20:])]
    r.release([sb])
    out_a += [feed(r, sa, a[13:14]), feed(r, sa, a[14:])]
    assert rel_err(torch.cat(out_a), O.forward(om, a)) < TOL["float32"]
    assert rel_err(torch.cat(out_b), O.forward(om, b)) < TOL["float32"]


def test_latent_rows_of_128_on_the_tcgen05_pipeline():
    """bfloat16 portions with key rows of 128 numbers and pages of 128 tokens take the tcgen05 portion kernel with the
    whole row as the value (the columns past the values are dropped): against the mma.sync kernel on the same inputs
    (test option) and against the oracle, with portions cut off the 128-row tiles and a borrowing layer."""
    from compactor_vllm import _native as N
    from oracle import batasun as O

    cfg = model_cfg([(latent(4, 48, 64, 40, 64, 56, base=1e4), None), (latent(2, 32, 64, 24, 64, 32, base=1e4, kv_from=0), None)],
                    vocab=64, width=64)
    r = make_runner(cfg, "bfloat16", pages=6, page_size=128)
    toks = tokens(400, 64, 12)
    want = O.forward(oracle_model(r.model), toks)
    got = {}
    for name, option in (("tcgen05", 0), ("mma", 2)):
        N.set_test_option("bias_attn_fma", option)
        try:
            got[name] = [run_in_portions(r, toks, sizes).float().cpu() for sizes in ([400], [130, 127, 143], [257, 2, 141])]
        finally:
            N.set_test_option("bias_attn_fma", 0)
    for a, b in zip(got["tcgen05"], got["mma"]):
        assert close(a, want, "bfloat16")
        assert rel_err(a, b.double()) < 3e-2


# ------------------------------------------------------------------------------------------------------ other sizes
@pytest.mark.parametrize("layers", [
    [(mamba(1, 4, 1, 1, 1, 1), moe(4, 1.0, 1, 1, 4, 1.0))],                                   # everything 1
    [(mamba(6, 8, 16, 6, 5, 3), None), (mamba(2, 32, 64, 2, 2, 1), None)],                    # no attention at all
    [(latent(5, 8, 2, 4, 6, 4), None), (latent(3, 4, 2, 8, 6, 5, kv_from=0), None),
     (latent(1, 6, 2, 3, 6, 4, kv_from=0), moe(6, 9.0, 2, 2, 6, 0.1))],                       # no recurrence; two borrowers
    [(latent(2, 64, 64, 64, 160, 48), None)],                                                 # key rows of 224 numbers
    [(latent(2, 40, 24, 48, 104, 48, base=1e6), moe(24, 1.0, 16, 8, 0)), (mamba(8, 8, 130, 4, 4, 8), None)],
    [(mamba(2, 8, 260, 1, 7, 2), None), (mamba(1, 70, 18, 1, 16, 5), None)],    # 16 state channels per thread; 16 taps
])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_sizes(layers, dtype):
    from oracle import batasun as O

    r = make_runner(model_cfg(layers, vocab=53, width=40), dtype, pages=10, page_size=16)
    toks = tokens(45, 53, 8)
    want = O.forward(oracle_model(r.model), toks)
    assert close(run_in_portions(r, toks, [45]), want, dtype)
    assert close(run_in_portions(r, toks, [7, 1, 2, 20]), want, dtype)
    seq = new_seq()
    out = [feed(r, seq, toks[:30])] + [feed(r, seq, [t]) for t in toks[30:]]
    r.release([seq])
    assert close(torch.cat(out), want, dtype)


def random_config(seed):
    """A model drawn at random: 1-5 layers of either mixer in any order, borrowed latents, odd and even sizes."""
    import random

    rnd = random.Random(seed)
    pick = lambda *xs: rnd.choice(xs)
    layers, owners = [], []
    for i in range(rnd.randint(1, 5)):
        mlp = None if rnd.random() < 0.3 else moe(pick(5, 8, 12, 16), pick(0.4, 1.0, 6.0), pick(1, 2, 5, 9), 1, pick(0, 7, 16),
                                                  pick(0.5, 2.0))
        if mlp is not None:
            mlp["router"]["top"] = rnd.randint(1, min(4, mlp["router"]["experts"]))
        if rnd.random() < 0.5:
            heads, vdim = pick(1, 2, 3, 4, 6), pick(3, 8, 10, 16, 24)
            groups = pick(*[g for g in (1, 2, 3, 4, 6) if heads % g == 0])
            parts = pick(*[k for k in (1, 2, 3, 4) if (heads * vdim) % k == 0])
            layers.append((mamba(heads, vdim, pick(1, 5, 16, 24, 40, 70), groups, pick(1, 2, 3, 4, 6), parts), mlp))
        elif owners and rnd.random() < 0.4:
            j = pick(*owners)
            o = layers[j][0]["mixer"]
            layers.append((latent(pick(1, 2, 5), pick(4, 8, 14), o["rot_dim"], pick(4, 9, 16), o["kv_rank"], pick(3, 8, 20),
                                  base=o["rot"]["base"], kv_from=j), mlp))
        else:
            owners.append(i)
            layers.append((latent(pick(1, 2, 3, 4), pick(4, 8, 14, 32), pick(2, 4, 8, 16), pick(4, 9, 16, 32),
                                  pick(6, 16, 24, 48, 112), pick(3, 8, 20), base=pick(10.0, 1e4, 5e5),
                                  scale=pick(0.1, 0.3)), mlp))
    return model_cfg(layers, vocab=pick(37, 64, 101), width=pick(24, 40, 64), eps=pick(1e-6, 1e-5, 1e-3))


@pytest.mark.parametrize("seed", range(10))
def test_random_configurations(seed):
    """Whatever config.json says is what runs: whole prompts, portions with single tokens between them, decoding from
    the graph, two requests in one batch."""
    from oracle import batasun as O

    cfg = random_config(seed)
    r = make_runner(cfg, "float32", pages=16, page_size=16, eager=False)
    om = oracle_model(r.model)
    V = cfg["vocab"]
    a, b = tokens(50, V, 100 + seed), tokens(21, V, 200 + seed)
    wa, wb = O.forward(om, a), O.forward(om, b)
    assert rel_err(run_in_portions(r, a, [50]), wa) < TOL["float32"]
    assert rel_err(run_in_portions(r, a, [9, 1, 1, 17, 2]), wa) < TOL["float32"]
    sa, sb = new_seq(), new_seq()
    out_a, out_b = [], []
    for lo_a, hi_a, lo_b, hi_b in ((0, 30, 0, 1), (30, 31, 1, 2), (31, 50, 2, 21)):
        sa.prompt_token_ids.extend(a[lo_a:hi_a])
        sb.prompt_token_ids.extend(b[lo_b:hi_b])
        na, nb = hi_a - lo_a, hi_b - lo_b
        logits = r.run_step([(sa, a[lo_a:hi_a]), (sb, b[lo_b:hi_b])], rows=list(range(na + nb)))
        out_a.append(logits[:na])
        out_b.append(logits[na:])
    r.release([sa, sb])
    assert rel_err(torch.cat(out_a), wa) < TOL["float32"]
    assert rel_err(torch.cat(out_b), wb) < TOL["float32"]


def test_config_refuses_a_bad_borrowed_latent():
    from compactor_vllm.config.model_config import BatasunConfig

    with pytest.raises(ValueError):
        BatasunConfig.from_json(model_cfg([(latent(kv_from=0), None)]))
    with pytest.raises(ValueError):
        BatasunConfig.from_json(model_cfg([(latent(), None), (latent(kv_rank=24, kv_from=0), None)]))
    with pytest.raises(ValueError):
        BatasunConfig.from_json(model_cfg([(mamba(), None), (latent(kv_from=0), None)]))


# ------------------------------------------------------------------------------ generation through the entry point
def test_greedy_generation_through_llm_generate():
    """`LLM.generate` with the step scheduler: prompts in portions of at most 16 tokens beside decoding requests, five
    requests on three slots.  Teacher forcing against the oracle: every generated token must be the oracle's argmax
    unless the oracle's two best logits are closer than the engine's rounding."""
    from compactor_vllm import LLM
    from compactor_vllm.api_types import SamplingParams
    from compactor_vllm.config.engine_config import LLMConfig
    from compactor_vllm.config.model_config import BatasunConfig
    from oracle import batasun as O

    hf = BatasunConfig.from_json(config_a())
    cfg = LLMConfig(model="synthetic", hf_config=hf, dtype="float32", max_num_seqs=3, kvcache_page_size=16,
                    max_model_len=160)
    llm = LLM(cfg, num_pages=14, device_allocator=False, max_batched_tokens=16)
    om = oracle_model(llm.model_runner.model)
    prompts = [tokens(n, 89, 30 + i) for i, n in enumerate((40, 3, 25, 1, 18))]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=12))
    assert llm.model_runner.kv.num_free_batches == 3
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        logits = O.forward(om, p + o[:-1])[len(p) - 1:]
        for k, tok in enumerate(o):
            best = torch.topk(logits[k], 2)
            assert tok == int(best.indices[0]) or float(best.values[0] - best.values[1]) < 1e-3, (k, tok)
