"""Host-side parts of the Batasun path (no GPU): configuration reader, and the oracle's own invariants (the slow
reference must agree with itself where two formulations of one mechanism exist)."""
import json
import math

import pytest
import torch

from compactor_vllm.config.model_config import BatasunConfig, load_model_config
from compactor_vllm.layers.latent_attention import rotation_frequencies
from oracle import batasun as O


def small_config():
    return {"architecture": "Batasun", "vocab": 31, "width": 12, "norm": {"eps": 1e-5},
            "layers": [
                {"type": "latent_attention",
                 "mixer": {"heads": 2, "dim": 6, "rot_dim": 4, "vdim": 5, "kv_rank": 7, "q_rank": 3, "scale": 0.3,
                           "rot": {"base": 50.0, "dims": 4}},
                 "mlp": {"kind": "moe", "expert": {"ff": 7, "limit": 2.5}, "shared": {"ff": 9, "limit": 0.5},
                         "router": {"experts": 5, "top": 2}}},
                {"type": "mamba2", "mixer": {"heads": 4, "vdim": 3, "state": 5, "groups": 2, "conv": 3, "norm_groups": 2},
                 "mlp": None},
                {"type": "latent_attention",
                 "mixer": {"heads": 3, "dim": 2, "rot_dim": 4, "vdim": 2, "kv_rank": 7, "q_rank": 4, "scale": 0.5,
                           "rot": {"base": 50.0, "dims": 4}, "kv_from": 0},
                 "mlp": {"kind": "moe", "expert": {"ff": 4, "limit": 1.0}, "router": {"experts": 2, "top": 1}}}]}


def test_config_reader_fields():
    cfg = BatasunConfig.from_json(small_config())
    assert (cfg.vocab_size, cfg.hidden_size, cfg.rms_norm_eps, cfg.model_type) == (31, 12, 1e-5, "batasun")
    a = cfg.layers[0].mixer
    assert (a.heads, a.dim, a.rot_dim, a.vdim, a.kv_rank, a.q_rank, a.scale, a.rot_base, a.kv_from) == \
        (2, 6, 4, 5, 7, 3, 0.3, 50.0, None)
    m = cfg.layers[0].mlp
    assert (m.ff, m.limit, m.experts, m.top, m.shared_ff, m.shared_limit) == (7, 2.5, 5, 2, 9, 0.5)
    s = cfg.layers[1].mixer
    assert (s.heads, s.vdim, s.state, s.groups, s.conv, s.norm_groups, s.inner, s.conv_channels) == (4, 3, 5, 2, 3, 2, 12, 32)
    assert cfg.layers[1].mlp is None
    assert cfg.layers[2].mixer.kv_from == 0 and cfg.layers[2].mlp.shared_ff == 0
    assert cfg.num_hidden_layers == 3 and cfg.num_key_value_heads == 1 and cfg.head_dim == 11


def test_config_reader_from_a_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(small_config()))
    cfg = load_model_config(str(tmp_path))
    assert isinstance(cfg, BatasunConfig) and len(cfg.layers) == 3


def test_config_reader_refuses_what_it_does_not_know():
    bad = small_config()
    bad["layers"][1]["type"] = "recurrent"
    with pytest.raises(ValueError):
        BatasunConfig.from_json(bad)
    bad = small_config()
    bad["layers"][2]["mixer"]["kv_from"] = 1          # a state-space layer has no latent to lend
    with pytest.raises(ValueError):
        BatasunConfig.from_json(bad)
    bad = small_config()
    bad["layers"][0]["mixer"]["rot"]["dims"] = 2      # the rotated part is rotated whole
    with pytest.raises(ValueError):
        BatasunConfig.from_json(bad)
    bad = small_config()
    bad["layers"][1]["mixer"]["groups"] = 3
    with pytest.raises(ValueError):
        BatasunConfig.from_json(bad)


def test_rotation_frequencies_and_pairing():
    f = rotation_frequencies(8, 10000.0)
    assert f.dtype == torch.float64 and f.tolist() == [10000.0 ** (-2.0 * i / 8) for i in range(4)]
    x = torch.arange(1.0, 9.0).view(1, 8).repeat(3, 1)
    y = O.rotate_half(x, torch.tensor([0, 1, 5]), 10000.0)
    assert torch.equal(y[0], x[0].double())                                  # position 0: no rotation
    a = 5 * 10000.0 ** (-2.0 / 8)                                            # element 1 pairs with element 5
    assert abs(float(y[2, 1]) - (2 * math.cos(a) - 6 * math.sin(a))) < 1e-12
    assert abs(float(y[2, 5]) - (6 * math.cos(a) + 2 * math.sin(a))) < 1e-12
    # a rotation keeps the dot product of two vectors at equal distance
    g = torch.Generator().manual_seed(0)
    u, v = torch.randn(1, 8, generator=g), torch.randn(1, 8, generator=g)
    d1 = (O.rotate_half(u, torch.tensor([7]), 30.0) * O.rotate_half(v, torch.tensor([3]), 30.0)).sum()
    d2 = (O.rotate_half(u, torch.tensor([104]), 30.0) * O.rotate_half(v, torch.tensor([100]), 30.0)).sum()
    assert abs(float(d1 - d2)) < 1e-9


def test_oracle_recurrence_equals_its_unrolled_sum():
    """y_t = sum_{s<=t} (prod_{s<r<=t} a_r) dt_s (C_t . B_s) x_s + D x_t, against the oracle's token-by-token state."""
    g = torch.Generator().manual_seed(3)
    W, Hh, P, N, G, taps = 10, 2, 3, 4, 1, 3
    inner = Hh * P
    m = {"type": "mamba2", "heads": Hh, "vdim": P, "state": N, "groups": G, "conv": taps, "norm_groups": 1,
         "in": torch.randn(2 * inner + 2 * G * N + Hh, W, generator=g) * 0.4,
         "conv_w": torch.randn(inner + 2 * G * N, taps, generator=g) * 0.5, "conv_b": torch.randn(inner + 2 * G * N, generator=g) * 0.1,
         "dt_bias": torch.randn(Hh, generator=g) * 0.3, "A_log": torch.randn(Hh, generator=g) * 0.3,
         "D": torch.randn(Hh, generator=g), "norm": torch.ones(inner), "o": torch.eye(inner, dtype=torch.float64)[:, :inner]}
    m["o"] = torch.eye(inner)
    h = torch.randn(9, W, generator=g)
    got = O.mamba2(h, m, 1e-5)                        # [T, inner] since o is the identity
    T = h.shape[0]
    proj = h.double() @ m["in"].double().T
    z, xbc, dt = proj[:, :inner], proj[:, inner:inner + inner + 2 * N], proj[:, -Hh:]
    xbc = O.silu(O.causal_conv(xbc, m["conv_w"], m["conv_b"]))
    x, B, C = xbc[:, :inner].view(T, Hh, P), xbc[:, inner:inner + N], xbc[:, inner + N:]
    dt = O.softplus(dt + m["dt_bias"].double())
    a = torch.exp(-torch.exp(m["A_log"].double()) * dt)
    y = torch.zeros(T, Hh, P, dtype=torch.float64)
    for t in range(T):
        for s in range(t + 1):
            decay = torch.prod(a[s + 1:t + 1], dim=0)                  # [Hh]
            y[t] += (decay * dt[s] * (C[t] @ B[s]))[:, None] * x[s]
        y[t] += m["D"].double()[:, None] * x[t]
    v = y.reshape(T, inner) * O.silu(z)
    want = O.rms_unit(v, 1e-5)
    assert torch.allclose(got, want, rtol=1e-9, atol=1e-9)


def test_oracle_latent_attention_equals_attention_in_the_latent_space():
    """Scores and outputs computed from per-head keys and values (the oracle) equal the ones computed against the cached
    latent with W_uk folded into the query and W_uv applied after the weighted sum."""
    g = torch.Generator().manual_seed(4)
    W, H, D, R, Dv, r, qr = 10, 2, 4, 2, 3, 5, 3
    m = {"type": "latent_attention", "heads": H, "dim": D, "rot_dim": R, "vdim": Dv, "kv_rank": r, "q_rank": qr,
         "scale": 0.4, "rot_base": 9.0, "kv_from": None,
         "dq": torch.randn(qr, W, generator=g), "dq_norm": torch.rand(qr, generator=g) + 0.5,
         "uq": torch.randn(H * (D + R), qr, generator=g), "dkv": torch.randn(r + R, W, generator=g),
         "dkv_norm": torch.rand(r, generator=g) + 0.5, "uk": torch.randn(H * D, r, generator=g),
         "uv": torch.randn(H * Dv, r, generator=g), "g": torch.randn(H * Dv, W, generator=g),
         "o": torch.eye(H * Dv)}
    h = torch.randn(7, W, generator=g)
    c, kr = O.latent_kv(h, m, 1e-5)
    got = O.latent_attention(h, m, 1e-5, c, kr)
    T = 7
    cq = O.plain_norm(h.double() @ m["dq"].double().T, m["dq_norm"], 1e-5)
    q = (cq @ m["uq"].double().T).view(T, H, D + R)
    q_rot = O.rotate_half(q[..., D:], torch.arange(T), 9.0)
    uk, uv = m["uk"].double().view(H, D, r), m["uv"].double().view(H, Dv, r)
    out = torch.zeros(T, H, Dv, dtype=torch.float64)
    for i in range(T):
        for hd in range(H):
            q_abs = q[i, hd, :D] @ uk[hd]
            s = (c[:i + 1] @ q_abs + kr[:i + 1] @ q_rot[i, hd]) * 0.4
            out[i, hd] = uv[hd] @ (torch.softmax(s, 0) @ c[:i + 1])
    want = out.reshape(T, H * Dv) * O.sigmoid(h.double() @ m["g"].double().T)
    assert torch.allclose(got, want, rtol=1e-9, atol=1e-9)


def test_oracle_router_ties_and_weights():
    idx, w = O.route_top_logits(torch.tensor([0.5, 2.0, 2.0, -1.0], dtype=torch.float64), 3)
    assert idx == [1, 2, 0]
    e = torch.exp(torch.tensor([0.0, 0.0, -1.5], dtype=torch.float64))
    assert torch.allclose(w, e / e.sum())
