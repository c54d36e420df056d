"""Oracle: the Batasun decoder in plain float64 torch on the CPU, one function per mechanism.

TEST INFRASTRUCTURE ONLY: nothing under compactor-vllm_b200/ imports this module and it imports nothing from
there.  Every function works on one whole sequence (no cache, no state slots, no batching): attention with dense
row-by-row loops, the recurrence token by token.

A model is a dict
  {"embed": [V, W], "embed_norm": [W], "eps": float, "final_norm": [W], "head": [V, W], "layers": [layer, ...]}
a layer is
  {"norm1": [W], "norm2": [W] | None, "mixer": mixer, "mlp": None | mlp}
a mixer is one of
  {"type": "latent_attention", "heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "rot_base",
   "kv_from": None | int, "dq", "dq_norm", "uq", "dkv" (absent with kv_from), "dkv_norm" (same), "uk", "uv", "g", "o"}
  {"type": "mamba2", "heads", "vdim", "state", "groups", "conv", "norm_groups",
   "in", "conv_w", "conv_b", "dt_bias", "A_log", "D", "norm", "o"}
and an mlp is
  {"experts": [{"gate","up","down"}...], "limit", "router", "router_b", "top",
   "shared": None | {"gate","up","down","sg","limit"}}
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    x = x.to(F64)
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def zero_centred_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose gain is stored around zero: unit(x) * (1 + w)."""
    return rms_unit(x, eps) * (1.0 + w.to(F64))


def plain_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w.to(F64)


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotate_half(x: torch.Tensor, pos: torch.Tensor, base: float) -> torch.Tensor:
    """x [T, ..., R] at positions pos [T]: element i pairs with i + R/2; angle = pos * base ** (-2 i / R)."""
    R = x.shape[-1]
    half = R // 2
    f = torch.tensor([base ** (-2.0 * i / R) for i in range(half)], dtype=F64)
    ang = pos.to(F64)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    u, v = x[..., :half].to(F64), x[..., half:].to(F64)
    return torch.cat([u * c - v * s, v * c + u * s], dim=-1)


def latent_kv(h: torch.Tensor, m: dict, eps: float):
    """What a latent-attention layer caches: (c [T, kv_rank] normed, shared rotated key part [T, rot_dim])."""
    T = h.shape[0]
    r = m["kv_rank"]
    d = h.to(F64) @ m["dkv"].to(F64).T
    c = plain_norm(d[:, :r], m["dkv_norm"], eps)
    kr = rotate_half(d[:, r:], torch.arange(T), m["rot_base"])
    return c, kr


def latent_attention(h: torch.Tensor, m: dict, eps: float, c: torch.Tensor, kr: torch.Tensor) -> torch.Tensor:
    """h [T, W] -> [T, W] with the latent c and the rotated shared key part given (the layer's own or another's)."""
    T = h.shape[0]
    H, D, R, Dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    h = h.to(F64)
    cq = plain_norm(h @ m["dq"].to(F64).T, m["dq_norm"], eps)
    q = (cq @ m["uq"].to(F64).T).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_half(q[..., D:], torch.arange(T), m["rot_base"])
    k_plain = (c @ m["uk"].to(F64).T).view(T, H, D)
    v = (c @ m["uv"].to(F64).T).view(T, H, Dv)
    out = torch.zeros(T, H, Dv, dtype=F64)
    for i in range(T):
        for hd in range(H):
            s = (k_plain[: i + 1, hd] @ q_plain[i, hd] + kr[: i + 1] @ q_rot[i, hd]) * m["scale"]
            p = torch.exp(s - s.max())
            p = p / p.sum()
            out[i, hd] = p @ v[: i + 1, hd]
    gate = sigmoid(h @ m["g"].to(F64).T)
    return (out.reshape(T, H * Dv) * gate) @ m["o"].to(F64).T


def causal_conv(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """x [T, C], w [C, taps] (last column = the current token), zeros before the start; + bias."""
    T, C = x.shape
    taps = w.shape[1]
    xp = torch.cat([torch.zeros(taps - 1, C, dtype=F64), x.to(F64)], 0)
    out = torch.zeros(T, C, dtype=F64)
    for k in range(taps):
        out += xp[k:k + T] * w[:, k].to(F64)[None, :]
    return out + b.to(F64)[None, :]


def mamba2(h: torch.Tensor, m: dict, eps: float) -> torch.Tensor:
    """h [T, W] -> [T, W]: the state-space recurrence token by token from a zero state."""
    T = h.shape[0]
    Hh, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hh * P
    proj = h.to(F64) @ m["in"].to(F64).T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, m["conv_w"], m["conv_b"]))
    x = xbc[:, :inner].view(T, Hh, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + m["dt_bias"].to(F64)[None, :])
    a = torch.exp(m["A_log"].to(F64))
    y = torch.zeros(T, Hh, P, dtype=F64)
    per = Hh // G
    for hd in range(Hh):
        g = hd // per
        S = torch.zeros(N, P, dtype=F64)
        for t in range(T):
            S = math.exp(-float(a[hd]) * float(dt[t, hd])) * S + float(dt[t, hd]) * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + float(m["D"][hd]) * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_unit(y.view(T, parts, inner // parts), eps).reshape(T, inner) * m["norm"].to(F64)
    return y @ m["o"].to(F64).T


def clamped_expert(h: torch.Tensor, e: dict, limit: float) -> torch.Tensor:
    """g = min(gate h, limit), u = clamp(up h, +-limit); down (g sigmoid(1.702 g) (u + 1))."""
    h = h.to(F64)
    g = torch.clamp(h @ e["gate"].to(F64).T, max=limit)
    u = torch.clamp(h @ e["up"].to(F64).T, min=-limit, max=limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ e["down"].to(F64).T


def route_top_logits(z: torch.Tensor, top: int):
    """The `top` largest logits of a token (lowest index first among equals) and the softmax over just those."""
    order = sorted(range(z.numel()), key=lambda e: (-float(z[e]), e))[:top]
    zz = torch.stack([z[e] for e in order])
    p = torch.exp(zz - zz.max())
    return order, p / p.sum()


def moe(h: torch.Tensor, m: dict) -> torch.Tensor:
    T = h.shape[0]
    h = h.to(F64)
    logits = h @ m["router"].to(F64).T + m["router_b"].to(F64)[None, :]
    out = torch.zeros(T, h.shape[1], dtype=F64)
    for t in range(T):
        idx, w = route_top_logits(logits[t], m["top"])
        for e, we in zip(idx, w):
            out[t] += we * clamped_expert(h[t:t + 1], m["experts"][e], m["limit"])[0]
    sh = m.get("shared")
    if sh is not None:
        gate = sigmoid(h @ sh["sg"].to(F64).T)          # [T, 1]
        out += gate * clamped_expert(h, sh, sh["limit"])
    return out


def forward(model: dict, tokens, residuals: list | None = None) -> torch.Tensor:
    """Logits [T, V] of every position of one sequence; `residuals` collects the stream after every layer."""
    eps = model["eps"]
    x = zero_centred_norm(model["embed"].to(F64)[torch.tensor(list(tokens))], model["embed_norm"], eps)
    cached = {}
    for i, layer in enumerate(model["layers"]):
        m = layer["mixer"]
        if m["type"] == "latent_attention":
            if m.get("kv_from") is None:
                cached[i] = latent_kv(x, m, eps)
                c, kr = cached[i]
            else:
                c, kr = cached[m["kv_from"]]
            y = latent_attention(x, m, eps, c, kr)
        elif m["type"] == "mamba2":
            y = mamba2(x, m, eps)
        else:
            raise ValueError(m["type"])
        x = x + zero_centred_norm(y, layer["norm1"], eps)
        if layer["mlp"] is not None:
            x = x + zero_centred_norm(moe(x, layer["mlp"]), layer["norm2"], eps)
        if residuals is not None:
            residuals.append(x.clone())
    return zero_centred_norm(x, model["final_norm"], eps) @ model["head"].to(F64).T


def from_checkpoint(cfg: dict, tensors: dict) -> dict:
    """config.json (as a dict) + named tensors -> the oracle's model dict."""
    t = {k: v.to(F64) if v.is_floating_point() else v for k, v in tensors.items()}
    layers = []
    for i, lc in enumerate(cfg["layers"]):
        p = f"l{i}."
        mc = lc["mixer"]
        if lc["type"] == "latent_attention":
            m = {"type": "latent_attention", "heads": mc["heads"], "dim": mc["dim"], "rot_dim": mc["rot_dim"],
                 "vdim": mc["vdim"], "kv_rank": mc["kv_rank"], "q_rank": mc["q_rank"], "scale": mc["scale"],
                 "rot_base": mc["rot"]["base"], "kv_from": mc.get("kv_from"),
                 "dq": t[p + "mix.dq"], "dq_norm": t[p + "mix.dq.norm"], "uq": t[p + "mix.uq"], "uk": t[p + "mix.uk"],
                 "uv": t[p + "mix.uv"], "g": t[p + "mix.g"], "o": t[p + "mix.o"]}
            if m["kv_from"] is None:
                m["dkv"], m["dkv_norm"] = t[p + "mix.dkv"], t[p + "mix.dkv.norm"]
        else:
            m = {"type": "mamba2", "heads": mc["heads"], "vdim": mc["vdim"], "state": mc["state"], "groups": mc["groups"],
                 "conv": mc["conv"], "norm_groups": mc["norm_groups"], "in": t[p + "mix.in"], "conv_w": t[p + "mix.conv"],
                 "conv_b": t[p + "mix.conv.b"], "dt_bias": t[p + "mix.dt_bias"], "A_log": t[p + "mix.A_log"],
                 "D": t[p + "mix.D"], "norm": t[p + "mix.norm"], "o": t[p + "mix.o"]}
        mlp = None
        fc = lc.get("mlp")
        if fc is not None:
            ex = [{"gate": t[p + f"mlp.e{e}.gate"], "up": t[p + f"mlp.e{e}.up"], "down": t[p + f"mlp.e{e}.down"]}
                  for e in range(fc["router"]["experts"])]
            sh = None
            if fc.get("shared"):
                sh = {"gate": t[p + "mlp.shared.gate"], "up": t[p + "mlp.shared.up"], "down": t[p + "mlp.shared.down"],
                      "sg": t[p + "mlp.shared.sg"], "limit": fc["shared"]["limit"]}
            mlp = {"experts": ex, "limit": fc["expert"]["limit"], "router": t[p + "mlp.router"],
                   "router_b": t[p + "mlp.router.b"], "top": fc["router"]["top"], "shared": sh}
        layers.append({"norm1": t[p + "norm1"], "norm2": t.get(p + "norm2") if fc is not None else None,
                       "mixer": m, "mlp": mlp})
    return {"embed": t["embed"], "embed_norm": t["embed.norm"], "eps": cfg["norm"]["eps"],
            "final_norm": t["final.norm"], "head": t["head"], "layers": layers}
