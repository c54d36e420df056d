"""Oracle: the Movolorn decoder in plain fp32 torch on the CPU, one function per mechanism.

TEST INFRASTRUCTURE ONLY: nothing under compactor-vllm_b200/ imports this module and it imports
nothing from there.  Every function works on whole sequences (no cache, no paging, no batching),
token by token or with dense [T, T] masks, so that what the engine computes through its paged
cache and scheduler can be compared with it.

Notation: T tokens, W model width, H query heads, G key/value heads, D query/key size, Dv value size,
E routed experts of which the last I are identity experts.

A model is a dict:
  {"embed": [V, W], "embed_scale": float, "eps": float, "final_norm": [W], "head": [V, W],
   "layers": [layer, ...], "loop": (start, stop, times)}
and a layer is
  {"norm1", "norm1b", "norm2", "norm2b": [W],
   "attn": {"q","k","v","o","q_norm","k_norm", "heads","kv_heads","dim","vdim","scale","chunk"},
   "mlp": None | {"kind": "dense", "gate","up","down"}
              | {"kind": "moe", "experts": [{"gate","up","down"}...], "router": [E, W], "correction": [E] | None,
                 "top", "groups", "keep", "identity", "shared": None | {"gate","up","down"}}}
"""
from __future__ import annotations

import math

import torch


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w over the last dimension."""
    x = x.float()
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w.float()


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def head_slopes(H: int) -> torch.Tensor:
    """slope of head h = 2 ** (-8 (h + 1) / H)."""
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=torch.float64)


def visible(i: int, j: int, chunk: int | None) -> bool:
    """Key j is seen from query i: causal, and in the same chunk counted from position 0."""
    if j > i:
        return False
    return chunk is None or i // chunk == j // chunk


def sink_softmax_row(s: torch.Tensor) -> torch.Tensor:
    """p_j = exp(s_j) / (1 + sum_j exp(s_j)): one extra term of score 0 and no value in the denominator.
    Done against max(s, 0) so that it cannot overflow."""
    m = max(float(s.max()) if s.numel() else 0.0, 0.0)
    e = torch.exp(s - m)
    return e / (math.exp(-m) + e.sum())


def attention_mixer(h: torch.Tensor, a: dict, eps: float) -> torch.Tensor:
    """h [T, W] -> [T, W].  Grouped heads, per-head RMS norm of q and k, no rotation, linear distance bias,
    chunk mask, softmax with a sink, output projection.  Row by row, in float64 inside the softmax."""
    T = h.shape[0]
    H, G, D, Dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
    h = h.float()
    q = (h @ a["q"].float().T).view(T, H, D)
    k = (h @ a["k"].float().T).view(T, G, D)
    v = (h @ a["v"].float().T).view(T, G, Dv)
    q = rms_norm(q, a["q_norm"], eps)
    k = rms_norm(k, a["k_norm"], eps)
    slopes = head_slopes(H)
    out = torch.zeros(T, H, Dv, dtype=torch.float64)
    per = H // G
    for hd in range(H):
        g = hd // per
        for i in range(T):
            js = [j for j in range(i + 1) if visible(i, j, a["chunk"])]
            kk = k[js, g].double()
            s = (kk @ q[i, hd].double()) * a["scale"]
            s = s - slopes[hd] * (i - torch.tensor(js, dtype=torch.float64))
            p = sink_softmax_row(s)
            out[i, hd] = p @ v[js, g].double()
    return out.float().reshape(T, H * Dv) @ a["o"].float().T


def gated_ff(h: torch.Tensor, w: dict, act) -> torch.Tensor:
    """down(act(gate h) * (up h))."""
    h = h.float()
    return (act(h @ w["gate"].float().T) * (h @ w["up"].float().T)) @ w["down"].float().T


def route(h: torch.Tensor, m: dict):
    """Router of one token batch: returns (chosen [T, top] expert indices, weights [T, top]).

    scores = softmax of the router logits over all E outputs; the choice is made on scores + correction,
    restricted to the `keep` groups (of `groups` equal runs of neighbouring experts) whose largest choice
    score is highest; the weights are the plain scores of the chosen experts, not renormalised."""
    z = h.float() @ m["router"].float().T
    s = torch.softmax(z, dim=-1)
    c = s if m.get("correction") is None else s + m["correction"].float()
    T, E = c.shape
    n_groups, keep, top = m["groups"], m["keep"], m["top"]
    chosen = torch.zeros(T, top, dtype=torch.long)
    weights = torch.zeros(T, top)
    size = E // n_groups
    for t in range(T):
        group_best = [max(float(c[t, e]) for e in range(g * size, (g + 1) * size)) for g in range(n_groups)]
        order = sorted(range(n_groups), key=lambda g: (-group_best[g], g))
        allowed = set(order[:keep])
        cand = [e for e in range(E) if e // size in allowed]
        cand.sort(key=lambda e: (-float(c[t, e]), e))
        for r, e in enumerate(cand[:top]):
            chosen[t, r] = e
            weights[t, r] = s[t, e]
    return chosen, weights


def moe_ff(h: torch.Tensor, m: dict) -> torch.Tensor:
    """Weighted sum of the chosen experts (silu-gated; the last `identity` router outputs return their input)
    plus the shared expert if there is one."""
    h = h.float()
    chosen, weights = route(h, m)
    E = m["router"].shape[0]
    n_real = E - m["identity"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t].tolist(), weights[t].tolist()):
            if e >= n_real:
                out[t] += w * h[t]
            else:
                out[t] += w * gated_ff(h[t:t + 1], m["experts"][e], silu)[0]
    if m.get("shared") is not None:
        out = out + gated_ff(h, m["shared"], silu)
    return out


def feed_forward(h: torch.Tensor, m: dict) -> torch.Tensor:
    if m["kind"] == "dense":
        return gated_ff(h, m, gelu_tanh)
    return moe_ff(h, m)


def layer_forward(x: torch.Tensor, layer: dict, eps: float) -> torch.Tensor:
    """x + norm1b(mixer(norm1 x)), then x + norm2b(ff(norm2 x))."""
    x = x + rms_norm(attention_mixer(rms_norm(x, layer["norm1"], eps), layer["attn"], eps), layer["norm1b"], eps)
    if layer.get("mlp") is not None:
        x = x + rms_norm(feed_forward(rms_norm(x, layer["norm2"], eps), layer["mlp"]), layer["norm2b"], eps)
    return x


def layer_runs(n_layers: int, loop) -> list[int]:
    """Layer index of every layer run: layers start..stop-1 repeated `times` times in a row."""
    if loop is None:
        return list(range(n_layers))
    start, stop, times = loop
    return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n_layers))


def forward(model: dict, tokens, collect: list | None = None) -> torch.Tensor:
    """tokens (list of ints) -> logits [T, V]; `collect` receives the residual stream after every layer run."""
    x = model["embed"].float()[torch.tensor(tokens, dtype=torch.long)] * model["embed_scale"]
    for li in layer_runs(len(model["layers"]), model.get("loop")):
        x = layer_forward(x, model["layers"][li], model["eps"])
        if collect is not None:
            collect.append(x.clone())
    return rms_norm(x, model["final_norm"], model["eps"]) @ model["head"].float().T
