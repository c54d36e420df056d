"""Movolorn: a decoder whose layers are  x += norm_b(mixer(norm(x))),  x += norm_b(ff(norm(x)))  on a 32-bit
residual stream, with a loop that runs a span of layers several times with the same weights.

Built from the engine's blocks:
  * mixer "attention" = `BiasedChunkAttention` (layers/attention.py): grouped heads, per-head q/k RMS norm, no
    rotation, a linear distance bias with slopes 2 ** (-8 (h + 1) / H), a chunk mask and a softmax sink;
  * feed-forward = `GatedMLP` with the tanh gelu, or `RoutedExperts` (layers/moe.py);
  * every norm is one half of a `sandwich_norm` launch (layers/layernorm.py): the post-norm of a sublayer, the residual
    sum and the pre-norm of the next sublayer — also across layer borders and into the final norm.
Each layer RUN has a cache layer of its own (`cache_specs`), so a looped layer owns one per pass.
Weights: `load_weights` takes the checkpoint's tensors (`embed`, `l<i>.norm1|norm1b|norm2|norm2b`,
`l<i>.mix.q|k|v|o|q.norm|k.norm`, `l<i>.mlp.gate|up|down`, `l<i>.mlp.e<j>.*`, `l<i>.mlp.router|correction`,
`l<i>.mlp.shared.*`, `final.norm`, `head`); `init_synthetic_weights` draws random ones.
"""
from __future__ import annotations

import sys
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F
from torch import nn

from compactor_vllm.config.model_config import FeedForwardConfig, MovolornConfig
from compactor_vllm.layers.attention import BiasedChunkAttention, linear_bias_slopes
from compactor_vllm.layers.layernorm import NormWeight, sandwich_norm
from compactor_vllm.layers.moe import ACT_GELU_TANH, ACT_SILU, GatedMLP, RoutedExperts
from compactor_vllm.utils.context import get_context


class _Pending:
    """A sublayer's output that still has to be post-normed and added into the residual stream."""
    __slots__ = ("branch", "weight")

    def __init__(self, branch: torch.Tensor, weight: torch.Tensor):
        self.branch, self.weight = branch, weight


def _advance(x: torch.Tensor, pending: Optional[_Pending], pre_weight: Optional[torch.Tensor], eps: float, dtype):
    """x += post_norm(pending) and, if asked, return pre_norm(x): one launch."""
    if pending is None and pre_weight is None:
        return None
    return sandwich_norm(x, branch=None if pending is None else pending.branch,
                         post_weight=None if pending is None else pending.weight,
                         pre_weight=pre_weight, eps=eps, out_dtype=dtype)


def make_feed_forward(width: int, m: Optional[FeedForwardConfig], dtype) -> Optional[nn.Module]:
    if m is None:
        return None
    if m.kind == "dense":
        return GatedMLP(width, m.ff, ACT_GELU_TANH)
    return RoutedExperts(width, m.ff, m.experts, m.identity, m.top, m.groups, m.keep, m.shared_ff, ACT_SILU, dtype)


class MovolornAttentionMixer(nn.Module):
    def __init__(self, width: int, a, eps: float):
        super().__init__()
        self.attn = BiasedChunkAttention(a.heads, a.kv_heads, a.dim, a.vdim, a.scale, slopes=linear_bias_slopes(a.heads),
                                         chunk=a.chunk, sink=True, qk_norm=True, eps=eps)
        self.qkv_proj = nn.Linear(width, self.attn.qkv_width, bias=False)
        self.o_proj = nn.Linear(a.heads * a.vdim, width, bias=False)

    def forward(self, h: torch.Tensor, attn: BiasedChunkAttention) -> torch.Tensor:
        return self.o_proj(attn(self.qkv_proj(h)))


class MovolornLayer(nn.Module):
    def __init__(self, cfg: MovolornConfig, index: int, dtype):
        super().__init__()
        lc = cfg.layers[index]
        W = cfg.hidden_size
        self.eps = cfg.rms_norm_eps
        self.mixer = MovolornAttentionMixer(W, lc.mixer, self.eps)
        self.mlp = make_feed_forward(W, lc.mlp, dtype)
        self.norm1, self.norm1b = NormWeight(W), NormWeight(W)
        if self.mlp is not None:
            self.norm2, self.norm2b = NormWeight(W), NormWeight(W)

    def forward(self, x: torch.Tensor, pending: Optional[_Pending], attn: BiasedChunkAttention, dtype) -> _Pending:
        h = _advance(x, pending, self.norm1.weight, self.eps, dtype)
        pending = _Pending(self.mixer(h, attn), self.norm1b.weight)
        if self.mlp is not None:
            h = _advance(x, pending, self.norm2.weight, self.eps, dtype)
            pending = _Pending(self.mlp(h), self.norm2b.weight)
        return pending


class MovolornForCausalLM(nn.Module):
    mixed_steps = True        # the runner may hand it portions of prompts beside single tokens in one step

    def __init__(self, cfg: MovolornConfig):
        super().__init__()
        self.config = cfg
        dtype = torch.get_default_dtype()
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList([MovolornLayer(cfg, i, dtype) for i in range(len(cfg.layers))])
        self.norm = NormWeight(cfg.hidden_size)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        self.layer_runs: List[int] = cfg.layer_runs
        # one attention object per layer RUN: same kernels and constants as the layer's, its own cache views
        self.run_attn = nn.ModuleList()
        seen = set()
        for li in self.layer_runs:
            base = self.layers[li].mixer.attn
            if li not in seen:
                seen.add(li)
                self.run_attn.append(base)
            else:
                a = cfg.layers[li].mixer
                twin = BiasedChunkAttention(a.heads, a.kv_heads, a.dim, a.vdim, a.scale, slopes=base.slopes,
                                            chunk=a.chunk, sink=True, qk_norm=False, eps=cfg.rms_norm_eps)
                twin.q_norm_weight, twin.k_norm_weight = base.q_norm_weight, base.k_norm_weight  # shared parameters
                self.run_attn.append(twin)
        self.debug_residuals: Optional[list] = None   # a list collects the residual stream after every layer run

    def cache_specs(self):
        """One entry per cache layer (= layer run): (attention module, kv heads, key size, value size)."""
        return [(a, a.num_kv_heads, a.head_dim, a.v_head_dim) for a in self.run_attn]

    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        cfg = self.config
        dtype = self.lm_head.weight.dtype
        x = (F.embedding(input_ids, self.embed_tokens.weight).float() * cfg.embedding_scale).contiguous()
        pending = None
        for run, li in enumerate(self.layer_runs):
            pending = self.layers[li](x, pending, self.run_attn[run], dtype)
            if self.debug_residuals is not None:
                _advance(x, pending, None, cfg.rms_norm_eps, dtype)
                pending = None
                self.debug_residuals.append(x.clone())
        return _advance(x, pending, self.norm.weight, cfg.rms_norm_eps, dtype)

    def compute_logits(self, hidden_states: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Logits of the given rows of the step (None: the last token of every sequence of the step)."""
        if rows is None:
            rows = get_context().cu_seqlens_q[1:].long() - 1
        return self.lm_head(hidden_states.index_select(0, rows))

    # ---- weights ---------------------------------------------------------------------------------------
    @torch.no_grad()
    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        used = set()

        def get(name):
            if name not in tensors:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            used.add(name)
            return tensors[name]

        def put(param, *names):
            src = torch.cat([get(n) for n in names], dim=0) if len(names) > 1 else get(names[0])
            if tuple(src.shape) != tuple(param.shape):
                raise ValueError(f"{names}: shape {tuple(src.shape)} does not fit {tuple(param.shape)}")
            param.copy_(src.to(param.dtype))

        put(self.embed_tokens.weight, "embed")
        put(self.norm.weight, "final.norm")
        put(self.lm_head.weight, "head")
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            put(layer.norm1.weight, p + "norm1")
            put(layer.norm1b.weight, p + "norm1b")
            mx = layer.mixer
            put(mx.qkv_proj.weight, p + "mix.q", p + "mix.k", p + "mix.v")
            put(mx.o_proj.weight, p + "mix.o")
            put(mx.attn.q_norm_weight, p + "mix.q.norm")
            put(mx.attn.k_norm_weight, p + "mix.k.norm")
            mlp = layer.mlp
            if mlp is None:
                continue
            put(layer.norm2.weight, p + "norm2")
            put(layer.norm2b.weight, p + "norm2b")
            if isinstance(mlp, GatedMLP):
                put(mlp.gate_up_proj.weight, p + "mlp.gate", p + "mlp.up")
                put(mlp.down_proj.weight, p + "mlp.down")
                continue
            put(mlp.router, p + "mlp.router")
            if p + "mlp.correction" in tensors:
                put(mlp.correction, p + "mlp.correction")
            for e in range(mlp.n_real):
                put(mlp.gate_up[e], p + f"mlp.e{e}.gate", p + f"mlp.e{e}.up")
                put(mlp.down[e], p + f"mlp.e{e}.down")
            if mlp.shared is not None:
                put(mlp.shared.gate_up_proj.weight, p + "mlp.shared.gate", p + "mlp.shared.up")
                put(mlp.shared.down_proj.weight, p + "mlp.shared.down")
        extra = sorted(set(tensors) - used)
        if extra:   # e.g. norms of a feed-forward that a layer does not have: nothing reads them
            print(f"movolorn: {len(extra)} checkpoint tensors are not used: {extra[:8]}", file=sys.stderr)

    @torch.no_grad()
    def init_synthetic_weights(self, seed: int = 0) -> None:
        """Random weights drawn on the parameters' device: matrices N(0, 1/fan_in), gains near 1, corrections small."""
        for i, (name, p) in enumerate(self.named_parameters()):
            gen = torch.Generator(device=p.device).manual_seed(seed * 100003 + i)
            val = torch.randn(p.shape, generator=gen, device=p.device, dtype=torch.float32)
            if p.dim() == 1:
                val = 0.01 * val if name.endswith("correction") else 1.0 + 0.1 * val
            elif name.endswith("embed_tokens.weight"):
                pass
            else:
                val = val * (p.shape[-1] ** -0.5)
            p.copy_(val.to(p.dtype))
