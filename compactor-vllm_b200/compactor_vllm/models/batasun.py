"""Batasun: a decoder that mixes latent-attention layers and state-space layers, each followed by a mixture of clamped
gated experts (or by nothing), on a 32-bit residual stream with norms on the sublayers' OUTPUTS only:

    x = norm(embed[token]);   per layer:  x += norm1(mixer(x)),  x += norm2(ff(x));   logits = head(norm(x))

Every norm is an RMS norm with its gain stored around zero (gain = 1 + w).  The sublayers read the stream itself, so one
`sandwich_norm` launch does the post-norm of a sublayer, the residual sum and the rounding of the new stream to the
activations' type for the next sublayer (the last one applies the final norm instead).

Built from the engine's blocks:
  * mixer "latent_attention" = `LatentAttention` (layers/latent_attention.py) over the paged cache; a layer with
    `kv_from` reads the cache rows of an earlier layer and owns no cache layer;
  * mixer "mamba2" = `StateSpaceMixer` (layers/ssm.py) with its state in the runner's state pool;
  * feed-forward = `RoutedExperts` (layers/moe.py) with ACT_CLAMPED_GLU experts, ROUTE_TOP_LOGITS routing with a bias,
    and a shared expert gated by one logit per token.
Weights: `load_weights` takes the checkpoint's tensors (`embed`, `embed.norm`, `final.norm`, `head`, `l<i>.norm1|norm2`,
`l<i>.mix.dq|dq.norm|uq|dkv|dkv.norm|uk|uv|g|o`, `l<i>.mix.in|conv|conv.b|dt_bias|A_log|D|norm|o`,
`l<i>.mlp.e<j>.gate|up|down`, `l<i>.mlp.router|router.b`, `l<i>.mlp.shared.gate|up|down|sg`);
`init_synthetic_weights` draws random ones.
"""
from __future__ import annotations

import sys
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F
from torch import nn

from compactor_vllm.config.model_config import BatasunConfig, ClampedMoEConfig
from compactor_vllm.layers.latent_attention import LatentAttention
from compactor_vllm.layers.layernorm import NormWeight, sandwich_norm
from compactor_vllm.layers.moe import ACT_CLAMPED_GLU, ROUTE_TOP_LOGITS, RoutedExperts
from compactor_vllm.layers.ssm import StateSpaceMixer
from compactor_vllm.utils.context import get_context

GAIN_OFFSET = 1.0     # every norm of the design: gain = 1 + stored weight


def make_experts(width: int, m: Optional[ClampedMoEConfig], dtype) -> Optional[RoutedExperts]:
    if m is None:
        return None
    return RoutedExperts(width, m.ff, m.experts, 0, m.top, 1, 1, m.shared_ff, ACT_CLAMPED_GLU, dtype,
                         route_mode=ROUTE_TOP_LOGITS, router_bias=True, limit=m.limit, shared_limit=m.shared_limit,
                         shared_gate=True)


class BatasunLayer(nn.Module):
    def __init__(self, cfg: BatasunConfig, index: int, layers: List["BatasunLayer"], dtype):
        super().__init__()
        lc = cfg.layers[index]
        W, eps = cfg.hidden_size, cfg.rms_norm_eps
        self.eps = eps
        a = lc.mixer
        if lc.mixer_type == "latent_attention":
            source = None if a.kv_from is None else layers[a.kv_from].mixer
            self.mixer = LatentAttention(W, a.heads, a.dim, a.rot_dim, a.vdim, a.kv_rank, a.q_rank, a.scale, a.rot_base,
                                         eps, source=source, dtype=dtype)
        else:
            self.mixer = StateSpaceMixer(W, a.heads, a.vdim, a.state, a.groups, a.conv, a.norm_groups, eps)
        self.mlp = make_experts(W, lc.mlp, dtype)
        self.norm1 = NormWeight(W)
        nn.init.zeros_(self.norm1.weight)
        if self.mlp is not None:
            self.norm2 = NormWeight(W)
            nn.init.zeros_(self.norm2.weight)


class BatasunForCausalLM(nn.Module):
    mixed_steps = True        # the runner may hand it portions of prompts beside single tokens in one step

    def __init__(self, cfg: BatasunConfig):
        super().__init__()
        self.config = cfg
        dtype = torch.get_default_dtype()
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.embed_norm = NormWeight(cfg.hidden_size)
        layers: List[BatasunLayer] = []
        for i in range(len(cfg.layers)):
            layers.append(BatasunLayer(cfg, i, layers, dtype))
        self.layers = nn.ModuleList(layers)
        self.norm = NormWeight(cfg.hidden_size)
        for n in (self.embed_norm, self.norm):
            nn.init.zeros_(n.weight)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        self.debug_residuals: Optional[list] = None   # a list collects the residual stream after every layer

    # ---- what the cache manager asks ----------------------------------------------------------------------
    def cache_specs(self):
        """One entry per cache layer: (attention module, kv heads, key row size, value row size).  Only layers with a
        latent of their own have one; the values are columns of the key rows (value row size 0)."""
        return [(l.mixer.attn, 1, l.mixer.row, 0) for l in self.layers
                if isinstance(l.mixer, LatentAttention) and l.mixer.own_latent]

    def state_layers(self):
        """The layers that carry a recurrent state between steps (each has `state_specs(dtype)`)."""
        return [l.mixer for l in self.layers if isinstance(l.mixer, StateSpaceMixer)]

    # ---- forward ----------------------------------------------------------------------------------------------
    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        cfg = self.config
        eps = cfg.rms_norm_eps
        dtype = self.lm_head.weight.dtype
        emb = F.embedding(input_ids, self.embed_tokens.weight)
        x = torch.empty(emb.shape, dtype=torch.float32, device=emb.device)
        # x = norm(embedding); h = x rounded to the activations' type
        h = sandwich_norm(x, branch=emb, post_weight=self.embed_norm.weight, eps=eps, out_dtype=dtype,
                          gain_offset=GAIN_OFFSET, assign=True, cast_out=True)
        last = len(self.layers) - 1

        def advance(branch, weight, final):
            if final:    # the last sublayer: the final norm instead of the next sublayer's input
                return sandwich_norm(x, branch=branch, post_weight=weight, pre_weight=self.norm.weight, eps=eps,
                                     out_dtype=dtype, gain_offset=GAIN_OFFSET)
            return sandwich_norm(x, branch=branch, post_weight=weight, eps=eps, out_dtype=dtype,
                                 gain_offset=GAIN_OFFSET, cast_out=True)

        for i, layer in enumerate(self.layers):
            collect = self.debug_residuals is not None
            h = advance(layer.mixer(h), layer.norm1.weight, i == last and layer.mlp is None and not collect)
            if layer.mlp is not None:
                h = advance(layer.mlp(h), layer.norm2.weight, i == last and not collect)
            if collect:
                self.debug_residuals.append(x.clone())
                if i == last:
                    h = sandwich_norm(x, pre_weight=self.norm.weight, eps=eps, out_dtype=dtype, gain_offset=GAIN_OFFSET)
        if not self.layers:
            h = sandwich_norm(x, pre_weight=self.norm.weight, eps=eps, out_dtype=dtype, gain_offset=GAIN_OFFSET)
        return h

    def compute_logits(self, hidden_states: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Logits of the given rows of the step (None: the last token of every sequence of the step)."""
        if rows is None:
            rows = get_context().cu_seqlens_q[1:].long() - 1
        return self.lm_head(hidden_states.index_select(0, rows))

    # ---- weights ----------------------------------------------------------------------------------------------
    @torch.no_grad()
    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        used = set()

        def get(name):
            if name not in tensors:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            used.add(name)
            return tensors[name]

        def put(param, *names, shape=None):
            src = torch.cat([get(n) for n in names], dim=0) if len(names) > 1 else get(names[0])
            if shape is not None:
                if src.numel() != param.numel():
                    raise ValueError(f"{names}: {tuple(src.shape)} does not fit {tuple(param.shape)}")
                src = src.reshape(shape)
            if tuple(src.shape) != tuple(param.shape):
                raise ValueError(f"{names}: shape {tuple(src.shape)} does not fit {tuple(param.shape)}")
            param.copy_(src.to(param.dtype))

        put(self.embed_tokens.weight, "embed")
        put(self.embed_norm.weight, "embed.norm")
        put(self.norm.weight, "final.norm")
        put(self.lm_head.weight, "head")
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            put(layer.norm1.weight, p + "norm1")
            mx = layer.mixer
            if isinstance(mx, LatentAttention):
                if mx.own_latent:
                    put(mx.in_proj.weight, p + "mix.dq", p + "mix.dkv", p + "mix.g")
                    put(mx.kv_norm, p + "mix.dkv.norm")
                else:
                    put(mx.in_proj.weight, p + "mix.dq", p + "mix.g")
                put(mx.q_norm, p + "mix.dq.norm")
                put(mx.uq_proj.weight, p + "mix.uq")
                put(mx.uk, p + "mix.uk", shape=mx.uk.shape)
                put(mx.uv, p + "mix.uv", shape=mx.uv.shape)
                put(mx.o_proj.weight, p + "mix.o")
            else:
                put(mx.in_proj.weight, p + "mix.in")
                put(mx.conv_weight, p + "mix.conv")
                put(mx.conv_bias, p + "mix.conv.b")
                put(mx.dt_bias, p + "mix.dt_bias")
                put(mx.A_log, p + "mix.A_log")
                put(mx.D, p + "mix.D")
                put(mx.norm_weight, p + "mix.norm")
                put(mx.o_proj.weight, p + "mix.o")
            mlp = layer.mlp
            if mlp is None:
                continue
            put(layer.norm2.weight, p + "norm2")
            E = mlp.n_real
            mlp.router[:E].copy_(get(p + "mlp.router").float())
            mlp.router_bias.zero_()
            mlp.router_bias[:E].copy_(get(p + "mlp.router.b").float())
            for e in range(E):
                put(mlp.gate_up[e], p + f"mlp.e{e}.gate", p + f"mlp.e{e}.up")
                put(mlp.down[e], p + f"mlp.e{e}.down")
            if mlp.shared is not None:
                put(mlp.shared.gate_up_proj.weight, p + "mlp.shared.gate", p + "mlp.shared.up")
                put(mlp.shared.down_proj.weight, p + "mlp.shared.down")
                mlp.router[E:].copy_(get(p + "mlp.shared.sg").float().reshape(1, -1))
        extra = sorted(set(tensors) - used)
        if extra:
            print(f"batasun: {len(extra)} checkpoint tensors are not used: {extra[:8]}", file=sys.stderr)

    @torch.no_grad()
    def init_synthetic_weights(self, seed: int = 0) -> None:
        """Random weights drawn on the parameters' device: matrices N(0, 1/fan_in), norm gains near their neutral value,
        small biases, decays and step sizes in the range where the recurrence neither dies nor saturates."""
        for i, (name, p) in enumerate(self.named_parameters()):
            gen = torch.Generator(device=p.device).manual_seed(seed * 100003 + i)
            val = torch.randn(p.shape, generator=gen, device=p.device, dtype=torch.float32)
            leaf = name.rsplit(".", 1)[-1]
            if name.endswith("embed_tokens.weight"):
                pass
            elif leaf in ("q_norm", "kv_norm", "norm_weight", "D"):
                val = 1.0 + 0.1 * val
            elif leaf == "A_log":
                val = 0.5 * val
            elif leaf == "dt_bias":
                val = -1.0 + 0.5 * val
            elif leaf in ("conv_bias", "router_bias") or (p.dim() == 1 and leaf == "weight"):
                val = 0.1 * val
            elif leaf == "conv_weight":
                val = val * 0.5
            else:
                val = val * (p.shape[-1] ** -0.5)
            p.copy_(val.to(p.dtype))
        for layer in self.layers:      # the shared expert's gate logit (the router's extra row) has no bias
            if layer.mlp is not None and layer.mlp.router_bias is not None:
                layer.mlp.router_bias[layer.mlp.total:].zero_()
