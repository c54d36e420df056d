"""Prefill and decode throughput of a Batasun model beside a Movolorn model of equal size (random weights), both through
the engine's runner, plus the design's kernels timed alone against the measured peaks.

Used by `bench.py --arch batasun`; the default workload of bench.py does not touch this module.  Movolorn with routed
experts is the closest existing model: the same runner path (mixed steps, decode graphs), the same 32-bit residual
stream with sandwich norms, routed experts with a shared one, and attention over the same paged kernels.
Timing as in arch_compare: CUDA events on the launching stream after warm-up, a buffer larger than L2 written between
timed kernel iterations; engine-level numbers include the runner's host work.
"""
from __future__ import annotations

import json
from typing import List

import torch

from compactor_vllm.benchmarks.arch_compare import (DECODE_BATCH, DECODE_CONTEXT, DECODE_STEPS, PREFILL_TOKENS, SIZES,
                                                    _events_ms, engine_throughput, movolorn_config)

# the latent sizes the tensor-core portion kernel serves: key rows of kv_rank + rot_dim = 128 numbers
LATENT = dict(dim=128, rot_dim=64, vdim=128, kv_rank=64)
STATE, VDIM, CONV = 128, 64, 4


def batasun_config(s: dict, pattern: str) -> dict:
    """`pattern`: one letter per layer, cycled over the size's layer count: A latent attention with a latent of its own,
    a latent attention that borrows the latent of the last A, M state-space mixer."""
    W = s["width"]
    heads_ssm = 2 * W // VDIM
    moe = {"kind": "moe", "expert": {"ff": s["ff"] // 4, "limit": 7.0}, "shared": {"ff": s["ff"] // 2, "limit": 7.0},
           "router": {"experts": 8, "top": 2}}
    layers, last_a = [], None
    for i in range(s["layers"]):
        kind = pattern[i % len(pattern)]
        if kind in "Aa":
            mixer = dict(LATENT, heads=s["heads"], q_rank=W // 4, scale=(LATENT["dim"] + LATENT["rot_dim"]) ** -0.5,
                         rot={"base": 10000.0, "dims": LATENT["rot_dim"]})
            if kind == "a" and last_a is not None:
                mixer["kv_from"] = last_a
            else:
                last_a = i
            layers.append({"type": "latent_attention", "mixer": mixer, "mlp": moe})
        else:
            layers.append({"type": "mamba2", "mlp": moe,
                           "mixer": {"heads": heads_ssm, "vdim": VDIM, "state": STATE, "groups": 8, "conv": CONV,
                                     "norm_groups": 8}})
    return {"architecture": "Batasun", "vocab": s["vocab"], "width": W, "norm": {"eps": 1e-6}, "layers": layers}


def kernel_rooflines(peaks: dict, reps: int) -> List[dict]:
    """The design's kernels alone at width 4096, bfloat16: achieved rate and its fraction of the measured copy
    bandwidth / cuBLAS bf16 rate."""
    from compactor_vllm import _native as N
    from compactor_vllm.config.constants import RESERVED_BATCH
    from compactor_vllm.kv_cache.page_table import KVAllocationStatus, PagedKVCache
    from compactor_vllm.layers.latent_attention import LatentAttention, sigmoid_gate
    from compactor_vllm.layers.layernorm import sandwich_norm
    from compactor_vllm.layers.moe import ACT_CLAMPED_GLU, ROUTE_TOP_LOGITS, gated_act, route
    from compactor_vllm.layers.ssm import StateSpaceMixer
    from compactor_vllm.utils.context import reset_context, set_context

    dev = torch.device("cuda", torch.cuda.current_device())
    bf = torch.bfloat16
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    hbm = float(peaks["hbm"]) * 1e9
    tflops = float(peaks["tensor_burst"]) * 1e12
    rows: List[dict] = []
    lib, code, st = N.lib(), N.CVLLM_BF16, N.stream(dev)

    def timed(fn):
        def run():
            flush_buf.zero_()
            fn()
        return max(_events_ms(run, reps) - _events_ms(lambda: flush_buf.zero_(), reps), 1e-4)

    def add(name, ms, *, nbytes=None, flops=None, like=None):
        r = {"kernel": name, "ms": round(ms, 4), "like": like}
        if nbytes is not None:
            r["GBs"] = round(nbytes / ms / 1e6, 1)
            r["frac_hbm_of_measured"] = round(nbytes / (ms * 1e-3) / hbm, 3)
        if flops is not None:
            r["TFLOPs"] = round(flops / ms / 1e9, 1)
            r["frac_bf16_of_measured"] = round(flops / (ms * 1e-3) / tflops, 4)
        rows.append(r)

    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    T, W, PS, L = 8192, 4096, 128, 4096
    # --- the residual update of this design: branch (2 B) + residual read and write (8 B) + rounded stream (2 B)
    x = torch.randn(T, W, device=dev)
    y = torch.randn(T, W, device=dev).to(bf)
    w1 = torch.zeros(W, device=dev)
    add("sandwich_norm (gain offset, cast)", timed(lambda: sandwich_norm(x, branch=y, post_weight=w1, out_dtype=bf,
                                                                       gain_offset=1.0, cast_out=True)),
        nbytes=12 * T * W, like="sandwich_norm (post + pre norm)")
    del x, y
    F_ = 3584
    gu = torch.randn(T, 2 * F_, device=dev).to(bf)
    add("gated_act (clamped unit)", timed(lambda: gated_act(gu, ACT_CLAMPED_GLU, limit=7.0)), nbytes=6 * T * F_,
        like="gated_act (silu)")
    del gu
    E = 64
    lg = torch.randn(T * 4, E + 1, device=dev)
    add("moe_route (top logits)", timed(lambda: route(lg, None, 6, 1, 1, ROUTE_TOP_LOGITS, experts=E)),
        nbytes=4 * T * 4 * (E + 1 + 12), like="moe_route (softmax, groups)")
    del lg
    # --- latent attention, 32 heads over one latent row of 64 + 64 numbers
    H = 32
    prev = torch.get_default_dtype()
    torch.set_default_dtype(bf)          # as the runner builds models: 16-bit matrices, fp32 gains, 64-bit frequencies
    try:
        with torch.device(dev):
            la = LatentAttention(W, H, LATENT["dim"], LATENT["rot_dim"], LATENT["vdim"], LATENT["kv_rank"], 1024,
                                 0.1, 10000.0, 1e-6, dtype=bf)
            mx = StateSpaceMixer(W, 2 * W // VDIM, VDIM, STATE, 8, CONV, 8, 1e-6)
    finally:
        torch.set_default_dtype(prev)
    attn = la.attn
    cache = PagedKVCache(1, L // PS + 1, (L // PS + 1) * 9, PS, 1, la.row, 9, bf, device=dev, v_head_dim=0)
    attn.k_cache, attn.v_cache, attn.page_table, attn.bh_seq_lens = cache.layer_slices(0)
    attn.page_size = PS
    slots = []
    for _ in range(8):
        s = cache.new_batch()
        assert cache.reserve_tokens(s, L + 1) == KVAllocationStatus.SUCCESS
        slots.append(s)
    pos_all = torch.arange(L, dtype=torch.int32, device=dev)
    tok_slot = torch.full((L,), slots[0], dtype=torch.int32, device=dev)
    set_context(is_prefill=True, cu_seqlens_q=i32([0, L]), max_seqlen_q=L, max_seqlen_k=L, batch_mapping=i32(slots[:1]),
                positions_i32=pos_all, token_slot=tok_slot, seq_start=i32([0]))
    proj = torch.randn(L, la.in_proj.out_features, device=dev).to(bf)
    cq = torch.empty(L, la.q_rank, dtype=bf, device=dev)
    pt = attn.page_table

    def norm_store():
        N.check(lib.cvllm_latent_norm_store(N.ptr(proj), proj.stride(0), 0, la.q_rank, la.q_rank, la.kv_rank, la.rot_dim,
                                            N.ptr(la.q_norm), N.ptr(la.kv_norm), 1e-6, N.ptr(la.inv_freq), N.ptr(pos_all),
                                            N.ptr(tok_slot), N.ptr(cq), N.ptr(attn.k_cache), N.ptr(pt), pt.stride(0), PS,
                                            N.ptr(attn.bh_seq_lens), L, RESERVED_BATCH, code, st), "norm_store")

    add("latent_norm_store (4096 tokens)", timed(norm_store), nbytes=2 * L * 2 * (la.q_rank + la.row),
        like="qknorm_store")
    q = torch.randn(L, H, la.dim + la.rot_dim, device=dev).to(bf)
    q_full = torch.randn(L, H, la.row, device=dev).to(bf)
    add("latent_q_rope (4096 tokens, 32 heads)",
        timed(lambda: N.check(lib.cvllm_latent_q_rope(N.ptr(q), q.stride(0), H, la.dim, la.rot_dim, N.ptr(la.inv_freq),
                                                      N.ptr(pos_all), N.ptr(q_full), q_full.stride(0), la.row, la.kv_rank,
                                                      L, code, st), "q_rope")),
        nbytes=2 * L * H * 2 * la.rot_dim, like="qknorm_store")
    add("portion attention, values in keys (4096 tokens, 32 heads, rows of 128, values of 64; tcgen05 pipeline with "
        "the whole row as the value)", timed(lambda: attn.attend(q_full)),
        flops=2.0 * (la.row + la.kv_rank) * H * L * (L + 1) / 2, like="prefill_attn_bias")
    N.set_test_option("bias_attn_fma", 2)
    add("portion attention, values in keys (the same on the mma.sync kernel)", timed(lambda: attn.attend(q_full)),
        flops=2.0 * (la.row + la.kv_rank) * H * L * (L + 1) / 2, like="bias_attn_varlen_mma")
    N.set_test_option("bias_attn_fma", 0)
    o = torch.randn(L, H * la.vdim, device=dev).to(bf)
    gsrc = torch.randn(L, H * la.vdim, device=dev).to(bf)
    add(f"sigmoid_gate (4096 x {H * la.vdim})", timed(lambda: sigmoid_gate(o, gsrc)), nbytes=6 * L * H * la.vdim, like="gated_act")
    B = 8
    set_context(is_prefill=False, batch_mapping=i32(slots), positions_i32=i32([L - 1] * B), token_slot=i32(slots),
                max_seqlen_q=1, max_seqlen_k=L)
    qd = torch.randn(B, H, la.row, device=dev).to(bf)
    add("bias_attn_decode, values in keys (8 x 4096 keys)", timed(lambda: attn.attend(qd)), nbytes=2 * B * L * la.row,
        like="bias_attn_decode")
    reset_context()
    # --- state-space mixer: 128 heads of 64 channels, state 128
    heads = mx.heads
    C = mx.channels
    mx.conv_state = torch.zeros(9, CONV - 1, C, dtype=bf, device=dev)
    mx.ssm_state = torch.zeros(9, heads, VDIM, STATE, dtype=torch.float32, device=dev)
    with torch.no_grad():
        mx.conv_weight.normal_(0, 0.3)
        mx.dt_bias.fill_(-1.0)
    projm = torch.randn(L, mx.in_proj.out_features, device=dev).to(bf)
    xbc = torch.empty(L, C, dtype=torch.float32, device=dev)
    ym = torch.empty(L, mx.inner, dtype=torch.float32, device=dev)
    outm = torch.empty(L, mx.inner, dtype=bf, device=dev)
    cu, st0, bm1 = i32([0, L]), i32([0]), i32(slots[:1])

    def conv(geom, Bn, mx_new):
        N.check(lib.cvllm_causal_conv(N.ptr(projm), projm.stride(0), mx.inner, C, CONV, N.ptr(mx.conv_weight),
                                      N.ptr(mx.conv_bias), N.ptr(mx.conv_state), *geom, Bn, mx_new, N.ptr(xbc),
                                      xbc.stride(0), code, st), "conv")

    def scan(geom, Bn, mx_new):
        nb = lib.cvllm_ssm_scan_workspace_bytes(Bn, mx_new, heads, VDIM, STATE)
        ws = N.workspace(dev, nb, "ssm_scan") if nb else None
        N.check(lib.cvllm_ssm_scan(N.ptr(xbc), xbc.stride(0), N.ptr(projm), projm.stride(0), mx.inner + C,
                                   N.ptr(mx.dt_bias), N.ptr(mx.A_log), N.ptr(mx.D), N.ptr(mx.ssm_state), *geom, Bn, mx_new,
                                   N.ptr(ym), ym.stride(0), heads, 8, VDIM, STATE, RESERVED_BATCH, N.ptr(ws), nb, code,
                                   st), "scan")

    pre = (N.ptr(cu), N.ptr(st0), None, N.ptr(bm1))
    add("causal_conv (4096 tokens, 10240 channels)", timed(lambda: conv(pre, 1, L)), nbytes=L * C * (2 + 4),
        like="qknorm_store")
    add("ssm_scan (one portion of 4096 tokens, the product's choice: whole portions at this CTA count)", timed(lambda: scan(pre, 1, L)),
        nbytes=4 * L * (C + mx.inner), like="bias_attn_varlen (the mixer's portion kernel)")
    N.set_test_option("ssm_segment", 256)
    add("ssm_scan (one portion of 4096 tokens, forced segments of 256)", timed(lambda: scan(pre, 1, L)),
        nbytes=4 * L * (C + mx.inner), like="bias_attn_varlen (the mixer's portion kernel)")
    N.set_test_option("ssm_segment", 0)
    add("gated_group_norm (4096 x 8192)",
        timed(lambda: N.check(lib.cvllm_gated_group_norm(N.ptr(ym), ym.stride(0), N.ptr(projm), projm.stride(0),
                                                         N.ptr(mx.norm_weight), 1e-6, N.ptr(outm), outm.stride(0), L,
                                                         mx.inner, 8, code, st), "norm")),
        nbytes=L * mx.inner * (4 + 2 + 2), like="sandwich_norm")
    posd, bmd = i32([L - 1] * B), i32(slots)
    dec = (None, None, N.ptr(posd), N.ptr(bmd))
    add("causal_conv (decode, 8 tokens)", timed(lambda: conv(dec, B, 1)), nbytes=B * C * (2 * CONV + 4), like=None)
    add("ssm_scan (decode, 8 sequences: state read + written)", timed(lambda: scan(dec, B, 1)),
        nbytes=2 * 4 * B * heads * VDIM * STATE, like="bias_attn_decode (the mixer's decode kernel)")
    return rows


def run(peaks: dict, sizes: List[str], reps: int) -> dict:
    from compactor_vllm.config.model_config import BatasunConfig, MovolornConfig

    result = {"arch": "batasun", "closest": "movolorn (routed experts)", "dtype": "bf16",
              "data": "synthetic (random weights)",
              "workload": {"prefill_tokens": PREFILL_TOKENS, "decode_batch": DECODE_BATCH,
                           "decode_context": DECODE_CONTEXT, "decode_steps": DECODE_STEPS}, "sizes": {}}
    for name in sizes:
        s = SIZES[name]
        row = {"shape": s}
        row["movolorn_moe_nochunk"] = engine_throughput("movolorn", MovolornConfig.from_json(movolorn_config(s, 0, True)), reps)
        for label, pattern in (("batasun_latent_only", "Aa"), ("batasun_state_space_only", "M"), ("batasun_mixed", "AaMM")):
            row[label] = engine_throughput("batasun", BatasunConfig.from_json(batasun_config(s, pattern)), reps)
        result["sizes"][name] = row
    result["kernels"] = kernel_rooflines(peaks, max(reps, 5))
    result["peaks"] = peaks
    return result


def main(peaks: dict, sizes: str, reps: int) -> None:
    print(json.dumps(run(peaks, [x for x in sizes.split(",") if x], reps)))
