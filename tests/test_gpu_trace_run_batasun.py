"""bin/trace_run end to end on a Batasun model from files: a config.json and a model.safetensors written by the test
(every tensor name of the design: both mixers, a layer that borrows a latent, a layer without feed-forward, a
feed-forward without a shared expert), a schedule on standard input with portions beside single tokens and requests
that end and give their pages and state slots to later ones, logits compared with the CPU oracle."""
import json
import os
import struct
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def default_config():
    la = {"heads": 3, "dim": 10, "rot_dim": 6, "vdim": 14, "kv_rank": 18, "q_rank": 12, "scale": 0.3,
          "rot": {"base": 500.0, "dims": 6}}
    moe = {"kind": "moe", "expert": {"ff": 14, "limit": 1.2}, "shared": {"ff": 22, "limit": 0.6},
           "router": {"experts": 4, "top": 2}}
    return {"architecture": "Batasun", "vocab": 50, "width": 36, "norm": {"eps": 2e-5},
            "layers": [
                {"type": "mamba2", "mixer": {"heads": 3, "vdim": 8, "state": 12, "groups": 3, "conv": 3, "norm_groups": 2},
                 "mlp": moe},
                {"type": "latent_attention", "mixer": la, "mlp": None},
                {"type": "latent_attention", "mixer": dict(la, heads=2, dim=8, vdim=6, q_rank=9, kv_from=1),
                 "mlp": {"kind": "moe", "expert": {"ff": 10, "limit": 3.0}, "router": {"experts": 3, "top": 1}}},
                {"type": "mamba2", "mixer": {"heads": 2, "vdim": 12, "state": 20, "groups": 1, "conv": 4, "norm_groups": 1},
                 "mlp": None}]}


def write_model(folder: Path, seed: int = 0):
    """Writes config.json and model.safetensors of a random model; returns (config, tensors as written)."""
    cfg = default_config()
    W, V = cfg["width"], cfg["vocab"]
    g = torch.Generator().manual_seed(seed)
    t = {}

    def mat(name, *shape, scale=None):
        t[name] = (torch.randn(*shape, generator=g) * (scale if scale is not None else shape[-1] ** -0.5)).to(torch.bfloat16)

    def vec(name, n, mean=0.0, spread=0.1):
        t[name] = (mean + spread * torch.randn(n, generator=g)).to(torch.bfloat16)

    mat("embed", V, W, scale=1.0)
    mat("head", V, W)
    vec("embed.norm", W)
    vec("final.norm", W)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        vec(p + "norm1", W)
        if layer["type"] == "latent_attention":
            H, D, R, Dv, r, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            mat(p + "mix.dq", qr, W); vec(p + "mix.dq.norm", qr, 1.0); mat(p + "mix.uq", H * (D + R), qr)
            if "kv_from" not in m:
                mat(p + "mix.dkv", r + R, W); vec(p + "mix.dkv.norm", r, 1.0)
            mat(p + "mix.uk", H * D, r); mat(p + "mix.uv", H * Dv, r); mat(p + "mix.g", H * Dv, W); mat(p + "mix.o", W, H * Dv)
        else:
            inner, GN = m["heads"] * m["vdim"], m["groups"] * m["state"]
            mat(p + "mix.in", 2 * inner + 2 * GN + m["heads"], W)
            mat(p + "mix.conv", inner + 2 * GN, m["conv"], scale=0.5); vec(p + "mix.conv.b", inner + 2 * GN)
            vec(p + "mix.dt_bias", m["heads"], -0.5, 0.5); vec(p + "mix.A_log", m["heads"], 0.0, 0.5)
            vec(p + "mix.D", m["heads"], 1.0); vec(p + "mix.norm", inner, 1.0); mat(p + "mix.o", W, inner)
        ml = layer["mlp"]
        if ml is None:
            continue
        vec(p + "norm2", W)
        f = ml["expert"]["ff"]
        for e in range(ml["router"]["experts"]):
            mat(p + f"mlp.e{e}.gate", f, W); mat(p + f"mlp.e{e}.up", f, W); mat(p + f"mlp.e{e}.down", W, f)
        mat(p + "mlp.router", ml["router"]["experts"], W, scale=0.5); vec(p + "mlp.router.b", ml["router"]["experts"], 0.0, 0.3)
        if ml.get("shared"):
            sf = ml["shared"]["ff"]
            mat(p + "mlp.shared.gate", sf, W); mat(p + "mlp.shared.up", sf, W); mat(p + "mlp.shared.down", W, sf)
            mat(p + "mlp.shared.sg", 1, W)
    header, blob = {}, b""
    for name, x in t.items():
        raw = x.contiguous().view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(x.shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    h = json.dumps(header).encode()
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    (folder / "model.safetensors").write_bytes(struct.pack("<Q", len(h)) + h + blob)
    return cfg, t


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-5), ("bfloat16", 8e-2)])
def test_trace_run_replays_a_schedule_from_files(tmp_path, dtype, tol):
    from oracle import batasun as O

    cfg, tensors = write_model(tmp_path / "model")
    om = O.from_checkpoint(cfg, tensors)
    g = torch.Generator().manual_seed(5)
    reqs = {k: torch.randint(0, 50, (n,), generator=g).tolist() for k, n in (("a", 40), ("b", 17), ("c", 5), ("d", 70), ("e", 1))}
    want = {k: O.forward(om, v) for k, v in reqs.items()}
    # pool: 3 pages of 64 tokens; a, b, c live together, then d (2 pages) beside b after a and c have ended, then e
    plan = [[("a", 16), ("b", 2)], [("a", 1), ("b", 1)], [("a", 23), ("c", 5)], [("b", 1)], [("b", 13), ("d", 33)],
            [("d", 1)], [("d", 36), ("e", 1)]]
    at = {k: 0 for k in reqs}
    lines, expect = [], []
    for n, step in enumerate(plan):
        entries, end, rows = [], [], []
        for k, c in step:
            lo, hi = at[k], at[k] + c
            entries.append({"id": "req-" + k, "tokens": reqs[k][lo:hi], "want": list(range(c))})
            rows.append(want[k][lo:hi])
            at[k] = hi
            if hi == len(reqs[k]):
                end.append("req-" + k)
        lines.append(json.dumps({"step": n, "entries": entries, "end": end}))
        expect.append(torch.cat(rows))
    assert all(at[k] == len(v) for k, v in reqs.items())
    out = tmp_path / "out"
    env = dict(os.environ, HOME=str(tmp_path), TMPDIR=str(tmp_path))
    res = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(tmp_path / "model"), "--dtype", dtype, "--out",
                          str(out), "--max-tokens", "192"], input="\n".join(lines) + "\n", capture_output=True, text=True,
                         env=env, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [l for l in res.stdout.splitlines() if l.startswith("done ")] == [f"done {n}" for n in range(len(plan))]
    scale = torch.cat(list(want.values())).std()
    errs = []
    for n, exp in enumerate(expect):
        got = torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(exp.shape)).double()
        d = (got - exp) - (got - exp).mean(-1, keepdim=True)
        errs.append(d.pow(2).mean(-1).sqrt() / scale)
    errs = torch.cat(errs)
    if dtype == "float32":
        assert errs.max() < tol
    else:   # rounding may flip a router's close call for single rows
        assert errs.median() < 0.04 and (errs > 2 * tol).float().mean() < 0.1
