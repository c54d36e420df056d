"""bin/trace_run end to end from files: a config.json and a model.safetensors written by the test (every tensor name of
the design, a layer without feed-forward, a loop, two cache geometries), a schedule on standard input with portions
beside single tokens and requests that end and give their pages to later ones, logits compared with the CPU oracle."""
import json
import os
import struct
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def default_config():
    W, V = 32, 50
    return {"architecture": "Movolorn", "vocab": V, "width": W, "embedding": {"scale": 0.7}, "norm": {"eps": 1e-5},
           "layers": [
               {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.2,
                                               "mask": {"size": 10}}, "mlp": {"kind": "dense", "ff": 40}},
               {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3,
                                               "mask": {"size": 7}},
                "mlp": {"kind": "moe", "expert": {"ff": 16}, "shared": {"ff": 24},
                        "router": {"experts": 3, "identity": 1, "top": 2, "groups": {"count": 2, "keep": 1}}}},
               {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.15},
                "mlp": None}],
           "loop": {"start": 1, "stop": 2, "times": 2}}


def write_model(folder: Path, seed: int = 0, cfg: dict | None = None):
    """Writes config.json and model.safetensors of a random model of `cfg`; returns the oracle's dict of the same
    tensors (after their bfloat16 rounding)."""
    cfg = default_config() if cfg is None else cfg
    W, V = cfg["width"], cfg["vocab"]
    g = torch.Generator().manual_seed(seed)
    t = {}

    def mat(name, *shape, scale=None):
        t[name] = (torch.randn(*shape, generator=g) * (scale if scale is not None else shape[-1] ** -0.5)).to(torch.bfloat16)

    def gain(name, n):
        t[name] = (1.0 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16)

    mat("embed", V, W, scale=1.0)
    mat("head", V, W)
    gain("final.norm", W)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        for n in ("norm1", "norm1b"):
            gain(p + n, W)
        mat(p + "mix.q", H * D, W); mat(p + "mix.k", G * D, W); mat(p + "mix.v", G * Dv, W); mat(p + "mix.o", W, H * Dv)
        gain(p + "mix.q.norm", D); gain(p + "mix.k.norm", D)
        ml = layer["mlp"]
        if ml is None:
            continue
        for n in ("norm2", "norm2b"):
            gain(p + n, W)
        if ml["kind"] == "dense":
            mat(p + "mlp.gate", ml["ff"], W); mat(p + "mlp.up", ml["ff"], W); mat(p + "mlp.down", W, ml["ff"])
        else:
            r, f = ml["router"], ml["expert"]["ff"]
            for e in range(r["experts"]):
                mat(p + f"mlp.e{e}.gate", f, W); mat(p + f"mlp.e{e}.up", f, W); mat(p + f"mlp.e{e}.down", W, f)
            total = r["experts"] + r.get("identity", 0)
            mat(p + "mlp.router", total, W, scale=0.5)
            t[p + "mlp.correction"] = (0.2 * torch.randn(total, generator=g)).to(torch.bfloat16)
            if ml.get("shared"):
                sf = ml["shared"]["ff"]
                mat(p + "mlp.shared.gate", sf, W); mat(p + "mlp.shared.up", sf, W); mat(p + "mlp.shared.down", W, sf)
    header, blob = {}, b""
    for name, x in t.items():
        raw = x.contiguous().view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(x.shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    h = json.dumps(header).encode()
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    (folder / "model.safetensors").write_bytes(struct.pack("<Q", len(h)) + h + blob)
    # the oracle's dict straight from the same tensors
    f = lambda n: t[n].float()
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        p, m, ml = f"l{i}.", layer["mixer"], layer["mlp"]
        attn = {"q": f(p + "mix.q"), "k": f(p + "mix.k"), "v": f(p + "mix.v"), "o": f(p + "mix.o"),
                "q_norm": f(p + "mix.q.norm"), "k_norm": f(p + "mix.k.norm"), "heads": m["heads"], "kv_heads": m["kv_heads"],
                "dim": m["dim"], "vdim": m["vdim"], "scale": m["scale"], "chunk": (m.get("mask") or {}).get("size")}
        entry = {"norm1": f(p + "norm1"), "norm1b": f(p + "norm1b"), "attn": attn, "mlp": None}
        if ml is not None:
            entry["norm2"], entry["norm2b"] = f(p + "norm2"), f(p + "norm2b")
            if ml["kind"] == "dense":
                entry["mlp"] = {"kind": "dense", "gate": f(p + "mlp.gate"), "up": f(p + "mlp.up"), "down": f(p + "mlp.down")}
            else:
                r = ml["router"]
                entry["mlp"] = {"kind": "moe", "router": f(p + "mlp.router"), "correction": f(p + "mlp.correction"),
                                "experts": [{k: f(p + f"mlp.e{e}.{k}") for k in ("gate", "up", "down")}
                                            for e in range(r["experts"])],
                                "top": r["top"], "groups": (r.get("groups") or {}).get("count", 1),
                                "keep": (r.get("groups") or {}).get("keep", 1), "identity": r.get("identity", 0),
                                "shared": ({k: f(p + f"mlp.shared.{k}") for k in ("gate", "up", "down")}
                                           if ml.get("shared") else None)}
        layers.append(entry)
    lp = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    return {"embed": f("embed"), "embed_scale": cfg["embedding"]["scale"], "eps": cfg["norm"]["eps"],
            "final_norm": f("final.norm"), "head": f("head"), "layers": layers,
            "loop": (lp["start"], lp["stop"], lp["times"])}


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-5), ("bfloat16", 8e-2)])
def test_trace_run_replays_a_schedule_from_files(tmp_path, dtype, tol):
    from oracle import movolorn as O

    om = write_model(tmp_path / "model")
    g = torch.Generator().manual_seed(5)
    reqs = {k: torch.randint(0, 50, (n,), generator=g).tolist() for k, n in (("a", 40), ("b", 17), ("c", 5), ("d", 70))}
    want = {k: O.forward(om, v) for k, v in reqs.items()}
    # pool: 3 pages of 64 tokens; a, b, c live together, then d (2 pages) beside b after a and c have ended
    plan = [[("a", 16), ("b", 2)], [("a", 1), ("b", 1)], [("a", 23), ("c", 5)], [("b", 1)], [("b", 13), ("d", 33)],
            [("d", 1)], [("d", 36)]]
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
        got = torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(exp.shape))
        d = (got - exp) - (got - exp).mean(-1, keepdim=True)
        errs.append(d.pow(2).mean(-1).sqrt() / scale)
    errs = torch.cat(errs)
    if dtype == "float32":
        assert errs.max() < tol
    else:   # rounding may flip a router's close call for single rows
        assert errs.median() < 0.03 and (errs > tol).float().mean() < 0.1
