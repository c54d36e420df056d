"""Host-side parts of the Movolorn path (no GPU): configuration reader, layer runs, checkpoint reader, the oracle's
own invariants."""
import json
import struct

import numpy as np
import pytest
import torch

from compactor_vllm.config.model_config import MovolornConfig, load_model_config
from compactor_vllm.layers.attention import linear_bias_slopes
from compactor_vllm.utils.safetensors_io import load_safetensors
from oracle import movolorn as O


def small_config(**over):
    c = {"architecture": "Movolorn", "vocab": 31, "width": 12, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5},
         "layers": [
             {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 10, "scale": 0.3,
                                             "mask": {"size": 5}}, "mlp": {"kind": "dense", "ff": 20}},
             {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.25},
              "mlp": {"kind": "moe", "expert": {"ff": 7}, "shared": {"ff": 9},
                      "router": {"experts": 5, "identity": 1, "top": 2, "groups": {"count": 3, "keep": 2}}}},
             {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.25,
                                             "mask": {"size": 9}}, "mlp": None}]}
    c.update(over)
    return c


def test_config_reader_fields_and_defaults():
    cfg = MovolornConfig.from_json(small_config())
    assert (cfg.vocab_size, cfg.hidden_size, cfg.embedding_scale, cfg.rms_norm_eps) == (31, 12, 2.0, 1e-5)
    a0, a1 = cfg.layers[0].mixer, cfg.layers[1].mixer
    assert (a0.heads, a0.kv_heads, a0.dim, a0.vdim, a0.scale, a0.chunk) == (4, 2, 6, 10, 0.3, 5)
    assert a1.chunk == 0                                   # no mask: plain causal
    m = cfg.layers[1].mlp
    assert (m.kind, m.ff, m.experts, m.identity, m.top, m.groups, m.keep, m.shared_ff) == ("moe", 7, 5, 1, 2, 3, 2, 9)
    assert cfg.layers[2].mlp is None
    assert cfg.layer_runs == [0, 1, 2] and cfg.num_hidden_layers == 3
    assert cfg.model_type == "movolorn"


@pytest.mark.parametrize("loop,runs", [
    ({"start": 0, "stop": 2, "times": 3}, [0, 1, 0, 1, 0, 1, 2]),
    ({"start": 1, "stop": 3, "times": 2}, [0, 1, 2, 1, 2]),
    ({"start": 2, "stop": 3, "times": 1}, [0, 1, 2]),
    ({"start": 1, "stop": 1, "times": 4}, [0, 1, 2]),
    ({"start": 0, "stop": 3, "times": 2}, [0, 1, 2, 0, 1, 2]),
])
def test_layer_runs_follow_the_loop(loop, runs):
    cfg = MovolornConfig.from_json(small_config(loop=loop))
    assert cfg.layer_runs == runs == O.layer_runs(3, (loop["start"], loop["stop"], loop["times"]))
    assert cfg.num_hidden_layers == len(runs)


def test_config_reader_refuses_what_it_does_not_know():
    bad = small_config()
    bad["layers"][0]["type"] = "recurrent"
    with pytest.raises(ValueError):
        MovolornConfig.from_json(bad)
    bad = small_config()
    bad["layers"][0]["mlp"]["kind"] = "sparse"
    with pytest.raises(ValueError):
        MovolornConfig.from_json(bad)
    with pytest.raises(ValueError):
        MovolornConfig.from_json(small_config(loop={"start": 2, "stop": 5, "times": 2}))


def test_load_model_config_reads_a_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(small_config()))
    cfg = load_model_config(str(tmp_path))
    assert isinstance(cfg, MovolornConfig) and cfg.hidden_size == 12


def test_safetensors_reader(tmp_path):
    a = np.arange(12, dtype="<f4").reshape(3, 4)
    b16 = torch.tensor([1.5, -2.0, 0.0078125, 3.0e5], dtype=torch.bfloat16)
    c = np.array([3, -1, 7], dtype="<i4")
    blobs = [("a", "F32", a.shape, a.tobytes()), ("b", "BF16", (2, 2), b16.view(torch.int16).numpy().tobytes()),
             ("c", "I32", c.shape, c.tobytes())]
    header, data = {"__metadata__": {"format": "pt"}}, b""
    for name, dt, shape, raw in blobs:
        header[name] = {"dtype": dt, "shape": list(shape), "data_offsets": [len(data), len(data) + len(raw)]}
        data += raw
    h = json.dumps(header).encode()
    path = tmp_path / "w.safetensors"
    path.write_bytes(struct.pack("<Q", len(h)) + h + data)
    t = load_safetensors(str(path))
    assert set(t) == {"a", "b", "c"}
    assert torch.equal(t["a"], torch.from_numpy(a.copy()))
    assert t["b"].dtype == torch.bfloat16 and torch.equal(t["b"], b16.view(2, 2))
    assert t["c"].dtype == torch.int32 and t["c"].tolist() == [3, -1, 7]


def test_slopes_match_the_oracle():
    for H in (1, 2, 3, 8, 12):
        assert torch.allclose(linear_bias_slopes(H).double(), O.head_slopes(H), rtol=1e-7)
    assert abs(float(linear_bias_slopes(8)[0]) - 0.5) < 1e-7 and abs(float(linear_bias_slopes(8)[-1]) - 2 ** -8) < 1e-9


def test_oracle_sink_softmax_and_chunks():
    p = O.sink_softmax_row(torch.tensor([0.0, 0.0, 0.0], dtype=torch.float64))
    assert torch.allclose(p, torch.full((3,), 0.25, dtype=torch.float64))         # the sink takes a quarter
    p = O.sink_softmax_row(torch.tensor([800.0, 799.0], dtype=torch.float64))      # no overflow
    assert torch.isfinite(p).all() and abs(float(p.sum()) - 1.0) < 1e-9
    p = O.sink_softmax_row(torch.tensor([-800.0], dtype=torch.float64))            # the sink takes everything
    assert float(p[0]) == 0.0
    assert O.visible(9, 5, 5) and not O.visible(10, 9, 5) and O.visible(10, 10, 5) and not O.visible(3, 4, None)
    assert O.visible(100, 0, None)


def test_oracle_router_keeps_to_the_best_groups():
    g = torch.Generator().manual_seed(0)
    m = {"router": torch.randn(8, 6, generator=g), "correction": torch.randn(8, generator=g), "top": 2,
         "groups": 4, "keep": 1}
    chosen, weights = O.route(torch.randn(40, 6, generator=g), m)
    assert ((chosen[:, 0] // 2) == (chosen[:, 1] // 2)).all()        # both from one group of two neighbours
    assert (weights > 0).all() and (weights.sum(-1) < 1).all()       # plain softmax scores, not renormalised
