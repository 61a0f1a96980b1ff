"""Zasesun without a GPU: config.json → typed configuration → parts and tensor names, refusals that
name the key, the random-weights folder, and hand-worked values of the plain implementation."""
from __future__ import annotations

import copy
import json
import math
import os

import pytest
import torch

import plain_zasesun as plain
from tiny_zasesun import ZTINY, load_folder, make_folder, zconfig


def test_registry_picks_the_architecture_by_its_name():
    from mrun_b200 import registry
    from mrun_b200.config import ZasesunConfig
    assert registry.resolve({"architecture": "Zasesun"}) is ZasesunConfig
    assert registry.resolve({"model_type": "zasesun"}) is ZasesunConfig
    with pytest.raises(Exception):
        registry.resolve({"architecture": "Nobody"})


@pytest.mark.parametrize("name", sorted(ZTINY))
def test_config_round_trip_and_spec(name):
    from mrun_b200.config import ZasesunConfig
    from mrun_b200.weights.loader import expected_tensors
    cfg = zconfig(name)
    assert ZasesunConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    spec = cfg.to_spec()
    raw = ZTINY[name]["config"]
    assert len(spec.layers) == len(raw["layers"]) and spec.tie_embeddings
    names = {t.name: t.shape for t in expected_tensors(spec)}
    assert names["embed"] == (raw["vocab"], raw["width"]) and names["final.norm"] == (raw["width"],)
    for i, entry in enumerate(raw["layers"]):
        m = entry["mixer"]
        assert names[f"l{i}.mix.dq"] == (m["q_rank"], raw["width"])
        assert names[f"l{i}.mix.dq.norm"] == (m["q_rank"],)
        assert names[f"l{i}.mix.uq"] == (m["heads"] * (m["dim"] + m["rot_dim"]), m["q_rank"])
        assert names[f"l{i}.mix.dkv"] == (m["kv_rank"] + m["rot_dim"], raw["width"])
        assert names[f"l{i}.mix.uk"] == (m["heads"] * m["dim"], m["kv_rank"])
        assert names[f"l{i}.mix.uv"] == (m["heads"] * m["vdim"], m["kv_rank"])
        assert names[f"l{i}.mix.o"] == (raw["width"], m["heads"] * m["vdim"])
        assert f"l{i}.norm1" in names and f"l{i}.norm1b" in names
        mlp = entry["mlp"]
        assert (f"l{i}.norm2" in names) == (mlp is not None) == (f"l{i}.norm2b" in names)
        if mlp and mlp["kind"] == "moe":
            assert names[f"l{i}.mlp.router"] == (mlp["router"]["experts"], raw["width"])
            assert names[f"l{i}.mlp.e0.up"] == (mlp["expert"]["ff"], raw["width"])
            assert (f"l{i}.mlp.shared.up" in names) == ("shared" in mlp)
            assert f"l{i}.mlp.e{mlp['router']['experts']}.up" not in names
        elif mlp:
            assert names[f"l{i}.mlp.gate"] == (mlp["ff"], raw["width"])
    spec.validate()


@pytest.mark.parametrize("path, value, key", [
    (("layers", 0, "type"), "ring", "layers[0].type"),
    (("layers", 1, "mixer", "heads"), 0, "layers[1].mixer.heads"),
    (("layers", 1, "mlp", "router", "top"), 9, "layers[1].mlp.router.top"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "layers[0].mixer.rot.dims"),
    (("norm",), None, "norm"),
    (("vocab",), "many", "vocab"),
])
def test_refusals_name_the_key(path, value, key):
    from mrun_b200.config import ConfigError, ZasesunConfig
    cfg = copy.deepcopy(ZTINY["P"]["config"])
    at = cfg
    for step in path[:-1]:
        at = at[step]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as error:
        ZasesunConfig.from_dict(cfg)
    assert key in str(error.value)


def test_random_folder_loads_back(tmp_path):
    from mrun_b200 import registry
    from mrun_b200.weights import load_tensors
    folder = make_folder("P", str(tmp_path / "p"))
    config = registry.load_config(folder)
    assert config == zconfig("P")
    tensors = load_tensors(folder, config.to_spec())
    cfg, stored = load_folder(folder)
    assert set(tensors) == set(stored)
    os.remove(os.path.join(folder, "model.safetensors"))


# ------------------------------------------------------------------ the plain implementation, by hand

def test_plain_rms_norm_and_gates():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    out = plain.rms_norm(x, torch.tensor([1.0, 2.0], dtype=torch.float64), 0.5)
    inv = 1.0 / math.sqrt(12.5 + 0.5)
    assert torch.allclose(out, torch.tensor([[3.0 * inv, 8.0 * inv]], dtype=torch.float64))
    z = torch.tensor([0.5], dtype=torch.float64)
    want = 0.25 * (1.0 + math.tanh(math.sqrt(2.0 / math.pi) * (0.5 + 0.044715 * 0.125)))
    assert abs(float(plain.gelu_tanh(z)) - want) < 1e-15
    assert float(plain.soft_cap(torch.tensor(2.0, dtype=torch.float64), 4.0)) == pytest.approx(4.0 * math.tanh(0.5))


def test_plain_rotary_frequencies_by_hand():
    rot = {"dims": 8, "base": 16.0}
    freq, magnitude = plain.rotary_frequencies(rot)
    assert magnitude == 1.0 and torch.allclose(freq, torch.tensor([1.0, 0.5, 0.25, 0.125], dtype=torch.float64))
    # original 64, base 16, dims 8: d(t) = 8 ln(64 / (2 pi t)) / (2 ln 16); d(4) = 1.348.., d(1) = 3.348..
    rot["scaling"] = {"factor": 4.0, "original": 64, "fast": 4.0, "slow": 1.0}
    freq, magnitude = plain.rotary_frequencies(rot)
    assert magnitude == pytest.approx(0.1 * math.log(4.0) + 1.0)
    lo, hi = 1, 4                                      # floor(1.348), ceil(3.348)
    ramp = [min(max((i - lo) / (hi - lo), 0.0), 1.0) for i in range(4)]
    base = [1.0, 0.5, 0.25, 0.125]
    want = [f / 4.0 * r + f * (1.0 - r) for f, r in zip(base, ramp)]
    assert torch.allclose(freq, torch.tensor(want, dtype=torch.float64))


def test_plain_rotation_pairs_neighbours():
    x = torch.tensor([[[1.0, 0.0, 0.0, 2.0, 5.0]]], dtype=torch.float64)          # one token, one head
    out = plain.rotate_interleaved(x, torch.tensor([3]), {"dims": 4, "base": 4.0})
    a0, a1 = 3.0, 3.0 * 0.5
    want = [math.cos(a0), math.sin(a0), -2.0 * math.sin(a1), 2.0 * math.cos(a1), 5.0]
    assert torch.allclose(out[0, 0], torch.tensor(want, dtype=torch.float64))


def test_plain_router_keeps_scores_unscaled():
    h = torch.eye(3, dtype=torch.float64)[:1]
    w = {"p.router": torch.tensor([[2.0, 0, 0], [1.0, 0, 0], [0.0, 0, 0]], dtype=torch.float64)}
    for e in range(3):
        w[f"p.e{e}.up"] = torch.tensor([[float(e + 1), 0, 0]], dtype=torch.float64)
        w[f"p.e{e}.down"] = torch.tensor([[1.0], [0.0], [0.0]], dtype=torch.float64)
    out = plain.routed_feed_forward(h, w, "p", {"router": {"experts": 3, "top": 2}})
    s = torch.softmax(torch.tensor([2.0, 1.0, 0.0], dtype=torch.float64), 0)
    assert float(out[0, 0]) == pytest.approx(float(s[0] * 1.0 + s[1] * 4.0))       # relu(e + 1)^2, no renormalising
