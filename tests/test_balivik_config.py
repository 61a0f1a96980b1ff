"""Balivik without a GPU: the registry, the configuration read back from its own dictionary, its refusals, the tensor
names and shapes of every part, the run order of a loop, the random-weights folder, and
hand-worked values of the plain implementation's functions."""
from __future__ import annotations

import copy
import json
import math
import os

import pytest
import torch

import plain_balivik as plain
from tiny_balivik import BTINY, bconfig, load_folder, make_folder, tokens_of


def test_registry_resolves_the_architecture():
    from mrun_b200 import registry
    from mrun_b200.config.balivik import BalivikConfig
    assert registry.resolve({"architecture": "Balivik"}) is BalivikConfig
    assert "balivik" in registry.supported()


@pytest.mark.parametrize("name", sorted(BTINY))
def test_read_back_and_spec(name):
    from mrun_b200.config.balivik import BalivikConfig
    from mrun_b200.weights.loader import expected_tensors
    config = bconfig(name)
    raw = BTINY[name]["config"]
    assert config.to_dict() == raw
    assert BalivikConfig.from_dict(json.loads(json.dumps(config.to_dict()))) == config
    spec = config.to_spec()
    assert [e.layer for e in spec.run_order()] == plain.run_order(raw)
    assert spec.streams == (raw.get("streams") or 1)
    names = {t.name: t.shape for t in expected_tensors(spec)}
    assert names["embed"] == names["head"] == (raw["vocab"], raw["width"]) and names["final.norm"] == ()
    for i, layer in enumerate(raw["layers"]):
        m, p = layer["mixer"], f"l{i}"
        assert names[f"{p}.norm1"] == ()
        assert (f"{p}.canon1" in names) == ("canon" in raw)
        if "canon" in raw:
            assert names[f"{p}.canon1"] == (raw["width"], raw["canon"]["taps"])
        assert (f"{p}.hc1.mix" in names) == ("streams" in raw)
        if "streams" in raw:
            s = raw["streams"]
            assert names[f"{p}.hc1.in"] == names[f"{p}.hc1.out"] == (s,) and names[f"{p}.hc1.mix"] == (s, s)
        assert (f"{p}.norm2" in names) == (f"{p}.hc2.in" in names or "streams" not in raw) == (layer["mlp"] is not None) \
            or "streams" not in raw
        if layer["type"] == "attention":
            assert names[f"{p}.mix.q"] == (m["heads"] * 2 * m["dim"], raw["width"])
            assert names[f"{p}.mix.k"] == (m["kv_heads"] * 2 * m["dim"], raw["width"])
            assert names[f"{p}.mix.v"] == (m["kv_heads"] * m["vdim"], raw["width"])
            assert names[f"{p}.mix.o"] == (raw["width"], m["heads"] * m["vdim"])
            assert names[f"{p}.mix.lq1"] == names[f"{p}.mix.lk2"] == (m["dim"],)
        elif layer["type"] == "lightning":
            assert names[f"{p}.mix.q"] == names[f"{p}.mix.k"] == (m["heads"] * m["dim"], raw["width"])
            assert names[f"{p}.mix.v"] == names[f"{p}.mix.g"] == (m["heads"] * m["vdim"], raw["width"])
            assert names[f"{p}.mix.norm"] == (m["heads"] * m["vdim"],)
        else:
            assert names[f"{p}.mix.q"] == (m["kv_heads"] * m["dim"], raw["width"])
            assert names[f"{p}.mix.k.conv"] == (m["kv_heads"] * m["dim"], m["conv"])
            assert names[f"{p}.mix.v.conv"] == (m["heads"] * m["vdim"], m["conv"])
            assert names[f"{p}.mix.a1"] == (m["decay_rank"], raw["width"])
            assert names[f"{p}.mix.a2"] == (m["heads"] * m["dim"], m["decay_rank"])
            assert names[f"{p}.mix.g2"] == (m["heads"] * m["vdim"], m["gate_rank"])
            assert names[f"{p}.mix.dt_bias"] == (m["heads"] * m["dim"],) and names[f"{p}.mix.A_log"] == (m["heads"],)
            assert names[f"{p}.mix.norm"] == (m["vdim"],) and names[f"{p}.mix.b"] == (m["heads"], raw["width"])
        mlp = layer["mlp"]
        if mlp and mlp["kind"] == "moe":
            assert names[f"{p}.mlp.table"] == (raw["vocab"], mlp["router"]["top"])
            last = mlp["router"]["experts"] - 1
            assert names[f"{p}.mlp.e{last}.gate"] == names[f"{p}.mlp.e0.up"] == (mlp["expert"]["ff"], raw["width"])
            assert f"{p}.mlp.e{last + 1}.gate" not in names
        elif mlp:
            assert names[f"{p}.mlp.down"] == (raw["width"], mlp["ff"])
    assert config.num_parameters() == sum(math.prod(shape) for shape in names.values())


def test_refusals_name_the_key():
    from mrun_b200.config.balivik import BalivikConfig
    from mrun_b200.config.base import ConfigError
    base = BTINY["U"]["config"]

    def refused(change, key):
        cfg = copy.deepcopy(base)
        change(cfg)
        with pytest.raises(ConfigError) as error:
            BalivikConfig.from_dict(cfg)
        assert key in str(error.value), str(error.value)

    refused(lambda c: c["layers"][0].update(type="mamba"), "layers[0].type")
    refused(lambda c: c["layers"][1]["mixer"].update(heads=5), "layers[1].mixer.heads")
    refused(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "layers[1].mixer.rot.dims")
    refused(lambda c: c["layers"][1]["mixer"].pop("diff"), "layers[1].mixer.diff")
    refused(lambda c: c["layers"][2]["mixer"].update(decay=[0.5]), "layers[2].mixer.decay")
    refused(lambda c: c["layers"][0]["mixer"].pop("decay_rank"), "layers[0].mixer.decay_rank")
    refused(lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "layers[1].mlp.router.top")
    refused(lambda c: c["layers"][1]["mlp"]["expert"].pop("limit"), "layers[1].mlp.expert.limit")
    refused(lambda c: c["layers"][0]["mlp"].update(kind="conv"), "layers[0].mlp.kind")
    refused(lambda c: c["loop"].update(stop=9), "loop")
    refused(lambda c: c["canon"].update(taps=0), "canon.taps")
    refused(lambda c: c.update(streams=9), "streams")
    refused(lambda c: c.pop("width"), "width")


def test_defaults_of_keys_a_config_may_leave_out():
    from mrun_b200.config.balivik import BalivikConfig
    cfg = copy.deepcopy(BTINY["V"]["config"])
    cfg["layers"][0]["mixer"].pop("kv_heads")               # as many key heads as heads
    cfg["layers"][2]["mixer"].pop("kv_heads")
    cfg["layers"][1]["mixer"]["decay"] = 0.9                # one decay for all heads
    config = BalivikConfig.from_dict(cfg)
    assert config.layers[0].mixer.kv_heads == 5 and config.layers[2].mixer.kv_heads == 2
    assert config.layers[1].mixer.decay == (0.9, 0.9)
    assert config.streams is None and config.canon_taps == 0 and config.loop is None and config.logit_scale is None
    spec = config.to_spec()
    assert spec.streams == 1 and spec.logits_transform is None and all(l.streams == 0 for l in spec.layers)


def test_random_folder_and_ranks_from_the_checkpoint(tmp_path):
    """The inner sizes of the delta rule's low-rank projections come from the checkpoint's shapes
    when config.json does not give them."""
    from mrun_b200 import registry
    from mrun_b200.weights import load_tensors
    folder = make_folder("X", str(tmp_path / "x"))
    cfg, weights = load_folder(folder)
    for layer in cfg["layers"]:
        layer["mixer"].pop("decay_rank", None)
        layer["mixer"].pop("gate_rank", None)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    config = registry.load_config(folder)
    assert config.layers[1].mixer.decay_rank == 10 and config.layers[1].mixer.gate_rank == 3
    tensors = load_tensors(folder, config.to_spec())
    table = tensors["l0.mlp.table"]
    assert table.dtype == torch.int32 and table.shape == (128, 2)
    assert int(table.min()) >= 0 and int(table.max()) < 7 and bool((table[:, 0] != table[:, 1]).all())
    assert tensors["l0.norm1"].shape == () and tensors["l1.hc1.mix"].shape == (4, 4)


# ------------------------------------------------------------------ hand-worked values of the plain functions

def test_plain_rms_norm_and_conv():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(plain.rms_norm(x, 2.0, 0.0), torch.tensor([[6.0, 8.0]], dtype=torch.float64) / math.sqrt(12.5))
    seq = torch.tensor([[1.0], [2.0], [3.0], [4.0]], dtype=torch.float64)
    w = torch.tensor([[0.5, -1.0, 2.0]], dtype=torch.float64)           # the last tap meets the token itself
    assert plain.causal_conv(seq, w).flatten().tolist() == [2.0, 3.0, 4.5, 6.0]


def test_plain_rotation_pairs_first_and_second_half():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]]], dtype=torch.float64)
    out = plain.rotate_half(x, torch.tensor([1]), 4, 4.0)              # frequencies 1 and 1/2; feature 4 stays
    c0, s0, c1, s1 = math.cos(1.0), math.sin(1.0), math.cos(0.5), math.sin(0.5)
    want = [1 * c0 - 3 * s0, 2 * c1 - 4 * s1, 3 * c0 + 1 * s0, 4 * c1 + 2 * s1, 5.0]
    assert torch.allclose(out.flatten(), torch.tensor(want, dtype=torch.float64))
    assert torch.equal(plain.rotate_half(x, torch.tensor([0]), 4, 4.0), x)


def test_plain_lightning_two_tokens():
    eye = torch.eye(2, dtype=torch.float64)
    big = 50.0                                                          # silu(50) = 50, sigmoid(50) = 1
    w = {"m.q": eye, "m.k": eye, "m.v": eye, "m.g": eye, "m.o": eye, "m.norm": torch.ones(2, dtype=torch.float64)}
    h = torch.tensor([[big, 0.0], [0.0, big]], dtype=torch.float64)
    out = plain.lightning(h, w, "m", {"heads": 1, "dim": 2, "vdim": 2, "decay": [0.5]}, 0.0)
    # token 0: S = k0 v0^T, o = S^T q0 = (2500 * 50, 0); token 1: S = S/2 + k1 v1^T, o = (0, 2500 * 50)
    norm = lambda v: [a / math.sqrt(sum(b * b for b in v) / 2) for a in v]
    assert torch.allclose(out[0], torch.tensor(norm([125000.0, 0.0]), dtype=torch.float64) * torch.sigmoid(h[0]))
    assert torch.allclose(out[1], torch.tensor(norm([0.0, 125000.0]), dtype=torch.float64) * torch.sigmoid(h[1]))


def test_plain_expert_clamps_and_table_weights():
    one = torch.ones(1, 1, dtype=torch.float64)
    w = {"f.e0.gate": 5 * one, "f.e0.up": -9 * one, "f.e0.down": one, "f.e1.gate": one, "f.e1.up": one, "f.e1.down": one,
         "f.table": torch.tensor([[0, 1], [1, 0]], dtype=torch.int32)}
    h = torch.ones(1, 1, dtype=torch.float64)
    sig = lambda z: 1 / (1 + math.exp(-z))
    e0 = 2.0 * sig(1.702 * 2.0) * (-2.0 + 1.0)                          # gate capped at 2, up clamped to -2
    e1 = 1.0 * sig(1.702) * 2.0
    assert math.isclose(float(plain.expert(h, w, "f.e0", 2.0)), e0)
    mlp = {"router": {"experts": 2, "top": 2}, "expert": {"limit": 2.0}}
    assert math.isclose(float(plain.table_moe(h, w, "f", mlp, [1])), (e0 + e1) / 2)


def test_plain_loop_order_and_streams():
    assert plain.run_order({"layers": [0] * 5, "loop": {"start": 1, "stop": 3, "times": 3}}) == [0, 1, 2, 1, 2, 1, 2, 3, 4]
    assert plain.run_order({"layers": [0] * 3}) == [0, 1, 2]
    streams = torch.tensor([[[1.0]], [[10.0]]], dtype=torch.float64)    # two streams, one token, width 1
    w = {"h.in": torch.tensor([1.0, 0.5], dtype=torch.float64), "h.out": torch.tensor([2.0, -1.0], dtype=torch.float64),
         "h.mix": torch.tensor([[1.0, 3.0], [0.0, 1.0]], dtype=torch.float64)}       # [from, to]
    out = plain.hyper_step(streams, w, "h", lambda h: h * 0 + 7.0, 1.0, 0.0)
    assert out.flatten().tolist() == [1.0 + 14.0, 3.0 + 10.0 - 7.0]
