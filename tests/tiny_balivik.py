"""Small Balivik configurations for the tests, none like another: every mixer kind in several
sizes (key sizes that fit one, two and four register tiles of the scans, value sizes that are no
multiple of 32, grouped and ungrouped key heads), with and without several streams, an input
convolution, a loop, a logit scale and a feed-forward; dense and table-routed feed-forwards with
one to all experts chosen; differential attention on the tensor-core path (value chunks of the
key size) and on the CUDA-core path."""
from __future__ import annotations

import json
import os

import numpy as np
import torch


def attention(heads, kv_heads, dim, vdim, scale, diff, rot_dims=0, base=10000.0):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if rot_dims is not None:
        out["rot"] = {"base": base, "dims": rot_dims}
    return out


def lightning(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def delta(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
            "decay_rank": decay_rank, "gate_rank": gate_rank}


def layer(kind, mix, mlp):
    return {"type": kind, "mixer": mix, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}


BTINY = {
    # two streams, three taps, the middle two layers run three times; the attention's values are two
    # chunks of the key size (tensor-core path in bfloat16), grouped heads everywhere, a layer
    # without a feed-forward, three of five experts
    "U": dict(
        config={"architecture": "Balivik", "vocab": 300, "width": 64, "norm": {"eps": 1e-6}, "streams": 2,
                "canon": {"taps": 3}, "loop": {"start": 1, "stop": 3, "times": 3}, "logit_scale": 0.5,
                "layers": [layer("channel_delta", delta(4, 2, 16, 24, 4, 8, 12), dense(96)),
                           layer("attention", attention(6, 3, 16, 32, 0.25, 0.2, rot_dims=8, base=500.0), moe(5, 3, 40, 1.5)),
                           layer("lightning", lightning(3, 24, 40, (0.5, 0.9, 0.99)), None),
                           layer("attention", attention(2, 2, 32, 32, 0.18, 0.35, rot_dims=32), dense(72))]},
        seed=3, std=0.1, norm_noise=0.2, page_size=16),
    # no streams, no input convolution, no loop, no logit scale; sizes that fit no vector width:
    # an odd width, key and value sizes that are no multiple of 16 (CUDA-core attention), a key
    # size of 72 (two register tiles), one expert of three and all of four
    "V": dict(
        config={"architecture": "Balivik", "vocab": 131, "width": 100, "norm": {"eps": 1e-5},
                "layers": [layer("attention", attention(5, 5, 20, 28, 0.22, 0.1, rot_dims=20, base=100.0), moe(3, 1, 22, 2.5)),
                           layer("lightning", lightning(2, 72, 33, (0.8, 0.97)), moe(4, 4, 18, 1.0)),
                           layer("channel_delta", delta(2, 1, 40, 70, 2, 6, 5), dense(90)),
                           layer("attention", attention(4, 1, 12, 36, 0.3, 0.5, rot_dims=None), None)]},
        seed=5, std=0.1, norm_noise=0.1, page_size=8),
    # one stream with coefficients of its own, two taps, a loop that runs once, key sizes of 64
    # (TMA and tcgen05 attention, one value chunk), 160 (two slices of the scan's key rows) and
    # 128, pages of four tokens, four streams would not fit here: see X
    "W": dict(
        config={"architecture": "Balivik", "vocab": 257, "width": 96, "norm": {"eps": 1e-4}, "streams": 1,
                "canon": {"taps": 2}, "loop": {"start": 0, "stop": 2, "times": 1}, "logit_scale": 2.0,
                "layers": [layer("attention", attention(4, 2, 64, 64, 0.125, 0.25, rot_dims=16, base=1000000.0), dense(136)),
                           layer("lightning", lightning(2, 160, 16, (0.95, 0.6)), moe(6, 2, 24, 3.0)),
                           layer("channel_delta", delta(3, 3, 128, 8, 3, 4, 4), moe(2, 1, 48, 0.5))]},
        seed=9, std=0.1, norm_noise=0.3, page_size=4),
    # four streams, five taps, the whole model is the loop, run twice
    "X": dict(
        config={"architecture": "Balivik", "vocab": 128, "width": 80, "norm": {"eps": 1e-5}, "streams": 4,
                "canon": {"taps": 5}, "loop": {"start": 0, "stop": 2, "times": 2},
                "layers": [layer("lightning", lightning(5, 16, 16, (0.3, 0.7, 0.9, 0.97, 1.0)), moe(7, 2, 16, 2.0)),
                           layer("channel_delta", delta(6, 2, 24, 20, 5, 10, 3), None)]},
        seed=13, std=0.1, norm_noise=0.2, page_size=16),
}


def bconfig(name: str):
    from mrun_b200.config.balivik import BalivikConfig
    return BalivikConfig.from_dict(BTINY[name]["config"])


def make_folder(name: str, folder: str) -> str:
    from mrun_b200.weights import write_random_model
    t = BTINY[name]
    return write_random_model(bconfig(name), folder, seed=t["seed"], std=t["std"], norm_noise=t["norm_noise"])


def load_folder(folder: str):
    """config.json as a dict and every tensor as stored."""
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, dict(load_file(os.path.join(folder, "model.safetensors")))


def tokens_of(vocab: int, length: int, seed: int) -> list:
    return np.random.default_rng(seed).integers(0, vocab, size=length).tolist()
