"""Small Zasesun configurations for the tests, none like another: layers of one model differ in
their head counts, latent ranks and rotary settings; cache rows of 32, 48, 64, 128 and 272 features
(the mma.sync, TMA / tcgen05 and CUDA-core attention kernels); dense, routed and absent
feed-forwards; one to all experts chosen; with and without a shared expert, a stretch of the
rotary frequencies, a soft cap; residual multipliers on both sides of one."""
from __future__ import annotations

import json
import os

import numpy as np
import torch


def mixer(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base=10000.0, scaling=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
            "scale": scale, "rot": rot}


def layer(mix, mlp):
    return {"type": "latent_attention", "mixer": mix, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


ZTINY = {
    # cache rows of 48 and 64 features; a layer without a feed-forward; a stretch whose band
    # lies inside the pairs; two of five experts
    "P": dict(
        config={"architecture": "Zasesun", "vocab": 300, "width": 64, "norm": {"eps": 1e-6}, "residual_mult": 0.7,
                "logit_softcap": 3.0,
                "layers": [layer(mixer(2, 16, 8, 24, 24, 40, 0.3), dense(96)),
                           layer(mixer(3, 32, 16, 16, 40, 48, 0.25, base=500.0, scaling=(4.0, 64, 8.0, 2.0)),
                                 moe(5, 2, 48, shared=32)),
                           layer(mixer(2, 8, 8, 40, 16, 40, 0.5, base=100.0, scaling=(1.5, 32, 4.0, 0.5)), None)]},
        seed=3, std=0.1, norm_noise=0.2, page_size=16),
    # a cache row of 128 features, five heads, one of three experts and no
    # shared expert, no soft cap, a multiplier above one, a width that is no multiple of 64
    "Q": dict(
        config={"architecture": "Zasesun", "vocab": 257, "width": 96, "norm": {"eps": 1e-5}, "residual_mult": 1.25,
                "layers": [layer(mixer(5, 24, 16, 24, 56, 112, 0.1, base=1000000.0), moe(3, 1, 40)),
                           layer(mixer(5, 24, 16, 24, 56, 112, 0.1, base=1000000.0, scaling=(8.0, 128, 16.0, 1.0)),
                                 dense(136))]},
        seed=5, std=0.1, norm_noise=0.1, page_size=8),
    # a cache row of 272 features (no tensor-core attention kernel takes it), twenty heads (more
    # than a decode kernel's group), every expert chosen, pages of four tokens
    "R": dict(
        config={"architecture": "Zasesun", "vocab": 128, "width": 80, "norm": {"eps": 1e-4}, "residual_mult": 0.4,
                "logit_softcap": 30.0,
                "layers": [layer(mixer(20, 8, 8, 8, 32, 264, 0.4, base=200.0, scaling=(2.0, 16, 2.0, 1.0)),
                                 moe(4, 4, 24, shared=8)),
                           layer(mixer(1, 48, 32, 56, 8, 24, 0.2), dense(72))]},
        seed=9, std=0.1, norm_noise=0.3, page_size=4),
    # sizes that fit no vector width or alignment: an odd width, latent ranks and head sizes that are
    # no multiple of 8, seven heads, three of seven experts of an odd size, an odd vocabulary
    "S": dict(
        config={"architecture": "Zasesun", "vocab": 131, "width": 100, "norm": {"eps": 1e-5}, "residual_mult": 0.9,
                "logit_softcap": 5.0,
                "layers": [layer(mixer(7, 10, 6, 14, 18, 50, 0.35, base=3000.0, scaling=(3.0, 48, 6.0, 1.5)),
                                 moe(7, 3, 22, shared=12)),
                           layer(mixer(3, 12, 10, 6, 30, 21, 0.3, base=700.0), dense(90))]},
        seed=13, std=0.1, norm_noise=0.2, page_size=16),
}


def zconfig(name: str):
    from mrun_b200.config import ZasesunConfig
    return ZasesunConfig.from_dict(ZTINY[name]["config"])


def make_folder(name: str, folder: str) -> str:
    from mrun_b200.weights import write_random_model
    t = ZTINY[name]
    return write_random_model(zconfig(name), folder, seed=t["seed"], std=t["std"], norm_noise=t["norm_noise"])


def load_folder(folder: str):
    """config.json as a dict and every tensor as stored."""
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, dict(load_file(os.path.join(folder, "model.safetensors")))


def tokens_of(vocab: int, length: int, seed: int) -> list:
    return np.random.default_rng(seed).integers(0, vocab, size=length).tolist()
