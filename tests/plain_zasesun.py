"""A plain, slow statement of the Zasesun decoder in torch on the CPU: one function per mechanism,
whole sequences at a time, no cache, no batching, nothing shared with the engine.

``cfg`` is the parsed config.json, ``w`` a dict of tensors by checkpoint name.  Everything is
computed in ``dtype`` (float64 by default) from the stored values, so the result is the design
itself, free of any rounding choice.
"""
from __future__ import annotations

import math

import torch


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_frequencies(rot, dtype=torch.float64):
    """(frequency of every pair, factor on cos and sin) of a rotary setting with optional
    YaRN-style scaling ``rot['scaling'] = {factor, original, fast, slow}``."""
    dims, base = int(rot["dims"]), float(rot["base"])
    pairs = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(pairs)], dtype=dtype)
    scaling = rot.get("scaling")
    if not scaling:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(pairs)], dtype=dtype)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x, positions, rot):
    """Rotates the first ``rot['dims']`` features of the last axis of ``x`` ([tokens, ..., n]);
    feature 2i pairs with 2i + 1.  ``positions``: one per token."""
    dims = int(rot["dims"])
    freq, magnitude = rotary_frequencies(rot, x.dtype)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]                 # [tokens, pairs]
    cos, sin = torch.cos(angle) * magnitude, torch.sin(angle) * magnitude
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def latent_attention(h, w, prefix, mixer, eps, positions):
    """The mixer of one layer over a whole sequence ``h`` [tokens, width]."""
    heads, dim, rot_dim = int(mixer["heads"]), int(mixer["dim"]), int(mixer["rot_dim"])
    vdim, kv_rank = int(mixer["vdim"]), int(mixer["kv_rank"])
    tokens = h.shape[0]
    g = lambda name: w[f"{prefix}.{name}"].to(h.dtype)
    cq = rms_norm(h @ g("dq").T, g("dq.norm"), eps)
    q = (cq @ g("uq").T).view(tokens, heads, dim + rot_dim)
    down = h @ g("dkv").T
    c = rms_norm(down[:, :kv_rank], g("dkv.norm"), eps)
    k_rot = rotate_interleaved(down[:, kv_rank:], positions, mixer["rot"])          # [tokens, rot_dim]
    q_rot = rotate_interleaved(q[..., dim:], positions, mixer["rot"])               # [tokens, heads, rot_dim]
    k_plain = (c @ g("uk").T).view(tokens, heads, dim)
    value = (c @ g("uv").T).view(tokens, heads, vdim)
    scores = torch.einsum("thd,shd->hts", q[..., :dim], k_plain) + torch.einsum("thd,sd->hts", q_rot, k_rot)
    scores = scores * float(mixer["scale"])
    visible = positions[None, :] <= positions[:, None]                              # [t, s]
    scores = scores.masked_fill(~visible[None], float("-inf"))
    weights = torch.softmax(scores, dim=-1)
    mixed = torch.einsum("hts,shd->thd", weights, value).reshape(tokens, heads * vdim)
    return mixed @ g("o").T


def dense_feed_forward(h, w, prefix):
    g = lambda name: w[f"{prefix}.{name}"].to(h.dtype)
    return (gelu_tanh(h @ g("gate").T) * (h @ g("up").T)) @ g("down").T


def expert(h, w, prefix):
    """down(relu(up h)^2)."""
    g = lambda name: w[f"{prefix}.{name}"].to(h.dtype)
    return torch.relu(h @ g("up").T) ** 2 @ g("down").T


def routed_feed_forward(h, w, prefix, mlp, margins=None):
    """``margins`` (a list) gets, per token, how far the router's logit of the last expert chosen
    lies above that of the first one left out (infinite when every expert is chosen)."""
    experts, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    logits = h @ w[f"{prefix}.router"].to(h.dtype).T
    scores = torch.softmax(logits, dim=-1)                                          # [tokens, experts]
    chosen = torch.topk(scores, top, dim=-1).indices
    if margins is not None:
        ranked = torch.sort(logits, dim=-1, descending=True).values
        margins.append(ranked[:, top - 1] - ranked[:, top] if top < experts
                       else torch.full((h.shape[0],), float("inf"), dtype=h.dtype))
    out = torch.zeros_like(h)
    for e in range(experts):
        uses = (chosen == e).any(-1)
        if uses.any():
            out[uses] += scores[uses, e:e + 1] * expert(h[uses], w, f"{prefix}.e{e}")
    if mlp.get("shared"):
        out = out + expert(h, w, f"{prefix}.shared")
    return out


def feed_forward(h, w, prefix, mlp, margins=None):
    if mlp["kind"] == "dense":
        return dense_feed_forward(h, w, prefix)
    if mlp["kind"] == "moe":
        return routed_feed_forward(h, w, prefix, mlp, margins)
    raise ValueError(mlp["kind"])


def soft_cap(logits, cap):
    return cap * torch.tanh(logits / cap)


def forward(cfg, w, tokens, dtype=torch.float64, return_layers=False, margins=None):
    """Logits [tokens, vocab] of one sequence of token ids (and the stream after every layer).
    ``margins``: a list that gets every routed layer's router margins (see
    :func:`routed_feed_forward`)."""
    eps, m = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    ids = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(ids))
    x = w["embed"].to(dtype)[ids]
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        norm = lambda v, name: rms_norm(v, w[f"{p}.{name}"].to(dtype), eps)
        if layer["type"] != "latent_attention":
            raise ValueError(layer["type"])
        a = latent_attention(norm(x, "norm1"), w, f"{p}.mix", layer["mixer"], eps, positions)
        x = x + m * norm(a, "norm1b")
        if layer.get("mlp"):
            f = feed_forward(norm(x, "norm2"), w, f"{p}.mlp", layer["mlp"], margins)
            x = x + m * norm(f, "norm2b")
        after.append(x)
    logits = rms_norm(x, w["final.norm"].to(dtype), eps) @ w["embed"].to(dtype).T
    if cfg.get("logit_softcap"):
        logits = soft_cap(logits, float(cfg["logit_softcap"]))
    return (logits, torch.stack(after)) if return_layers else logits
