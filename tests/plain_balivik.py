"""A plain, slow statement of the Balivik decoder in torch on the CPU: one function per mechanism,
whole sequences at a time, token-by-token loops for the recurrences, no cache, no batching,
nothing shared with the engine.

``cfg`` is the parsed config.json, ``w`` a dict of tensors by checkpoint name.  Everything is
computed in ``dtype`` (float64 by default) from the stored values.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis; weight may be one number."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def silu(z):
    return z * torch.sigmoid(z)


def causal_conv(x, weight):
    """y[t, c] = sum_j weight[c, j] * x[t - taps + 1 + j, c], zeros before the start.
    ``x``: [tokens, channels]; ``weight``: [channels, taps]; the last tap meets the token itself."""
    tokens, channels = x.shape
    taps = weight.shape[1]
    padded = torch.cat([x.new_zeros(taps - 1, channels), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + padded[j:j + tokens] * weight[:, j]
    return y


def rotate_half(x, positions, dims, base):
    """Rotates the first ``dims`` features of the last axis of ``x`` ([tokens, ..., n]); feature i
    pairs with i + dims/2 and turns by position * base^(-2i/dims)."""
    if not dims:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle), torch.sin(angle)
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


def differential_attention(h, w, prefix, m, eps, positions):
    """Two softmax maps a head over the same values, o = a1 - lambda * a2, normed over the head's
    values without a weight and multiplied by 1 - diff."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ w[f"{prefix}.q"].T).view(T, H, 2, D)
    k = (h @ w[f"{prefix}.k"].T).view(T, G, 2, D)
    v = (h @ w[f"{prefix}.v"].T).view(T, G, V)
    rot = m.get("rot") or {}
    dims = int(rot.get("dims", 0))
    if dims:
        q = rotate_half(q, positions, dims, float(rot["base"]))
        k = rotate_half(k, positions, dims, float(rot["base"]))
    lam = (torch.exp((w[f"{prefix}.lq1"] * w[f"{prefix}.lk1"]).sum())
           - torch.exp((w[f"{prefix}.lq2"] * w[f"{prefix}.lk2"]).sum()) + m["diff"])
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    out = h.new_zeros(T, H, V)
    for head in range(H):
        g = head // (H // G)
        maps = []
        for which in range(2):
            s = (q[:, head, which] @ k[:, g, which].T) * m["scale"]
            s = s.masked_fill(~mask, float("-inf"))
            maps.append(torch.softmax(s, dim=-1) @ v[:, g])
        o = maps[0] - lam * maps[1]
        o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps)
        out[:, head] = o * (1.0 - m["diff"])
    return out.reshape(T, H * V) @ w[f"{prefix}.o"].T


def lightning(h, w, prefix, m, eps):
    """Linear attention with one decay a head: S = decay * S + k v^T, o = S^T q."""
    H, D, V = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(h @ w[f"{prefix}.q"].T).view(T, H, D)
    k = silu(h @ w[f"{prefix}.k"].T).view(T, H, D)
    v = silu(h @ w[f"{prefix}.v"].T).view(T, H, V)
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    S = h.new_zeros(H, D, V)
    out = h.new_zeros(T, H, V)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(out.reshape(T, H * V), w[f"{prefix}.norm"], eps)
    o = o * torch.sigmoid(h @ w[f"{prefix}.g"].T)
    return o @ w[f"{prefix}.o"].T


def channel_delta(h, w, prefix, m, eps):
    """Gated delta rule with a decay per head and key channel."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(h @ w[f"{prefix}.q"].T, w[f"{prefix}.q.conv"])).view(T, G, D)
    k = silu(causal_conv(h @ w[f"{prefix}.k"].T, w[f"{prefix}.k.conv"])).view(T, G, D)
    v = silu(causal_conv(h @ w[f"{prefix}.v"].T, w[f"{prefix}.v.conv"])).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[f"{prefix}.b"].T)                                   # [T, H]
    a = (h @ w[f"{prefix}.a1"].T) @ w[f"{prefix}.a2"].T + w[f"{prefix}.dt_bias"]
    g = torch.exp(-torch.exp(w[f"{prefix}.A_log"])[None, :, None] * F.softplus(a).view(T, H, D))
    S = h.new_zeros(H, D, V)
    out = h.new_zeros(T, H, V)
    rep = H // G
    for t in range(T):
        kt = k[t].repeat_interleave(rep, dim=0)                                    # [H, D]
        qt = q[t].repeat_interleave(rep, dim=0)
        S = g[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, kt))
        S = S + kt[:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, qt)
    o = out / torch.sqrt((out * out).mean(-1, keepdim=True) + eps) * w[f"{prefix}.norm"]
    gate = torch.sigmoid((h @ w[f"{prefix}.g1"].T) @ w[f"{prefix}.g2"].T).view(T, H, V)
    return (o * gate).reshape(T, H * V) @ w[f"{prefix}.o"].T


def dense_ff(h, w, prefix):
    return (silu(h @ w[f"{prefix}.gate"].T) * (h @ w[f"{prefix}.up"].T)) @ w[f"{prefix}.down"].T


def expert(h, w, prefix, limit):
    g = torch.clamp(h @ w[f"{prefix}.gate"].T, max=limit)
    u = torch.clamp(h @ w[f"{prefix}.up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[f"{prefix}.down"].T


def table_moe(h, w, prefix, mlp, tokens):
    """Every token's experts come from a table by its token id; each weighs 1/top."""
    top = mlp["router"]["top"]
    table = w[f"{prefix}.table"]
    out = torch.zeros(h.shape[0], w[f"{prefix}.e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e in table[int(tokens[t])].tolist():
            out[t] = out[t] + expert(h[t:t + 1], w, f"{prefix}.e{int(e)}", mlp["expert"]["limit"])[0] / top
    return out


def feed_forward(h, w, prefix, mlp, tokens):
    if mlp["kind"] == "dense":
        return dense_ff(h, w, prefix)
    return table_moe(h, w, prefix, mlp, tokens)


def mixer(kind, h, w, prefix, m, eps, positions):
    if kind == "attention":
        return differential_attention(h, w, prefix, m, eps, positions)
    if kind == "lightning":
        return lightning(h, w, prefix, m, eps)
    if kind == "channel_delta":
        return channel_delta(h, w, prefix, m, eps)
    raise ValueError(kind)


def run_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))


def hyper_step(streams, w, prefix, sublayer, norm_weight, eps):
    """One sublayer under hyper-connections.  ``streams``: [S, tokens, width]."""
    u = torch.einsum("s,stw->tw", w[f"{prefix}.in"], streams)
    y = sublayer(rms_norm(u, norm_weight, eps))
    return torch.einsum("sr,stw->rtw", w[f"{prefix}.mix"], streams) + w[f"{prefix}.out"][:, None, None] * y[None]


def forward(cfg, w, tokens, dtype=torch.float64, layers_out=None):
    """Logits [tokens, vocab] of one sequence.  ``layers_out``: a list that gets the residual
    stream (the sum of the streams) after every layer run."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(tokens))
    x = w["embed"][tokens]
    S = cfg.get("streams")
    canon = cfg.get("canon")
    streams = x[None].repeat(S, 1, 1) if S else None
    for i in run_order(cfg):
        layer, p = cfg["layers"][i], f"l{i}"

        def mix(h):
            if canon:
                h = h + causal_conv(h, w[f"{p}.canon1"])
            return mixer(layer["type"], h, w, f"{p}.mix", layer["mixer"], eps, positions)

        ff = (lambda h: feed_forward(h, w, f"{p}.mlp", layer["mlp"], tokens)) if layer.get("mlp") else None
        if S:
            streams = hyper_step(streams, w, f"{p}.hc1", mix, w[f"{p}.norm1"], eps)
            if ff:
                streams = hyper_step(streams, w, f"{p}.hc2", ff, w[f"{p}.norm2"], eps)
            x = streams.sum(0)
        else:
            x = x + mix(rms_norm(x, w[f"{p}.norm1"], eps))
            if ff:
                x = x + ff(rms_norm(x, w[f"{p}.norm2"], eps))
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms_norm(x, w["final.norm"], eps) @ w["head"].T) * cfg.get("logit_scale", 1.0)
