"""Typed configuration of the Balivik decoder: layers that are each a differential softmax
attention, a linear attention with a decay per head or a gated delta rule with a decay per key
channel, under hyper-connections (several residual streams a token) with a causal convolution in
front of every mixer; dense SiLU-gated feed-forwards and mixtures of gated experts chosen by a
table over token ids; norms with a single weight; a block of layers that runs several times.

config.json of this design is nested: ``layers`` lists the layers (``type``, ``mixer`` with the
mixer's sizes, ``mlp`` with the feed-forward's or null), beside ``vocab``, ``width``, ``norm.eps``
and the optional ``streams``, ``canon.taps``, ``loop`` (``start``, ``stop``, ``times``: layers
start .. stop - 1 run ``times`` times in a row, each pass with a cache of its own) and
``logit_scale``.  The inner sizes of the delta rule's two low-rank projections are not in
config.json: they are the shapes of ``l<i>.mix.a1`` and ``l<i>.mix.g1`` in the checkpoint (or,
for a configuration made without one, the mixer's ``decay_rank`` and ``gate_rank`` keys).
Checkpoint tensors are named ``embed``, ``head``, ``final.norm`` and ``l<i>.<part>`` without a
``.weight`` suffix.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .base import ConfigError, eos_token_ids, req_int, req_num
from .spec import (ChannelDeltaSpec, DecayAttentionSpec, DifferentialAttentionSpec, GatedMLPSpec, LayerSpec,
                   ModelSpec, RMSNormSpec, ScaledRotarySpec, ScaleSpec, ScheduleEntry, TableRoutedMLPSpec)
from .zasesun import _count, _positive, _section


def _number(cfg: Mapping[str, Any], key: str, where: str) -> float:
    try:
        return req_num(cfg, key)
    except ConfigError as error:
        raise ConfigError(f"{where}{key}", error.reason) from None


def checkpoint_shapes(model_dir: Optional[str]) -> dict:
    """name -> shape of every tensor in the folder's safetensors files (empty without a folder)."""
    if not model_dir or not os.path.isdir(model_dir):
        return {}
    from ..weights.safetensors_io import iter_tensors, open_model_files
    try:
        files = open_model_files(model_dir)
    except (OSError, ValueError):
        return {}
    return {name: tuple(f.info(name)[1]) for name, f in iter_tensors(files)}


@dataclass(frozen=True)
class BalivikLayer:
    mixer: Any                       # DifferentialAttentionSpec | DecayAttentionSpec | ChannelDeltaSpec
    feed_forward: Optional[Any]      # GatedMLPSpec | TableRoutedMLPSpec | None
    raw: Any                         # the layer's entry of config.json, kept for to_dict()


@dataclass(frozen=True)
class BalivikConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[BalivikLayer, ...]
    streams: Optional[int] = None
    canon_taps: int = 0
    loop: Optional[Tuple[int, int, int]] = None      # (start, stop, times)
    logit_scale: Optional[float] = None
    max_positions: int = 1 << 20
    eos_token_id: Tuple[int, ...] = ()

    architecture = "Balivik"
    model_type = "balivik"

    # ------------------------------------------------------------------ reading
    @staticmethod
    def _mixer(i: int, layer: Mapping[str, Any], where: str, width: int, eps: float, shapes: dict):
        kind = layer.get("type")
        m = _section(layer, "mixer", where)
        mw = f"{where}mixer."
        if kind == "attention":
            heads = _count(m, "heads", mw)
            kv_heads = _count(m, "kv_heads", mw) if m.get("kv_heads") is not None else heads
            if heads % kv_heads:
                raise ConfigError(f"{mw}heads", f"({heads}) is not a multiple of kv_heads ({kv_heads})")
            dim = _count(m, "dim", mw)
            position = None
            rot = m.get("rot")
            if rot is not None:
                if not isinstance(rot, dict):
                    raise ConfigError(f"{mw}rot", "is not an object")
                dims = _count(rot, "dims", f"{mw}rot.", 0)
                if dims:
                    if dims % 2 or dims > dim:
                        raise ConfigError(f"{mw}rot.dims", f"must be even and at most dim={dim}, got {dims}")
                    position = ScaledRotarySpec(dims=dims, base=_positive(rot, "base", f"{mw}rot."), pairing="half")
            diff = _number(m, "diff", mw)
            return DifferentialAttentionSpec(hidden=width, heads=heads, kv_heads=kv_heads, dim=dim,
                                             vdim=_count(m, "vdim", mw), softmax_scale=_positive(m, "scale", mw),
                                             diff=diff, eps=eps, position=position)
        if kind == "lightning":
            heads = _count(m, "heads", mw)
            decay = m.get("decay")
            if isinstance(decay, (int, float)) and not isinstance(decay, bool):
                decay = [decay] * heads             # one number for all heads
            if not isinstance(decay, list) or len(decay) != heads or \
                    any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
                raise ConfigError(f"{mw}decay", f"must list one number for each of the {heads} heads")
            return DecayAttentionSpec(hidden=width, heads=heads, dim=_count(m, "dim", mw), vdim=_count(m, "vdim", mw),
                                      decay=tuple(float(d) for d in decay), eps=eps)
        if kind == "channel_delta":
            heads = _count(m, "heads", mw)
            kv_heads = _count(m, "kv_heads", mw) if m.get("kv_heads") is not None else heads
            if heads % kv_heads:
                raise ConfigError(f"{mw}heads", f"({heads}) is not a multiple of kv_heads ({kv_heads})")
            ranks = {}
            for key, tensor in (("decay_rank", f"l{i}.mix.a1"), ("gate_rank", f"l{i}.mix.g1")):
                if tensor in shapes and len(shapes[tensor]) == 2:
                    ranks[key] = int(shapes[tensor][0])
                elif m.get(key) is not None:
                    ranks[key] = _count(m, key, mw)
                else:
                    raise ConfigError(f"{mw}{key}", f"is given neither by the checkpoint tensor {tensor} nor by the key")
            return ChannelDeltaSpec(hidden=width, heads=heads, kv_heads=kv_heads, dim=_count(m, "dim", mw),
                                    vdim=_count(m, "vdim", mw), conv=_count(m, "conv", mw), eps=eps, **ranks)
        raise ConfigError(f"{where}type", f"names the unknown mixer {kind!r}")

    @staticmethod
    def _feed_forward(layer: Mapping[str, Any], where: str, width: int, vocab: int):
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        if not isinstance(mlp, dict):
            raise ConfigError(f"{where}mlp", "is neither an object nor null")
        fw = f"{where}mlp."
        kind = mlp.get("kind")
        if kind == "dense":
            return GatedMLPSpec(width, _count(mlp, "ff", fw), "silu", tensor_names=("gate", "up", "down"))
        if kind == "moe":
            router = _section(mlp, "router", fw)
            experts = _count(router, "experts", f"{fw}router.")
            top = _count(router, "top", f"{fw}router.")
            if top > experts:
                raise ConfigError(f"{fw}router.top", f"({top}) exceeds the {experts} experts")
            expert = _section(mlp, "expert", fw)
            return TableRoutedMLPSpec(hidden=width, vocab=vocab, experts=experts, top=top,
                                      expert_ff=_count(expert, "ff", f"{fw}expert."),
                                      limit=_positive(expert, "limit", f"{fw}expert."))
        raise ConfigError(f"{fw}kind", f"names the unknown feed-forward {kind!r}")

    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any], model_dir: Optional[str] = None) -> "BalivikConfig":
        vocab, width = req_int(cfg, "vocab"), req_int(cfg, "width")
        eps = _positive(_section(cfg, "norm", ""), "eps", "norm.")
        entries = cfg.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("layers", "is missing or empty")
        shapes = checkpoint_shapes(model_dir)
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"layers[{i}]", "is not an object")
            layers.append(BalivikLayer(cls._mixer(i, entry, where, width, eps, shapes),
                                       cls._feed_forward(entry, where, width, vocab), entry))
        streams = req_int(cfg, "streams") if cfg.get("streams") is not None else None
        if streams is not None and streams > 8:
            raise ConfigError("streams", f"must be at most 8, got {streams}")
        taps = 0
        if cfg.get("canon") is not None:
            taps = _count(_section(cfg, "canon", ""), "taps", "canon.")
        loop = None
        if cfg.get("loop") is not None:
            section = _section(cfg, "loop", "")
            start, stop = _count(section, "start", "loop.", 0), _count(section, "stop", "loop.", 0)
            times = _count(section, "times", "loop.", 1)
            if not start <= stop <= len(layers):
                raise ConfigError("loop", f"start={start} stop={stop} do not lie in the {len(layers)} layers")
            loop = (start, stop, times)
        scale = _number(cfg, "logit_scale", "") if cfg.get("logit_scale") is not None else None
        positions = cfg.get("max_positions")
        return cls(vocab=vocab, width=width, eps=eps, layers=tuple(layers), streams=streams, canon_taps=taps, loop=loop,
                   logit_scale=scale, max_positions=req_int(cfg, "max_positions") if positions is not None else 1 << 20,
                   eos_token_id=eos_token_ids(model_dir, cfg))

    def to_dict(self) -> dict:
        """config.json contents that :meth:`from_dict` reads back to an equal configuration."""
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "layers": [layer.raw for layer in self.layers]}
        if self.streams is not None:
            out["streams"] = self.streams
        if self.canon_taps:
            out["canon"] = {"taps": self.canon_taps}
        if self.loop is not None:
            out["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        if self.logit_scale is not None:
            out["logit_scale"] = self.logit_scale
        if self.max_positions != 1 << 20:
            out["max_positions"] = self.max_positions
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out

    # ------------------------------------------------------------------ derived
    def run_order(self) -> Tuple[int, ...]:
        n = len(self.layers)
        if self.loop is None:
            return tuple(range(n))
        start, stop, times = self.loop
        return tuple(range(start)) + tuple(range(start, stop)) * times + tuple(range(stop, n))

    def num_parameters(self) -> int:
        from ..weights.loader import expected_tensors
        total = 0
        for t in expected_tensors(self.to_spec()):
            count = 1
            for extent in t.shape:
                count *= extent
            total += count
        return total

    def to_spec(self) -> ModelSpec:
        norm = RMSNormSpec(self.width, self.eps, bare=True, scalar=True)
        layers = tuple(
            LayerSpec(prefix=f"l{i}", mixer=layer.mixer, feed_forward=layer.feed_forward,
                      mixer_norm=norm, feed_forward_norm=norm if layer.feed_forward is not None else None,
                      arrangement="streams", mixer_prefix="mix", feed_forward_prefix="mlp",
                      mixer_norm_prefix="norm1", feed_forward_norm_prefix="norm2",
                      streams=self.streams or 0, mixer_streams_prefix="hc1", feed_forward_streams_prefix="hc2",
                      input_conv_taps=self.canon_taps, input_conv_name="canon1")
            for i, layer in enumerate(self.layers))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width,
            max_positions=self.max_positions, layers=layers, final_norm=norm, tie_embeddings=False,
            schedule=tuple(ScheduleEntry(i) for i in self.run_order()),
            embedding_name="embed", final_norm_prefix="final.norm", head_name="head",
            eos_token_ids=self.eos_token_id,
            logits_transform=ScaleSpec(self.logit_scale) if self.logit_scale is not None else None,
            streams=self.streams or 1, ignored_prefixes=(), ignored_containing=())
