"""Typed configuration of the Zasesun decoder: latent attention with scaled rotary positions,
sandwich norms with a residual multiplier, dense (tanh-GELU gated) and routed (squared-ReLU
experts plus a shared expert) feed-forwards, a tied output head with a soft cap on the logits.

config.json of this design is nested: ``layers`` is a list with one entry per layer (``type``,
``mixer`` with the mixer's sizes, ``mlp`` with the feed-forward's or null), beside ``vocab``,
``width``, ``norm.eps``, ``residual_mult`` and ``logit_softcap``.  Every size and constant is read
from there; layers may differ from one another in all of them.  Checkpoint tensors are named
``embed``, ``final.norm`` and ``l<i>.<part>`` without a ``.weight`` suffix.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .base import ConfigError, eos_token_ids, req_int, req_num
from .spec import (GatedMLPSpec, LatentAttentionSpec, LayerSpec, ModelSpec, RMSNormSpec, RoutedMLPSpec,
                   ScaledRotarySpec, SoftCapSpec)


def _section(cfg: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = cfg.get(key)
    if not isinstance(value, dict):
        raise ConfigError(f"{where}{key}", "is missing or not an object")
    return value


def _positive(cfg: Mapping[str, Any], key: str, where: str) -> float:
    try:
        value = req_num(cfg, key)
    except ConfigError as error:
        raise ConfigError(f"{where}{key}", error.reason) from None
    if not value > 0:
        raise ConfigError(f"{where}{key}", f"must be positive, got {value}")
    return value


def _count(cfg: Mapping[str, Any], key: str, where: str, minimum: int = 1) -> int:
    try:
        return req_int(cfg, key, minimum)
    except ConfigError as error:
        raise ConfigError(f"{where}{key}", error.reason) from None


@dataclass(frozen=True)
class ZasesunLayer:
    mixer: LatentAttentionSpec
    feed_forward: Optional[Any]      # GatedMLPSpec | RoutedMLPSpec | None
    raw: Any                         # the layer's entry of config.json, kept for to_dict()


@dataclass(frozen=True)
class ZasesunConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    logit_softcap: Optional[float]
    layers: Tuple[ZasesunLayer, ...]
    max_positions: int = 1 << 20
    eos_token_id: Tuple[int, ...] = ()

    architecture = "Zasesun"
    model_type = "zasesun"

    # ------------------------------------------------------------------ reading
    @staticmethod
    def _rotary(rot: Mapping[str, Any], where: str, rot_dim: int) -> Optional[ScaledRotarySpec]:
        dims = _count(rot, "dims", where, 0)
        if dims == 0:
            return None
        if dims % 2 or dims > rot_dim:
            raise ConfigError(f"{where}dims", f"must be even and at most rot_dim={rot_dim}, got {dims}")
        base = _positive(rot, "base", where)
        scaling = rot.get("scaling")
        stretch = None
        if scaling is not None:
            if not isinstance(scaling, dict):
                raise ConfigError(f"{where}scaling", "is not an object")
            sw = f"{where}scaling."
            stretch = (_positive(scaling, "factor", sw), _positive(scaling, "original", sw),
                       _positive(scaling, "fast", sw), _positive(scaling, "slow", sw))
        return ScaledRotarySpec(dims=dims, base=base, pairing="interleaved", scaling=stretch)

    @classmethod
    def _mixer(cls, layer: Mapping[str, Any], where: str, width: int, eps: float) -> LatentAttentionSpec:
        kind = layer.get("type")
        if kind != "latent_attention":
            raise ConfigError(f"{where}type", f"names the unknown mixer {kind!r}")
        m = _section(layer, "mixer", where)
        mw = f"{where}mixer."
        rot_dim = _count(m, "rot_dim", mw, 0)
        position = cls._rotary(_section(m, "rot", mw), f"{mw}rot.", rot_dim) if rot_dim else None
        return LatentAttentionSpec(
            hidden=width, heads=_count(m, "heads", mw), dim=_count(m, "dim", mw), rot_dim=rot_dim,
            vdim=_count(m, "vdim", mw), q_rank=_count(m, "q_rank", mw), kv_rank=_count(m, "kv_rank", mw),
            softmax_scale=_positive(m, "scale", mw), eps=eps, position=position)

    @staticmethod
    def _feed_forward(layer: Mapping[str, Any], where: str, width: int):
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        if not isinstance(mlp, dict):
            raise ConfigError(f"{where}mlp", "is neither an object nor null")
        fw = f"{where}mlp."
        kind = mlp.get("kind")
        if kind == "dense":
            return GatedMLPSpec(width, _count(mlp, "ff", fw), "gelu_tanh", tensor_names=("gate", "up", "down"))
        if kind == "moe":
            router = _section(mlp, "router", fw)
            experts = _count(router, "experts", f"{fw}router.")
            top = _count(router, "top", f"{fw}router.")
            if top > experts:
                raise ConfigError(f"{fw}router.top", f"({top}) exceeds the {experts} experts")
            shared = mlp.get("shared")
            if shared is not None and not isinstance(shared, dict):
                raise ConfigError(f"{fw}shared", "is neither an object nor null")
            return RoutedMLPSpec(hidden=width, experts=experts, top=top,
                                 expert_ff=_count(_section(mlp, "expert", fw), "ff", f"{fw}expert."),
                                 shared_ff=_count(shared, "ff", f"{fw}shared.") if shared else 0,
                                 activation="relu2", score="softmax", renormalize=False)
        raise ConfigError(f"{fw}kind", f"names the unknown feed-forward {kind!r}")

    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any], model_dir: Optional[str] = None) -> "ZasesunConfig":
        vocab, width = req_int(cfg, "vocab"), req_int(cfg, "width")
        eps = _positive(_section(cfg, "norm", ""), "eps", "norm.")
        mult = req_num(cfg, "residual_mult") if cfg.get("residual_mult") is not None else 1.0
        cap = cfg.get("logit_softcap")
        if cap is not None:
            cap = _positive(cfg, "logit_softcap", "")
        entries = cfg.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("layers", "is missing or empty")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"layers[{i}]", "is not an object")
            layers.append(ZasesunLayer(cls._mixer(entry, where, width, eps), cls._feed_forward(entry, where, width),
                                       entry))
        positions = cfg.get("max_positions")
        return cls(vocab=vocab, width=width, eps=eps, residual_mult=mult, logit_softcap=cap, layers=tuple(layers),
                   max_positions=req_int(cfg, "max_positions") if positions is not None else 1 << 20,
                   eos_token_id=eos_token_ids(model_dir, cfg))

    def to_dict(self) -> dict:
        """config.json contents that :meth:`from_dict` reads back to an equal configuration."""
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.eps}, "residual_mult": self.residual_mult,
               "layers": [layer.raw for layer in self.layers]}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if self.max_positions != 1 << 20:
            out["max_positions"] = self.max_positions
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out

    # ------------------------------------------------------------------ derived
    def num_parameters(self) -> int:
        """Elements of every tensor the checkpoint holds."""
        from ..weights.loader import expected_tensors
        total = 0
        for t in expected_tensors(self.to_spec()):
            count = 1
            for extent in t.shape:
                count *= extent
            total += count
        return total

    def to_spec(self) -> ModelSpec:
        norm = RMSNormSpec(self.width, self.eps, bare=True)
        layers = tuple(
            LayerSpec(prefix=f"l{i}", mixer=layer.mixer, feed_forward=layer.feed_forward,
                      mixer_norm=norm, feed_forward_norm=norm if layer.feed_forward is not None else None,
                      arrangement="sandwich", mixer_prefix="mix", feed_forward_prefix="mlp",
                      mixer_norm_prefix="norm1", feed_forward_norm_prefix="norm2",
                      mixer_post_norm=norm, feed_forward_post_norm=norm if layer.feed_forward is not None else None,
                      mixer_post_norm_prefix="norm1b", feed_forward_post_norm_prefix="norm2b",
                      residual_scale=self.residual_mult)
            for i, layer in enumerate(self.layers))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width,
            max_positions=self.max_positions, layers=layers, final_norm=norm, tie_embeddings=True,
            embedding_name="embed", final_norm_prefix="final.norm", head_name="head",
            eos_token_ids=self.eos_token_id,
            logits_transform=SoftCapSpec(self.logit_softcap) if self.logit_softcap is not None else None,
            ignored_prefixes=(), ignored_containing=())
