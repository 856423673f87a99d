"""Typed configuration of the Vefulix decoder, read from the keys of its own config.json, and its
`ModelSpec` builder.

A Vefulix model is a list of layers, each with one of three token mixers (a matrix-memory mLSTM, a
gated delta rule with short convolutions, latent attention with a softmax sink) and an optional
mixture-of-experts feed-forward with a shared expert; LayerNorm with bias everywhere (also on the
embedded rows); optionally a residual kept as several streams (hyper-connections); logits through a
soft cap.  Every size and every constant that can differ between models comes from config.json:

    architecture   "Vefulix"
    vocab, width
    norm.eps
    streams        (optional) number of residual streams; absent: one plain residual
    logit_softcap  (optional)
    layers[i]      {"type": "mlstm" | "delta" | "latent_attention", "mixer": {...}, "mlp": {...} | null}
      mlstm             heads, dim, vdim, gate_cap
      delta             heads, kv_heads, dim, vdim, conv
      latent_attention  heads, dim, vdim, q_rank, kv_rank, scale
      mlp               kind "moe", expert.ff, router.experts, router.top, shared.ff (optional)
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .registry import ConfigError, register_architecture
from .specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Vefulix"
MIXER_TYPES = ("mlstm", "delta", "latent_attention")
_MIXER_KEYS = {
    "mlstm": (("heads", int), ("dim", int), ("vdim", int), ("gate_cap", float)),
    "delta": (("heads", int), ("kv_heads", int), ("dim", int), ("vdim", int), ("conv", int)),
    "latent_attention": (("heads", int), ("dim", int), ("vdim", int), ("q_rank", int), ("kv_rank", int), ("scale", float)),
}


def _number(where: str, raw: Mapping[str, Any], key: str, typ):
    if not isinstance(raw, Mapping) or key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: {where}: required key {key!r} is missing")
    v = raw[key]
    if isinstance(v, bool) or not isinstance(v, (int, float) if typ is float else int):
        raise ConfigError(f"config.json: {where}.{key} must be {'a number' if typ is float else 'an integer'}, got {v!r}")
    v = typ(v)
    if not (v > 0 and math.isfinite(v)):
        raise ConfigError(f"config.json: {where}.{key} must be positive and finite, got {v!r}")
    return v


@dataclass(frozen=True)
class VefulixConfig:
    vocab: int
    width: int
    eps: float
    streams: Optional[int]
    logit_softcap: Optional[float]
    layers: Tuple[Mapping[str, Any], ...]       # validated copies of config.json's entries
    architecture: str = ARCHITECTURE

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "VefulixConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(lr, Mapping) or lr.get("type") not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type must be one of {MIXER_TYPES}, got "
                                  f"{lr.get('type') if isinstance(lr, Mapping) else lr!r}")
            kind = lr["type"]
            given = lr.get("mixer")
            if kind == "delta" and isinstance(given, Mapping) and given.get("kv_heads") is None and "heads" in given:
                given = dict(given, kv_heads=given["heads"])          # no grouping given: every head has its own q and k
            mixer = {k: _number(where + ".mixer", given, k, t) for k, t in _MIXER_KEYS[kind]}
            if kind == "delta" and mixer["heads"] % mixer["kv_heads"]:
                raise ConfigError(f"config.json: {where}.mixer: heads {mixer['heads']} is not a multiple of "
                                  f"kv_heads {mixer['kv_heads']}")
            mlp = lr.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "moe":
                    raise ConfigError(f"config.json: {where}.mlp.kind must be 'moe' (or mlp null), got "
                                      f"{mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r}")
                experts = _number(where + ".mlp.router", mlp.get("router"), "experts", int)
                top = _number(where + ".mlp.router", mlp.get("router"), "top", int)
                if top > experts:
                    raise ConfigError(f"config.json: {where}.mlp.router: top {top} exceeds experts {experts}")
                shared = mlp.get("shared")
                mlp = {"kind": "moe", "expert": {"ff": _number(where + ".mlp.expert", mlp.get("expert"), "ff", int)},
                       "router": {"experts": experts, "top": top},
                       "shared": None if shared is None else {"ff": _number(where + ".mlp.shared", shared, "ff", int)}}
            layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
        streams = raw.get("streams")
        if streams is not None:
            streams = _number("top level", raw, "streams", int)
            if streams > 8:
                raise ConfigError(f"config.json: streams {streams}: at most 8 residual streams are supported")
        cap = raw.get("logit_softcap")
        return cls(vocab=_number("top level", raw, "vocab", int), width=_number("top level", raw, "width", int),
                   eps=_number("norm", raw.get("norm"), "eps", float), streams=streams,
                   logit_softcap=None if cap is None else _number("top level", raw, "logit_softcap", float),
                   layers=tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                             "norm": {"eps": self.eps}, "layers": copy.deepcopy(list(self.layers))}
        for layer in d["layers"]:
            if layer["mlp"] is not None and layer["mlp"]["shared"] is None:
                del layer["mlp"]["shared"]
        if self.streams is not None:
            d["streams"] = self.streams
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        return d


def build_spec(cfg: VefulixConfig) -> ModelSpec:
    """Tensor names: `embed`, `embed.norm(.b)`, `l<i>.norm1(.b)`, `l<i>.norm2(.b)`, `l<i>.mix.*`, `l<i>.mlp.*`,
    `l<i>.hc1.*` / `l<i>.hc2.*` (with streams), `final.norm(.b)`, `head`."""
    norm = PartSpec("layernorm", {"eps": cfg.eps})
    block = PartSpec("prenorm", {}) if cfg.streams is None else PartSpec("hyper", {"streams": cfg.streams})
    kinds = {"mlstm": "mlstm", "delta": "gated_delta", "latent_attention": "latent_attention"}
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        mixer = PartSpec(kinds[layer["type"]], {"hidden_size": cfg.width, "eps": cfg.eps, **layer["mixer"]})
        mlp = layer["mlp"]
        ffn = None if mlp is None else PartSpec("moe", {
            "hidden_size": cfg.width, "experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
            "expert_ff": mlp["expert"]["ff"], "shared_ff": None if mlp["shared"] is None else mlp["shared"]["ff"]})
        layers.append(LayerSpec(block=block, norm=norm, mixer=mixer, ffn=ffn, mixer_prefix=p + "mix.",
                                ffn_prefix=p + "mlp.", mixer_norm_name=p + "norm1", ffn_norm_name=p + "norm2",
                                block_prefix=p))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))), final_norm=norm, embedding_name="embed",
        final_norm_name="final.norm", lm_head_name="head", embedding_scale=1.0,
        max_position=1 << 30,                      # no positions: a sequence is as long as the cache allows
        bos_token_id=None, eos_token_id=None,
        head=PartSpec("linear") if cfg.logit_softcap is None else PartSpec("softcap", {"cap": cfg.logit_softcap}),
        inputs=((PartSpec("embed_norm", {"norm": norm}), "embed."),),
        residual_streams=cfg.streams)


register_architecture(ARCHITECTURE, VefulixConfig, build_spec)
