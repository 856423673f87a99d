"""Typed configuration of the Sifasun decoder, read from the keys of its own config.json, and its
`ModelSpec` builder.

A Sifasun model is a list of layers that norm each sublayer's OUTPUT (x <- x + norm(sublayer(x)), RMS norm
with a weight stored around zero); a layer's mixer is either attention whose keys double as values (partial
rotary positions with stretched frequencies, unit RMS per head, capped scores, a sliding window, a softmax
sink), or a PAIR of mixers side by side: such an attention with one RMS norm over the whole query / key
projection, and a gated linear recurrence with a short convolution.  The feed-forward is a dense SiLU-gated
one, or absent.  A layer may run with another layer's weights and a cache of its own.  The output head is
the embedding table, times a fixed factor.  Every size and every constant that can differ between models
comes from config.json:

    architecture   "Sifasun"
    vocab, width, logit_scale
    norm.eps
    layers[i]      {"type": "attention" | "parallel", "mixer": {...}, "mlp": {"kind": "dense", "ff": n} | null,
                    "weights_of": j (optional)}
      attention    heads, kv_heads, dim, vdim (= dim), scale, softcap (optional), mask.size (optional),
                   rot.base, rot.dims, rot.scaling.factor (optional)
      parallel     left: {as attention, without a sink}, left_scale, right: {width, blocks, conv}, right_scale
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .registry import ConfigError, register_architecture
from .specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Sifasun"
LAYER_TYPES = ("attention", "parallel")


def _number(where: str, raw: Any, key: str, typ, positive: bool = True):
    if not isinstance(raw, Mapping) or key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: {where}: required key {key!r} is missing")
    v = raw[key]
    if isinstance(v, bool) or not isinstance(v, (int, float) if typ is float else int):
        raise ConfigError(f"config.json: {where}.{key} must be {'a number' if typ is float else 'an integer'}, got {v!r}")
    v = typ(v)
    if not math.isfinite(v) or (positive and not v > 0):
        raise ConfigError(f"config.json: {where}.{key} must be {'positive and ' if positive else ''}finite, got {v!r}")
    return v


def _attention(where: str, raw: Any) -> Dict[str, Any]:
    heads, kv_heads = _number(where, raw, "heads", int), _number(where, raw, "kv_heads", int)
    dim = _number(where, raw, "dim", int)
    vdim = _number(where, raw, "vdim", int) if isinstance(raw, Mapping) and raw.get("vdim") is not None else dim
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}: heads {heads} is not a multiple of kv_heads {kv_heads}")
    if vdim != dim:
        raise ConfigError(f"config.json: {where}: vdim {vdim} differs from dim {dim}, but the values are the keys")
    rot = raw.get("rot")
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": _number(where, raw, "scale", float)}
    if rot is not None:
        dims = _number(where + ".rot", rot, "dims", int, positive=False)
        if dims < 0 or dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where}.rot.dims {dims} must be even, not negative and at most dim {dim}")
        out["rot"] = {"base": _number(where + ".rot", rot, "base", float), "dims": dims}
        if rot.get("scaling") is not None:
            out["rot"]["scaling"] = {"factor": _number(where + ".rot.scaling", rot["scaling"], "factor", float)}
    if raw.get("mask") is not None:
        out["mask"] = {"size": _number(where + ".mask", raw["mask"], "size", int)}
    if raw.get("softcap") is not None:
        out["softcap"] = _number(where, raw, "softcap", float)
    return out


def _recurrent(where: str, raw: Any) -> Dict[str, Any]:
    width, blocks = _number(where, raw, "width", int), _number(where, raw, "blocks", int)
    if width % blocks:
        raise ConfigError(f"config.json: {where}: width {width} is not a multiple of blocks {blocks}")
    return {"width": width, "blocks": blocks, "conv": _number(where, raw, "conv", int)}


@dataclass(frozen=True)
class SifasunConfig:
    vocab: int
    width: int
    eps: float
    logit_scale: float
    layers: Tuple[Mapping[str, Any], ...]       # validated copies of config.json's entries
    architecture: str = ARCHITECTURE

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "SifasunConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(lr, Mapping) or lr.get("type") not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}.type must be one of {LAYER_TYPES}, got "
                                  f"{lr.get('type') if isinstance(lr, Mapping) else lr!r}")
            given = lr.get("mixer")
            if not isinstance(given, Mapping):
                raise ConfigError(f"config.json: {where}: required key 'mixer' is missing")
            if lr["type"] == "attention":
                mixer = _attention(where + ".mixer", given)
            else:
                mixer = {"left": _attention(where + ".mixer.left", given.get("left")),
                         "left_scale": _number(where + ".mixer", given, "left_scale", float, positive=False),
                         "right": _recurrent(where + ".mixer.right", given.get("right")),
                         "right_scale": _number(where + ".mixer", given, "right_scale", float, positive=False)}
            mlp = lr.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind must be 'dense' (or mlp null), got "
                                      f"{mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r}")
                mlp = {"kind": "dense", "ff": _number(where + ".mlp", mlp, "ff", int)}
            entry = {"type": lr["type"], "mixer": mixer, "mlp": mlp}
            if lr.get("weights_of") is not None:
                j = lr["weights_of"]
                if isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < len(layers_raw) or j == i:
                    raise ConfigError(f"config.json: {where}.weights_of must name another layer, got {j!r}")
                entry["weights_of"] = j
            layers.append(entry)
        for i, layer in enumerate(layers):        # a layer that borrows weights is built like their owner
            j = layer.get("weights_of")
            if j is not None and layers[j]["type"] != layer["type"]:
                raise ConfigError(f"config.json: layers[{i}] is of type {layer['type']!r} but takes the weights of "
                                  f"layers[{j}], of type {layers[j]['type']!r}")
        return cls(vocab=_number("top level", raw, "vocab", int), width=_number("top level", raw, "width", int),
                   eps=_number("norm", raw.get("norm"), "eps", float),
                   logit_scale=_number("top level", raw, "logit_scale", float) if raw.get("logit_scale") is not None else 1.0,
                   layers=tuple(layers))

    def owner(self, i: int) -> int:
        """The layer whose tensors layer `i` uses (itself, unless it names another)."""
        seen = set()
        while self.layers[i].get("weights_of") is not None:
            if i in seen:
                raise ConfigError(f"config.json: layers[{i}].weights_of goes round in a circle")
            seen.add(i)
            i = self.layers[i]["weights_of"]
        return i

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "logit_scale": self.logit_scale, "layers": copy.deepcopy(list(self.layers))}


def _attention_spec(cfg: SifasunConfig, m: Mapping[str, Any], qk_norm: str, sink: bool) -> PartSpec:
    rot = m.get("rot") or {"base": 10000.0, "dims": 0}
    position = {"theta": rot["base"], "rotary_dim": rot["dims"], "pairing": "half"}
    if rot.get("scaling") is not None:         # stretched positions: every frequency divided by the factor
        position["freq_factors"] = [rot["scaling"]["factor"]] * (rot["dims"] // 2)
    return PartSpec("tied_kv_attention", {
        "hidden_size": cfg.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "head_dim": m["dim"],
        "window": (m.get("mask") or {}).get("size"), "scale": m["scale"], "softcap": m.get("softcap"), "sink": sink,
        "qk_norm": qk_norm, "eps": cfg.eps, "position": PartSpec("rope", position)})


def build_spec(cfg: SifasunConfig) -> ModelSpec:
    """Tensor names: `embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*` (a pair: `l<i>.mix.left.*`, `l<i>.mix.right.*`),
    `l<i>.mlp.gate|up|down`, `final.norm`; i is the layer's place in config.json, and a layer with `weights_of` has none."""
    norm = PartSpec("rmsnorm", {"eps": cfg.eps, "offset": 1.0})
    block = PartSpec("outnorm", {})
    owners = sorted({cfg.owner(i) for i in range(len(cfg.layers))})
    index_of = {i: n for n, i in enumerate(owners)}
    layers = []
    for i in owners:
        layer, p = cfg.layers[i], f"l{i}."
        m = layer["mixer"]
        if layer["type"] == "attention":
            mixer = _attention_spec(cfg, m, "head", sink=True)
        else:
            mixer = PartSpec("parallel", {
                "left": _attention_spec(cfg, m["left"], "whole", sink=False), "left_scale": m["left_scale"],
                "right": PartSpec("rglru", {"hidden_size": cfg.width, **m["right"]}), "right_scale": m["right_scale"]})
        ffn = None if layer["mlp"] is None else PartSpec("swiglu", {
            "hidden_size": cfg.width, "intermediate_size": layer["mlp"]["ff"], "tensor_names": ("gate", "up", "down")})
        layers.append(LayerSpec(block=block, norm=norm, mixer=mixer, ffn=ffn, mixer_prefix=p + "mix.", ffn_prefix=p + "mlp.",
                                mixer_norm_name=p + "norm1", ffn_norm_name=p + "norm2"))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, layers=tuple(layers),
        schedule=tuple(ScheduleEntry(index_of[cfg.owner(i)]) for i in range(len(cfg.layers))),
        final_norm=norm, embedding_name="embed", final_norm_name="final.norm",
        lm_head_name=None,                          # the output head is the embedding table
        embedding_scale=1.0, max_position=1 << 30, bos_token_id=None, eos_token_id=None,
        head=PartSpec("scaled", {"scale": cfg.logit_scale}))


register_architecture(ARCHITECTURE, SifasunConfig, build_spec)
