"""Typed configuration of the Dogilorn decoder (config.json ``"architecture": "Dogilorn"``).

A stack of pre-norm layers around a 32-bit residual stream: ``x += ls1 * mixer(c(norm1(x)))`` then ``x += ls2 * ff(norm2(x))``.
The norms are layer norms with weight and bias (``norm.eps``), ``ls1`` / ``ls2`` a learned multiplier for every channel, and
``c(h) = h + conv(h)`` a causal convolution over time on every channel with ``canon.taps`` taps (tensor ``canon1 [width,
taps]``) whose last ``taps - 1`` inputs are part of a request's state.  The embedding output is multiplied by
``embedding.scale``; the logits are the final norm's output times the embedding table itself.  config.json lists the
layers (``layers[i]``: ``type``, ``mixer``, ``mlp``), and every layer may differ:

* ``type: "attention"``: grouped-query attention (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``) whose queries and keys
  are normed over the whole projection, with the rotation of the interleaved pairs of each head's first ``rot.dims`` elements
  (``rot.base``), values of unit root mean square, a temperature a head, a window of ``mask.size`` positions that also keeps a
  sequence's first ``mask.keep_first`` tokens in view, and a softmax with one added to its denominator.  ``kv_from: j``: the
  layer has no keys and values of its own and reads those of layer ``j``, which has its own projections.
* ``mlp``: null, ``{"kind": "dense", "ff", "limit"}`` (``down(g * sigmoid(1.702 g) * (u + 1))`` with clamped ``g`` and ``u``, biases on
  all three projections) or ``{"kind": "moe", "router": {"experts", "top", "identity", "groups": {"count", "keep"}}, "expert":
  {"ff"}, "shared": {"ff"} or null}``: experts ``down(silu(gate h) * up h)`` without biases, the choice by the softmax scores plus
  the tensor ``correction`` among the best groups of router outputs, the last ``identity`` outputs standing for experts that
  return their input, the weights the plain scores, and a shared expert behind a sigmoid gate of one number a token.

Tensor names: ``embed``, ``l<i>.{norm1,norm1.b,norm2,norm2.b,ls1,ls2,canon1}``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``,
``final.norm.b``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List

from .model_config import ArchitectureConfig, ConfigError, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

MAX_POSITION = 1 << 20      # the design sets no limit of its own; the engine's max_model_len is the one that counts
DENSE_SLOPE = 1.702         # the dense feed-forward's activation is g * sigmoid(1.702 g) * (u + 1)


def _int(d, key, where, least=1):
    v = d.get(key) if isinstance(d, dict) else None
    if not isinstance(v, int) or isinstance(v, bool) or v < least:
        raise ConfigError(f"Dogilorn config.json: {where}.{key} must be an integer of at least {least}, found {v!r}")
    return v


def _num(d, key, where, positive=False):
    v = d.get(key) if isinstance(d, dict) else None
    if not isinstance(v, (int, float)) or isinstance(v, bool) or (positive and not v > 0):
        raise ConfigError(f"Dogilorn config.json: {where}.{key} must be a{' positive' if positive else ''} number, found {v!r}")
    return float(v)


def _check_mixer(i, kind, m, layers):
    where = f"layers[{i}].mixer"
    if kind != "attention":
        raise ConfigError(f"Dogilorn config.json: layers[{i}].type {kind!r} is not a known layer type (attention)")
    if not isinstance(m, dict):
        raise ConfigError(f"Dogilorn config.json: {where} must be an object")
    heads, groups = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % groups:
        raise ConfigError(f"Dogilorn config.json: {where}: {heads} heads do not group over {groups} key/value heads")
    dim = _int(m, "dim", where)
    _int(m, "vdim", where)
    if m.get("scale") is None:
        m["scale"] = float(dim) ** -0.5
    _num(m, "scale", where, positive=True)
    rot = m.get("rot")
    if rot is not None and rot.get("dims"):
        dims = _int(rot, "dims", where + ".rot", least=2)
        if dims % 2 or dims > dim:
            raise ConfigError(f"Dogilorn config.json: {where}.rot.dims {dims} must be even and at most dim ({dim})")
        _num(rot, "base", where + ".rot", positive=True)
    mask = m.get("mask")
    if mask is not None:
        _int(mask, "size", where + ".mask")
        if mask.get("keep_first") is not None:
            _int(mask, "keep_first", where + ".mask", least=0)
    src = m.get("kv_from")
    if src is not None:
        if not isinstance(src, int) or isinstance(src, bool) or not 0 <= src < i:
            raise ConfigError(f"Dogilorn config.json: {where}.kv_from {src!r} must name an earlier layer")
        o = layers[src]["mixer"]
        if o.get("kv_from") is not None:
            raise ConfigError(f"Dogilorn config.json: {where}.kv_from names layer {src}, which has no keys and values of its own")
        same = ("kv_heads", "dim", "vdim")
        if any(o.get(k) != m.get(k) for k in same) or (o.get("rot") or {}) != (m.get("rot") or {}):
            raise ConfigError(f"Dogilorn config.json: {where}.kv_from: layer {src} differs in key/value heads, sizes or rotation")


def _check_mlp(mlp, where):
    if mlp is None:
        return
    kind = mlp.get("kind") if isinstance(mlp, dict) else None
    if kind == "dense":
        _int(mlp, "ff", where)
        _num(mlp, "limit", where, positive=True)
    elif kind == "moe":
        r = mlp.get("router")
        experts, top = _int(r, "experts", where + ".router"), _int(r, "top", where + ".router")
        identity = _int(r, "identity", where + ".router", least=0) if r.get("identity") is not None else 0
        if top > experts + identity:
            raise ConfigError(f"Dogilorn config.json: {where}.router.top {top} exceeds the {experts + identity} router outputs")
        g = r.get("groups")
        if g is not None:
            count, keep = _int(g, "count", where + ".router.groups"), _int(g, "keep", where + ".router.groups")
            if (experts + identity) % count or keep > count or keep * ((experts + identity) // count) < top:
                raise ConfigError(f"Dogilorn config.json: {where}.router.groups: {count} groups, {keep} kept do not fit {experts + identity} outputs, top {top}")
        _int(mlp.get("expert"), "ff", where + ".expert")
        if mlp.get("shared") is not None:
            _int(mlp.get("shared"), "ff", where + ".shared")
    else:
        raise ConfigError(f"Dogilorn config.json: {where}.kind {kind!r} is not implemented (dense, moe)")


@register_architecture("Dogilorn", model_type="dogilorn")
@dataclass
class DogilornConfig(ArchitectureConfig):
    vocab: int
    width: int
    norm_eps: float
    taps: int
    embedding_scale: float
    layers: List[Dict[str, Any]]
    extra: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_json(cls, data: Dict[str, Any]) -> "DogilornConfig":
        vocab, width = _int(data, "vocab", "config"), _int(data, "width", "config")
        eps = _num(data.get("norm"), "eps", "norm", positive=True)
        taps = _int(data.get("canon"), "taps", "canon") if data.get("canon") is not None else 0      # 0: no input convolution
        scale = _num(data.get("embedding"), "scale", "embedding") if data.get("embedding") is not None else 1.0
        layers = copy.deepcopy(data.get("layers"))
        if not isinstance(layers, list) or not layers:
            raise ConfigError("Dogilorn config.json: 'layers' must list at least one layer")
        for i, layer in enumerate(layers):
            _check_mixer(i, layer.get("type"), layer.get("mixer"), layers)
            _check_mlp(layer.get("mlp"), f"layers[{i}].mlp")
        known = {"architecture", "architectures", "model_type", "vocab", "width", "norm", "canon", "embedding", "layers"}
        return cls(vocab=vocab, width=width, norm_eps=eps, taps=taps, embedding_scale=scale, layers=layers,
                   extra={k: v for k, v in data.items() if k not in known})

    def to_json(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "canon": {"taps": self.taps} if self.taps else None, "embedding": {"scale": self.embedding_scale}, "layers": copy.deepcopy(self.layers)}
        for k, v in self.extra.items():
            d.setdefault(k, v)
        return d

    # ---- parts -------------------------------------------------------------------------------
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("layer_norm", {"size": self.width, "eps": self.norm_eps, "weight": name, "bias": name + ".b"})

    @staticmethod
    def _mask(m):
        mask = m.get("mask")
        return (int(mask["size"]), int(mask.get("keep_first") or 0)) if mask is not None else (None, 0)

    def _mixer(self, i: int) -> PartSpec:
        m = self.layers[i]["mixer"]
        rot, position = m.get("rot"), None
        if rot is not None and rot.get("dims"):
            position = PartSpec("rotary_interleaved", {"theta": float(rot["base"]), "rotary_dim": int(rot["dims"])})
        window, keep = self._mask(m)
        # what a layer's cache keeps serves the layer itself and every later layer that reads it: the widest window, the most kept tokens
        cache_window, cache_keep = window, keep
        for other in self.layers[i + 1:]:
            if other["mixer"].get("kv_from") == i:
                w, k = self._mask(other["mixer"])
                cache_window = None if (w is None or cache_window is None) else max(cache_window, w)
                cache_keep = max(cache_keep, k)
        return PartSpec("sink_window_attention", {
            "hidden_size": self.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"], "scale": float(m["scale"]),
            "eps": self.norm_eps, "window": window, "keep_first": keep, "sink": True, "temperature": True, "shares_cache": m.get("kv_from") is not None,
            "cache_window": cache_window, "cache_keep_first": cache_keep, "position": position, "prefix": "mix."})

    def _feed_forward(self, mlp: Dict[str, Any]) -> PartSpec:
        W = self.width
        if mlp["kind"] == "dense":
            return PartSpec("gated_mlp", {"hidden_size": W, "intermediate_size": mlp["ff"], "activation": "clamped_swish", "limit": float(mlp["limit"]),
                                          "slope": DENSE_SLOPE, "bias": True, "prefix": "mlp.", "names": {"gate": "gate", "up": "up", "down": "down"}})
        r, shared = mlp["router"], mlp.get("shared")
        g = r.get("groups")
        return PartSpec("expert_mixture", {
            "hidden_size": W, "experts": r["experts"], "top": r["top"], "ff": mlp["expert"]["ff"], "activation": "silu",
            "identity": int(r.get("identity") or 0), "correction": True, "groups": (int(g["count"]), int(g["keep"])) if g is not None else None,
            "shared_ff": shared["ff"] if shared is not None else 0, "prefix": "mlp."})

    def run_order(self) -> List[RunEntry]:
        return [RunEntry(i, cache_of=layer["mixer"].get("kv_from")) for i, layer in enumerate(self.layers)]

    def to_spec(self) -> ModelSpec:
        layers, ignorable = [], []
        for i, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            more = {"mixer_scale": PartSpec("channel_scale", {"size": self.width, "weight": "ls1"})}
            if self.taps:
                more["mixer_conv"] = PartSpec("causal_conv", {"channels": self.width, "taps": self.taps, "weight": "canon1", "residual": True})
            else:
                ignorable.append(f"l{i}.canon1")
            if mlp is not None:
                more["ffn_scale"] = PartSpec("channel_scale", {"size": self.width, "weight": "ls2"})
            else:
                ignorable += [f"l{i}.norm2", f"l{i}.norm2.b", f"l{i}.ls2"]
            layers.append(LayerSpec(
                block="pre_norm_scaled", mixer_norm=self._norm("norm1"), mixer=self._mixer(i),
                ffn_norm=self._norm("norm2") if mlp is not None else None, feed_forward=self._feed_forward(mlp) if mlp is not None else None,
                weight_prefix=f"l{i}.", more=more))
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width, "weight": "embed", "scale": self.embedding_scale}),
            layers=layers, run_order=self.run_order(), final_norm=self._norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": True, "weight": "head", "tied_to": "embed"}),
            max_position=MAX_POSITION, ignorable=ignorable)
        spec.validate()
        return spec
