"""Typed configuration of the Naforax decoder (config.json ``"architecture": "Naforax"``).

A stack of layers around a 32-bit residual stream with a norm on both sides of every sublayer,
``x += m * norm1b(mixer(c1(norm1(x))))`` then ``x += m * norm2b(ff(c2(norm2(x))))``: ``m`` is ``residual_mult``, every norm
an RMS norm in ``norm.groups`` equal consecutive groups with a plain gain (``norm.eps``), and ``c(h) = h + conv(h)`` a
causal convolution over time on every channel with ``canon.taps`` taps (tensors ``canon1``, ``canon2`` ``[width, taps]``),
whose last ``taps - 1`` inputs are part of a request's state.  config.json lists the layers (``layers[i]``: ``type``,
``mixer``, ``mlp``), and every layer may differ:

* ``type: "attention"``: differential softmax attention (``heads``, ``kv_heads``, per map ``dim``, ``vdim``, ``diff``,
  ``scale``, ``rot.base`` / ``rot.dims`` for the rotation of the interleaved pairs of each map's first elements,
  ``mask.size`` for the chunk a query sees), with biases on q, k, v and o, a norm on every map of q and k, and a sigmoid
  output gate.
* ``type: "mingru"``: the minimal gated recurrent unit over ``width`` channels.
* ``type: "mamba1"``: the selective scan (``inner`` channels of ``state`` states, ``dt_rank``, a convolution of ``conv`` taps).
* ``mlp``: null, ``{"kind": "dense", "ff": n}`` (``down(gelu_tanh(gate h) * up h)``) or ``{"kind": "moe", "router":
  {"experts", "top"}, "expert": {"ff", "limit"}, "shared": {"ff", "limit"} or null}``.

``loop: {start, stop, times}``: the layers ``start .. stop - 1`` run ``times`` times in a row with the same weights and a
cache of its own for every pass; ahead of each pass but the first the embedding output is added to the stream again, and
ahead of every pass row ``t`` of ``loop.step [times, width]``.  ``logits = cap * tanh(head(norm(x)) / cap)`` with
``logit_softcap`` (absent or 0: no cap).  Tensor names: ``embed``, ``loop.step``, ``l<i>.{norm1,norm1b,norm2,norm2b,canon1,
canon2}``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .model_config import ArchitectureConfig, ConfigError, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry, StreamAdd

MAX_POSITION = 1 << 20      # the design sets no limit of its own; the engine's max_model_len is the one that counts
EXPERT_SLOPE = 1.702        # the experts' activation is g * sigmoid(1.702 g)


def _int(d, key, where, least=1):
    v = d.get(key) if isinstance(d, dict) else None
    if not isinstance(v, int) or isinstance(v, bool) or v < least:
        raise ConfigError(f"Naforax config.json: {where}.{key} must be an integer of at least {least}, found {v!r}")
    return v


def _num(d, key, where, positive=False):
    v = d.get(key) if isinstance(d, dict) else None
    if not isinstance(v, (int, float)) or isinstance(v, bool) or (positive and not v > 0):
        raise ConfigError(f"Naforax config.json: {where}.{key} must be a{' positive' if positive else ''} number, found {v!r}")
    return float(v)


def _check_mixer(kind, m, where):
    if not isinstance(m, dict):
        raise ConfigError(f"Naforax config.json: {where} must be an object")
    if kind == "attention":
        heads, groups = _int(m, "heads", where), _int(m, "kv_heads", where)
        if heads % groups:
            raise ConfigError(f"Naforax config.json: {where}: {heads} heads do not group over {groups} key/value heads")
        dim = _int(m, "dim", where)
        _int(m, "vdim", where)
        _num(m, "diff", where)
        if m.get("scale") is None:
            m["scale"] = float(dim) ** -0.5
        _num(m, "scale", where, positive=True)
        rot = m.get("rot")
        if rot is not None and rot.get("dims"):
            dims = _int(rot, "dims", where + ".rot", least=2)
            if dims % 2 or dims > dim:
                raise ConfigError(f"Naforax config.json: {where}.rot.dims {dims} must be even and at most dim ({dim})")
            _num(rot, "base", where + ".rot", positive=True)
        if m.get("mask") is not None:
            _int(m["mask"], "size", where + ".mask")
    elif kind == "mingru":
        _int(m, "width", where)
    elif kind == "mamba1":
        for k in ("inner", "state", "dt_rank", "conv"):
            _int(m, k, where)
    else:
        raise ConfigError(f"Naforax config.json: {where[:-6]}.type {kind!r} is not a known layer type (attention, mingru, mamba1)")


def _check_mlp(mlp, where):
    if mlp is None:
        return
    kind = mlp.get("kind") if isinstance(mlp, dict) else None
    if kind == "dense":
        _int(mlp, "ff", where)
    elif kind == "moe":
        experts, top = _int(mlp.get("router"), "experts", where + ".router"), _int(mlp.get("router"), "top", where + ".router")
        if top > experts:
            raise ConfigError(f"Naforax config.json: {where}.router.top {top} exceeds the {experts} experts")
        for name in ("expert",) + (("shared",) if mlp.get("shared") is not None else ()):
            _int(mlp.get(name), "ff", f"{where}.{name}")
            _num(mlp.get(name), "limit", f"{where}.{name}", positive=True)
    else:
        raise ConfigError(f"Naforax config.json: {where}.kind {kind!r} is not implemented (dense, moe)")


@register_architecture("Naforax", model_type="naforax")
@dataclass
class NaforaxConfig(ArchitectureConfig):
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    taps: int
    residual_mult: float
    logit_softcap: float
    layers: List[Dict[str, Any]]
    loop: Optional[Dict[str, int]] = None
    extra: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_json(cls, data: Dict[str, Any]) -> "NaforaxConfig":
        vocab, width = _int(data, "vocab", "config"), _int(data, "width", "config")
        eps = _num(data.get("norm"), "eps", "norm", positive=True)
        groups = _int(data.get("norm"), "groups", "norm") if (data.get("norm") or {}).get("groups") is not None else 1
        if width % groups:
            raise ConfigError(f"Naforax config.json: norm.groups {groups} does not divide the width {width}")
        taps = _int(data.get("canon"), "taps", "canon") if data.get("canon") is not None else 0      # 0: no input convolution
        mult = _num(data, "residual_mult", "config") if data.get("residual_mult") is not None else 1.0
        cap = _num(data, "logit_softcap", "config") if data.get("logit_softcap") is not None else 0.0
        if cap < 0.0:
            raise ConfigError(f"Naforax config.json: logit_softcap {cap} must not be negative")
        layers = copy.deepcopy(data.get("layers"))
        if not isinstance(layers, list) or not layers:
            raise ConfigError("Naforax config.json: 'layers' must list at least one layer")
        for i, layer in enumerate(layers):
            _check_mixer(layer.get("type"), layer.get("mixer"), f"layers[{i}].mixer")
            _check_mlp(layer.get("mlp"), f"layers[{i}].mlp")
        loop = copy.deepcopy(data.get("loop"))
        if loop is not None:
            start, stop, times = _int(loop, "start", "loop", least=0), _int(loop, "stop", "loop", least=0), _int(loop, "times", "loop")
            if not start <= stop <= len(layers):
                raise ConfigError(f"Naforax config.json: loop {start} .. {stop} does not lie within the {len(layers)} layers")
        known = {"architecture", "architectures", "model_type", "vocab", "width", "norm", "canon", "residual_mult", "logit_softcap", "layers", "loop"}
        return cls(vocab=vocab, width=width, norm_eps=eps, norm_groups=groups, taps=taps, residual_mult=mult, logit_softcap=cap, layers=layers,
                   loop=loop, extra={k: v for k, v in data.items() if k not in known})

    def to_json(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
             "canon": {"taps": self.taps} if self.taps else None, "residual_mult": self.residual_mult, "logit_softcap": self.logit_softcap,
             "layers": copy.deepcopy(self.layers), "loop": copy.deepcopy(self.loop)}
        for k, v in self.extra.items():
            d.setdefault(k, v)
        return d

    # ---- parts -------------------------------------------------------------------------------
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("group_rms_norm", {"size": self.width, "groups": self.norm_groups, "eps": self.norm_eps, "weight": name})

    def _conv(self, name: str) -> PartSpec:
        return PartSpec("causal_conv", {"channels": self.width, "taps": self.taps, "weight": name, "residual": True})

    def _mixer(self, layer: Dict[str, Any]) -> PartSpec:
        W, m, kind = self.width, layer["mixer"], layer["type"]
        if kind == "mingru":
            return PartSpec("mingru", {"hidden_size": W, "width": m["width"], "prefix": "mix."})
        if kind == "mamba1":
            return PartSpec("selective_scan", {"hidden_size": W, "inner": m["inner"], "state": m["state"], "dt_rank": m["dt_rank"], "taps": m["conv"],
                                               "prefix": "mix."})
        rot, position = m.get("rot"), None
        if rot is not None and rot.get("dims"):
            position = PartSpec("rotary_interleaved", {"theta": float(rot["base"]), "rotary_dim": int(rot["dims"])})
        return PartSpec("differential_attention", {
            "hidden_size": W, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"], "diff": float(m["diff"]),
            "scale": float(m["scale"]), "eps": self.norm_eps, "chunk": int(m["mask"]["size"]) if m.get("mask") is not None else None,
            "position": position, "prefix": "mix."})

    def _feed_forward(self, mlp: Dict[str, Any]) -> PartSpec:
        W = self.width
        if mlp["kind"] == "dense":
            return PartSpec("gated_mlp", {"hidden_size": W, "intermediate_size": mlp["ff"], "activation": "gelu_tanh", "prefix": "mlp.",
                                          "names": {"gate": "gate", "up": "up", "down": "down"}})
        shared = mlp.get("shared")
        return PartSpec("expert_mixture", {
            "hidden_size": W, "experts": mlp["router"]["experts"], "top": mlp["router"]["top"], "ff": mlp["expert"]["ff"],
            "limit": float(mlp["expert"]["limit"]), "shared_ff": shared["ff"] if shared is not None else 0,
            "shared_limit": float(shared["limit"]) if shared is not None else 0.0, "slope": EXPERT_SLOPE, "prefix": "mlp."})

    def run_order(self) -> List[RunEntry]:
        n, loop = len(self.layers), self.loop
        if loop is None or loop["start"] == loop["stop"]:
            return [RunEntry(i) for i in range(n)]
        order = [RunEntry(i) for i in range(loop["start"])]
        for t in range(loop["times"]):
            ahead = StreamAdd(embedding=t > 0, tensor="loop.step", rows=loop["times"], row=t)
            order += [RunEntry(i, before=ahead if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
        return order + [RunEntry(i) for i in range(loop["stop"], n)]

    def to_spec(self) -> ModelSpec:
        layers, ignorable = [], []
        for i, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            more = {"mixer_out_norm": self._norm("norm1b")}
            if self.taps:
                more["mixer_conv"] = self._conv("canon1")
            else:
                ignorable.append(f"l{i}.canon1")
            if mlp is not None:
                more["ffn_out_norm"] = self._norm("norm2b")
                if self.taps:
                    more["ffn_conv"] = self._conv("canon2")
            if mlp is None or not self.taps:
                ignorable.append(f"l{i}.canon2")
            if mlp is None:
                ignorable += [f"l{i}.norm2", f"l{i}.norm2b"]
            layers.append(LayerSpec(
                block="sandwich_norm", mixer_norm=self._norm("norm1"), mixer=self._mixer(layer),
                ffn_norm=self._norm("norm2") if mlp is not None else None, feed_forward=self._feed_forward(mlp) if mlp is not None else None,
                weight_prefix=f"l{i}.", more=more, block_params={"residual_scale": self.residual_mult}))
        order = self.run_order()
        if not any(e.before is not None for e in order):
            ignorable.append("loop.step")
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width, "weight": "embed"}),
            layers=layers, run_order=order, final_norm=self._norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": False, "weight": "head", "tied_to": "embed",
                                      "softcap": self.logit_softcap}),
            max_position=MAX_POSITION, ignorable=ignorable)
        spec.validate()
        return spec
