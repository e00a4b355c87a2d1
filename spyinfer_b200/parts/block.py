"""Block arrangements around the 32-bit residual stream.

``pre_norm``: ``h += mixer(norm(h)); h += ffn(norm(h))`` (spymaster2h/spyinfer
src/models/qwen3.hpp:127-133, 216-230, 272-277).  Each residual sum is fused into the norm
that follows it: a block receives the previous block's output as ``delta``, still to be
added, and hands its own feed-forward output on in the same way.
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import Block

_BLOCKS = {}


def register_block(kind: str):
    def wrap(cls):
        cls.kind = kind
        _BLOCKS[kind] = cls
        return cls

    return wrap


def build_block(kind: str, parts, params=None) -> Block:
    """``parts``: role -> built part (``LayerSpec.roles()`` with every ``PartSpec`` built); ``params``: the
    arrangement's own constants (``LayerSpec.block_params``)."""
    if kind not in _BLOCKS:
        raise KeyError(f"unknown block arrangement {kind!r}; registered: {', '.join(sorted(_BLOCKS))}")
    cls = _BLOCKS[kind]
    return cls(dict(parts), dict(params)) if params else cls(dict(parts))


@register_block("pre_norm")
class PreNormBlock(Block):
    graph_safe = True

    def forward(self, hidden, delta, batch, cache):
        x = self.mixer_norm.forward_add(hidden, delta)
        a = self.mixer.forward(x, batch, cache)
        x = self.ffn_norm.forward_add(hidden, a)
        return hidden, self.feed_forward.forward(x)


@register_block("post_norm")
class PostNormBlock(Block):
    """``h += norm1(mixer(h)); h += norm2(ffn(h))``: the sublayers read the residual stream itself and the norm sits on
    their output only; a layer may do without the feed-forward half.  The norms must offer ``add_normed``.  On the
    bfloat16 path the products read a copy of the stream in that type, which the kernel that adds a sublayer's normed
    output also writes (one launch a sublayer); the copy that a block leaves is handed to the next block through the
    batch's ``extras``."""

    graph_safe = True
    required = ("mixer_norm", "mixer")
    optional = ("ffn_norm", "feed_forward")

    def __init__(self, parts, params=None):
        super().__init__(parts, params)
        if (self.ffn_norm is None) != (self.feed_forward is None):
            raise ValueError("block arrangement 'post_norm': the feed-forward and its norm come together or not at all")
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None and not hasattr(norm, "add_normed"):
                raise ValueError(f"block arrangement 'post_norm': the norm {norm.kind!r} cannot add its result to the stream")
            if norm is not None:
                norm.adds_to_stream = True

    def forward(self, hidden, delta, batch, cache):
        if delta is not None:
            raise ValueError("block arrangement 'post_norm' follows a block that left its residual sum to the next norm; it has none ahead of its mixer")
        held = batch.extras.get("stream_copy")
        if held is not None and held[0] is hidden:
            x = held[1]
        elif self.mixer_norm.ctx.dtype == hidden.dtype:
            x = hidden
        else:
            x = torch.empty(hidden.shape, dtype=self.mixer_norm.ctx.dtype, device=hidden.device)
            kernels.residual_norm(hidden, None, None, 0.0, copy=x)
        x = self.mixer_norm.add_normed(hidden, self.mixer.forward(x, batch, cache))
        if self.feed_forward is not None:
            x = self.ffn_norm.add_normed(hidden, self.feed_forward.forward(x))
        batch.extras["stream_copy"] = (hidden, x)
        return hidden, None


@register_block("pre_norm_scaled")
class ScaledPreNormBlock(Block):
    """``h += m * mixer(norm(h)); h += m * ffn(norm(h))`` with one multiplier ``m`` (param ``residual_scale``) for both
    sums, and a layer may do without the feed-forward half.  Its norms must take a scale (``Norm.takes_scaled_parts``);
    then the mixer may also hand over a weighted sum that is still to be formed (``ScaledParts``).

    Optional parts: ``mixer_conv``, an input convolution over time between the first norm and the mixer (a part with
    ``forward(x, batch, cache)`` and ``cache_need()``, such as ``causal_conv``: the mixer reads ``c(norm(h))``), and
    ``mixer_scale`` / ``ffn_scale`` (``channel_scale``), a multiplier for every channel of a sublayer's output, which the
    next norm of the stream applies inside its kernel (it must say ``takes_channel_scale``).  With a convolution the
    layer's need is the composite (convolution state, the mixer's need), and a layer that reads another entry's cache
    still keeps its own convolution state."""

    graph_safe = True
    required = ("mixer_norm", "mixer")
    optional = ("ffn_norm", "feed_forward", "mixer_conv", "mixer_scale", "ffn_scale")

    def __init__(self, parts, params=None):
        super().__init__(parts, params)
        self.residual_scale = float(self.params.get("residual_scale", 1.0))
        if (self.ffn_norm is None) != (self.feed_forward is None):
            raise ValueError("block arrangement 'pre_norm_scaled': the feed-forward and its norm come together or not at all")
        if self.ffn_scale is not None and self.feed_forward is None:
            raise ValueError("block arrangement 'pre_norm_scaled': a scale of the feed-forward's output needs the feed-forward")
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None and not norm.takes_scaled_parts:
                raise ValueError(f"block arrangement 'pre_norm_scaled': the norm {norm.kind!r} takes no scale")
            if norm is not None and (self.mixer_scale is not None or self.ffn_scale is not None) and not norm.takes_channel_scale:
                raise ValueError(f"block arrangement 'pre_norm_scaled': the norm {norm.kind!r} takes no per-channel multiplier")
        if hasattr(self.mixer, "scaled_parts_ok"):
            self.mixer.scaled_parts_ok = self.ffn_norm is not None and self.mixer_scale is None      # the sum is formed by this layer's second norm
        self._conv_state = self.mixer_conv is not None and self.mixer_conv.cache_need() is not None
        if self.ffn_scale is not None:
            self.feed_forward.leave_output_bias = True       # the norm that applies the scale adds the last projection's bias too

    def cache_need(self):
        from ..config.spec import CompositeCacheNeed
        own = self.mixer.cache_need()
        if not self._conv_state:
            return own
        return CompositeCacheNeed((self.mixer_conv.cache_need(),) + ((own,) if own is not None else ()))

    def cache_need_reading(self):
        from ..config.spec import CompositeCacheNeed, SharedCacheNeed
        if not self._conv_state:
            return None
        return CompositeCacheNeed((self.mixer_conv.cache_need(), SharedCacheNeed()))

    def forward(self, hidden, delta, batch, cache):
        x = self.mixer_norm.forward_add(hidden, delta, scale=self.residual_scale)
        if self.mixer_conv is not None:
            x = self.mixer_conv.forward(x, batch, cache.parts[0] if self._conv_state else None)
        if self._conv_state:
            cache = cache.parts[1] if len(cache.parts) > 1 else None
        a = self.mixer.forward(x, batch, cache)
        if self.mixer_scale is not None:
            a = self.mixer_scale.defer(a)
        if self.feed_forward is None:
            return hidden, a
        x = self.ffn_norm.forward_add(hidden, a, scale=self.residual_scale)
        f = self.feed_forward.forward(x)
        return hidden, self.ffn_scale.defer(f, self.feed_forward.output_bias, self.feed_forward.output_rows) if self.ffn_scale is not None else f


@register_block("sandwich_norm")
class SandwichNormBlock(Block):
    """``h += m * out_norm(mixer(c(norm(h))))`` and the same around the feed-forward: a norm on both sides of every sublayer,
    one multiplier ``m`` (param ``residual_scale``) on what the stream takes, and optionally an input convolution ``c`` over
    time (a part that offers ``forward(x, batch, cache)`` and ``cache_need()``, such as ``causal_conv``) between the first
    norm and the sublayer.  A layer may do without the feed-forward half.

    The output norms must offer ``defer``/``add_normed`` (``group_rms_norm``): a sublayer's output is handed on as a record
    that the next norm of the stream adds, normed and weighted, in the launch that also norms the stream for the next
    sublayer.  What the convolutions keep between steps lies beside the mixer's cache: the layer's need is a composite of
    (the mixer convolution's state, the feed-forward convolution's state, the mixer's need), parts that are absent left out."""

    graph_safe = True
    required = ("mixer_norm", "mixer", "mixer_out_norm")
    optional = ("mixer_conv", "ffn_norm", "ffn_conv", "feed_forward", "ffn_out_norm")

    def __init__(self, parts, params=None):
        super().__init__(parts, params)
        self.mult = float(self.params.get("residual_scale", 1.0))
        if len({self.ffn_norm is None, self.feed_forward is None, self.ffn_out_norm is None}) > 1:
            raise ValueError("block arrangement 'sandwich_norm': the feed-forward and its two norms come together or not at all")
        if self.ffn_conv is not None and self.feed_forward is None:
            raise ValueError("block arrangement 'sandwich_norm': an input convolution of the feed-forward needs the feed-forward")
        for norm in (self.mixer_out_norm, self.ffn_out_norm):
            if norm is not None and not (hasattr(norm, "defer") and hasattr(norm, "add_normed")):
                raise ValueError(f"block arrangement 'sandwich_norm': the norm {norm.kind!r} cannot hand a normed output on to the stream")
        self.mixer.output_dtype = torch.float32      # what an output norm reads is not rounded to 16 bits first
        # where each holder of state finds its view among the parts of the layer's composite need
        self._order = [role for role in ("mixer_conv", "ffn_conv", "mixer") if self.parts.get(role) is not None and self.parts[role].cache_need() is not None]

    def cache_need(self):
        from ..config.spec import CompositeCacheNeed
        needs = tuple(self.parts[role].cache_need() for role in self._order)
        if self._order == ["mixer"]:
            return needs[0]
        return CompositeCacheNeed(needs) if needs else None

    def _view(self, cache, role):
        if role not in self._order:
            return None
        return cache if self._order == ["mixer"] else cache.parts[self._order.index(role)]

    def forward(self, hidden, delta, batch, cache):
        x = self.mixer_norm.forward_add(hidden, delta)
        if self.mixer_conv is not None:
            x = self.mixer_conv.forward(x, batch, self._view(cache, "mixer_conv"))
        delta = self.mixer_out_norm.defer(self.mixer.forward(x, batch, self._view(cache, "mixer")), self.mult)
        if self.feed_forward is None:
            return hidden, delta
        x = self.ffn_norm.forward_add(hidden, delta)
        if self.ffn_conv is not None:
            x = self.ffn_conv.forward(x, batch, self._view(cache, "ffn_conv"))
        return hidden, self.ffn_out_norm.defer(self.feed_forward.forward(x), self.mult)

    def settle(self, hidden, delta):
        return self.mixer_out_norm.add_normed(hidden, delta) if delta is not None else hidden
