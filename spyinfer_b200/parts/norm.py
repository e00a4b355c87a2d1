"""RMSNorm: ``x * (1 / sqrt(mean(x^2) + eps)) * weight``, statistics in 32-bit, plain weight
(or, with ``weight_offset``, a weight that is stored around zero: ``offset + weight``).

Formula: spymaster2h/spyinfer src/backends/cpu/x64/kernels.cpp:168-180; used before the
mixer, before the feed-forward and before the head (src/models/qwen3.hpp:127-133, 224-230,
287-293).  The residual sum of the block is fused into the same kernel.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import WeightDecl
from .base import ChannelScaled, Norm, NormedDelta, ScaledParts
from .registry import register_part


@register_part("rms_norm")
class RMSNorm(Norm):
    graph_safe = True
    """params: ``size``, ``eps``, ``weight`` (the tensor's relative name), ``weight_offset`` (default 0; with 1 the stored
    tensor is the gain's distance from one and the norm multiplies by ``1 + weight``)."""

    #: set by a block arrangement that has this norm on a sublayer's output (``add_normed``): it then runs the kernel
    #: that adds the normed result to the stream, not the one that norms the stream
    adds_to_stream = False

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.size, self.eps, self.weight_name = int(params["size"]), float(params["eps"]), params.get("weight", "weight")
        self.weight_offset = float(params.get("weight_offset", 0.0))
        self.weight = None

    def weight_decls(self):
        return [WeightDecl(self.weight_name, (self.size,), init="normal" if self.weight_offset else "one_plus_normal")]

    def bind(self, tensors):
        self.weight = tensors[self.weight_name]
        if self.weight_offset:
            self.weight = (self.weight.float() + self.weight_offset).contiguous()     # the gain itself, in 32-bit

    def modules(self):
        return ["residual_norm"] if self.adds_to_stream else ["rmsnorm"]

    def add_normed(self, residual, y):
        """``residual += norm(y)`` (32-bit, in place) for a block whose norm sits on a sublayer's output; ``y`` may be a
        stack of float32 partial products.  Returns what the next sublayer reads: the stream itself when the activations
        are 32-bit, else a copy of it in their type, made by the same kernel."""
        copy = None if self.ctx.dtype == torch.float32 else torch.empty(residual.shape, dtype=self.ctx.dtype, device=residual.device)
        kernels.residual_norm(residual, y, self.weight, self.eps, copy=copy)
        return residual if copy is None else copy

    def forward(self, x, out_dtype=None):
        out = torch.empty(x.shape, dtype=out_dtype or self.ctx.dtype, device=x.device)
        return kernels.rmsnorm(x, self.weight, self.eps, out)

    def forward_add(self, residual, delta, rows=None, out_dtype=None):
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.size), dtype=out_dtype or self.ctx.dtype, device=residual.device)
        return kernels.rmsnorm(residual, self.weight, self.eps, out, delta=delta, rows=rows, write_back=delta is not None and rows is None)


@register_part("layer_norm")
class LayerNorm(Norm):
    """``(x - mean) / sqrt(var + eps) * weight (+ bias)`` with ``var`` the mean squared deviation, statistics in 32-bit, a
    plain weight.  params: ``size``, ``eps``, ``weight`` (the tensor's relative name), ``bias`` (a relative name, or None:
    no bias), ``center`` (default true; false keeps the mean: an RMS norm).  The residual sum fused into the kernel may carry
    a scale and may be a weighted sum of two results (``ScaledParts``): ``residual += scale * (s1 * d1 + s2 * d2)``, or one
    result times a vector along the row (``ChannelScaled``): ``residual += scale * weight * d``."""

    graph_safe = True
    takes_scaled_parts = True
    takes_channel_scale = True
    kernel_modules = ("layernorm",)

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.size, self.eps, self.weight_name = int(params["size"]), float(params["eps"]), params.get("weight", "weight")
        self.center = bool(params.get("center", True))
        self.bias_name = params.get("bias")
        self.weight = self.bias = None

    def weight_decls(self):
        return [WeightDecl(self.weight_name, (self.size,), init="one_plus_normal")] + ([WeightDecl(self.bias_name, (self.size,))] if self.bias_name else [])

    def bind(self, tensors):
        self.weight = tensors[self.weight_name]
        if self.bias_name:
            self.bias = tensors[self.bias_name].to(self.weight.dtype).contiguous()

    def forward(self, x, out_dtype=None):
        out = torch.empty(x.shape, dtype=out_dtype or self.ctx.dtype, device=x.device)
        return kernels.layernorm(x, self.weight, self.eps, out, center=self.center, bias=self.bias)

    def forward_add(self, residual, delta, rows=None, out_dtype=None, scale=1.0):
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.size), dtype=out_dtype or self.ctx.dtype, device=residual.device)
        if isinstance(delta, ChannelScaled):
            return kernels.layernorm(residual, self.weight, self.eps, out, delta=delta.y, delta_scale=scale, delta_weight=delta.weight.to(self.weight.dtype),
                                     delta_bias=delta.bias, delta_rows=delta.rows, rows=rows, write_back=rows is None, center=self.center, bias=self.bias)
        terms = delta.terms if isinstance(delta, ScaledParts) else ([(delta, 1.0)] if delta is not None else [])
        if len(terms) > 2:
            raise ValueError(f"layer_norm: a weighted sum of {len(terms)} results (at most two)")
        if len(terms) == 2 and terms[0][0].dtype != terms[1][0].dtype:
            terms = [(t.float() if t.dim() == 2 else t, s) for t, s in terms]
        (d1, s1), (d2, s2) = (terms + [(None, 1.0), (None, 1.0)])[:2]
        return kernels.layernorm(residual, self.weight, self.eps, out, delta=d1, delta_scale=scale * s1, delta2=d2, delta2_scale=scale * s2,
                                 rows=rows, write_back=bool(terms) and rows is None, center=self.center, bias=self.bias)


@register_part("channel_scale")
class ChannelScale(Norm):
    """A learned multiplier for every channel of a sublayer's output (a layer scale): ``y * weight``.  It launches nothing:
    ``defer(y)`` hands the product on as a ``ChannelScaled`` record that the next norm of the stream forms inside its own
    kernel, in 32-bit.  params: ``size``, ``weight`` (the tensor's relative name)."""

    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.size, self.weight_name = int(params["size"]), params.get("weight", "weight")
        self.weight = None

    def weight_decls(self):
        return [WeightDecl(self.weight_name, (self.size,), init="one_plus_normal")]

    def bind(self, tensors):
        self.weight = tensors[self.weight_name].contiguous()

    def defer(self, y, bias=None, rows=None):
        return ChannelScaled(y, self.weight, bias, rows)


@register_part("group_rms_norm")
class GroupRMSNorm(Norm):
    """RMS norm in groups: the row is cut into ``groups`` equal consecutive parts, each divided by its own
    ``sqrt(mean(part^2) + eps)``, and the whole multiplied by a plain weight.  params: ``size``, ``groups``, ``eps``,
    ``weight`` (the tensor's relative name).

    It serves on both sides of a sublayer.  Ahead of one, ``forward_add(residual, delta)`` norms the stream; ``delta`` may
    be a ``NormedDelta`` that a norm of this kind (same size, groups and eps) left behind a sublayer (``defer``), and the
    one kernel then first adds ``scale * norm(y) * weight`` to the stream.  Behind one, ``defer(y, scale)`` makes that
    record, and ``add_normed`` adds it at once."""

    graph_safe = True
    kernel_modules = ("group_norm",)

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.size, self.groups, self.eps = int(params["size"]), int(params.get("groups", 1)), float(params["eps"])
        if self.groups <= 0 or self.size % self.groups:
            raise ValueError(f"group_rms_norm: rows of {self.size} cannot be cut into {self.groups} equal groups")
        self.weight_name = params.get("weight", "weight")
        self.weight = None

    def weight_decls(self):
        return [WeightDecl(self.weight_name, (self.size,), init="one_plus_normal")]

    def bind(self, tensors):
        self.weight = tensors[self.weight_name].contiguous()

    def defer(self, y, scale=1.0):
        return NormedDelta(y, self.weight, float(scale))

    def _pending(self, delta):
        if delta is None:
            return None, None, 1.0
        if not isinstance(delta, NormedDelta):
            raise ValueError("group_rms_norm: what is pending on the stream must be a sublayer output that a norm of this kind deferred")
        return delta.y, delta.weight, delta.scale

    def add_normed(self, residual, delta):
        """``residual += scale * norm(y) * weight`` for a ``NormedDelta`` (32-bit, in place)."""
        y, w, scale = self._pending(delta)
        if y is not None:
            kernels.group_norm(residual, self.groups, self.eps, y=y, y_weight=w, y_scale=scale)
        return residual

    def forward(self, x, out_dtype=None):
        out = torch.empty(x.shape, dtype=out_dtype or self.ctx.dtype, device=x.device)
        return kernels.group_norm(x, self.groups, self.eps, weight=self.weight, out=out)

    def forward_add(self, residual, delta, rows=None, out_dtype=None):
        y, w, scale = self._pending(delta)
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.size), dtype=out_dtype or self.ctx.dtype, device=residual.device)
        return kernels.group_norm(residual, self.groups, self.eps, y=y, y_weight=w, y_scale=scale, weight=self.weight, out=out, rows=rows)
