"""A causal convolution over time on every channel, whose past inputs are a request's state.

``conv(x)_t = sum_j w[:, j] * x_(t - taps + 1 + j)`` with zeros before a sequence's start (the kernel's last column meets the
current token), then ``act(conv + bias (+ x_t))``.  The ``taps - 1`` inputs ahead of a step's first token live in the
request's slot of the cache manager in 32-bit, so a token's result does not depend on where its sequence was cut into steps.
A block arrangement puts it ahead of a sublayer (``residual``: the sublayer reads ``x + conv(x)``); a mixer uses it on a
part of its projection (``channels`` of a wider row).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.spec import StateCacheNeed
from ..weights.loader import WeightDecl
from .base import Part
from .registry import register_part


@register_part("causal_conv")
class CausalConv(Part):
    """params: ``channels``, ``taps`` (at least 1; with 1 tap there is no state), ``weight`` (the tensor's relative name,
    ``[channels, taps]``), ``bias`` (a relative name or None), ``residual`` (default false: the input is added to the
    result), ``activation`` (None or ``"silu"``)."""

    graph_safe = True
    kernel_modules = ("time_conv",)

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.channels, self.taps = int(params["channels"]), int(params["taps"])
        if self.channels <= 0 or not 1 <= self.taps <= 16:
            raise ValueError(f"causal_conv: {self.channels} channels and {self.taps} taps (1 to 16) are not served")
        self.weight_name, self.bias_name = params.get("weight", "weight"), params.get("bias")
        self.residual, self.activation = bool(params.get("residual", False)), params.get("activation")
        if self.activation not in (None, "silu"):
            raise ValueError(f"causal_conv: activation {self.activation!r} is not implemented (only \"silu\")")
        self.weight = self.bias = None

    def weight_decls(self):
        decls = [WeightDecl(self.weight_name, (self.channels, self.taps))]
        if self.bias_name is not None:
            decls.append(WeightDecl(self.bias_name, (self.channels,)))
        return decls

    def bind(self, tensors):
        self.weight = tensors[self.weight_name].contiguous()
        if self.bias_name is not None:
            self.bias = tensors[self.bias_name].to(self.weight.dtype).contiguous()

    def cache_need(self):
        return StateCacheNeed(((self.taps - 1) * self.channels,), "float32") if self.taps > 1 else None

    def forward(self, x: torch.Tensor, batch, cache, out_dtype=None) -> torch.Tensor:
        """``x [T, >= channels]`` (the first ``channels`` columns are read) -> ``[T, channels]``; ``cache`` is the view of this
        part's state (not looked at with one tap)."""
        out = torch.empty((x.shape[0], self.channels), dtype=out_dtype or self.ctx.dtype, device=x.device)
        return kernels.time_conv(x, self.channels, self.weight, self.bias, cache.state if self.taps > 1 else None, batch.q_start, batch.state_slot,
                                 batch.num_seqs, 1 if batch.one_token_each else batch.num_tokens, out, residual=self.residual,
                                 activation=self.activation)
