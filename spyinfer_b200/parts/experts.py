"""A mixture of small gated feed-forward experts, of which every token uses the few with the largest router scores.

Router: ``s = softmax(W_router h)`` over all experts, in 32-bit; the ``top`` largest scores are the chosen experts' weights
as they are (no renormalising).  An expert: ``g = min(W_gate h, limit)``, ``u = clamp(W_up h, -limit, limit)``,
``W_down (g * sigmoid(slope * g) * (u + 1))``, no biases.  An optional shared expert of the same form (sizes and limit of its
own) runs for every token, weighted by ``sigmoid(W_sg h)``, one number a token.

All experts' gate and up projections are one product, their down projections one product over the activations side by
side; the kernel between the two multiplies each expert's activation by the token's weight for it, which is exactly zero
for an expert that the token did not choose.  A token's result therefore does not depend on what else is in the batch.

A step of many tokens (``routed_from`` or more: by default so many that an expert gets 1,024 rows on average, below which its
products fill too little of the GPU to gain; ``SPYINFER_MOE_ROUTED_FROM`` in the environment sets the number, 0 turns the form
off; never inside a captured graph) takes the routed form instead: the (token, chosen expert) pairs are sorted by expert on the
device, the tokens' rows gathered in that order, each expert's two products run on its own run of rows (views of the same
fused weights, nothing stored twice), and every token's ``top`` results and the shared expert's are added in a fixed order in
32-bit.  The experts' row counts are read back once a layer to size the products.  Weights and arithmetic are the same, so the
two forms differ by the order of sums only.  Both forms serve the options of the choice (a correction for the choice only, groups
of router outputs, identity experts, whose pairs take no rows) and both activations.
"""
from __future__ import annotations

import os

import torch

from .. import kernels
from ..weights.loader import WeightDecl
from .base import FeedForward
from .linear import Linear
from .registry import register_part


@register_part("expert_mixture")
class ExpertMixture(FeedForward):
    """params: ``hidden_size``, ``experts``, ``top``, ``ff`` (an expert's inner size), ``limit``, ``shared_ff`` (0: no shared
    expert), ``shared_limit``, ``slope`` (default 1.702), ``prefix``; ``activation`` (``clamped_swish``, the default, or ``silu``:
    ``W_down (silu(W_gate h) * W_up h)`` without clamps, ``limit`` then unused); and the options of the choice: ``identity``
    (default 0: so many further router outputs, behind the experts', stand for experts without tensors that return their
    input), ``correction`` (default false: a tensor ``correction [experts + identity]`` is added to the scores for the choice
    only), ``groups`` (None or ``(count, keep)``: the router's outputs form ``count`` equal groups of neighbours, a group counts
    by its best choice score, and only the ``keep`` best groups' outputs can be chosen).  Tensors: ``router [experts +
    identity, hidden]``, ``e<i>.{gate,up} [ff, hidden]``, ``e<i>.down [hidden, ff]``, and with a shared expert
    ``shared.{gate,up,down}`` and ``shared.sg [1, hidden]``."""

    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden, self.experts, self.top, self.ff = int(params["hidden_size"]), int(params["experts"]), int(params["top"]), int(params["ff"])
        self.slope = float(params.get("slope", 1.702))
        self.shared_ff, self.shared_limit = int(params.get("shared_ff") or 0), float(params.get("shared_limit") or 0.0)
        self.limit = float(params.get("limit") or 0.0)
        self.activation = params.get("activation", "clamped_swish")
        self.identity, self.has_correction = int(params.get("identity") or 0), bool(params.get("correction", False))
        self.groups = tuple(int(v) for v in params["groups"]) if params.get("groups") else None
        self.outputs = self.experts + self.identity                 # the router's outputs
        if min(self.hidden, self.experts, self.top, self.ff) <= 0 or self.top > self.outputs or self.shared_ff < 0 or self.identity < 0:
            raise ValueError(f"expert_mixture: {self.experts} experts of {self.ff}, top {self.top}, shared {self.shared_ff} are not served")
        if self.activation not in ("clamped_swish", "silu") or (self.activation == "clamped_swish" and not self.limit > 0.0):
            raise ValueError(f"expert_mixture: activation {self.activation!r} (clamped_swish with a positive limit, or silu)")
        if self.groups is not None:
            count, keep = self.groups
            if count <= 0 or self.outputs % count or not 0 < keep <= count or keep * (self.outputs // count) < self.top:
                raise ValueError(f"expert_mixture: {count} groups of which {keep} are kept do not fit {self.outputs} router outputs and top {self.top}")
        self.plain_choice = not self.identity and not self.has_correction and self.groups is None and self.activation == "clamped_swish"
        self.correction = None
        self.prefix = params.get("prefix", "")
        self.cols = self.experts * self.ff + self.shared_ff
        self.router = self.gate_up = self.down = None
        default = -(-1024 * self.experts // self.top)
        try:
            self.routed_from = int(os.environ.get("SPYINFER_MOE_ROUTED_FROM", params.get("routed_from", default)))
        except ValueError:
            self.routed_from = default

    def weight_decls(self):
        p, W = self.prefix, self.hidden
        decls = [WeightDecl(p + "router", (self.outputs, W))] + ([WeightDecl(p + "correction", (self.outputs,))] if self.has_correction else [])
        for e in range(self.experts):
            decls += [WeightDecl(f"{p}e{e}.gate", (self.ff, W)), WeightDecl(f"{p}e{e}.up", (self.ff, W)), WeightDecl(f"{p}e{e}.down", (W, self.ff))]
        if self.shared_ff:
            decls += [WeightDecl(p + "shared.gate", (self.shared_ff, W)), WeightDecl(p + "shared.up", (self.shared_ff, W)),
                      WeightDecl(p + "shared.down", (W, self.shared_ff)), WeightDecl(p + "shared.sg", (1, W))]
        return decls

    def bind(self, tensors):
        p = self.prefix
        names = [f"e{e}." for e in range(self.experts)] + (["shared."] if self.shared_ff else [])
        rows = [tensors[p + n + half] for n in names for half in ("gate", "up")]
        downs = [tensors[p + n + "down"] for n in names]
        if len({t.dtype for t in rows + downs}) > 1:
            rows, downs = [t.float() for t in rows], [t.float() for t in downs]
        self.gate_up = Linear(torch.cat(rows, dim=0).contiguous(), self.ctx.dtype)
        self.down = Linear(torch.cat(downs, dim=1).contiguous(), self.ctx.dtype)
        # the router (and the shared expert's gate behind it) in 32-bit
        routes = [tensors[p + "router"].float()] + ([tensors[p + "shared.sg"].float()] if self.shared_ff else [])
        self.router = Linear(torch.cat(routes, dim=0).contiguous(), self.ctx.dtype)
        if self.has_correction:
            self.correction = tensors[p + "correction"].float().contiguous()

    def modules(self):
        return ["moe"] + self.router.modules() + self.gate_up.modules() + self.down.modules()

    def linears(self):
        return [self.router, self.gate_up, self.down]

    def forward(self, x):
        if 0 < self.routed_from <= x.shape[0] and self.top < self.outputs and not torch.cuda.is_current_stream_capturing():
            return self._routed(x)
        logits = self.router(x, out_dtype=torch.float32)
        gu = self.gate_up(x)
        y = torch.empty((x.shape[0], self.cols), dtype=self.ctx.dtype, device=x.device)
        if self.plain_choice:
            kernels.moe_activation(gu, logits, y, self.experts, self.top, self.ff, self.limit, self.shared_ff, self.shared_limit, self.slope)
            return self.down(y, defer=self.defer_output)
        idw = torch.empty((x.shape[0],), dtype=torch.float32, device=x.device) if self.identity else None
        kernels.moe_activation(gu, logits, y, self.experts, self.top, self.ff, self.limit, self.shared_ff, self.shared_limit, self.slope,
                               identity=self.identity, correction=self.correction, groups=self.groups, activation=self.activation, id_weight=idw)
        if not self.identity:
            return self.down(y, defer=self.defer_output)
        # the identity experts' share, weight * input, joins the experts' sum in 32-bit: in the consumer's kernel where it offers that
        # (the block arrangement said so), else here
        if self.leave_output_bias:
            self.output_rows = (x, idw)
            return self.down(y, defer=self.defer_output)
        return kernels.add_scaled_rows(self.down(y, out_dtype=torch.float32), x, idw)

    def _routed(self, x):
        T, E, top, ff, sff, dev = x.shape[0], self.experts, self.top, self.ff, self.shared_ff, x.device
        logits = self.router(x, out_dtype=torch.float32)
        idw = None
        if self.plain_choice:
            offsets, slot, row_token, row_w, shared_w = kernels.moe_route(logits, E, top, bool(sff))
        else:
            offsets, slot, row_token, row_w, shared_w, idw = kernels.moe_route_general(logits, E, top, self.identity, self.correction, self.groups, bool(sff))
        starts = offsets.cpu().tolist()                      # the layer's one read-back: the experts' row counts size their products
        R, n = T * top, starts[E]                            # n rows are in use: a token may have chosen fewer real experts than `top`
        results = torch.empty((R, self.hidden), dtype=torch.float32, device=dev)
        if n:
            rows = kernels.gather_rows(x, row_token[:n], torch.empty((n, self.hidden), dtype=x.dtype, device=dev))
            gu = torch.empty((n, 2 * ff), dtype=self.ctx.dtype, device=dev)
            for e in range(E):
                a, b = starts[e], starts[e + 1]
                if b > a:
                    self.gate_up.part(rows[a:b], rows=(2 * ff * e, 2 * ff * (e + 1)), out=gu[a:b])
            y = kernels.expert_activation(gu, row_w, torch.empty((n, ff), dtype=self.ctx.dtype, device=dev), self.limit, self.slope, activation=self.activation)
            for e in range(E):
                a, b = starts[e], starts[e + 1]
                if b > a:
                    self.down.part(y[a:b], cols=(ff * e, ff * (e + 1)), out=results[a:b])
        shared = None
        if sff:
            sgu = self.gate_up.part(x, rows=(2 * ff * E, 2 * ff * E + 2 * sff), out_dtype=self.ctx.dtype)
            sy = kernels.expert_activation(sgu, shared_w, torch.empty((T, sff), dtype=self.ctx.dtype, device=dev), self.shared_limit, self.slope,
                                           activation=self.activation)
            shared = self.down.part(sy, cols=(ff * E, ff * E + sff), out_dtype=torch.float32)
        out = kernels.moe_combine(results, slot, shared, torch.empty((T, self.hidden), dtype=torch.float32, device=dev))
        if idw is None:
            return out
        if self.leave_output_bias:                           # the identity experts' share is the consumer's to add
            self.output_rows = (x, idw)
            return out
        return kernels.add_scaled_rows(out, x, idw)
