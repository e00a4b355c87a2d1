"""Mixers that carry a vector (or a few states per channel) from token to token, element by element, in 32-bit.

``mingru`` (the minimal gated recurrent unit, whose gates read the current token only): with ``h`` the input,
``z = sigmoid(W_z h + b_z)``, ``u = W_x h + b_x``, the candidate ``c = u + 1/2`` where ``u >= 0`` and ``sigmoid(u)``
elsewhere; ``S_t = (1 - z) S_(t-1) + z c`` over ``width`` channels, output ``W_o (S_t * silu(W_g h))``.

``selective_scan`` (the selective state-space scan): ``W_in h = [x | z]`` (``inner`` each); ``x`` passes a causal convolution
over time with a bias and silu; ``W_x x = [dt (dt_rank) | B (state) | C (state)]``, ``dt = softplus(W_dt dt + b_dt)`` per
channel, ``A = -exp(A_log)``; per channel ``c`` and state ``n``: ``S[c, n] = exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n``,
``y_c = sum_n S[c, n] C_n + D_c x_c``; output ``W_o (y * silu(z))``.

The projections that feed a recurrence come back in 32-bit (nothing that enters it is rounded to 16 bits but ``x``, which is
the product's input as well); the states live in the request's slot of the cache manager and start at zero.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.spec import CompositeCacheNeed, PartSpec, StateCacheNeed
from ..weights.loader import WeightDecl
from .base import Mixer
from .linear import Linear
from .registry import build_part, register_part


def _cat_rows(tensors):
    if len({t.dtype for t in tensors}) > 1:
        tensors = [t.float() for t in tensors]
    return torch.cat(tensors, dim=0).contiguous()


@register_part("mingru")
class MinGRU(Mixer):
    """params: ``hidden_size``, ``width`` (channels of the recurrence), ``prefix``.  Tensors: ``z, x, g [width, hidden]``,
    ``z.b, x.b [width]``, ``o [hidden, width]``."""

    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden, self.width = int(params["hidden_size"]), int(params["width"])
        if min(self.hidden, self.width) <= 0:
            raise ValueError("mingru: sizes must be positive")
        self.prefix = params.get("prefix", "")
        self.fused = self.o = self.bias_z = self.bias_x = None

    def weight_decls(self):
        p, n, W = self.prefix, self.width, self.hidden
        return [WeightDecl(p + "z", (n, W)), WeightDecl(p + "z.b", (n,)), WeightDecl(p + "x", (n, W)), WeightDecl(p + "x.b", (n,)),
                WeightDecl(p + "g", (n, W)), WeightDecl(p + "o", (W, n))]

    def bind(self, tensors):
        p = self.prefix
        self.fused = Linear(_cat_rows([tensors[p + n] for n in ("z", "x", "g")]), self.ctx.dtype)
        self.o = Linear(tensors[p + "o"], self.ctx.dtype)
        self.bias_z, self.bias_x = tensors[p + "z.b"].float().contiguous(), tensors[p + "x.b"].float().contiguous()

    def modules(self):
        return ["gated_scan"] + self.fused.modules() + self.o.modules()

    def linears(self):
        return [self.fused, self.o]

    def cache_need(self):
        return StateCacheNeed((self.width,), "float32")

    def forward(self, x, batch, cache):
        n = self.width
        proj = self.fused(x, out_dtype=torch.float32)
        y = torch.empty((x.shape[0], n), dtype=self.ctx.dtype, device=x.device)
        kernels.mingru_scan(proj, 0, n, 2 * n, self.bias_z, self.bias_x, cache.state, batch.q_start, batch.state_slot, batch.num_seqs, y, n,
                            longest=1 if batch.one_token_each else batch.num_tokens)
        return self.o(y, defer=self.defer_output, out_dtype=self.output_dtype)


@register_part("selective_scan")
class SelectiveScan(Mixer):
    """params: ``hidden_size``, ``inner`` (channels), ``state`` (states a channel), ``dt_rank``, ``taps`` (of the convolution on
    ``x``), ``prefix``.  Tensors: ``in [2 inner, hidden]``, ``conv [inner, taps]``, ``conv.b [inner]``,
    ``x [dt_rank + 2 state, inner]``, ``dt [inner, dt_rank]``, ``dt.b [inner]``, ``A_log [inner, state]``, ``D [inner]``,
    ``o [hidden, inner]``."""

    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden, self.inner, self.n, self.rank = int(params["hidden_size"]), int(params["inner"]), int(params["state"]), int(params["dt_rank"])
        if min(self.hidden, self.inner, self.n, self.rank) <= 0:
            raise ValueError("selective_scan: sizes must be positive")
        self.prefix = params.get("prefix", "")
        p = self.prefix
        self.conv = build_part(PartSpec("causal_conv", {"channels": self.inner, "taps": int(params["taps"]), "weight": p + "conv", "bias": p + "conv.b",
                                                        "activation": "silu"}), ctx)
        self.w_in = self.w_x = self.w_dt = self.o = self.dt_bias = self.a_log = self.d_skip = None

    def weight_decls(self):
        p, I, N, R, W = self.prefix, self.inner, self.n, self.rank, self.hidden
        return ([WeightDecl(p + "in", (2 * I, W))] + self.conv.weight_decls()
                + [WeightDecl(p + "x", (R + 2 * N, I)), WeightDecl(p + "dt", (I, R)), WeightDecl(p + "dt.b", (I,)),
                   WeightDecl(p + "A_log", (I, N)), WeightDecl(p + "D", (I,), init="one_plus_normal"), WeightDecl(p + "o", (W, I))])

    def bind(self, tensors):
        p = self.prefix
        self.conv.bind({d.name: tensors[d.name] for d in self.conv.weight_decls()})
        self.w_in = Linear(tensors[p + "in"], self.ctx.dtype)
        self.w_x = Linear(tensors[p + "x"], self.ctx.dtype)
        self.w_dt = Linear(tensors[p + "dt"], self.ctx.dtype)
        self.o = Linear(tensors[p + "o"], self.ctx.dtype)
        self.dt_bias, self.a_log, self.d_skip = (tensors[p + n].float().contiguous() for n in ("dt.b", "A_log", "D"))

    def modules(self):
        return ["gated_scan", "recurrence"] + self.conv.modules() + self.w_in.modules() + self.w_x.modules() + self.w_dt.modules() + self.o.modules()

    def linears(self):
        return [self.w_in, self.w_x, self.w_dt, self.o]

    def cache_need(self):
        conv = self.conv.cache_need()
        scan = StateCacheNeed((self.inner * self.n,), "float32")
        return CompositeCacheNeed((scan, conv)) if conv is not None else scan

    def forward(self, x, batch, cache):
        T, I, N, R = x.shape[0], self.inner, self.n, self.rank
        scan_state, conv_state = (cache.parts[0], cache.parts[1]) if cache.kind == "composite" else (cache, None)
        xz = self.w_in(x, out_dtype=torch.float32)                                   # [x | z]
        xc = self.conv.forward(xz, batch, conv_state)                                # silu(conv(x) + b), the products' input type
        proj = self.w_x(xc, out_dtype=torch.float32)                                 # [dt | B | C]
        low = torch.empty((T, R), dtype=self.ctx.dtype, device=x.device)
        kernels.tanh_cols(proj, 0, R, low, activation="none")
        dt_pre = self.w_dt(low, out_dtype=torch.float32)
        y = torch.empty((T, I), dtype=self.ctx.dtype, device=x.device)
        kernels.selective_scan(xc, dt_pre, self.dt_bias, proj, R, R + N, xz, I, self.a_log, self.d_skip, scan_state.state, batch.q_start, batch.state_slot,
                               batch.num_seqs, y, longest=1 if batch.one_token_each else batch.num_tokens)
        return self.o(y, defer=self.defer_output, out_dtype=self.output_dtype)
