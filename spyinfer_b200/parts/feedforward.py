"""Dense gated feed-forward: ``down(act(gate(x)) * up(x))``, no biases.

spymaster2h/spyinfer src/models/qwen3.hpp:233-263 with SiLU as the activation (SwiGLU:
src/backends/cpu/x64/kernels.cpp:242-247).  The gate and up projections are fused into one
matrix at load; on the bfloat16 path their rows are interleaved and the activation runs in
the product's epilogue, so the gate and up activations never reach memory.  The output may
come back as a stack of split-K partial products, which the next norm adds to the residual.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import WeightDecl
from .base import FeedForward
from .linear import Linear
from .registry import register_part


@register_part("mlp")
class MLP(FeedForward):
    """``down(act(up(x)))`` without a gate, no biases.  params: ``hidden_size``, ``intermediate_size``, ``activation``
    (``relu2``: the square of relu; ``gelu_tanh``; ``silu``; ``relu``), ``prefix``, ``names`` (the two tensors' names after the
    prefix: ``up``, ``down``)."""

    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        self.activation = params.get("activation", "relu2")
        if self.activation not in kernels._ACTIVATIONS:
            raise ValueError(f"mlp: activation {self.activation!r} is not implemented ({', '.join(kernels._ACTIVATIONS)})")
        self.prefix = params.get("prefix", "")
        self.names = {"up": "up_proj.weight", "down": "down_proj.weight"}
        self.names.update(params.get("names") or {})
        self.up = self.down = None

    def weight_decls(self):
        p, n = self.prefix, self.names
        return [WeightDecl(p + n["up"], (self.inter, self.hidden)), WeightDecl(p + n["down"], (self.hidden, self.inter))]

    def bind(self, tensors):
        p, n = self.prefix, self.names
        self.up = Linear(tensors[p + n["up"]], self.ctx.dtype)
        self.down = Linear(tensors[p + n["down"]], self.ctx.dtype)
        self.up.hint_next = False       # only the activation runs between the two products

    def linears(self):
        return [self.up, self.down]

    def _fused(self):
        # the tensor-core product applies the square of relu in its epilogue: the activation costs no launch and no pass over memory
        return self.activation == "relu2" and self.up is not None and self.up.fast and self.ctx.dtype == torch.bfloat16

    def modules(self):
        return ([] if self._fused() else ["swiglu"]) + self.up.modules() + self.down.modules()

    def forward(self, x):
        if self._fused():
            return self.down(self.up(x, epilogue="relu2"), defer=self.defer_output)
        a = self.up(x)
        kernels.activation(a, a, self.activation)
        return self.down(a, defer=self.defer_output)


@register_part("gated_mlp")
class GatedMLP(FeedForward):
    graph_safe = True
    """params: ``hidden_size``, ``intermediate_size``, ``activation`` (``silu``; ``gelu_tanh``: the tanh form of gelu; or
    ``clamped_swish``: ``g * sigmoid(slope g) * (u + 1)`` with ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``, which
    needs ``limit`` and takes ``slope``, default 1.702), ``bias`` (default false: the three projections have biases, named
    as the weights with ``.b`` behind), ``prefix``, ``names`` (the three tensors' names after the prefix: ``gate``, ``up``,
    ``down``; default ``gate_proj.weight`` and so on)."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        self.activation = params.get("activation", "silu")
        if self.activation not in kernels._GATED_ACTIVATIONS + ("clamped_swish",):
            raise ValueError(f"gated_mlp: activation {self.activation!r} is not implemented ({', '.join(kernels._GATED_ACTIVATIONS)}, clamped_swish)")
        self.limit, self.slope, self.has_bias = float(params.get("limit") or 0.0), float(params.get("slope", 1.702)), bool(params.get("bias", False))
        if self.activation == "clamped_swish" and not self.limit > 0.0:
            raise ValueError("gated_mlp: the clamped activation needs a positive limit")
        self.gate_up_bias = None
        self.prefix = params.get("prefix", "")
        self.names = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        self.names.update(params.get("names") or {})
        self.gate_up = self.down = None
        self.fused = False

    def weight_decls(self):
        p, n = self.prefix, self.names
        decls = [WeightDecl(p + n["gate"], (self.inter, self.hidden)),
                 WeightDecl(p + n["up"], (self.inter, self.hidden)),
                 WeightDecl(p + n["down"], (self.hidden, self.inter))]
        if self.has_bias:
            decls += [WeightDecl(p + n["gate"] + ".b", (self.inter,)), WeightDecl(p + n["up"] + ".b", (self.inter,)), WeightDecl(p + n["down"] + ".b", (self.hidden,))]
        return decls

    def bind(self, tensors):
        p, n = self.prefix, self.names
        gate, up = tensors[p + n["gate"]], tensors[p + n["up"]]
        if gate.dtype != up.dtype:
            gate, up = gate.float(), up.float()
        # silu and gelu_tanh without biases, and the clamped activation with or without them, run in the tensor-core product's epilogue
        self.fused = (self.ctx.dtype == torch.bfloat16 and gate.dtype == torch.bfloat16 and kernels.tensor_core_gemm_takes(2 * self.inter, self.hidden)
                      and (self.activation == "clamped_swish" or (self.activation in ("silu", "gelu_tanh") and not self.has_bias)))
        if self.fused:
            # rows alternate gate_i, up_i: the tensor-core product applies act(gate) * up in its epilogue
            self.gate_up = Linear(torch.stack([gate, up], dim=1).reshape(2 * self.inter, self.hidden).contiguous(), self.ctx.dtype)
        else:
            self.gate_up = Linear(torch.cat([gate, up], dim=0).contiguous(), self.ctx.dtype)
        if self.has_bias:
            # the gate and up biases are added where the activation is computed (32-bit; in the rows' order: alternating when the
            # product's epilogue does it), the down bias by a pass behind its product or by the consumer
            gb, ub = tensors[p + n["gate"] + ".b"].float(), tensors[p + n["up"] + ".b"].float()
            self.gate_up_bias = (torch.stack([gb, ub], dim=1).reshape(-1) if self.fused else torch.cat([gb, ub])).contiguous()
        down_bias = tensors[p + n["down"] + ".b"].float().contiguous() if self.has_bias else None
        if self.leave_output_bias:           # the consumer adds it (and may then take the down product's split-K parts unsummed)
            self.output_bias, down_bias = down_bias, None
        self.down = Linear(tensors[p + n["down"]], self.ctx.dtype, bias=down_bias)
        self.gate_up.hint_next = not self.fused       # fused: the down product follows at once

    def linears(self):
        return [self.gate_up, self.down]

    def modules(self):
        return ([] if self.fused else ["swiglu"]) + self.gate_up.modules() + self.down.modules()

    def forward(self, x):
        if self.fused and self.activation == "clamped_swish":
            return self.down(self.gate_up(x, epilogue="clamped_swish", glu=(self.gate_up_bias, self.limit, self.slope)), defer=self.defer_output)
        if self.fused:
            return self.down(self.gate_up(x, epilogue="swiglu" if self.activation == "silu" else "geglu_tanh"), defer=self.defer_output)
        z = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
        if self.activation == "clamped_swish":
            kernels.clamped_glu(self.gate_up(x), self.gate_up_bias, z, self.limit, self.slope)     # the biases are added and the clamps applied in 32-bit
            return self.down(z, defer=self.defer_output)
        gu = self.gate_up(x)
        if self.has_bias:
            kernels.add_bias(gu, self.gate_up_bias)
        if self.activation == "silu":
            kernels.swiglu(gu, z)
        else:
            kernels.gated_activation(gu, z, self.activation)
        return self.down(z, defer=self.defer_output)
