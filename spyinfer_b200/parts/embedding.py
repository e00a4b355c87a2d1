"""Token embedding and output head.

``token_embedding``: ``h[t] = E[ids[t]]`` into the 32-bit residual stream, no scaling
(spymaster2h/spyinfer src/models/qwen3.hpp:114-119); optionally times a ``scale``, and optionally plus
a row of a second table chosen by a hash of the pair (previous token, token), for which the part keeps
each request's last token as state.  ``lm_head``: ``logits = x @ W^T`` in
32-bit out, ``W`` the embedding table when tied (qwen3.hpp:46, 295-301).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.spec import StateCacheNeed
from ..weights.loader import WeightDecl
from .base import Part
from .linear import Linear
from .registry import register_part


@register_part("token_embedding")
class TokenEmbedding(Part):
    graph_safe = True
    """params: ``vocab_size``, ``hidden_size``, ``weight`` (full tensor name); optional ``scale`` (default 1) and
    ``pairs``: ``{"weight": name, "buckets": B, "mul_prev": a, "mul_cur": b}``: the row
    ``(previous * a + token * b) mod B`` of the table ``[B + 1, hidden]`` is added, its last row for a
    request's first token.  With ``pairs`` the part needs a state (``cache_need``): the request's last token."""

    kernel_modules = ("embedding",)

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.vocab, self.hidden, self.weight_name = int(params["vocab_size"]), int(params["hidden_size"]), params["weight"]
        self.scale = float(params.get("scale", 1.0))
        self.pairs = dict(params["pairs"]) if params.get("pairs") else None
        if self.pairs is not None and (int(self.pairs["buckets"]) <= 0 or int(self.pairs["mul_prev"]) < 0 or int(self.pairs["mul_cur"]) < 0):
            raise ValueError("token_embedding: the pair table needs a positive number of buckets and multipliers that are not negative")
        self.table = self.pair_table = None

    def weight_decls(self):
        decls = [WeightDecl(self.weight_name, (self.vocab, self.hidden))]
        if self.pairs is not None:
            decls.append(WeightDecl(self.pairs["weight"], (int(self.pairs["buckets"]) + 1, self.hidden)))
        return decls

    def bind(self, tensors):
        self.table = tensors[self.weight_name]
        if self.pairs is not None:
            self.pair_table = tensors[self.pairs["weight"]]

    def cache_need(self):
        return StateCacheNeed((1,), "int32") if self.pairs is not None else None

    def forward(self, token_ids, status=None, batch=None, cache=None):
        out = torch.empty((token_ids.shape[0], self.hidden), dtype=torch.float32, device=token_ids.device)
        if self.pairs is None:
            if self.scale == 1.0:
                return kernels.embedding(self.table, token_ids, out, status)
            return kernels.embedding_scaled(self.table, token_ids, out, self.scale, status)
        return kernels.embedding_scaled(self.table, token_ids, out, self.scale, status, pairs=self.pair_table, mul_prev=int(self.pairs["mul_prev"]),
                                        mul_cur=int(self.pairs["mul_cur"]), positions=batch.positions, seq_of_token=batch.seq_of_token,
                                        q_start=batch.q_start, state_slot=batch.state_slot, prev_state=cache.state)


@register_part("lm_head")
class LMHead(Part):
    graph_safe = True
    """params: ``vocab_size``, ``hidden_size``, ``tied``, ``weight`` (full name when untied),
    ``tied_to`` (full name of the embedding table when tied), ``scale`` (default 1: the logits' multiplier), ``softcap``
    (default 0: none; else ``logits = cap * tanh(logits / cap)``, after the scale)."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.vocab, self.hidden, self.tied = int(params["vocab_size"]), int(params["hidden_size"]), bool(params["tied"])
        self.weight_name = params["tied_to"] if self.tied else params["weight"]
        self.ignorable = [params["weight"]] if self.tied else []
        self.scale = float(params.get("scale", 1.0))
        self.softcap = float(params.get("softcap") or 0.0)
        if self.softcap < 0.0:
            raise ValueError(f"lm_head: the logits' cap {self.softcap} must not be negative")
        self.linear = None

    def weight_decls(self):
        return [] if self.tied else [WeightDecl(self.weight_name, (self.vocab, self.hidden))]

    def bind(self, tensors):
        self.linear = Linear(tensors[self.weight_name], self.ctx.dtype)

    def modules(self):
        return self.linear.modules() + (["swiglu"] if self.scale != 1.0 or self.softcap else [])

    def linears(self):
        return [self.linear]

    def forward(self, x):
        logits = self.linear(x, out_dtype=torch.float32)
        if self.scale != 1.0:
            kernels.scale_(logits, self.scale)
        return kernels.softcap_(logits, self.softcap) if self.softcap else logits
