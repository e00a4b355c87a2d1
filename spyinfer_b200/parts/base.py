"""Interfaces of the parts a model is put together from.

A part is built from its own sizes and constants (``params``) and a ``BuildContext``; it
declares the tensors it needs by names relative to its layer's prefix, gets them bound, and
then only computes.  No part knows which model it is in, which layer it is, or what other
parts the model has.

* ``Norm``: ``forward(x)`` and ``forward_add(residual, delta)`` (residual sum fused in).
* ``PositionEncoding``: owned by a mixer; hands out what the mixer's kernel needs.
* ``Mixer``: ``forward(x, batch, cache)``; declares what it keeps between steps through
  ``cache_need()`` (pages of keys and values, a fixed-size state per request, or nothing).
* ``FeedForward``: ``forward(x)``.
* ``Block``: the arrangement of a layer's parts around the residual stream (for the usual
  pre-norm block two norms, a mixer and a feed-forward; an arrangement states the roles it
  needs): ``forward(hidden, delta, batch, cache) -> (hidden, delta)``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from ..weights.loader import WeightDecl


@dataclass
class BuildContext:
    """What every part is built with.  ``dtype`` is the storage type of activations and of
    the cache: bfloat16 (the serving path) or float32 (everything in true 32-bit)."""

    dtype: torch.dtype
    device: torch.device
    max_model_len: int


@dataclass
class ScaledParts:
    """A result that is still a weighted sum, ``sum_i scale_i * term_i``: each term is ``[rows, size]`` or a stack
    ``[splits, rows, size]`` of float32 partial products.  A mixer made of several mixers side by side hands this on,
    and a norm that says ``takes_scaled_parts`` adds it to the residual in its own kernel."""

    terms: List[Tuple[torch.Tensor, float]]


@dataclass
class ChannelScaled:
    """A sublayer output that the stream takes multiplied element by element along the row: ``residual += y * weight``
    with ``weight [size]`` (a layer scale).  ``y`` is ``[rows, size]`` or a stack ``[splits, rows, size]`` of float32 partial
    products.  ``bias`` (optional, float32 ``[size]``): the bias of the projection that made ``y``, still to be added:
    ``residual += (y + bias) * weight``.  ``rows`` (optional, ``(x [rows, size] of the activations' type, w [rows] float32)``): one
    more term with a weight a row, ``residual += (y + bias + w[t] * x[t]) * weight``.  A norm that says ``takes_channel_scale`` forms
    the product in its own kernel."""

    y: torch.Tensor
    weight: torch.Tensor
    bias: Optional[torch.Tensor] = None
    rows: Optional[Tuple[torch.Tensor, torch.Tensor]] = None


@dataclass
class NormedDelta:
    """A sublayer output that is still to be normed, weighted and added: ``residual += scale * norm(y) * weight``, the norm
    being that of the part which made this record (and which the next norm of the same kind folds into its own launch).
    ``y`` is ``[rows, size]`` or a stack ``[splits, rows, size]`` of float32 partial products."""

    y: torch.Tensor
    weight: torch.Tensor
    scale: float = 1.0


class Part:
    kind: str = ""
    #: kernel modules (``csrc/<name>.cu``) this part launches; built before the first step
    kernel_modules: Sequence[str] = ()
    #: True when ``forward`` launches the same kernels with the same arguments for every batch of the same sizes
    #: (tokens, requests, wanted rows): no look at the batch's content on the host, no wait for the device, no
    #: allocation that outlives the call.  A model whose parts all say so has its small steps captured in CUDA
    #: graphs and replayed; one part that does not keeps the whole model on launches one by one.
    graph_safe: bool = False

    def __init__(self, params: Dict[str, Any], ctx: BuildContext):
        self.params = params
        self.ctx = ctx

    def weight_decls(self) -> List[WeightDecl]:
        """Tensors this part needs, named relative to its layer's prefix."""
        return []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receives the declared tensors (same relative names), already on the device."""

    def modules(self) -> List[str]:
        return list(self.kernel_modules)

    def linears(self) -> List:
        """The part's ``Linear`` products in the order ``forward`` runs them (the model tells each
        which weight is read next, so that it can ask for it ahead of time)."""
        return []


class Norm(Part):
    #: True: ``forward_add`` also takes a ``ScaledParts`` as ``delta`` and a ``scale`` other than 1
    takes_scaled_parts: bool = False
    #: True: ``forward_add`` also takes a ``ChannelScaled`` as ``delta``
    takes_channel_scale: bool = False

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        raise NotImplementedError

    def forward_add(self, residual: torch.Tensor, delta: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None,
                    out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """``residual += delta`` (32-bit, in place, skipped when ``delta`` is None), then the
        norm of the sum.  With ``rows`` only those rows are normed and nothing is written back.
        ``delta`` is ``[rows, size]``, or a stack ``[splits, rows, size]`` of float32 partial
        products (a mixer or feed-forward may hand its last product over unsummed); all are added.
        A norm that ``takes_scaled_parts`` has one more argument, ``scale`` (default 1): the residual
        takes ``scale * delta``, and ``delta`` may be a ``ScaledParts``."""
        raise NotImplementedError


class PositionEncoding(Part):
    #: which two elements of a head the table's angle ``j`` rotates: "half" ``(j, j + r)`` or
    #: "interleaved" ``(2j, 2j + 1)``
    pairing: str = "half"

    def rotation_table(self) -> Optional[torch.Tensor]:
        """For encodings that rotate pairs of each head's elements: float32 ``[positions, r, 2]``
        of (cos, sin) per position and pair, which the fused q/k kernel applies by the part's
        ``pairing`` rule; None for no rotation."""
        return None


class Mixer(Part):
    #: True: ``forward`` may hand its result over as a stack ``[splits, rows, size]`` of float32 partial
    #: products (its last product then skips its own reduction), which ``Norm.forward_add`` adds to the
    #: residual.  A block arrangement that does anything else with the result sets this to False on
    #: the part and always gets ``[rows, size]``.
    defer_output: bool = True
    #: None: the result has the activations' dtype; a mixer that is one of several side by side is asked for float32
    #: here, so that the norm which adds the weighted results reads them all in one format (parts that cannot do not)
    output_dtype: Optional[torch.dtype] = None

    def cache_need(self):
        """A ``PagedCacheNeed``, a ``StateCacheNeed``, a ``CompositeCacheNeed`` of them, or None."""
        return None

    def forward(self, x: torch.Tensor, batch, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    defer_output: bool = True     # as ``Mixer.defer_output``
    #: set by a block arrangement whose next norm adds a projection's bias itself: a feed-forward whose last projection has a
    #: bias then leaves it out and offers it as ``output_bias`` (float32 ``[size]``, None when there is none)
    leave_output_bias: bool = False
    output_bias: Optional[torch.Tensor] = None
    #: set with ``leave_output_bias``: a feed-forward whose result has a term ``w[t] * x[t]`` (a weight a row times its input) may
    #: leave that to the consumer as well and offers it, after every ``forward``, as ``output_rows = (x, w)`` (else None)
    output_rows: Optional[Tuple[torch.Tensor, torch.Tensor]] = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block:
    """An arrangement of a layer's parts.  ``required`` and ``optional`` name the roles it takes
    (``LayerSpec.roles()``); the parts arrive as ``self.parts[role]`` and as attributes of the
    same names (None for an optional role that the layer does not have)."""

    kind: str = ""
    graph_safe: bool = False      # as ``Part.graph_safe``, for the arrangement's own code
    required: Sequence[str] = ("mixer_norm", "mixer", "ffn_norm", "feed_forward")
    optional: Sequence[str] = ()

    #: what the residual stream takes of a part's output (``hidden += residual_scale * part(norm(hidden))``); the model
    #: hands the last block's to the final norm
    residual_scale: float = 1.0

    def __init__(self, parts: Dict[str, Part], params: Optional[Dict[str, Any]] = None):
        self.params = dict(params or {})
        missing = [r for r in self.required if r not in parts]
        unknown = [r for r in parts if r not in self.required and r not in self.optional]
        if missing or unknown:
            raise ValueError(f"block arrangement {self.kind!r} takes the roles {list(self.required)} (optional {list(self.optional)}): "
                             f"missing {missing}, unknown {unknown}")
        self.parts = dict(parts)
        for role in list(self.required) + list(self.optional):
            setattr(self, role, parts.get(role))

    def forward(self, hidden: torch.Tensor, delta: Optional[torch.Tensor], batch, cache):
        """``hidden`` is the 32-bit residual stream; ``delta`` the previous block's output
        that is still to be added to it (None for the first).  Returns the same pair."""
        raise NotImplementedError

    def cache_need(self):
        """What the layer keeps between steps: its mixer's need, unless the arrangement keeps something of its own beside
        it (it then returns a ``CompositeCacheNeed`` and hands the mixer its part of the view)."""
        mixer = self.parts.get("mixer")
        return mixer.cache_need() if mixer is not None else None

    def cache_need_reading(self):
        """The layer's need when its run-order entry reads another entry's cache (``RunEntry.cache_of``): None, the whole
        view is then the other entry's; or a need whose ``SharedCacheNeed`` part stands for the other entry's pages, for an
        arrangement that keeps state of its own beside them."""
        return None

    def settle(self, hidden: torch.Tensor, delta):
        """Adds what ``forward`` left pending to the stream (the model asks for this when something else is added to the
        stream between two blocks).  Returns the stream."""
        if delta is None:
            return hidden
        raise NotImplementedError(f"block arrangement {self.kind!r} cannot add its pending output to the stream on its own")
