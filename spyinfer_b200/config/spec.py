"""The data that describes a model to the engine: parts, layers, and the order they run in.

A model is a list of layers; a layer is a block arrangement over named parts (for the usual
pre-norm block: a norm before the mixer, the mixer, a norm before the feed-forward, the
feed-forward; an arrangement may name others, or fewer); each part is a
``PartSpec``: the registry key of its kind plus its sizes and constants.  The order in
which layers run is a list of ``RunEntry`` and may name a layer twice, or let an entry
read the cache that an earlier entry wrote.  Nothing here knows a model by name: an
architecture's typed configuration produces a ``ModelSpec`` and the engine builds from it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: ``kind`` is a key of the part registry, ``params`` its sizes and constants."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)

    def __hash__(self):
        return hash((self.kind, repr(sorted(self.params.items(), key=lambda kv: kv[0]))))


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the arrangement (a key of the block registry), its parts by the role they play
    in it, and the prefix of its tensors' names in the checkpoint.

    The four roles of the usual block have fields of their own; an arrangement that needs other
    parts (norms after the mixer and the feed-forward, a second feed-forward, ...) names them in
    ``more``, and one that needs fewer leaves fields at None.  Which roles are required is the
    arrangement's statement (``Block.required`` / ``Block.optional``), checked when the layer is
    built.  The role ``mixer``, if present, is the part that owns the layer's cache."""

    block: str
    mixer_norm: Optional[PartSpec] = None
    mixer: Optional[PartSpec] = None
    ffn_norm: Optional[PartSpec] = None
    feed_forward: Optional[PartSpec] = None
    weight_prefix: str = ""
    more: Dict[str, PartSpec] = field(default_factory=dict)
    block_params: Dict[str, Any] = field(default_factory=dict)     # the arrangement's own constants

    def roles(self) -> Dict[str, PartSpec]:
        """role -> part, in the order the parts' tensors are declared."""
        out = {r: getattr(self, r) for r in ("mixer_norm", "mixer", "ffn_norm", "feed_forward") if getattr(self, r) is not None}
        for r, p in self.more.items():
            if r in out:
                raise ValueError(f"layer role {r!r} is given twice")
            out[r] = p
        return out

    def __hash__(self):
        return hash((self.block, self.weight_prefix, tuple(self.roles().items()), repr(sorted(self.block_params.items()))))


@dataclass(frozen=True)
class StreamAdd:
    """Something a model adds to its residual stream right before an entry of the run order runs: the embedding output
    of the step's tokens once more (``embedding``), and/or row ``row`` of the tensor ``tensor`` (``[rows, hidden]``, a
    learned offset for each pass of a repeated stretch of layers)."""

    embedding: bool = False
    tensor: Optional[str] = None
    rows: int = 0
    row: int = 0


@dataclass(frozen=True)
class RunEntry:
    """One position in the run order.

    ``layer`` indexes ``ModelSpec.layers``.  Every entry owns a cache of its own unless
    ``cache_of`` names an earlier entry (by its index in the run order): then this entry's
    mixer reads that entry's cache and stores nothing.  ``before`` is added to the residual
    stream ahead of the entry.
    """

    layer: int
    cache_of: Optional[int] = None
    before: Optional[StreamAdd] = None


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: List[LayerSpec]
    run_order: List[RunEntry]
    final_norm: PartSpec
    head: PartSpec
    max_position: int
    eos_token_id: int = -1
    bos_token_id: int = -1
    ignorable: List[str] = field(default_factory=list)     # tensors a checkpoint may hold without the model using them

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        for i, e in enumerate(self.run_order):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"run order entry {i} names layer {e.layer}, the model has {len(self.layers)}")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ValueError(f"run order entry {i} reads the cache of entry {e.cache_of}, which is not an earlier entry")
                if self.run_order[e.cache_of].cache_of is not None:
                    raise ValueError(f"run order entry {i} reads the cache of entry {e.cache_of}, which owns none")


@dataclass(frozen=True)
class PagedCacheNeed:
    """A mixer that keeps keys and values of past tokens in pages.

    ``window`` is ``None`` when every past key is kept, else the number of most recent
    positions (the query's own included) whose entries the mixer still reads; older pages are
    given back.  ``stride`` above 1: the mixer keeps one entry for every ``stride`` tokens (a
    summary of each block of that many tokens, stored when the block's last token is), so a
    request of ``L`` tokens holds ``L // stride`` entries; such a need has no window.  ``planes``
    is 2 for keys and values, 1 for a mixer whose values are its keys (or a part of them, as a
    latent that keys and values are both projected from): a page then holds keys only.
    ``keep_first`` (with a window): the entries of a sequence's first so many positions stay
    visible to every later query, so the pages that hold them are never given back.  Entries of
    the run order with equal needs share one group of pages in the cache manager.
    """

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    stride: int = 1
    planes: int = 2
    keep_first: int = 0

    def __post_init__(self):
        if self.planes not in (1, 2):
            raise ValueError(f"a paged need has 1 or 2 planes, found {self.planes}")
        if self.keep_first < 0:
            raise ValueError(f"a paged need keeps the first {self.keep_first} positions: not negative")
        if self.stride < 1 or (self.stride > 1 and self.window is not None):
            raise ValueError(f"a paged need's stride must be at least 1, and with a stride above 1 there is no window (found stride {self.stride}, window {self.window})")

    def group_key(self) -> Tuple:
        return ("paged", self.num_kv_heads, self.head_dim, self.window, self.stride, self.planes, self.keep_first if self.window is not None else 0)


@dataclass(frozen=True)
class StateCacheNeed:
    """A mixer that keeps a state of fixed size for each live request, in that request's slot."""

    shape: Tuple[int, ...]
    dtype: str = "float32"

    def group_key(self) -> Tuple:
        return ("state", tuple(self.shape), self.dtype)


@dataclass(frozen=True)
class SharedCacheNeed:
    """Inside the need of a run-order entry that names another entry in ``cache_of``: this part is that entry's paged
    cache (its only one), read and never written.  It lets an entry read another's keys and values and still keep
    things of its own beside them (the state of an input convolution, say)."""

    def group_key(self) -> Tuple:
        return ("shared",)


@dataclass(frozen=True)
class CompositeCacheNeed:
    """A mixer that keeps several things: each part is a ``PagedCacheNeed`` or a ``StateCacheNeed``
    (or None), and the mixer's ``CacheView`` holds one view for each in ``parts``, in this order."""

    parts: Tuple

    def flat(self):
        out = []
        for p in self.parts:
            out += p.flat() if isinstance(p, CompositeCacheNeed) else [p]
        return out
