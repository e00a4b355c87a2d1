"""Grouped-query softmax attention over the paged cache, with optional per-head q/k RMSNorm,
a position encoding of its own, and an optional window.

Order of operations (spymaster2h/spyinfer src/models/qwen3.hpp:136-213): q, k, v projections
(fused into one matrix here), RMSNorm over head_dim on q and k with one shared weight each,
position encoding on q and k, keys and values stored into the cache, attention, output
projection.  kv head = head * nkv / nh, score = q.k / sqrt(head_dim), causal on absolute
positions (src/backends/cpu/cpu_attention.cpp:59, :96, :100-110).  A windowed layer sees
the last ``window`` keys, the query's own included.
"""
from __future__ import annotations

import math

import torch

from .. import kernels
from ..config.spec import CompositeCacheNeed, PagedCacheNeed
from ..weights.loader import WeightDecl
from .base import Mixer
from .linear import Linear
from .registry import build_part, register_part


@register_part("attention")
class Attention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``qk_norm_eps``
    (None: no q/k norm), ``position`` (a PartSpec or None), ``window`` (None: all keys),
    ``chunk`` (None, or a size: a query sees the earlier keys of its own block of that many positions only, blocks counted
    from position 0 of the sequence; not together with a window), ``scale`` (None: 1/sqrt(head_dim)), ``prefix``,
    ``qkv_bias`` and ``o_bias`` (default false: the projections have bias tensors ``{q,k,v}_proj.bias`` / ``o_proj.bias``)."""

    graph_safe = True
    #: False: the head size must be a multiple of 4 (the kernel that rotates and stores q, k and v reads quads)
    any_head_dim = False

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(params["hidden_size"])
        self.nh, self.nkv, self.hd = int(params["num_heads"]), int(params["num_kv_heads"]), int(params["head_dim"])
        if self.nh % self.nkv:
            raise ValueError(f"attention: {self.nh} heads do not group over {self.nkv} key/value heads")
        if (self.hd % 4 and not self.any_head_dim) or self.hd > 1024:
            raise ValueError(f"attention: head_dim {self.hd} must be a multiple of 4 and at most 1024")
        self.qk_norm_eps = params.get("qk_norm_eps")
        self.window = params.get("window")
        if self.window is not None and int(self.window) <= 0:
            raise ValueError(f"attention: window {self.window} must be positive")
        self.chunk = params.get("chunk")
        if self.chunk is not None and (int(self.chunk) <= 0 or self.window is not None):
            raise ValueError(f"attention: chunk {self.chunk} must be positive, and a layer has a window or chunks, not both")
        self.scale = float(params["scale"]) if params.get("scale") is not None else 1.0 / math.sqrt(float(self.hd))
        self.prefix = params.get("prefix", "")
        self.qkv_bias, self.o_bias = bool(params.get("qkv_bias", False)), bool(params.get("o_bias", False))
        pos = params.get("position")
        self.position = build_part(pos, ctx) if pos is not None else None
        self.qkv = self.o = self.q_norm = self.k_norm = self.rope_table = None
        # which attention kernels take these sizes (the page size, known at the first step, decides between them)
        self.tc = kernels.attention_tc_takes(self.nh, self.nkv, self.hd, ctx.dtype)        # tcgen05, pages that are one TMA box
        self.mma = kernels.attention_mma_takes(self.nh, self.nkv, self.hd, ctx.dtype)      # mma.sync, any page size
        self._split_plans = {}

    def weight_decls(self):
        p, nh, nkv, hd, H = self.prefix, self.nh, self.nkv, self.hd, self.hidden
        decls = [WeightDecl(p + "q_proj.weight", (nh * hd, H)), WeightDecl(p + "k_proj.weight", (nkv * hd, H)),
                 WeightDecl(p + "v_proj.weight", (nkv * hd, H)), WeightDecl(p + "o_proj.weight", (H, nh * hd))]
        if self.qk_norm_eps is not None:
            decls += [WeightDecl(p + "q_norm.weight", (hd,), init="one_plus_normal"),
                      WeightDecl(p + "k_norm.weight", (hd,), init="one_plus_normal")]
        if self.qkv_bias:
            decls += [WeightDecl(p + "q_proj.bias", (nh * hd,)), WeightDecl(p + "k_proj.bias", (nkv * hd,)), WeightDecl(p + "v_proj.bias", (nkv * hd,))]
        if self.o_bias:
            decls += [WeightDecl(p + "o_proj.bias", (H,))]
        return decls

    def bind(self, tensors):
        p = self.prefix
        qkv = [tensors[p + n] for n in ("q_proj.weight", "k_proj.weight", "v_proj.weight")]
        if len({t.dtype for t in qkv}) > 1:
            qkv = [t.float() for t in qkv]
        bias = None
        if self.qkv_bias:
            bias = torch.cat([tensors[p + n].float() for n in ("q_proj.bias", "k_proj.bias", "v_proj.bias")]).contiguous()
        self.qkv = Linear(torch.cat(qkv, dim=0).contiguous(), self.ctx.dtype, bias=bias)
        self.o = Linear(tensors[p + "o_proj.weight"], self.ctx.dtype, bias=tensors[p + "o_proj.bias"] if self.o_bias else None)
        if self.qk_norm_eps is not None:
            self.q_norm, self.k_norm = tensors[p + "q_norm.weight"], tensors[p + "k_norm.weight"]
            if self.q_norm.dtype != self.k_norm.dtype:
                self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()

    def modules(self):
        mods = ["qk_rope_store"] + (["attention_tc", "attention_decode"] if self.tc else []) + (["attention_mma"] if self.mma else ["attention_generic"]) + self.qkv.modules() + self.o.modules()
        if self.position is not None:
            mods += self.position.modules()
        return mods

    def linears(self):
        return [self.qkv, self.o]

    def cache_need(self):
        return PagedCacheNeed(self.nkv, self.hd, int(self.window) if self.window is not None else None)

    @property
    def key_mask(self):
        """What the attention kernels take as ``window``: None (every earlier key), the window, or minus the chunk size."""
        return -int(self.chunk) if self.chunk is not None else self.window

    def split_plan(self, num_seqs: int):
        """(split_keys, max_splits) for decoding ``num_seqs`` requests: the keys of every request
        are cut into ranges so that (requests x key/value heads x ranges) blocks fill whole waves
        of the GPU's block slots (two a SM) as evenly as possible; at most 16 ranges, ranges of at
        least 256 keys and a multiple of 64.  The plan depends on the (padded) batch size only."""
        plan = self._split_plans.get(num_seqs)
        if plan is None:
            slots, per_split, best = 2 * torch.cuda.get_device_properties(self.ctx.device).multi_processor_count, num_seqs * self.nkv, None
            most = max(1, min(16, self.ctx.max_model_len // 256))
            for splits in range(1, most + 1):
                blocks = per_split * splits
                waves = -(-blocks // slots)
                fill = min(blocks, slots) / slots if waves == 1 else blocks / (waves * slots)
                keys = self.ctx.max_model_len / splits
                score = (fill * keys / (keys + 200.0), -splits)       # a block's fixed cost is worth about 200 keys
                if best is None or score > best[0]:
                    best = (score, splits)
            splits = best[1]
            split_keys = max(256, (-(-self.ctx.max_model_len // splits) + 63) // 64 * 64)
            plan = (split_keys, -(-self.ctx.max_model_len // split_keys))
            self._split_plans[num_seqs] = plan
        return plan

    def forward(self, x, batch, cache):
        if self.rope_table is None and self.position is not None:
            self.rope_table = self.position.rotation_table()   # built by the first step (an eager one)
        qkv = self.qkv(x, defer=True)
        q = None
        if qkv.dim() == 3:   # split-K partial products: summed inside the next kernel, q gets a buffer of its own
            q = torch.empty((x.shape[0], self.nh * self.hd), dtype=x.dtype, device=x.device)
        q = kernels.qk_rope_store(qkv, self.nh, self.nkv, self.hd, self.q_norm, self.k_norm, float(self.qk_norm_eps or 0.0),
                                  self.rope_table, batch.positions, batch.seq_of_token, cache.block_table, cache.pages,
                                  store=cache.writes, status=batch.status, q_out=q,
                                  pairing=self.position.pairing if self.position is not None else "half")
        out = torch.empty((x.shape[0], self.nh * self.hd), dtype=x.dtype, device=x.device)
        self.attend(q, out, batch, cache)
        return self.o(out, defer=self.defer_output)

    def attend(self, q, out, batch, cache):
        """The attention itself, ``q [T, >= nh hd]`` over the cache into ``out [T, nh hd]``, on the kernel that the sizes, the
        page size and the kind of batch call for."""
        x = q
        decoding = batch.one_token_each         # every request brings one token
        boxes = self.tc and cache.page_size in kernels.ATTENTION_TMA_PAGE_SIZES        # a page is one TMA box
        if (boxes and decoding and batch.num_seqs <= kernels.ATTENTION_DECODE_MAX_SEQS and batch.num_seqs * self.nkv <= kernels.ATTENTION_DECODE_MAX_PAIRS
                and kernels.attention_decode_takes(self.nh, self.nkv, self.hd, cache.page_size, x.dtype)):
            # memory-bound: one persistent block per SM, the batch's key tiles shared out evenly, pages by TMA
            kernels.attention_decode(q, self.nh, self.hd, out, cache.pages, cache.block_table, batch.positions, batch.q_start,
                                     batch.num_seqs, self.scale, window=self.key_mask, status=batch.status)
        elif decoding and self.mma:
            # page sizes that are no TMA box, or very many requests: keys split across blocks by a plan per batch size
            split_keys, max_splits = self.split_plan(batch.num_seqs)
            kernels.attention_mma(q, self.nh, self.hd, out, cache.pages, cache.block_table, batch.positions, batch.q_start,
                                  batch.num_seqs, self.scale, window=self.key_mask, split_keys=split_keys, max_splits=max_splits,
                                  status=batch.status)
        elif boxes:
            # prompt portions on blocks of 256 query rows; requests that decode beside them (laid out first in the batch)
            # go through the decode kernel, which reads a cache two to three times faster for one token than a 256-row block does
            head = batch.one_token_head      # the step function says whether a launch of the decode kernel pays for them
            if not (0 < head <= kernels.ATTENTION_DECODE_MAX_SEQS and head * self.nkv <= kernels.ATTENTION_DECODE_MAX_PAIRS
                    and kernels.attention_decode_takes(self.nh, self.nkv, self.hd, cache.page_size, x.dtype)):
                head = 0
            if head:
                kernels.attention_decode(q, self.nh, self.hd, out, cache.pages, cache.block_table[:head], batch.positions, batch.q_start[:head + 1],
                                         head, self.scale, window=self.key_mask, status=batch.status)
            kernels.attention_tc(q, self.nh, self.hd, out, cache.pages, cache.block_table[head:], batch.positions, batch.q_start[head:],
                                 batch.num_seqs - head, self.scale, window=self.key_mask, status=batch.status)
        elif self.mma:
            kernels.attention_mma(q, self.nh, self.hd, out, cache.pages, cache.block_table, batch.positions, batch.q_start,
                                  batch.num_seqs, self.scale, window=self.key_mask, status=batch.status)
        else:
            # the float32 path, head sizes above 128 or no multiple of 8, more than 16 query heads a key/value head
            kernels.attention_generic(q, self.nh, self.hd, out, cache.pages, cache.block_table, batch.positions, batch.seq_of_token,
                                      self.scale, window=self.key_mask, status=batch.status)
        return out


@register_part("pooled_window_attention")
class PooledWindowAttention(Attention):
    """Grouped-query attention over a window of the last ``window`` keys plus one pooled key and value for every block
    of ``pool`` tokens that lies wholly before the window (the means of the block's keys and values as the cache holds
    them), all under one softmax.  A token that has left the window while its block is not yet wholly before it is
    seen by no query.

    params, beside those of ``attention`` that it shares (``hidden_size``, ``num_heads``, ``num_kv_heads``,
    ``head_dim``, ``position``, ``scale``, ``prefix``): ``window``, ``pool`` (0 or None: no pooled entries),
    ``values_are_keys`` (true: there is no value projection, a token's value is its key as projected, before the
    position encoding) and ``names`` (the projections' tensor names: ``q``, ``k``, ``v``, ``o``).

    The pooled entries live in a paged cache of their own with one entry for every ``pool`` tokens; an entry is made,
    from the token cache, in the step that stores its block's last token, which is why the token cache keeps
    ``max(window, pool)`` positions."""

    graph_safe = True

    def __init__(self, params, ctx):
        base = dict(params)
        base.setdefault("qk_norm_eps", None)
        super().__init__(base, ctx)
        if self.window is None:
            raise ValueError("pooled_window_attention: a window is required")
        self.window = int(self.window)
        self.pool = int(params.get("pool") or 0)
        if self.pool < 0:
            raise ValueError(f"pooled_window_attention: pool {self.pool} must not be negative")
        self.values_are_keys = bool(params.get("values_are_keys", False))
        names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight"}
        names.update(params.get("names") or {})
        self.names = names

    def weight_decls(self):
        p, nh, nkv, hd, H, n = self.prefix, self.nh, self.nkv, self.hd, self.hidden, self.names
        decls = [WeightDecl(p + n["q"], (nh * hd, H)), WeightDecl(p + n["k"], (nkv * hd, H))]
        if not self.values_are_keys:
            decls.append(WeightDecl(p + n["v"], (nkv * hd, H)))
        return decls + [WeightDecl(p + n["o"], (H, nh * hd))]

    def bind(self, tensors):
        p, n = self.prefix, self.names
        q, k = tensors[p + n["q"]], tensors[p + n["k"]]
        v = k if self.values_are_keys else tensors[p + n["v"]]     # the key projection's rows once more: the value IS the key before rotation
        qkv = [q, k, v]
        if len({t.dtype for t in qkv}) > 1:
            qkv = [t.float() for t in qkv]
        self.qkv = Linear(torch.cat(qkv, dim=0).contiguous(), self.ctx.dtype)
        self.o = Linear(tensors[p + n["o"]], self.ctx.dtype)

    def modules(self):
        mods = ["qk_rope_store", "attention_pool"] + (["attention_tc", "attention_decode"] if self.tc else []) + self.qkv.modules() + self.o.modules()
        if self.position is not None:
            mods += self.position.modules()
        return mods

    def cache_need(self):
        if not self.pool:
            return PagedCacheNeed(self.nkv, self.hd, self.window)
        return CompositeCacheNeed((PagedCacheNeed(self.nkv, self.hd, max(self.window, self.pool)),
                                   PagedCacheNeed(self.nkv, self.hd, None, stride=self.pool)))

    def forward(self, x, batch, cache):
        if self.rope_table is None and self.position is not None:
            self.rope_table = self.position.rotation_table()
        tokens, pooled = (cache.parts[0], cache.parts[1]) if self.pool else (cache, None)
        qkv = self.qkv(x, defer=True)
        q = None
        if qkv.dim() == 3:
            q = torch.empty((x.shape[0], self.nh * self.hd), dtype=x.dtype, device=x.device)
        q = kernels.qk_rope_store(qkv, self.nh, self.nkv, self.hd, None, None, 0.0, self.rope_table, batch.positions, batch.seq_of_token,
                                  tokens.block_table, tokens.pages, store=tokens.writes, status=batch.status, q_out=q,
                                  pairing=self.position.pairing if self.position is not None else "half")
        if self.pool and pooled.writes:
            kernels.pool_store(tokens.pages, tokens.block_table, pooled.pages, pooled.block_table, self.pool, batch.positions, batch.seq_of_token,
                               status=batch.status)
        out = torch.empty((x.shape[0], self.nh * self.hd), dtype=x.dtype, device=x.device)
        lse = None
        if self.tc and tokens.page_size in kernels.ATTENTION_TMA_PAGE_SIZES:
            # The window's keys on the tensor cores, by the kernels that attention over a plain window uses (the persistent
            # decode kernel for requests that bring one token, the kernel for portions for the rest), which also leave each
            # row's logarithm of its sum of exponentials; the pooled entries are then merged into that softmax.
            decode_ok = kernels.attention_decode_takes(self.nh, self.nkv, self.hd, tokens.page_size, x.dtype)
            fits = lambda n: 0 < n <= kernels.ATTENTION_DECODE_MAX_SEQS and n * self.nkv <= kernels.ATTENTION_DECODE_MAX_PAIRS
            head = batch.num_seqs if batch.one_token_each else batch.one_token_head
            if not (decode_ok and fits(head)):
                head = 0
            if head or not batch.one_token_each:
                lse = torch.empty((x.shape[0], self.nh), dtype=torch.float32, device=x.device) if self.pool else None
                if head:
                    kernels.attention_decode(q, self.nh, self.hd, out, tokens.pages, tokens.block_table[:head], batch.positions, batch.q_start[:head + 1],
                                             head, self.scale, window=self.window, status=batch.status, lse=lse)
                if head < batch.num_seqs:
                    kernels.attention_tc(q, self.nh, self.hd, out, tokens.pages, tokens.block_table[head:], batch.positions, batch.q_start[head:],
                                         batch.num_seqs - head, self.scale, window=self.window, status=batch.status, lse=lse)
                if not self.pool:
                    return self.o(out, defer=self.defer_output, out_dtype=self.output_dtype)
        # decoding batches, the float32 path and sizes the tensor-core kernel does not take: one plain kernel for both parts
        kernels.attention_pool(q, self.nh, self.hd, out, tokens.pages, tokens.block_table, pooled.pages if self.pool else None,
                               pooled.block_table if self.pool else None, batch.positions, batch.seq_of_token, self.scale, self.window, self.pool,
                               status=batch.status, lse=lse)
        return self.o(out, defer=self.defer_output, out_dtype=self.output_dtype)


@register_part("latent_attention")
class LatentAttention(Attention):
    """Softmax attention whose keys and values are per-head projections of one small latent per token, which is all the
    cache keeps beside one rotated key part that the heads share; the queries go through a latent of their own.

    With ``h`` the input: ``c_q = rms_norm(W_dq h)``, ``q = W_uq c_q`` laid out head by head as ``[dim | rot_dim]``;
    ``W_dkv h = [kv_rank | rot_dim]``, ``c = rms_norm`` of the first part, ``k_r`` the rotated second part; per head
    ``score = (q_n . U_k c + rot(q_r) . k_r) * scale``, ``o = U_v (sum p c)``; optionally ``o * sigmoid(W_g h)``; then ``W_o``.
    It is computed in the absorbed form, ``(U_k^T q_n) . c``, so the attention runs over one key/value head of size
    ``kv_rank + rot_dim`` on a cache of one plane (the value is the key row's first ``kv_rank`` elements) with the kernels
    of ``attention``; see ``csrc/latent.cu``.

    params: ``hidden_size``, ``num_heads``, ``head_dim`` (the unrotated part), ``rot_dim``, ``v_head_dim``, ``q_rank``,
    ``kv_rank``, ``eps`` (of the two latent norms), ``scale``, ``window`` (None: every earlier key), ``position`` (a rotary
    part whose ``rotary_dim`` is at most ``rot_dim``, or None), ``gate`` (default false), ``shares_cache`` (true: the layer
    has no ``W_dkv`` and reads the cache of the run-order entry that its ``RunEntry.cache_of`` names), ``prefix``.  Tensors:
    ``dq``, ``dq.norm``, ``uq``, ``dkv``, ``dkv.norm``, ``uk``, ``uv``, ``g``, ``o``."""

    graph_safe = True
    any_head_dim = True

    def __init__(self, params, ctx):
        self.d, self.rd, self.vd = int(params["head_dim"]), int(params["rot_dim"]), int(params["v_head_dim"])
        self.q_rank, self.kv_rank = int(params["q_rank"]), int(params["kv_rank"])
        if min(self.d, self.vd, self.q_rank, self.kv_rank) <= 0 or self.rd < 0:
            raise ValueError("latent_attention: sizes must be positive")
        base = dict(params)
        base.update(num_kv_heads=1, head_dim=self.kv_rank + self.rd, qk_norm_eps=None)
        if base.get("scale") is None:
            base["scale"] = 1.0 / math.sqrt(float(self.d + self.rd))
        if (self.kv_rank + self.rd) > 1024:
            raise ValueError(f"latent_attention: a latent of {self.kv_rank} with a rotated part of {self.rd} exceeds the attention kernels' 1024")
        super().__init__(base, ctx)
        self.mma = False                        # that kernel reads keys and values from two planes
        self.eps = float(params["eps"])
        self.gated, self.shares_cache = bool(params.get("gate", False)), bool(params.get("shares_cache", False))
        if self.position is not None and 2 * (self.position.rotary_dim // 2) > self.rd:
            raise ValueError(f"latent_attention: a rotation of {self.position.rotary_dim} elements exceeds the rotated part of {self.rd}")
        self.width = self.kv_rank + self.rd      # a cache row, and a head of the absorbed query
        self.c_offset = self.q_rank
        self.gate_offset = self.q_rank + (0 if self.shares_cache else self.width)
        self.fused = self.uq = self.uk = self.uv = self.q_norm_w = self.c_norm_w = None

    def weight_decls(self):
        p, H, W = self.prefix, self.nh, self.hidden
        decls = [WeightDecl(p + "dq", (self.q_rank, W)), WeightDecl(p + "dq.norm", (self.q_rank,), init="one_plus_normal"),
                 WeightDecl(p + "uq", (H * (self.d + self.rd), self.q_rank))]
        if not self.shares_cache:
            decls += [WeightDecl(p + "dkv", (self.width, W)), WeightDecl(p + "dkv.norm", (self.kv_rank,), init="one_plus_normal")]
        decls += [WeightDecl(p + "uk", (H * self.d, self.kv_rank)), WeightDecl(p + "uv", (H * self.vd, self.kv_rank))]
        if self.gated:
            decls.append(WeightDecl(p + "g", (H * self.vd, W)))
        return decls + [WeightDecl(p + "o", (W, H * self.vd))]

    def bind(self, tensors):
        p, H = self.prefix, self.nh
        rows = [tensors[p + "dq"]] + ([] if self.shares_cache else [tensors[p + "dkv"]]) + ([tensors[p + "g"]] if self.gated else [])
        if len({t.dtype for t in rows}) > 1:
            rows = [t.float() for t in rows]
        self.fused = Linear(torch.cat(rows, dim=0).contiguous(), self.ctx.dtype)
        self.uq = Linear(tensors[p + "uq"], self.ctx.dtype)
        self.o = Linear(tensors[p + "o"], self.ctx.dtype)
        self.uk = tensors[p + "uk"].reshape(H, self.d, self.kv_rank).contiguous()                      # [head][unrotated element][latent]: as stored
        self.uv = tensors[p + "uv"].reshape(H, self.vd, self.kv_rank).transpose(1, 2).contiguous()     # [head][latent][value element]
        self.q_norm_w = tensors[p + "dq.norm"].float().contiguous()
        if not self.shares_cache:
            self.c_norm_w = tensors[p + "dkv.norm"].float().contiguous()

    def modules(self):
        mods = ["latent"] + (["attention_tc", "attention_decode"] if self.tc else []) + ["attention_generic"] + self.fused.modules() + self.uq.modules() + self.o.modules()
        if self.position is not None:
            mods += self.position.modules()
        return mods

    def linears(self):
        return [self.fused, self.uq, self.o]

    def cache_need(self):
        return PagedCacheNeed(1, self.width, int(self.window) if self.window is not None else None, planes=1)

    def forward(self, x, batch, cache):
        if self.rope_table is None and self.position is not None:
            self.rope_table = self.position.rotation_table()
        if cache.writes == self.shares_cache:
            raise ValueError("latent_attention: a layer with a key/value projection of its own owns its cache, one without reads another layer's")
        T, H = x.shape[0], self.nh
        interleaved = self.position is not None and self.position.pairing == "interleaved"
        fused = self.fused(x, out_dtype=torch.float32)
        cq = torch.empty((T, self.q_rank), dtype=x.dtype, device=x.device)
        kernels.latent_prep(fused, 0, self.q_rank, self.q_norm_w, cq, self.c_offset if cache.writes else -1, self.kv_rank, self.c_norm_w, self.rd,
                            self.rope_table, interleaved, batch.positions, batch.seq_of_token, cache.block_table, cache.pages, self.eps, status=batch.status)
        q = self.uq(cq)
        q_abs = torch.empty((T, H * self.width), dtype=x.dtype, device=x.device)
        kernels.head_product(q, self.d + self.rd, self.uk, q_abs, self.width, tail=self.rd, rope_table=self.rope_table, interleaved=interleaved,
                             positions=batch.positions, status=batch.status)
        mixed = torch.empty((T, H * self.width), dtype=x.dtype, device=x.device)      # per head: [sum p c | sum p k_r]; the second part is not used
        self.attend(q_abs, mixed, batch, cache)
        o = torch.empty((T, H * self.vd), dtype=x.dtype, device=x.device)
        kernels.head_product(mixed, self.width, self.uv, o, self.vd, gate=fused if self.gated else None, gate_offset=self.gate_offset)
        return self.o(o, defer=self.defer_output)


@register_part("differential_attention")
class DifferentialAttention(Attention):
    """Softmax attention with two score maps a head over the same values, the second map's result subtracted from the
    first's: with ``a1``, ``a2`` the two maps' results, ``o = a1 - lambda * a2``, brought to unit root mean square over the
    head's values (no weight) and multiplied by ``1 - diff``; ``lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff`` is one
    number for the layer.  Queries and keys are laid out head by head as ``[map 1 | map 2]``; each map of each head gets an
    RMS norm over ``dim`` with a weight shared by all heads and maps, then the rotation.  The concatenated heads are
    multiplied by ``sigmoid(W_g h)`` ahead of the output projection.  q, k, v and o have biases.

    The two maps run as two query heads of the ordinary attention kernels over one key/value head whose key row is
    ``[key of map 1 | key of map 2]`` and whose query has zeros in the other map's columns (``csrc/diff_attention.cu``): the
    kernels see ``2 heads`` query heads over ``kv_heads`` key/value heads of rows ``max(2 dim, vdim)`` wide, rounded up to 8.

    params: ``hidden_size``, ``heads``, ``kv_heads``, ``dim`` (a map's query/key size), ``vdim``, ``diff``, ``scale``
    (None: ``dim^(-1/2)``), ``eps`` (of the norms), ``window`` or ``chunk`` (as ``attention``), ``position`` (a rotary part
    with the interleaved pairing, or None), ``prefix``.  Tensors: ``q [2 heads dim, hidden]``, ``k [2 kv_heads dim, hidden]``,
    ``v [kv_heads vdim, hidden]`` with biases ``q.b, k.b, v.b``, ``q.norm, k.norm, lq1, lk1, lq2, lk2 [dim]``,
    ``g [heads vdim, hidden]``, ``o [hidden, heads vdim]``, ``o.b``."""

    graph_safe = True
    any_head_dim = True

    def __init__(self, params, ctx):
        self.heads, self.groups = int(params["heads"]), int(params["kv_heads"])
        self.d, self.vd, self.diff, self.eps = int(params["dim"]), int(params["vdim"]), float(params["diff"]), float(params["eps"])
        if min(self.heads, self.groups, self.d, self.vd) <= 0:
            raise ValueError("differential_attention: sizes must be positive")
        row = (max(2 * self.d, self.vd) + 7) // 8 * 8
        base = dict(params)
        base.update(num_heads=2 * self.heads, num_kv_heads=self.groups, head_dim=row, qk_norm_eps=None)
        if base.get("scale") is None:
            base["scale"] = 1.0 / math.sqrt(float(self.d))
        super().__init__(base, ctx)
        if self.position is not None and (self.position.pairing != "interleaved" or self.position.rotary_dim > self.d):
            raise ValueError("differential_attention: the rotation pairs neighbouring elements and fits within a map")
        n_q, n_k, n_v = 2 * self.heads * self.d, 2 * self.groups * self.d, self.groups * self.vd
        self.cols = (0, n_q, n_q + n_k, n_q + n_k + n_v)          # q, k, v, gate in the fused projection
        self.fused = self.o = self.bias = self.q_norm_w = self.k_norm_w = None
        self.lam = 0.0

    def weight_decls(self):
        p, H, G, d, vd, W = self.prefix, self.heads, self.groups, self.d, self.vd, self.hidden
        return ([WeightDecl(p + "q", (2 * H * d, W)), WeightDecl(p + "q.b", (2 * H * d,)), WeightDecl(p + "k", (2 * G * d, W)),
                 WeightDecl(p + "k.b", (2 * G * d,)), WeightDecl(p + "v", (G * vd, W)), WeightDecl(p + "v.b", (G * vd,)),
                 WeightDecl(p + "q.norm", (d,), init="one_plus_normal"), WeightDecl(p + "k.norm", (d,), init="one_plus_normal")]
                + [WeightDecl(p + n, (d,)) for n in ("lq1", "lk1", "lq2", "lk2")]
                + [WeightDecl(p + "g", (H * vd, W)), WeightDecl(p + "o", (W, H * vd)), WeightDecl(p + "o.b", (W,))])

    def bind(self, tensors):
        p = self.prefix
        rows = [tensors[p + n] for n in ("q", "k", "v", "g")]
        if len({t.dtype for t in rows}) > 1:
            rows = [t.float() for t in rows]
        self.fused = Linear(torch.cat(rows, dim=0).contiguous(), self.ctx.dtype)
        self.bias = torch.cat([tensors[p + n].float() for n in ("q.b", "k.b", "v.b")]
                              + [torch.zeros(self.heads * self.vd, dtype=torch.float32, device=rows[0].device)]).contiguous()
        self.o = Linear(tensors[p + "o"], self.ctx.dtype, bias=tensors[p + "o.b"])
        self.q_norm_w, self.k_norm_w = tensors[p + "q.norm"].float().contiguous(), tensors[p + "k.norm"].float().contiguous()
        l = [tensors[p + n].double() for n in ("lq1", "lk1", "lq2", "lk2")]
        self.lam = float(torch.exp((l[0] * l[1]).sum()) - torch.exp((l[2] * l[3]).sum())) + self.diff

    def modules(self):
        mods = (["diff_attention"] + (["attention_tc", "attention_decode"] if self.tc else []) + (["attention_mma"] if self.mma else ["attention_generic"])
                + self.fused.modules() + self.o.modules())
        if self.position is not None:
            mods += self.position.modules()
        return mods

    def linears(self):
        return [self.fused, self.o]

    def cache_need(self):
        return PagedCacheNeed(self.groups, self.hd, int(self.window) if self.window is not None else None)

    def forward(self, x, batch, cache):
        if self.rope_table is None and self.position is not None:
            self.rope_table = self.position.rotation_table()
        T = x.shape[0]
        proj = self.fused(x, out_dtype=torch.float32)
        q = torch.empty((T, self.nh * self.hd), dtype=x.dtype, device=x.device)
        kernels.diff_qkv_store(proj, self.cols[0], self.cols[1], self.cols[2], self.bias, self.q_norm_w, self.k_norm_w, self.eps, self.rope_table,
                               batch.positions, batch.seq_of_token, q, cache.block_table, cache.pages, self.heads, self.groups, self.d, self.vd,
                               status=batch.status)
        maps = torch.empty((T, self.nh * self.hd), dtype=x.dtype, device=x.device)
        self.attend(q, maps, batch, cache)
        o = torch.empty((T, self.heads * self.vd), dtype=x.dtype, device=x.device)
        kernels.diff_combine(maps, self.hd, proj, self.cols[3], o, self.heads, self.vd, self.lam, 1.0 - self.diff, self.eps)
        return self.o(o, defer=self.defer_output, out_dtype=self.output_dtype)


@register_part("sink_window_attention")
class SinkWindowAttention(Attention):
    """Grouped-query attention over a sliding window that also keeps a sequence's first tokens in view, under a softmax with
    a sink: a query at position ``i`` sees ``j <= i`` with ``i - j < window`` or ``j < keep_first`` (kept keys stay at their
    true positions), and ``p_j = exp(s_j) / (1 + sum exp(s_j))`` when ``sink`` is set (a key of score 0 that has no value).
    Queries and keys are normed over the WHOLE projection (one root mean square for all of a token's query heads together,
    a weight of that size; the same for its keys), then rotated; ``s = q . k * scale * temp[head]`` with a learned number a
    head; every value head is brought to unit root mean square over ``vdim`` (no weight) and cached so.

    A layer that ``shares_cache`` has no key or value tensors: its run-order entry names the entry whose keys and values it
    reads (``RunEntry.cache_of``), with queries, mask, temperatures and output projection of its own; ``cache_window`` /
    ``cache_keep_first`` then tell the owning layer what its readers need kept (the widest window, the most kept tokens).

    The attention kernels see rows of ``max(dim, vdim)`` rounded up to 8 (zeros behind a row's content).  On the bfloat16
    path the window's keys run on the tensor-core kernels of ``attention``, which leave each row's logarithm of its sum of
    exponentials, and ``sink_merge`` adds the kept first keys and the sink; the plain kernel does all of it in one pass.

    params: ``hidden_size``, ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``eps``, ``scale`` (None: ``dim^(-1/2)``), ``window``
    (None: every earlier key), ``keep_first`` (default 0), ``sink`` (default true), ``temperature`` (default true),
    ``shares_cache``, ``cache_window``, ``cache_keep_first``, ``position`` (a rotary part with the interleaved pairing, or None),
    ``prefix``.  Tensors: ``q [heads dim, hidden]``, ``k [kv_heads dim, hidden]``, ``v [kv_heads vdim, hidden]``, ``q.norm [heads
    dim]``, ``k.norm [kv_heads dim]``, ``temp [heads]``, ``o [hidden, heads vdim]``."""

    graph_safe = True
    any_head_dim = True

    def __init__(self, params, ctx):
        self.heads, self.groups = int(params["heads"]), int(params["kv_heads"])
        self.d, self.vd, self.eps = int(params["dim"]), int(params["vdim"]), float(params["eps"])
        if min(self.heads, self.groups, self.d, self.vd) <= 0:
            raise ValueError("sink_window_attention: sizes must be positive")
        row = (max(self.d, self.vd) + 7) // 8 * 8
        base = dict(params)
        base.update(num_heads=self.heads, num_kv_heads=self.groups, head_dim=row, qk_norm_eps=None, chunk=None)
        if base.get("scale") is None:
            base["scale"] = 1.0 / math.sqrt(float(self.d))
        super().__init__(base, ctx)
        self.mma = False                 # the plain kernel is the one that knows the kept keys and the sink
        self.keep_first = int(params.get("keep_first") or 0)
        if self.keep_first < 0 or (self.keep_first and self.window is None):
            self.keep_first = max(self.keep_first, 0) if self.window is not None else 0     # without a window every key is seen anyway
        self.sink, self.temperature = bool(params.get("sink", True)), bool(params.get("temperature", True))
        self.shares_cache = bool(params.get("shares_cache", False))
        self.cache_window = params.get("cache_window", self.window)
        self.cache_keep_first = int(params.get("cache_keep_first", self.keep_first) or 0)
        if self.position is not None and (self.position.pairing != "interleaved" or self.position.rotary_dim > self.d):
            raise ValueError("sink_window_attention: the rotation pairs neighbouring elements and fits within a head")
        self.n_q, self.n_k, self.n_v = self.heads * self.d, self.groups * self.d, self.groups * self.vd
        self.q_norm_w = self.k_norm_w = self.temp = None

    def weight_decls(self):
        p, W = self.prefix, self.hidden
        decls = [WeightDecl(p + "q", (self.n_q, W)), WeightDecl(p + "q.norm", (self.n_q,), init="one_plus_normal")]
        if not self.shares_cache:
            decls += [WeightDecl(p + "k", (self.n_k, W)), WeightDecl(p + "v", (self.n_v, W)), WeightDecl(p + "k.norm", (self.n_k,), init="one_plus_normal")]
        if self.temperature:
            decls.append(WeightDecl(p + "temp", (self.heads,), init="one_plus_normal"))
        return decls + [WeightDecl(p + "o", (W, self.heads * self.vd))]

    def bind(self, tensors):
        p = self.prefix
        rows = [tensors[p + "q"]] + ([] if self.shares_cache else [tensors[p + "k"], tensors[p + "v"]])
        if len({t.dtype for t in rows}) > 1:
            rows = [t.float() for t in rows]
        self.qkv = Linear(torch.cat(rows, dim=0).contiguous() if len(rows) > 1 else rows[0], self.ctx.dtype)
        o = tensors[p + "o"]
        if self.hd != self.vd:           # the attention's rows are wider than a value: the matching columns of the output projection are zero
            o = torch.nn.functional.pad(o.reshape(self.hidden, self.heads, self.vd), (0, self.hd - self.vd)).reshape(self.hidden, self.heads * self.hd).contiguous()
        self.o = Linear(o, self.ctx.dtype)
        names = ["q.norm"] + ([] if self.shares_cache else ["k.norm"]) + (["temp"] if self.temperature else [])
        small = {n: tensors[p + n] for n in names}
        if len({t.dtype for t in small.values()}) > 1:
            small = {n: t.float() for n, t in small.items()}
        self.q_norm_w, self.k_norm_w, self.temp = small["q.norm"].contiguous(), small.get("k.norm"), small.get("temp")

    def modules(self):
        mods = ["sink_attention", "attention_generic"] + (["attention_tc", "attention_decode"] if self.tc else []) + self.qkv.modules() + self.o.modules()
        if self.position is not None:
            mods += self.position.modules()
        return mods

    def linears(self):
        return [self.qkv, self.o]

    def cache_need(self):
        if self.shares_cache:
            return None
        window = int(self.cache_window) if self.cache_window is not None else None
        return PagedCacheNeed(self.groups, self.hd, window, keep_first=self.cache_keep_first if window is not None else 0)

    def forward(self, x, batch, cache):
        if self.rope_table is None and self.position is not None:
            self.rope_table = self.position.rotation_table()
        if cache.writes == self.shares_cache:
            raise ValueError("sink_window_attention: a layer with key and value projections owns its cache, one without reads another layer's")
        T = x.shape[0]
        proj = self.qkv(x, out_dtype=torch.float32)          # the norms over the whole projection read it unrounded
        q = torch.empty((T, self.nh * self.hd), dtype=x.dtype, device=x.device)
        kernels.sink_qkv_store(proj, 0, self.n_q, self.n_q + self.n_k, self.q_norm_w, self.k_norm_w, self.temp, self.eps, self.rope_table,
                               batch.positions, batch.seq_of_token, q, cache.block_table if cache.writes else None, cache.pages if cache.writes else None,
                               self.heads, self.groups, self.d, self.vd, self.hd, status=batch.status)
        out = torch.empty((T, self.nh * self.hd), dtype=x.dtype, device=x.device)
        self.attend(q, out, batch, cache)
        return self.o(out, defer=self.defer_output, out_dtype=self.output_dtype)

    def attend(self, q, out, batch, cache):
        if not (self.tc and cache.page_size in kernels.ATTENTION_TMA_PAGE_SIZES):
            # the float32 path, and sizes or pages that the tensor-core kernels do not take: everything in one plain kernel
            return kernels.attention_generic(q, self.nh, self.hd, out, cache.pages, cache.block_table, batch.positions, batch.seq_of_token, self.scale,
                                             window=self.window, status=batch.status, keep_first=self.keep_first, sink=self.sink)
        head = batch.num_seqs if batch.one_token_each else batch.one_token_head
        if not (0 < head <= kernels.ATTENTION_DECODE_MAX_SEQS and head * self.nkv <= kernels.ATTENTION_DECODE_MAX_PAIRS
                and kernels.attention_decode_takes(self.nh, self.nkv, self.hd, cache.page_size, q.dtype)):
            head = 0
        merges = self.sink or self.keep_first > 0
        lse = torch.empty((q.shape[0], self.nh), dtype=torch.float32, device=q.device) if merges else None
        if head:
            kernels.attention_decode(q, self.nh, self.hd, out, cache.pages, cache.block_table[:head], batch.positions, batch.q_start[:head + 1], head,
                                     self.scale, window=self.window, status=batch.status, lse=lse)
        if head < batch.num_seqs:
            kernels.attention_tc(q, self.nh, self.hd, out, cache.pages, cache.block_table[head:], batch.positions, batch.q_start[head:],
                                 batch.num_seqs - head, self.scale, window=self.window, status=batch.status, lse=lse)
        if merges:
            kernels.sink_merge(q, self.nh, self.hd, out, lse, cache.pages, cache.block_table, batch.positions, batch.seq_of_token, self.scale,
                               self.window, self.keep_first, self.sink, status=batch.status)
        return out
