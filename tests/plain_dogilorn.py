"""A plain, slow implementation of the Dogilorn decoder in float64 on the CPU: one function a mechanism, whole
sequences at once, no cache.  It shares no code with the engine; the tests hold the engine to it.

``cfg`` is the dictionary of config.json, ``W`` a dictionary name -> float64 tensor.
"""
import math

import torch

F = torch.float64


def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b over the last axis, var = mean of squared deviations."""
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w + b


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def time_conv(h, w):
    """h [T, C], w [C, taps]: out_t = sum_j w[:, j] * h_(t - taps + 1 + j), zeros before the start."""
    T, taps = h.shape[0], w.shape[1]
    out = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def rotate_pairs(x, positions, dims, base):
    """x [T, heads, d]: the pairs (2i, 2i + 1), i < dims / 2, of every head turn by positions * base^(-2i / dims)."""
    if not dims:
        return x
    out = x.clone()
    for i in range(dims // 2):
        a = positions.to(F) * (float(base) ** (-2.0 * i / dims))
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def visible(i, j, size, keep_first):
    """Does the query at position i see the key at position j?  ``size`` None: every earlier key."""
    if j > i:
        return False
    return size is None or i - j < size or j < keep_first


def keys_and_values(h, m, W, p, eps, positions):
    """What a layer's cache holds: keys after the whole-row norm and rotation [T, G, dim], values of unit rms [T, G, vdim]."""
    T, G, d, vd = h.shape[0], m["kv_heads"], m["dim"], m["vdim"]
    k = unit_rms(h @ W[p + "k"].T, eps) * W[p + "k.norm"]
    rot = m.get("rot") or {}
    k = rotate_pairs(k.reshape(T, G, d), positions, int(rot.get("dims") or 0), rot.get("base", 1.0))
    v = unit_rms((h @ W[p + "v"].T).reshape(T, G, vd), eps)
    return k, v


def visibility(T, size, keep_first):
    """[query, key] of ``visible`` for a sequence of T tokens."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = j <= i
    if size is not None:
        seen = seen & ((i - j < size) | (j < keep_first))
    return seen


def sink_softmax_attention(q, k, v, scale, temp, size, keep_first, probs=None):
    """q [T, H, d], k [T, G, d], v [T, G, vd]; weights exp(s) / (1 + sum exp(s)) over the visible keys (the one in the
    denominator is a sink: a key of score 0 that has no value).  ``probs`` (a list) receives the weights [H, T, T]."""
    T, H = q.shape[0], q.shape[1]
    G = k.shape[1]
    seen = visibility(T, size, keep_first)
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    kept = []
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * scale * temp[hh]
        s = torch.where(seen, s, torch.full_like(s, -math.inf))
        m = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)          # the sink's score is 0
        e = torch.exp(s - m)
        p = e / (torch.exp(-m) + e.sum(-1, keepdim=True))
        out[:, hh] = p @ v[:, g]
        kept.append(p)
    if probs is not None:
        probs.append(torch.stack(kept))
    return out


def attention_mixer(h, m, W, p, eps, positions, shared=None, probs=None):
    """``shared``: (keys, values) of the layer that ``kv_from`` names, or None for a layer with projections of its own.
    Returns the mixer's output and the (keys, values) it used."""
    T, H, d = h.shape[0], m["heads"], m["dim"]
    q = unit_rms(h @ W[p + "q"].T, eps) * W[p + "q.norm"]
    rot = m.get("rot") or {}
    q = rotate_pairs(q.reshape(T, H, d), positions, int(rot.get("dims") or 0), rot.get("base", 1.0))
    kv = shared if shared is not None else keys_and_values(h, m, W, p, eps, positions)
    mask = m.get("mask") or {}
    o = sink_softmax_attention(q, kv[0], kv[1], float(m["scale"]), W[p + "temp"], mask.get("size"), int(mask.get("keep_first") or 0), probs)
    return o.reshape(T, -1) @ W[p + "o"].T, kv


def dense_ff(h, mlp, W, p):
    lim = float(mlp["limit"])
    g = torch.clamp(h @ W[p + "gate"].T + W[p + "gate.b"], max=lim)
    u = torch.clamp(h @ W[p + "up"].T + W[p + "up.b"], -lim, lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T + W[p + "down.b"]


def silu_expert(h, W, p):
    z = h @ W[p + "gate"].T
    return (z * torch.sigmoid(z) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(h, mlp, W, p):
    """Per token: the chosen outputs of the router (indices among experts + identity experts) and their weights."""
    r = mlp["router"]
    n_id, top = int(r.get("identity") or 0), int(r["top"])
    total = int(r["experts"]) + n_id
    s = torch.softmax(h @ W[p + "router"].T, dim=-1)
    choice = s + W[p + "correction"] if (p + "correction") in W else s.clone()
    groups = r.get("groups")
    if groups:
        count, keep = int(groups["count"]), int(groups["keep"])
        per = total // count
        best = choice.reshape(-1, count, per).max(-1).values
        kept = torch.topk(best, keep, dim=-1).indices
        allowed = torch.zeros(h.shape[0], count, dtype=torch.bool)
        allowed.scatter_(1, kept, True)
        choice = torch.where(allowed.repeat_interleave(per, dim=1), choice, torch.full_like(choice, -math.inf))
    idx = torch.topk(choice, top, dim=-1).indices
    return idx, torch.gather(s, 1, idx)


def mixture_ff(h, mlp, W, p):
    n_exp = int(mlp["router"]["experts"])
    idx, w = route(h, mlp, W, p)
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for e, wt in zip(idx[t].tolist(), w[t]):
            out[t] += wt * (h[t] if e >= n_exp else silu_expert(h[t:t + 1], W, f"{p}e{e}.")[0])
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ W[p + "shared.sg"].T) * silu_expert(h, W, p + "shared.")
    return out


def forward(cfg, W, tokens, return_layers=False, probs=None):
    """Logits [T, vocab] of one sequence (and, asked for, the stream after every layer; ``probs``, a list, receives every
    layer's attention weights)."""
    eps, taps = float(cfg["norm"]["eps"]), int((cfg.get("canon") or {}).get("taps") or 0)
    positions = torch.arange(len(tokens))
    x = W["embed"][torch.tensor(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    caches, streams = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = layer_norm(x, W[p + "norm1"], W[p + "norm1.b"], eps)
        if taps:
            h = h + time_conv(h, W[p + "canon1"])
        a, caches[i] = attention_mixer(h, m, W, p + "mix.", eps, positions, caches[m["kv_from"]] if m.get("kv_from") is not None else None, probs)
        x = x + a * W[p + "ls1"]
        mlp = layer.get("mlp")
        if mlp is not None:
            h = layer_norm(x, W[p + "norm2"], W[p + "norm2.b"], eps)
            f = dense_ff(h, mlp, W, p + "mlp.") if mlp["kind"] == "dense" else mixture_ff(h, mlp, W, p + "mlp.")
            x = x + f * W[p + "ls2"]
        streams.append(x.clone())
    logits = layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["embed"].T
    return (logits, torch.stack(streams)) if return_layers else logits


# ---- what a checkpoint of a configuration holds, and seeded random ones ------------------------------------

def tensor_shapes(cfg):
    W, V = int(cfg["width"]), int(cfg["vocab"])
    taps = int((cfg.get("canon") or {}).get("taps") or 0)
    out = {"embed": (V, W), "final.norm": (W,), "final.norm.b": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m, mlp = f"l{i}.", layer["mixer"], layer.get("mlp")
        out.update({p + "norm1": (W,), p + "norm1.b": (W,), p + "ls1": (W,)})
        if taps:
            out[p + "canon1"] = (W, taps)
        H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out.update({p + "mix.q": (H * d, W), p + "mix.q.norm": (H * d,), p + "mix.temp": (H,), p + "mix.o": (W, H * vd)})
        if m.get("kv_from") is None:
            out.update({p + "mix.k": (G * d, W), p + "mix.v": (G * vd, W), p + "mix.k.norm": (G * d,)})
        if mlp is None:
            continue
        out.update({p + "norm2": (W,), p + "norm2.b": (W,), p + "ls2": (W,)})
        if mlp["kind"] == "dense":
            ff = mlp["ff"]
            out.update({p + "mlp.gate": (ff, W), p + "mlp.gate.b": (ff,), p + "mlp.up": (ff, W), p + "mlp.up.b": (ff,), p + "mlp.down": (W, ff),
                        p + "mlp.down.b": (W,)})
        else:
            r, ff = mlp["router"], mlp["expert"]["ff"]
            total = r["experts"] + int(r.get("identity") or 0)
            out.update({p + "mlp.router": (total, W), p + "mlp.correction": (total,)})
            for e in range(r["experts"]):
                out.update({f"{p}mlp.e{e}.gate": (ff, W), f"{p}mlp.e{e}.up": (ff, W), f"{p}mlp.e{e}.down": (W, ff)})
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                out.update({p + "mlp.shared.gate": (sf, W), p + "mlp.shared.up": (sf, W), p + "mlp.shared.down": (W, sf), p + "mlp.shared.sg": (1, W)})
    return out


def random_weights(cfg, seed, gain=1.0):
    """Seeded weights in bfloat16 (as a checkpoint stores them): matrices of a size that keeps activations of order one, norm
    weights, layer scales and temperatures around one, small biases and corrections."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if name == "embed":
            t = torch.randn(shape, generator=g)
        elif last in ("norm1", "norm2", "norm") or name.endswith((".q.norm", ".k.norm")):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif last in ("ls1", "ls2"):
            t = 0.6 + 0.2 * torch.randn(shape, generator=g)
        elif last == "temp":
            t = 1.0 + 0.3 * torch.rand(shape, generator=g)
        elif last == "b":
            t = 0.2 * torch.randn(shape, generator=g)
        elif last == "correction":
            t = 0.05 * torch.randn(shape, generator=g)
        elif last == "canon1":
            t = 0.4 * torch.randn(shape, generator=g)
        elif last == "router" or last == "sg":
            t = gain * 2.0 * torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        else:
            t = gain * torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16)
    return out


def as_float64(W):
    return {k: v.to(F) for k, v in W.items()}
