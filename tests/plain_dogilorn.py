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


def sink_softmax_attention(q, k, v, scale, temp, size, keep_first):
    """q [T, H, d], k [T, G, d], v [T, G, vd]; weights exp(s) / (1 + sum exp(s)) over the visible keys."""
    T, H = q.shape[0], q.shape[1]
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * scale * temp[hh]
        for i in range(T):
            js = [j for j in range(T) if visible(i, j, size, keep_first)]
            e = torch.exp(s[i, js])
            out[i, hh] = (e / (1.0 + e.sum())) @ v[js, g]
    return out


def attention_mixer(h, m, W, p, eps, positions, shared=None):
    """``shared``: (keys, values) of the layer that ``kv_from`` names, or None for a layer with projections of its own.
    Returns the mixer's output and the (keys, values) it used."""
    T, H, d = h.shape[0], m["heads"], m["dim"]
    q = unit_rms(h @ W[p + "q"].T, eps) * W[p + "q.norm"]
    rot = m.get("rot") or {}
    q = rotate_pairs(q.reshape(T, H, d), positions, int(rot.get("dims") or 0), rot.get("base", 1.0))
    kv = shared if shared is not None else keys_and_values(h, m, W, p, eps, positions)
    mask = m.get("mask") or {}
    o = sink_softmax_attention(q, kv[0], kv[1], float(m["scale"]), W[p + "temp"], mask.get("size"), int(mask.get("keep_first") or 0))
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


def forward(cfg, W, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (and, asked for, the stream after every layer)."""
    eps, taps = float(cfg["norm"]["eps"]), int((cfg.get("canon") or {}).get("taps") or 0)
    positions = torch.arange(len(tokens))
    x = W["embed"][torch.tensor(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    caches, streams = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = layer_norm(x, W[p + "norm1"], W[p + "norm1.b"], eps)
        if taps:
            h = h + time_conv(h, W[p + "canon1"])
        a, caches[i] = attention_mixer(h, m, W, p + "mix.", eps, positions, caches[m["kv_from"]] if m.get("kv_from") is not None else None)
        x = x + a * W[p + "ls1"]
        mlp = layer.get("mlp")
        if mlp is not None:
            h = layer_norm(x, W[p + "norm2"], W[p + "norm2.b"], eps)
            f = dense_ff(h, mlp, W, p + "mlp.") if mlp["kind"] == "dense" else mixture_ff(h, mlp, W, p + "mlp.")
            x = x + f * W[p + "ls2"]
        streams.append(x.clone())
    logits = layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["embed"].T
    return (logits, torch.stack(streams)) if return_layers else logits
