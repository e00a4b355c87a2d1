"""A plain, slow implementation of the Naforax decoder in float64 on the CPU, one function per mechanism, written from
the design's equations and sharing no code with the engine.  A whole sequence at a time, no cache, no batching.

Notation: ``h`` is a sublayer's input ``[T, width]``; weights ``w`` are a dictionary name -> float64 tensor, stored
``[out, in]`` and applied as ``h @ W.T``; positions count from 0; ``cfg`` is the model's config.json as a dictionary.
"""
import math

import torch

F = torch.float64


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def group_norm(x, weight, groups, eps):
    """The last axis in ``groups`` equal consecutive parts, each brought to unit root mean square; then the gain."""
    T, W = x.shape
    return unit_rms(x.reshape(T, groups, W // groups), eps).reshape(T, W) * weight


def time_conv(h, kernel, bias=None):
    """Causal convolution over time on each channel: ``kernel [channels, taps]``, whose last column meets the current
    token; zeros stand before the sequence's start."""
    T, C = h.shape
    taps = kernel.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=h.dtype), h], dim=0)
    out = torch.zeros_like(h)
    for j in range(taps):
        out = out + padded[j:j + T] * kernel[:, j]
    return out if bias is None else out + bias


def sublayer_input(h, kernel):
    """What a sublayer reads: its normed input plus that input's convolution over time (no kernel: the input itself)."""
    return h if kernel is None else h + time_conv(h, kernel)


def rotate_pairs(x, positions, base, dims):
    """Rotates the pairs ``(2i, 2i + 1)``, ``i < dims / 2``, of the last axis of ``x [T, ..., D]`` by ``position * base^(-2i / dims)``."""
    out = x.clone()
    for i in range(dims // 2):
        angle = positions.to(F) * (base ** (-2.0 * i / dims))
        while angle.dim() < x.dim() - 1:
            angle = angle[:, None]
        c, s = torch.cos(angle), torch.sin(angle)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def chunk_visible(T, size):
    """[query, key] -> bool: earlier keys (and the query's own) of the query's own chunk of ``size`` positions."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    return (j <= i) & ((i // size) == (j // size))


def diff_lambda(w, p, diff):
    return math.exp(float((w[p + "lq1"] * w[p + "lk1"]).sum())) - math.exp(float((w[p + "lq2"] * w[p + "lk2"]).sum())) + diff


def diff_attention(h, w, p, m, eps, probs=None):
    """Two softmax maps a head over the same values, the second subtracted ``lambda`` times; per-head unit norm; a
    sigmoid gate from the input.  ``probs`` (a list) receives the maps ``[2, heads, query, key]``."""
    T, H, G, d, vd, diff = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["diff"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, 2, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, 2, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, vd)
    q = unit_rms(q, eps) * w[p + "q.norm"]
    k = unit_rms(k, eps) * w[p + "k.norm"]
    pos = torch.arange(T)
    rot = m.get("rot")
    if rot is not None and rot["dims"] > 0:
        q, k = rotate_pairs(q, pos, rot["base"], rot["dims"]), rotate_pairs(k, pos, rot["base"], rot["dims"])
    rep = H // G
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihmd,jhmd->mhij", q, k) * m["scale"]
    size = m["mask"]["size"] if m.get("mask") is not None else T + 1          # no mask: every earlier key
    s = s.masked_fill(~chunk_visible(T, size)[None, None], -math.inf)
    a = torch.softmax(s, dim=-1)
    if probs is not None:
        probs.append(a)
    o = torch.einsum("mhij,jhv->mihv", a, v)
    o = o[0] - diff_lambda(w, p, diff) * o[1]
    o = unit_rms(o, eps) * (1.0 - diff)
    o = o.reshape(T, H * vd) * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T + w[p + "o.b"]


def mingru(h, w, p, state=None):
    """``S_t = (1 - z_t) S_(t-1) + z_t c_t`` element by element, gates from the current token only."""
    z = torch.sigmoid(h @ w[p + "z"].T + w[p + "z.b"])
    u = h @ w[p + "x"].T + w[p + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    gate = torch.nn.functional.silu(h @ w[p + "g"].T)
    S = torch.zeros(z.shape[1], dtype=F) if state is None else state
    rows = []
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        rows.append(S * gate[t])
    return torch.stack(rows) @ w[p + "o"].T


def mamba1(h, w, p, m):
    """Selective scan: a state ``[inner, state]`` that decays by ``exp(dt A)`` and takes in ``dt x B``."""
    T, inner, N, R = h.shape[0], m["inner"], m["state"], m["dt_rank"]
    xz = h @ w[p + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = torch.nn.functional.silu(time_conv(x, w[p + "conv"], w[p + "conv.b"]))
    proj = x @ w[p + "x"].T
    dt, B, C = proj[:, :R], proj[:, R:R + N], proj[:, R + N:R + 2 * N]
    dt = torch.nn.functional.softplus(dt @ w[p + "dt"].T + w[p + "dt.b"])
    A = -torch.exp(w[p + "A_log"])
    S = torch.zeros(inner, N, dtype=F)
    rows = []
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        rows.append(S @ C[t] + w[p + "D"] * x[t])
    y = torch.stack(rows) * torch.nn.functional.silu(z)
    return y @ w[p + "o"].T


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def dense_ff(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def expert(h, w, p, limit):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def moe_ff(h, w, p, mlp, chosen=None):
    """Softmax over all experts, the ``top`` largest scores keep their values as weights; a shared expert with a sigmoid
    gate of its own beside them.  ``chosen`` (a list) receives the chosen experts ``[T, top]``."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    scores = torch.softmax(h @ w[p + "router"].T, dim=-1)
    best = torch.topk(scores, top, dim=-1)
    if chosen is not None:
        chosen.append(best.indices)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F)
    for e in range(E):
        y = expert(h, w, f"{p}e{e}.", mlp["expert"]["limit"])
        weight = (scores[:, e:e + 1] * (best.indices == e).any(-1, keepdim=True))
        out = out + weight * y
    if mlp.get("shared") is not None:
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * expert(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


def run_order(cfg):
    """(layer, pass number or None, first of its pass) in the order the layers run."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    order = [(i, None, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None, False) for i in range(loop["stop"], n)]


def layer(x, w, cfg, i, probs=None, chosen=None):
    L, p = cfg["layers"][i], f"l{i}."
    m, groups, eps = cfg.get("residual_mult", 1.0), cfg["norm"].get("groups", 1), cfg["norm"]["eps"]
    h = sublayer_input(group_norm(x, w[p + "norm1"], groups, eps), w.get(p + "canon1"))
    if L["type"] == "attention":
        a = diff_attention(h, w, p + "mix.", L["mixer"], eps, probs)
    elif L["type"] == "mingru":
        a = mingru(h, w, p + "mix.")
    elif L["type"] == "mamba1":
        a = mamba1(h, w, p + "mix.", L["mixer"])
    else:
        raise ValueError(L["type"])
    x = x + m * group_norm(a, w[p + "norm1b"], groups, eps)
    mlp = L.get("mlp")
    if mlp is not None:
        h = sublayer_input(group_norm(x, w[p + "norm2"], groups, eps), w.get(p + "canon2"))
        f = dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp, chosen)
        x = x + m * group_norm(f, w[p + "norm2b"], groups, eps)
    return x


def model(tokens, w, cfg, streams=None, probs=None, chosen=None):
    """Logits ``[T, vocab]`` of one whole sequence.  ``streams`` (a list) receives the residual stream after every layer run,
    ``probs`` the attention maps of every attention layer run, ``chosen`` the experts that every mixture layer run chose."""
    w = {k: v.to(F) for k, v in w.items()}
    first = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = first
    for i, t, opens in run_order(cfg):
        if opens:
            if t > 0:
                x = x + first
            x = x + w["loop.step"][t]
        x = layer(x, w, cfg, i, probs, chosen)
        if streams is not None:
            streams.append(x)
    x = group_norm(x, w["final.norm"], cfg["norm"].get("groups", 1), cfg["norm"]["eps"])
    logits = x @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits


def forward(w, cfg, tokens, **more):
    return model(tokens, w, cfg, **more)


def tensor_shapes(cfg):
    """name -> shape of every tensor a checkpoint of this configuration holds."""
    W, out = cfg["width"], {}
    out["embed"], out["head"], out["final.norm"] = (cfg["vocab"], W), (cfg["vocab"], W), (W,)
    loop = cfg.get("loop")
    if loop and loop["start"] < loop["stop"]:
        out["loop.step"] = (loop["times"], W)
    taps = (cfg.get("canon") or {}).get("taps", 0)
    for i, L in enumerate(cfg["layers"]):
        p, m, mlp = f"l{i}.", L["mixer"], L.get("mlp")
        out[p + "norm1"], out[p + "norm1b"] = (W,), (W,)
        if taps:
            out[p + "canon1"] = (W, taps)
        if L["type"] == "attention":
            H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (2 * H * d, W), p + "mix.q.b": (2 * H * d,), p + "mix.k": (2 * G * d, W), p + "mix.k.b": (2 * G * d,),
                        p + "mix.v": (G * vd, W), p + "mix.v.b": (G * vd,), p + "mix.q.norm": (d,), p + "mix.k.norm": (d,),
                        p + "mix.g": (H * vd, W), p + "mix.o": (W, H * vd), p + "mix.o.b": (W,)})
            out.update({p + "mix." + n: (d,) for n in ("lq1", "lk1", "lq2", "lk2")})
        elif L["type"] == "mingru":
            n = m["width"]
            out.update({p + "mix.z": (n, W), p + "mix.z.b": (n,), p + "mix.x": (n, W), p + "mix.x.b": (n,), p + "mix.g": (n, W), p + "mix.o": (W, n)})
        else:
            I, N, R = m["inner"], m["state"], m["dt_rank"]
            out.update({p + "mix.in": (2 * I, W), p + "mix.conv": (I, m["conv"]), p + "mix.conv.b": (I,), p + "mix.x": (R + 2 * N, I),
                        p + "mix.dt": (I, R), p + "mix.dt.b": (I,), p + "mix.A_log": (I, N), p + "mix.D": (I,), p + "mix.o": (W, I)})
        if mlp is None:
            continue
        out[p + "norm2"], out[p + "norm2b"] = (W,), (W,)
        if taps:
            out[p + "canon2"] = (W, taps)
        if mlp["kind"] == "dense":
            out.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
        else:
            names = [(f"e{e}.", mlp["expert"]["ff"]) for e in range(mlp["router"]["experts"])]
            if mlp.get("shared") is not None:
                names.append(("shared.", mlp["shared"]["ff"]))
                out[p + "mlp.shared.sg"] = (1, W)
            out[p + "mlp.router"] = (mlp["router"]["experts"], W)
            for n, ff in names:
                out.update({p + "mlp." + n + "gate": (ff, W), p + "mlp." + n + "up": (ff, W), p + "mlp." + n + "down": (W, ff)})
    return out


def random_weights(cfg, seed, gain=1.0):
    """Seeded bfloat16 tensors: matrices ``N(0, gain^2 / in)``, gains of norms near one, small biases, decays and step sizes
    of the scan in a range where the state neither dies at once nor keeps everything, a router whose scores differ."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if name.endswith("A_log"):
            t = torch.log(1.0 + torch.arange(shape[1], dtype=torch.float32) * 0.5)[None, :] + 0.2 * torch.randn(shape, generator=g) - 1.0
        elif name.endswith("dt.b"):
            t = torch.randn(shape, generator=g) * 0.5 - 1.0
        elif last in ("norm1", "norm1b", "norm2", "norm2b") or name in ("final.norm",) or name.endswith(".D") or name.endswith("q.norm") or name.endswith("k.norm"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif last == "b":
            t = 0.3 * torch.randn(shape, generator=g)
        elif last in ("canon1", "canon2", "conv"):
            t = 0.5 * torch.randn(shape, generator=g)
        elif name in ("embed", "loop.step"):
            t = torch.randn(shape, generator=g)
        elif last == "router" or last == "sg":
            t = 3.0 * torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        else:
            t = gain * torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16)
    return out
