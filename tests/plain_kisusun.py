"""A plain, slow implementation of the Kisusun design: one function per mechanism, 64-bit torch on
the CPU, whole sequences at once.  It shares no code with the engine; the tests compare the engine
with it.

``config`` is the config.json dictionary, ``w`` maps checkpoint tensor names to tensors.

Notation: T tokens, H query heads, G key/value heads, d the query/key head size, dv the value head
size, W the model width.  A layer is ``x <- x + N1(mix(x))``, ``x <- x + N2(ff(x))`` with
``N(y) = y / sqrt(mean(y^2) + eps) * weight``.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64
EXPERT_SLOPE = 1.702


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


def rotation_frequencies(rot):
    """One frequency per rotated pair: base^(-2i/dims), divided by the scaling factor if there is one."""
    dims = rot["dims"]
    f = torch.tensor([rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    factor = (rot.get("scaling") or {}).get("factor")
    return f / factor if factor else f


def rotate_half_pairs(x, positions, rot):
    """x [T, heads, D]: dim i of the first ``dims`` is paired with dim i + dims/2; the rest pass."""
    if not rot or not rot["dims"]:
        return x
    dims = rot["dims"]
    half = dims // 2
    ang = positions.to(F64)[:, None] * rotation_frequencies(rot)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def capped(s, cap):
    return cap * torch.tanh(s / cap) if cap else s


def seen_keys(T, window):
    """[T, T] bool: query i sees key j when 0 <= i - j (< window, if there is one)."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = i - j >= 0
    return seen & (i - j < window) if window else seen


def softmax_plus_one(scores, seen):
    """Weights exp(s_j) / (1 + sum_j exp(s_j)) over the seen keys: a key of score 0 without a value
    shares the softmax."""
    s = scores.masked_fill(~seen, float("-inf"))
    top = s.max(-1, keepdim=True).values.clamp(min=0.0)
    e = torch.exp(s - top)
    return e / (torch.exp(-top) + e.sum(-1, keepdim=True))


def values_of(h, w, p, m):
    T = h.shape[0]
    return (h @ w[p + "v"].T).view(T, m.get("kv_heads") or m["heads"], m.get("vdim") or m["dim"])


def attention(h, w, p, m, eps, v_first=None):
    """h [T, W]; tensors ``p + name``; ``m`` the mixer's configuration.  ``v_first``: the values
    [T, G, dv] this layer blends its own with (None: it keeps its own)."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    G, dv = m.get("kv_heads") or H, m.get("vdim") or d
    pos = torch.arange(T)
    q = rms_norm(h @ w[p + "q"].T, w[p + "q.norm"], eps).view(T, H, d)          # the norm spans all heads
    k = rms_norm(h @ w[p + "k"].T, w[p + "k.norm"], eps).view(T, G, d)
    q, k = rotate_half_pairs(q, pos, m.get("rot")), rotate_half_pairs(k, pos, m.get("rot"))
    v = values_of(h, w, p, m)
    if v_first is not None:
        lam = w[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    k, v = k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1)        # head h uses key/value head h // (H/G)
    scale = m["scale"] if m.get("scale") is not None else d ** -0.5
    scores = capped(torch.einsum("ihd,jhd->hij", q, k) * scale, m.get("softcap"))
    weights = softmax_plus_one(scores, seen_keys(T, (m.get("mask") or {}).get("size"))[None])
    heads = torch.einsum("hij,jhd->ihd", weights, v).reshape(T, H * dv)
    return (heads * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def silu(z):
    return z * torch.sigmoid(z)


def dense_ff(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def clamped_expert(h, w, p, limit):
    g = (h @ w[p + "gate"].T).clamp(max=limit)
    u = (h @ w[p + "up"].T).clamp(-limit, limit)
    return (g * torch.sigmoid(EXPERT_SLOPE * g) * (u + 1.0)) @ w[p + "down"].T


def open_experts(scores, groups, margins=None):
    """[T, E] bool: the experts of the ``keep`` groups whose two best scores sum highest.  ``margins``: a
    list that receives, per token, how far the last kept group's rating lies above the first one left out."""
    T, E = scores.shape
    count, keep = (groups or {}).get("count", 1), (groups or {}).get("keep", 1)
    if count <= 1:
        return torch.ones(T, E, dtype=torch.bool)
    per = E // count
    by_group = scores.view(T, count, per)
    rating = by_group.topk(min(2, per), -1).values.sum(-1)                      # [T, count]
    best = rating.topk(keep, -1).indices
    if margins is not None and keep < count:
        ordered = rating.sort(-1, descending=True).values
        margins.append(ordered[:, keep - 1] - ordered[:, keep])
    open_groups = torch.zeros(T, count, dtype=torch.bool).scatter_(1, best, True)
    return open_groups[:, :, None].expand(T, count, per).reshape(T, E)


def route(h, w, p, router, margins=None):
    """(chosen experts [T, top], their weights [T, top]).  ``margins``: a list that receives per-token
    distances between what was chosen and what was not (a small one marks a choice that rounding can turn)."""
    scores = torch.sigmoid(h @ w[p + "router"].T)
    allowed = open_experts(scores, router.get("groups"), margins)
    masked = scores.masked_fill(~allowed, -1.0)
    chosen = masked.topk(router["top"], -1).indices
    if margins is not None and router["top"] < int(allowed[0].sum()):
        ordered = masked.sort(-1, descending=True).values
        margins.append(ordered[:, router["top"] - 1] - ordered[:, router["top"]])
    return chosen, scores.gather(1, chosen) * router.get("scale", 1.0)


def moe_ff(h, w, p, mlp, margins=None):
    chosen, weights = route(h, w, p, mlp["router"], margins)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weights[t]):
            out[t] += a * clamped_expert(h[t:t + 1], w, p + f"e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out = out + clamped_expert(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


def feed_forward(h, w, p, mlp, margins=None):
    return dense_ff(h, w, p) if mlp["kind"] == "dense" else moe_ff(h, w, p, mlp, margins)


def first_mixing_layer(config):
    return next((i for i, layer in enumerate(config["layers"]) if layer["mixer"].get("v_mix")), None)


def forward(config, weights, tokens, taps=None, margins=None):
    """Logits [T, vocab] of one sequence (64-bit).  ``taps``: a list that receives the stream after
    every layer.  ``margins``: a list that receives the routers' per-token margins (see :func:`route`)."""
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * (config.get("embedding") or {}).get("scale", 1.0)
    first = first_mixing_layer(config)
    v_first = None
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if i == first:
            v_first = values_of(x, w, p + "mix.", m)
        blend = v_first if (m.get("v_mix") and i != first) else None
        x = x + rms_norm(attention(x, w, p + "mix.", m, eps, blend), w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + rms_norm(feed_forward(x, w, p + "mlp.", layer["mlp"], margins), w[p + "norm2"], eps)
        if taps is not None:
            taps.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["embed"].T * config.get("logit_scale", 1.0)


def tensor_shapes(config):
    """Checkpoint tensor name -> shape, for a configuration dictionary."""
    W = config["width"]
    out = {"embed": (config["vocab"], W), "final.norm": (W,)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, d = m["heads"], m["dim"]
        G, dv = m.get("kv_heads") or H, m.get("vdim") or d
        out.update({p + "norm1": (W,), p + "mix.q": (H * d, W), p + "mix.k": (G * d, W), p + "mix.v": (G * dv, W),
                    p + "mix.q.norm": (H * d,), p + "mix.k.norm": (G * d,), p + "mix.g": (H * dv, W),
                    p + "mix.o": (W, H * dv)})
        if m.get("v_mix"):
            out[p + "mix.vmix"] = ()
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        out[p + "norm2"] = (W,)
        if mlp["kind"] == "dense":
            out.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
            continue
        E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
        out[p + "mlp.router"] = (E, W)
        for name, n in [(f"e{e}.", ff) for e in range(E)] + ([("shared.", mlp["shared"]["ff"])] if mlp.get("shared") else []):
            out.update({p + "mlp." + name + "gate": (n, W), p + "mlp." + name + "up": (n, W), p + "mlp." + name + "down": (W, n)})
    return out


def random_weights(config, seed, gain=1.0):
    """bfloat16 tensors of a size that keeps activations of order one: the stream has elements of
    size embedding.scale, so matrices that read it are smaller by that factor."""
    g = torch.Generator().manual_seed(seed)
    stream = max(1.0, (config.get("embedding") or {}).get("scale", 1.0))
    out = {}
    for name, shape in tensor_shapes(config).items():
        x = torch.randn(shape, generator=g)
        if name.endswith(("norm", "norm1", "norm2")):
            t = 1.0 + 0.2 * x
        elif name.endswith("vmix"):
            t = torch.sigmoid(x)
        elif name == "embed":
            t = x / math.sqrt(stream)
        elif name.endswith(("down", "mix.o")):
            t = gain * x / math.sqrt(shape[-1])
        else:
            t = gain * x / (math.sqrt(shape[-1]) * math.sqrt(stream))
        out[name] = t.to(torch.bfloat16)
    return out
