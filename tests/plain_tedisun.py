"""A plain, slow implementation of the Tedisun design: one function per mechanism, 64-bit torch on
the CPU, whole sequences at once (the recurrences token by token).  It shares no code with the
engine; the tests compare the engine with it.

``config`` is the config.json dictionary, ``w`` maps checkpoint tensor names to tensors.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def log_sigmoid(z):
    return -softplus(-z)


def one_plus_norm(x, weight, eps):
    """RMS norm whose stored weight lies around zero."""
    return unit_rms(x, eps) * (1.0 + weight)


# ---- positions ---------------------------------------------------------------------------------

def scaled_frequencies(rot):
    """One frequency per rotated pair; wavelengths beyond ``original / low`` are slowed by ``factor``,
    those under ``original / high`` kept, the band between blended."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F64)
    factor, low, high, orig = sc["factor"], sc["low"], sc["high"], sc["original"]
    out = []
    for x in f:
        wave = 2.0 * math.pi / x
        if wave < orig / high:
            out.append(x)
        elif wave > orig / low:
            out.append(x / factor)
        else:
            s = (orig / wave - low) / (high - low)
            out.append((1.0 - s) * x / factor + s * x)
    return torch.tensor(out, dtype=F64)


def rotate_half_pairs(x, positions, rot):
    """x [T, H, D]: dim i of the first ``dims`` is paired with dim i + dims/2; the rest pass."""
    dims = rot["dims"]
    half = dims // 2
    ang = positions.to(F64)[:, None] * scaled_frequencies(rot)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


# ---- mixers ------------------------------------------------------------------------------------

def causal_conv(x, taps_w):
    """x [T, C], taps_w [C, taps]: the last column weighs the current token; zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], 0)
    out = torch.zeros_like(x)
    for j in range(taps):
        out = out + padded[j:j + T] * taps_w[:, j][None, :]
    return out


def delta_mixer(h, w, p, m, eps):
    """Gated delta rule with one decay per head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, d)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, d)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    rep = H // G
    q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                  # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    S = torch.zeros(H, d, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = decay[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = unit_rms(o, eps) * w[p + "norm"] * silu(h @ w[p + "g"].T).view(T, H, dv)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def sink_window_attention(h, w, p, m, eps):
    """Grouped-query softmax attention: biases, a norm per head on q and k, partial rotation, a
    sliding window that also keeps the first tokens, a learned sink per head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    q = unit_rms(q, eps) * w[p + "q.norm"]
    k = unit_rms(k, eps) * w[p + "k.norm"]
    rot = m.get("rot")
    if rot and rot["dims"]:
        q, k = rotate_half_pairs(q, pos, rot), rotate_half_pairs(k, pos, rot)
    rep = H // G
    k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    i, j = pos[:, None], pos[None, :]
    seen = j <= i
    mask = m.get("mask")
    if mask:
        seen = seen & ((i - j < mask["size"]) | (j < mask.get("keep_first", 0)))
    scores = scores.masked_fill(~seen[None], float("-inf"))
    sink = w[p + "sink"].to(F64)[:, None, None].expand(H, T, 1)
    prob = torch.softmax(torch.cat([scores, sink], -1), -1)[..., :T]          # the sink has no value
    out = torch.einsum("hij,jhd->ihd", prob, v).reshape(T, H * dv)
    return out @ w[p + "o"].T + w[p + "o.b"]


def matrix_memory(h, w, p, m, eps):
    """Matrix memory with exponential gates held stable by a running maximum that starts at 0."""
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[p + "q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, d)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    gi = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)              # [T, H]
    gf = log_sigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    S = torch.zeros(H, d, dv, dtype=F64)
    n = torch.zeros(H, d, dtype=F64)
    mx = torch.zeros(H, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        new = torch.maximum(gf[t] + mx, gi[t])
        keep, take = torch.exp(gf[t] + mx - new), torch.exp(gi[t] - new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        mx = new
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        o[t] = torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None]
    o = unit_rms(o, eps).reshape(T, H * dv) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    return (m["left_scale"] * sink_window_attention(h, w, p + "left.", m["left"], eps)
            + m["right_scale"] * matrix_memory(h, w, p + "right.", m["right"], eps))


MIXERS = {"delta": delta_mixer, "parallel": parallel_mixer}


# ---- feed-forward ------------------------------------------------------------------------------

def routed_ff(h, w, p, mlp):
    """Softmax scores over experts and identity experts; the choice adds a correction, the weights
    are the plain scores of the chosen, not renormalised."""
    r = mlp["router"]
    E, ident, top = r["experts"], r.get("identity", 0), r["top"]
    s = torch.softmax(h @ w[p + "router"].T, -1)                                # [T, E + ident]
    choice = s + w[p + "correction"] if (p + "correction") in w else s
    chosen = torch.topk(choice, top, -1).indices
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            if e >= E:
                y = h[t]
            else:
                y = (silu(h[t] @ w[p + f"e{e}.gate"].T) * (h[t] @ w[p + f"e{e}.up"].T)) @ w[p + f"e{e}.down"].T
            out[t] = out[t] + s[t, e] * y
    return out


# ---- the model ---------------------------------------------------------------------------------

def forward(config, w, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence.  ``layers_out``: a list that receives the sum of the streams
    after every layer."""
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in w.items()}
    eps = config["norm"]["eps"]
    n_streams = int(config.get("streams", 1))
    x0 = w["embed"][torch.as_tensor(tokens)] * config["embedding"]["scale"]
    xs = [x0.clone() for _ in range(n_streams)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        subs = [(1, lambda hh: MIXERS[layer["type"]](hh, w, p + "mix.", layer["mixer"], eps))]
        if layer.get("mlp") is not None:
            subs.append((2, lambda hh: routed_ff(hh, w, p + "mlp.", layer["mlp"])))
        for q, fn in subs:
            hc = f"{p}hc{q}."
            if hc + "in" in w:
                u = sum(w[hc + "in"][s] * xs[s] for s in range(n_streams))
            else:
                u = xs[0]
            hh = one_plus_norm(u, w[f"{p}norm{q}"], eps)
            y = fn(hh)
            if f"{p}rg{q}" in w:
                y = y * torch.sigmoid(hh @ w[f"{p}rg{q}"].T + w[f"{p}rg{q}.b"])
            if hc + "in" in w:
                xs = [sum(w[hc + "mix"][s, t] * xs[s] for s in range(n_streams)) + w[hc + "out"][t] * y
                      for t in range(n_streams)]
            else:
                xs = [xs[0] + y]
        if layers_out is not None:
            layers_out.append(sum(xs))
    x = one_plus_norm(sum(xs), w["final.norm"], eps)
    logits = x @ w["head"].T if "head" in w else x @ w["embed"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits


# ---- random weights ----------------------------------------------------------------------------

def random_weights(config, seed):
    """Checkpoint tensors (bfloat16) for ``config``, spread so that every mechanism matters."""
    g = torch.Generator().manual_seed(seed)
    W, V, S = config["width"], config["vocab"], int(config.get("streams", 1))
    out = {}

    def put(name, shape, std=1.0, mean=0.0):
        out[name] = (torch.randn(*shape, generator=g) * std + mean).to(torch.bfloat16)

    def lin(name, rows, cols, gain=1.0):
        put(name, (rows, cols), gain * cols ** -0.5)

    put("embed", (V, W), W ** -0.5)
    lin("head", V, W)
    put("final.norm", (W,), 0.1)
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        subs = (1, 2) if layer.get("mlp") is not None else (1,)
        for q in subs:
            put(f"{p}norm{q}", (W,), 0.1)
            if "streams" in config:
                put(f"{p}hc{q}.in", (S,), 0.2, 1.0 / S)
                put(f"{p}hc{q}.out", (S,), 0.3, 0.8)
                out[f"{p}hc{q}.mix"] = (torch.eye(S) + 0.15 * torch.randn(S, S, generator=g)).to(torch.bfloat16)
            lin(f"{p}rg{q}", W, W)
            put(f"{p}rg{q}.b", (W,), 0.5, 0.5)
        if layer["type"] == "delta":
            H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for name, rows in (("q", G * d), ("k", G * d), ("v", H * dv)):
                lin(p + "mix." + name, rows, W, 2.0)
                put(p + "mix." + name + ".conv", (rows, taps), 0.6)
            lin(p + "mix.b", H, W)
            lin(p + "mix.a", H, W)
            put(p + "mix.A_log", (H,), 0.7, -1.0)
            put(p + "mix.dt_bias", (H,), 0.7, -1.0)
            put(p + "mix.norm", (dv,), 0.1, 1.0)
            lin(p + "mix.g", H * dv, W)
            lin(p + "mix.o", W, H * dv)
        else:
            a, r = m["left"], m["right"]
            H, G, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            for name, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                lin(p + "mix.left." + name, rows, W)
                put(p + "mix.left." + name + ".b", (rows,), 0.3)
            put(p + "mix.left.q.norm", (d,), 0.2, 1.0)
            put(p + "mix.left.k.norm", (d,), 0.2, 1.0)
            put(p + "mix.left.sink", (H,), 1.0)
            lin(p + "mix.left.o", W, H * dv)
            put(p + "mix.left.o.b", (W,), 0.2)
            H, d, dv = r["heads"], r["dim"], r["vdim"]
            for name, rows in (("q", H * d), ("k", H * d), ("v", H * dv), ("g", H * dv)):
                lin(p + "mix.right." + name, rows, W)
            lin(p + "mix.right.o", W, H * dv)
            put(p + "mix.right.norm", (H * dv,), 0.1, 1.0)
            lin(p + "mix.right.i", H, W, 2.0)
            put(p + "mix.right.i.b", (H,), 1.0)
            lin(p + "mix.right.f", H, W, 2.0)
            put(p + "mix.right.f.b", (H,), 1.0, 2.0)
        mlp = layer.get("mlp")
        if mlp is not None:
            E, ident, ff = mlp["router"]["experts"], mlp["router"].get("identity", 0), mlp["expert"]["ff"]
            for e in range(E):
                lin(f"{p}mlp.e{e}.gate", ff, W)
                lin(f"{p}mlp.e{e}.up", ff, W)
                lin(f"{p}mlp.e{e}.down", W, ff)
            lin(p + "mlp.router", E + ident, W, 2.0)
            put(p + "mlp.correction", (E + ident,), 0.05)
    return out
