"""Tedisun: a decoder-only design whose ``config.json`` lists its layers one by one, over several
copies of the residual stream.

The stream is kept in ``streams`` 32-bit copies, all equal to the scaled embedding at the start
(``parts.streams``).  A sublayer q of layer i (1: the mixer, 2: the feed-forward) reads the mixture
``sum_s hc<q>.in[s] x_s`` through an RMS norm whose stored weight lies around zero (applied as 1 + w),
its result is multiplied by ``sigmoid(rg<q> h + rg<q>.b)`` with ``h`` the normed input, and goes back
into all copies, ``x_t <- sum_s hc<q>.mix[s, t] x_s + hc<q>.out[t] y``.  The last norm reads the sum of
the copies; the logits are capped.  A layer's mixer is one of

* ``delta``: a gated delta rule with one decay per head (``parts.recurrent.GatedDeltaMixer``,
  ``decay_per="head"``, a silu output gate);
* ``parallel``: two mixers on the same input whose results are added with weights from the
  configuration (``parts.parallel``): grouped-query attention with biases, a norm per head on q and
  k, partial rotation with scaled frequencies, a sliding window that keeps the first tokens visible
  and a learned sink per head; and a matrix memory with exponential gates
  (``parts.recurrent.MatrixMemoryMixer``).

The feed-forward is routed: softmax scores over the experts and a few identity experts (their
output is their input), the choice by score plus a correction, the weights the plain scores of the
chosen.  A checkpoint without ``hc*`` tensors has one plain residual stream, one without ``rg*``
tensors no gate on the sublayers' results, one without ``correction`` no correction.

Tensor names: ``embed``, ``head``, ``final.norm``, ``l<i>.norm1|norm2``, ``l<i>.hc1|hc2.in|out|mix``,
``l<i>.rg1|rg2[.b]``, ``l<i>.mix.*``, ``l<i>.mlp.router|correction``, ``l<i>.mlp.e<j>.gate|up|down``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..config.registry import register_architecture
from ..config.specs import (AttentionSpec, GatedDeltaSpec, LayerSpec, MatrixMemorySpec, ModelSpec, MoESpec,
                            ParallelMixerSpec, RMSNormSpec, RotarySpec, ScheduleEntry, Source, StreamMixSpec)

ARCHITECTURE = "Tedisun"
MIXER_TYPES = ("delta", "parallel")
DEFAULT_MAX_POSITION = 1 << 20      # the design has no position table; the cache manager wants a bound

_DELTA_KEYS = ("heads", "kv_heads", "dim", "vdim", "conv")
_LEFT_KEYS = ("heads", "kv_heads", "dim", "vdim")
_RIGHT_KEYS = ("heads", "dim", "vdim", "gate_cap")


@dataclass(frozen=True)
class TedisunConfig:
    vocab: int
    width: int
    streams: int
    layers: tuple                      # of dicts {"type", "mixer", "mlp"} as in config.json (validated)
    embedding_scale: float
    norm_eps: float
    logit_softcap: Optional[float]
    max_position: int
    learned_streams: tuple             # per layer: the checkpoint has hc1 / hc2 tensors
    gated: tuple                       # per layer: the checkpoint has rg1 / rg2 tensors
    corrected: tuple                   # per layer: the router has a correction
    own_head: bool

    uses_checkpoint_shapes = True

    @classmethod
    def from_dict(cls, raw: dict, shapes: Optional[dict] = None) -> "TedisunConfig":
        problems = []
        for key in ("vocab", "width", "layers"):
            if raw.get(key) is None:
                problems.append(f"missing key {key!r}")
        layers = raw.get("layers") or []
        if not isinstance(layers, list) or not layers:
            problems.append("'layers' must be a non-empty list")
            layers = []
        for i, layer in enumerate(layers):
            kind, m = layer.get("type"), layer.get("mixer") or {}
            if kind not in MIXER_TYPES:
                problems.append(f"layer {i}: unknown mixer type {kind!r} (known: {', '.join(MIXER_TYPES)})")
                continue
            if kind == "delta":
                missing = [k for k in _DELTA_KEYS if m.get(k) is None]
            else:
                left, right = m.get("left") or {}, m.get("right") or {}
                missing = [f"left.{k}" for k in _LEFT_KEYS if left.get(k) is None] + \
                          [f"right.{k}" for k in _RIGHT_KEYS if right.get(k) is None]
                rot = left.get("rot")
                if rot is not None and rot.get("dims") and rot.get("base") is None:
                    problems.append(f"layer {i}: 'rot' needs 'base'")
                sc = (rot or {}).get("scaling")
                if sc is not None and any(sc.get(k) is None for k in ("factor", "low", "high", "original")):
                    problems.append(f"layer {i}: 'rot.scaling' needs factor, low, high and original")
                mask = left.get("mask")
                if mask is not None and mask.get("size") is None:
                    problems.append(f"layer {i}: 'mask' needs 'size'")
            if missing:
                problems.append(f"layer {i} ({kind}): missing mixer keys {missing}")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "moe") != "moe" or (mlp.get("expert") or {}).get("ff") is None \
                        or (mlp.get("router") or {}).get("experts") is None or (mlp.get("router") or {}).get("top") is None:
                    problems.append(f"layer {i}: the feed-forward must be a 'moe' with expert.ff, router.experts and "
                                    "router.top, or null")
        if problems:
            raise ValueError("Tedisun config.json cannot be used: " + "; ".join(problems))
        has = (lambda name: name in shapes) if shapes is not None else None
        streams = int(raw.get("streams", 1))
        n = len(layers)
        cap = raw.get("logit_softcap")
        return cls(vocab=int(raw["vocab"]), width=int(raw["width"]), streams=streams, layers=tuple(layers),
                   embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
                   norm_eps=float((raw.get("norm") or {}).get("eps", 1e-6)),
                   logit_softcap=float(cap) if cap else None,
                   max_position=int(raw.get("max_position", DEFAULT_MAX_POSITION)),
                   # without a checkpoint to look at: what the configuration implies
                   learned_streams=tuple(has(f"l{i}.hc1.in") if has else "streams" in raw for i in range(n)),
                   gated=tuple(has(f"l{i}.rg1") if has else True for i in range(n)),
                   corrected=tuple(has(f"l{i}.mlp.correction") if has else True for i in range(n)),
                   own_head=has("head") if has else True)


def _rows(prefix, parts):
    """Sources that stack the named tensors along the first dimension."""
    out, at = [], 0
    for name, n in parts:
        out.append(Source(prefix + name, ((at, n),)))
        at += n
    return tuple(out)


def _delta(cfg, m, p):
    d, dv, H, G = int(m["dim"]), int(m["vdim"]), int(m["heads"]), int(m["kv_heads"])
    spec = GatedDeltaSpec(hidden_size=cfg.width, num_heads=H, num_kv_heads=G, head_dim=d, v_head_dim=dv,
                          conv_taps=int(m["conv"]), norm_eps=cfg.norm_eps, unit_eps=1e-6, decay_per="head",
                          gate_activation="silu")
    qk, vv = G * d, H * dv
    sources = {"mixer.in_proj": _rows(p, (("q", qk), ("k", qk), ("v", vv), ("b", H), ("a", H), ("g", vv))),
               "mixer.conv_w": _rows(p, (("q.conv", qk), ("k.conv", qk), ("v.conv", vv))),
               "mixer.dt_bias": (Source(p + "dt_bias"),), "mixer.a_log": (Source(p + "A_log"),),
               "mixer.norm_w": (Source(p + "norm"),), "mixer.o": (Source(p + "o"),)}
    return spec, sources


def _attention(cfg, m, p, name):
    d, dv, H, G = int(m["dim"]), int(m["vdim"]), int(m["heads"]), int(m["kv_heads"])
    rot, position = m.get("rot"), None
    if rot is not None and int(rot.get("dims") or 0) > 0:
        sc = rot.get("scaling")
        scaling = None
        if sc is not None:
            scaling = tuple(sorted({"rope_type": "llama3", "factor": float(sc["factor"]),
                                    "low_freq_factor": float(sc["low"]), "high_freq_factor": float(sc["high"]),
                                    "original_max_position_embeddings": float(sc["original"])}.items()))
        position = RotarySpec(rotary_dim=int(rot["dims"]), theta=float(rot["base"]), pairing="split_half",
                              frequency_scaling=scaling)
    mask = m.get("mask")
    spec = AttentionSpec(hidden_size=cfg.width, num_heads=H, num_kv_heads=G, head_dim=d,
                         scale=float(m.get("scale", d ** -0.5)), qk_norm="per_head", qk_norm_eps=cfg.norm_eps,
                         window=int(mask["size"]) if mask else None, position=position, prep="general",
                         v_head_dim=None if dv == d else dv, sink="learned",
                         keep_first=int(mask.get("keep_first", 0)) if mask else 0, bias=True)
    parts = (("q", H * d), ("k", G * d), ("v", G * dv))
    k = f"mixer.{name}_"
    sources = {k + "qkv": _rows(p, parts), k + "qkv_bias": _rows(p, tuple((n + ".b", c) for n, c in parts)),
               k + "q_norm": (Source(p + "q.norm"),), k + "k_norm": (Source(p + "k.norm"),),
               k + "sink": (Source(p + "sink"),), k + "o": (Source(p + "o"),), k + "o_bias": (Source(p + "o.b"),)}
    return spec, sources


def _memory(cfg, m, p, name):
    d, dv, H = int(m["dim"]), int(m["vdim"]), int(m["heads"])
    spec = MatrixMemorySpec(hidden_size=cfg.width, num_heads=H, head_dim=d, v_head_dim=dv, gate_cap=float(m["gate_cap"]),
                            norm_eps=cfg.norm_eps, den_eps=1e-6)
    k = f"mixer.{name}_"
    sources = {k + "in_proj": _rows(p, (("q", H * d), ("k", H * d), ("v", H * dv), ("g", H * dv), ("i", H), ("f", H))),
               k + "gate_bias": _rows(p, (("i.b", H), ("f.b", H))), k + "norm_w": (Source(p + "norm"),),
               k + "o": (Source(p + "o"),)}
    return spec, sources


def _parallel(cfg, m, p):
    left, sources = _attention(cfg, m["left"], p + "left.", "left")
    right, more = _memory(cfg, m["right"], p + "right.", "right")
    sources.update(more)
    spec = ParallelMixerSpec(hidden_size=cfg.width, branches=(left, right),
                             scales=(float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0))),
                             names=("left", "right"))
    return spec, sources


_MIXERS = {"delta": _delta, "parallel": _parallel}


def _feed_forward(cfg, mlp, p, corrected):
    r = mlp["router"]
    E, top, ff, ident = int(r["experts"]), int(r["top"]), int(mlp["expert"]["ff"]), int(r.get("identity", 0))
    spec = MoESpec(hidden_size=cfg.width, num_experts=E, top_k=top, intermediate_size=ff, score_fn="softmax",
                   selection_bias=corrected, renormalize=False, routed_scale=1.0, activation="silu",
                   identity_experts=ident)
    w13, w2 = [], []
    for e in range(E):
        w13 += [Source(p + f"e{e}.gate", (e, (0, ff))), Source(p + f"e{e}.up", (e, (ff, ff)))]
        w2.append(Source(p + f"e{e}.down", (e,)))
    sources = {"feed_forward.gate": (Source(p + "router"),), "feed_forward.w13": tuple(w13), "feed_forward.w2": tuple(w2)}
    if corrected:
        sources["feed_forward.selection_bias"] = (Source(p + "correction"),)
    return spec, sources


def _streams(cfg, i, q, part):
    """The StreamMixSpec of sublayer q of layer i and its parameters' sources."""
    spec = StreamMixSpec(hidden_size=cfg.width, streams=cfg.streams, gated=bool(cfg.gated[i]),
                         learned=bool(cfg.learned_streams[i]))
    sources = {}
    if spec.learned:
        sources.update({f"{part}.in_w": (Source(f"l{i}.hc{q}.in"),), f"{part}.out_w": (Source(f"l{i}.hc{q}.out"),),
                        f"{part}.mix": (Source(f"l{i}.hc{q}.mix"),)})
    if spec.gated:
        sources.update({f"{part}.gate": (Source(f"l{i}.rg{q}"),), f"{part}.gate_bias": (Source(f"l{i}.rg{q}.b"),)})
    return spec, sources


def build_tedisun(cfg: TedisunConfig) -> ModelSpec:
    norm = RMSNormSpec(size=cfg.width, eps=cfg.norm_eps, offset=1.0)
    layers = []
    for i, layer in enumerate(cfg.layers):
        mixer, sources = _MIXERS[layer["type"]](cfg, layer["mixer"], f"l{i}.mix.")
        sources["mixer_norm.weight"] = (Source(f"l{i}.norm1"),)
        extra = {}
        extra["mixer_streams"], more = _streams(cfg, i, 1, "mixer_streams")
        sources.update(more)
        ff = None
        if layer.get("mlp") is not None:
            ff, more = _feed_forward(cfg, layer["mlp"], f"l{i}.mlp.", bool(cfg.corrected[i]))
            sources.update(more)
            sources["feed_forward_norm.weight"] = (Source(f"l{i}.norm2"),)
            extra["feed_forward_streams"], more = _streams(cfg, i, 2, "feed_forward_streams")
            sources.update(more)
        layers.append(LayerSpec(mixer=mixer, feed_forward=ff, mixer_norm=norm,
                                feed_forward_norm=norm if ff is not None else None, arrangement="stream_mix",
                                extra=extra, sources=sources))
    order = [ScheduleEntry(layer=i) for i in range(len(layers))]
    return ModelSpec(architecture=ARCHITECTURE, hidden_size=cfg.width, vocab_size=cfg.vocab,
                     max_position=cfg.max_position, layers=layers, order=order, final_norm=norm,
                     final_norm_source="final.norm", embed_source="embed", head_source="head" if cfg.own_head else None,
                     embed_scale=cfg.embedding_scale, logit_softcap=cfg.logit_softcap, residual_stream="float32",
                     streams=cfg.streams)


register_architecture(ARCHITECTURE, TedisunConfig, build_tedisun)
