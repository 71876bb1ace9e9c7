"""Kisusun: a decoder-only design whose ``config.json`` lists its layers one by one.

The residual stream is 32-bit and the norms sit on the sublayers' outputs: ``x <- x + norm1(mixer(x))``
and, where the layer has a feed-forward, ``x <- x + norm2(ff(x))`` with RMS norms; the sublayers read
``x`` itself.  The embedding is scaled; the LM head is the embedding table, and the logits are scaled.

The mixer is grouped-query softmax attention (``parts.attention.PagedAttention``, general
preparation): RMS norms over the whole query and key projections, rotary positions on the first
``rot.dims`` dims of every head (split halves, every frequency divided by ``rot.scaling.factor``), a
score scale from the configuration, scores capped by ``c tanh(s / c)``, a sliding window, a sink of score 0
in the softmax's denominator, value heads of their own size, an output gate ``sigmoid(W_g x)`` on the
concatenated heads, and, in layers that say ``v_mix``, values blended with those of the first such
layer by a learned number before they are cached.

The feed-forward is ``dense`` (SwiGLU) or ``moe``: experts ``g sigmoid(1.702 g) (u + 1)`` with
``g = min(gate, limit)`` and ``u = clamp(up, -limit, limit)``; sigmoid router scores; experts in equal groups
of neighbours, a group scored by its two best, only the best groups open to the choice; weights are the
chosen scores times ``router.scale``, not renormalised; a shared expert of the same form is added.

Tensor names: ``embed``, ``final.norm``, ``l<i>.norm1|norm2``, ``l<i>.mix.q|k|v|g|o|q.norm|k.norm|vmix``,
``l<i>.mlp.gate|up|down`` or ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.gate|up|down`` and
``l<i>.mlp.shared.gate|up|down``.
"""
from __future__ import annotations

import re
from dataclasses import dataclass

from ..config.registry import register_architecture
from ..config.specs import (AttentionSpec, DenseMLPSpec, LayerSpec, ModelSpec, MoESpec, RMSNormSpec, RotarySpec,
                            ScheduleEntry, Source)

ARCHITECTURE = "Kisusun"
MIXER_TYPES = ("attention",)
DEFAULT_MAX_POSITION = 1 << 20      # the design has no position table; the cache manager wants a bound
EXPERT_SLOPE = 1.702                # the experts' gate is g * sigmoid(EXPERT_SLOPE * g)


@dataclass(frozen=True)
class KisusunConfig:
    vocab: int
    width: int
    layers: tuple                      # of dicts {"type", "mixer", "mlp"} as in config.json (validated)
    norm_eps: float
    embed_scale: float
    logit_scale: float
    max_position: int

    @classmethod
    def from_dict(cls, raw: dict) -> "KisusunConfig":
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
            missing = [k for k in ("heads", "dim") if m.get(k) is None]
            if missing:
                problems.append(f"layer {i} ({kind}): missing mixer keys {missing}")
                continue
            if int(m["heads"]) % int(m.get("kv_heads") or m["heads"]):
                problems.append(f"layer {i}: 'heads' must be a multiple of 'kv_heads'")
            rot = m.get("rot")
            if rot is not None and (rot.get("dims") is None or rot.get("base") is None):
                problems.append(f"layer {i}: 'rot' needs 'dims' and 'base'")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") == "dense":
                    if mlp.get("ff") is None:
                        problems.append(f"layer {i}: a dense feed-forward needs 'ff'")
                elif mlp.get("kind") == "moe":
                    expert, router = mlp.get("expert") or {}, mlp.get("router") or {}
                    if expert.get("ff") is None or expert.get("limit") is None or router.get("experts") is None \
                            or router.get("top") is None:
                        problems.append(f"layer {i}: a moe feed-forward needs expert.ff, expert.limit, router.experts "
                                        "and router.top")
                    shared = mlp.get("shared")
                    if shared is not None and (shared.get("ff") is None or shared.get("limit") is None):
                        problems.append(f"layer {i}: a shared expert needs 'ff' and 'limit'")
                else:
                    problems.append(f"layer {i}: the feed-forward's kind must be 'dense' or 'moe', or the entry null")
        if problems:
            raise ValueError("Kisusun config.json cannot be used: " + "; ".join(problems))
        return cls(vocab=int(raw["vocab"]), width=int(raw["width"]), layers=tuple(layers),
                   norm_eps=float((raw.get("norm") or {}).get("eps", 1e-6)),
                   embed_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
                   logit_scale=float(raw.get("logit_scale", 1.0)),
                   max_position=int(raw.get("max_position", DEFAULT_MAX_POSITION)))


def _rotary(m):
    rot = m.get("rot")
    if rot is None or int(rot["dims"]) == 0:
        return None
    factor = (rot.get("scaling") or {}).get("factor")
    scaling = None
    if factor is not None and float(factor) != 1.0:
        scaling = (("factor", float(factor)), ("rope_type", "linear"))
    return RotarySpec(rotary_dim=int(rot["dims"]), theta=float(rot["base"]), pairing="split_half",
                      frequency_scaling=scaling)


def _attention(cfg, m, p, mix_role):
    H, d = int(m["heads"]), int(m["dim"])
    G, dv = int(m.get("kv_heads") or H), int(m.get("vdim") or d)
    window = (m.get("mask") or {}).get("size")
    cap = m.get("softcap")
    spec = AttentionSpec(hidden_size=cfg.width, num_heads=H, num_kv_heads=G, head_dim=d,
                         scale=float(m["scale"]) if m.get("scale") is not None else d ** -0.5,
                         qk_norm="whole_projection", qk_norm_eps=cfg.norm_eps, window=int(window) if window else None,
                         position=_rotary(m), prep="general", v_head_dim=dv,
                         score_softcap=float(cap) if cap else None, sink="zero", output_gate=True, value_mix=mix_role)
    rows, at = [], 0
    for name, n in (("q", H * d), ("k", G * d), ("v", G * dv), ("g", H * dv)):
        rows.append(Source(p + name, ((at, n),)))
        at += n
    sources = {"mixer.qkv": tuple(rows), "mixer.q_norm": (Source(p + "q.norm"),), "mixer.k_norm": (Source(p + "k.norm"),),
               "mixer.o": (Source(p + "o"),)}
    if mix_role is not None:
        sources["mixer.v_mix"] = (Source(p + "vmix"),)
    return spec, sources


def _expert_sources(p, ff, e=0):
    return ((Source(p + "gate", (e, (0, ff))), Source(p + "up", (e, (ff, ff)))), (Source(p + "down", (e,)),))


def _feed_forward(cfg, mlp, p):
    if mlp["kind"] == "dense":
        ff = int(mlp["ff"])
        w13, w2 = _expert_sources(p, ff)
        return (DenseMLPSpec(hidden_size=cfg.width, intermediate_size=ff, activation="silu"),
                {"feed_forward.w13": w13, "feed_forward.w2": w2})
    router, expert = mlp["router"], mlp["expert"]
    E, top, ff = int(router["experts"]), int(router["top"]), int(expert["ff"])
    groups = router.get("groups") or {}
    shared = sources_shared = None
    if mlp.get("shared") is not None:
        sff = int(mlp["shared"]["ff"])
        shared = DenseMLPSpec(hidden_size=cfg.width, intermediate_size=sff, activation="clamped_swiglu",
                              activation_limit=float(mlp["shared"]["limit"]), activation_alpha=EXPERT_SLOPE)
        sources_shared = _expert_sources(p + "shared.", sff)
    spec = MoESpec(hidden_size=cfg.width, num_experts=E, top_k=top, intermediate_size=ff, score_fn="sigmoid",
                   selection_bias=False, renormalize=False, routed_scale=float(router.get("scale", 1.0)),
                   activation="clamped_swiglu", activation_limit=float(expert["limit"]), activation_alpha=EXPERT_SLOPE,
                   groups=int(groups.get("count", 1)), keep_groups=int(groups.get("keep", groups.get("count", 1))),
                   shared=shared)
    w13, w2 = [], []
    for e in range(E):
        a, b = _expert_sources(p + f"e{e}.", ff, e)
        w13 += a
        w2 += b
    sources = {"feed_forward.gate": (Source(p + "router"),), "feed_forward.w13": tuple(w13), "feed_forward.w2": tuple(w2)}
    if shared is not None:
        sources["feed_forward.shared_w13"], sources["feed_forward.shared_w2"] = sources_shared
    return spec, sources


_UNUSED_BLEND_WEIGHT = re.compile(r"l\d+\.mix\.vmix")


def build_kisusun(cfg: KisusunConfig) -> ModelSpec:
    norm = RMSNormSpec(size=cfg.width, eps=cfg.norm_eps)
    layers = []
    mixing_seen = False
    for i, layer in enumerate(cfg.layers):
        role = None
        if layer["mixer"].get("v_mix"):
            role = "blend" if mixing_seen else "first"
            mixing_seen = True
        mixer, sources = _attention(cfg, layer["mixer"], f"l{i}.mix.", role)
        sources["mixer_norm.weight"] = (Source(f"l{i}.norm1"),)
        ff = None
        if layer.get("mlp") is not None:
            ff, more = _feed_forward(cfg, layer["mlp"], f"l{i}.mlp.")
            sources.update(more)
            sources["feed_forward_norm.weight"] = (Source(f"l{i}.norm2"),)
        layers.append(LayerSpec(mixer=mixer, feed_forward=ff, mixer_norm=norm,
                                feed_forward_norm=norm if ff is not None else None, arrangement="sublayer_norm",
                                sources=sources))
    return ModelSpec(architecture=ARCHITECTURE, hidden_size=cfg.width, vocab_size=cfg.vocab,
                     max_position=cfg.max_position, layers=layers,
                     order=[ScheduleEntry(layer=i) for i in range(len(layers))], final_norm=norm,
                     final_norm_source="final.norm", embed_source="embed", head_source=None,
                     embed_scale=cfg.embed_scale, logit_scale=cfg.logit_scale, residual_stream="float32",
                     # a blending weight stored for a layer that does not blend is not read
                     ignored_rule=lambda name: bool(_UNUSED_BLEND_WEIGHT.fullmatch(name)))


register_architecture(ARCHITECTURE, KisusunConfig, build_kisusun)
