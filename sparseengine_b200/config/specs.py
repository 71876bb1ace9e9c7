"""Typed descriptions of the parts a model is assembled from.

A model is data: a list of :class:`LayerSpec` (which mixer, feed-forward, norm and
position encoding a layer has, with every size and constant as a field) and an
execution order, a list of :class:`ScheduleEntry` that may name a layer twice or let
an entry read the cache another entry wrote.  Nothing here knows an architecture's
name; architecture builders (``sparseengine_b200.models``) turn a ``config.json``
into these records, and ``sparseengine_b200.parts`` turns the records into parts.

The reference keeps the same facts spread over ``ModelSpec``
(src/sparseengine/models/spec.py:11-211), ``RuntimeLayout``
(src/sparseengine/models/layout.py:77-357) and per-op ``*OpSpec`` records
(src/sparseengine/operators/moe_router.py:19-42, src/sparseengine/operators/moe.py:23-82).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Sequence


@dataclass(frozen=True)
class Source:
    """One checkpoint tensor that fills a slice of a parameter.

    ``index`` addresses the destination along the leading dimensions of the parameter:
    an ``int`` selects (and drops) a dimension, a ``(start, length)`` pair narrows it;
    the remaining dimensions are taken whole.
    """
    name: str
    index: tuple = ()


@dataclass(frozen=True)
class ParamSpec:
    """A parameter a part owns.

    ``dtype`` is ``"act"`` (the engine's activation dtype: bfloat16 or float32) or
    ``"float32"`` (kept in 32-bit whatever the engine dtype, e.g. router weights).
    ``init`` names the random-weights distribution: ``"matrix"`` N(0, std),
    ``"norm"`` 1 + N(0, norm_std), ``"bias"`` N(0, bias_std), ``"unit"`` sigmoid(N(0, 1)).
    """
    shape: tuple
    dtype: str = "act"
    init: str = "matrix"
    sources: tuple = ()          # tuple[Source, ...]; filled by the architecture builder


@dataclass(frozen=True)
class RotarySpec:
    kind: str = "rotary"
    rotary_dim: int = 0
    theta: float = 10000.0
    # which dims form rotated pair i: "split_half" (i, i + rotary_dim/2), "interleaved"
    # (2i, 2i+1), "interleaved_to_split_half" (reads 2i, 2i+1; writes i, i + rotary_dim/2)
    pairing: str = "split_half"
    scaling: float = 1.0          # multiplies cos and sin (beside what frequency_scaling brings)
    # the configuration's frequency-scaling entries (linear, llama3, yarn) as a sorted tuple of
    # (key, value) pairs, or None; worked into the frequency table on the host
    frequency_scaling: Optional[tuple] = None


@dataclass(frozen=True)
class RMSNormSpec:
    kind: str = "rms"
    size: int = 0
    eps: float = 1e-6
    # the stored weight w is applied as (offset + w): 1.0 for weights kept around zero.  Such a norm keeps its
    # weight in 32-bit (the sum would lose the stored digits in a 16-bit type).
    offset: float = 0.0


@dataclass(frozen=True)
class LayerNormSpec:
    """Layer norm with a weight and (``bias``) a bias: (x - mean) / sqrt(var + eps) * w + b."""
    kind: str = "layer_norm"
    size: int = 0
    eps: float = 1e-6
    bias: bool = True


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query attention over a paged key/value cache."""
    kind: str = "attention"
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 1.0
    # None | "whole_projection" (one root mean square over all heads, a weight per column) | "per_head" (one per
    # head, a weight of head_dim elements shared by the heads; needs prep="general")
    qk_norm: Optional[str] = None
    qk_norm_eps: float = 1e-6
    window: Optional[int] = None      # keys p-window+1..p; None = all keys
    position: Optional[Any] = None    # a position-encoding spec (e.g. RotarySpec)
    # "rotary": the fused norm + rotation kernel (values as wide as keys).  "general": no rotation;
    # the fields below apply, and norms and temperature are computed in 32-bit and rounded once.
    prep: str = "rotary"
    v_head_dim: Optional[int] = None  # the values' head size (None: head_dim)
    # (coef, every): the query at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1)
    q_temperature: Optional[tuple] = None
    own_kv: bool = True               # False: no key/value projections; the layer attends over another's cache
    # The fields below need prep="general", which then also rotates (``position``: split halves, no factor).
    score_softcap: Optional[float] = None   # c: the scaled score becomes c * tanh(score / c)
    # "zero": a key of score 0 that has no value joins the softmax: p_j = exp(s_j) / (1 + sum exp(s_j)).
    # "learned": the same with a learned logit per head (parameter ``sink``) in place of 0, unscaled.
    sink: Optional[str] = None
    # with a window: the first keep_first positions stay visible to every later query (at their true positions),
    # beside the window's keys
    keep_first: int = 0
    # biases on the q, k, v rows of the packed projection (parameter ``qkv_bias``) and on the output projection
    # (``o_bias``); needs prep="general"
    bias: bool = False
    # the concatenated heads are multiplied by sigmoid(W_g x) before the output projection; W_g's
    # rows follow the values' in the packed projection
    output_gate: bool = False
    # "first": this layer's values (of this step's tokens) are kept for the layers after it.
    # "blend": the values become (1 - m) v + m v_first with a learned number m, before they are cached.
    # Both kinds own the parameter ``v_mix`` (a "first" layer does not use it).
    value_mix: Optional[str] = None

    @property
    def value_dim(self) -> int:
        return self.v_head_dim or self.head_dim


@dataclass(frozen=True)
class StateSpaceSpec:
    """Selective state-space mixer (state-space duality form): per head a state of
    ``state_size x head_dim`` with a scalar decay, inputs through a short causal convolution,
    output gated and RMS-normed in ``norm_groups`` equal parts."""
    kind: str = "mamba2"
    hidden_size: int = 0
    num_heads: int = 0
    head_dim: int = 0
    state_size: int = 0
    groups: int = 1                   # heads of one group share B and C
    conv_taps: int = 4
    norm_groups: int = 1
    norm_eps: float = 1e-6


@dataclass(frozen=True)
class GatedDeltaSpec:
    """Gated delta rule: per head a state of ``head_dim x v_head_dim``; q, k, v through short causal
    convolutions.  ``decay_per="channel"``: one decay per head and key channel; the decay and the output
    gate come through low-rank projections of the given ranks, the gate is a sigmoid.
    ``decay_per="head"``: one decay per head, straight from a projection of the input (no ranks); the
    output gate is ``gate_activation`` of a full projection."""
    kind: str = "channel_delta"
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0             # q/k heads; value head h uses q/k head h // (num_heads / num_kv_heads)
    head_dim: int = 0
    v_head_dim: int = 0
    conv_taps: int = 4
    decay_rank: int = 0
    gate_rank: int = 0
    norm_eps: float = 1e-6
    unit_eps: float = 1e-6            # q and k become x / sqrt(sum(x^2) + unit_eps)
    decay_per: str = "channel"        # "channel" | "head"
    gate_activation: str = "sigmoid"  # "sigmoid" | "silu" (of the output gate)


@dataclass(frozen=True)
class MatrixMemorySpec:
    """Matrix memory with exponential gates (the mLSTM cell): per head a state ``S [head_dim, v_head_dim]``, a
    vector ``n [head_dim]`` and a running maximum ``m`` of the gates' logarithms, all starting at 0.  With
    ``i = cap tanh(a / cap)`` and ``f = logsigmoid(cap tanh(b / cap))`` (a, b: projections with bias, one per
    head): ``m' = max(f + m, i)``, ``S' = exp(f + m - m') S + exp(i - m') k v^T``, ``n'`` likewise with k alone,
    ``o = S'^T q / (max(|n' . q|, exp(-m')) + den_eps)`` with ``q`` scaled by ``head_dim ** -0.5``.  Each head's
    ``o`` is divided by its root mean square, the concatenated heads are multiplied by a weight and by
    ``sigmoid(W_g x)``, then projected."""
    kind: str = "matrix_memory"
    hidden_size: int = 0
    num_heads: int = 0
    head_dim: int = 0
    v_head_dim: int = 0
    gate_cap: float = 15.0
    norm_eps: float = 1e-6
    den_eps: float = 1e-6


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Mixers side by side on the same input: the result is ``sum_i scales[i] * branch_i(x)``.  At most one
    branch may ask for pages and at most one for a state slot."""
    kind: str = "parallel"
    hidden_size: int = 0
    branches: tuple = ()              # mixer specs
    scales: tuple = ()                # one factor per branch
    names: tuple = ()                 # a name per branch: its parameters are "<name>_<parameter>"


@dataclass(frozen=True)
class StreamMixSpec:
    """How one sublayer reads from and writes to ``streams`` copies of the residual stream
    (hyper-connections): it reads ``sum_s in[s] x_s`` and writes ``x_t <- sum_s mix[s, t] x_s + out[t] y``.
    ``gated``: ``y`` is first multiplied by ``sigmoid(W h + b)``, ``h`` being the sublayer's (normed) input.
    ``learned=False`` (one stream only): in, out and mix are 1, the plain residual sum."""
    kind: str = "stream_mix"
    hidden_size: int = 0
    streams: int = 1
    gated: bool = False
    learned: bool = True


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Softmax attention whose keys and values are up-projections of one cached latent per position.

    Queries go through a latent of their own (``q_rank``, RMS-normed); a head's query and key have
    ``head_dim`` unrotated dims followed by ``rot_dim`` rotated ones.  The key/value projection gives
    ``kv_rank`` latent dims (RMS-normed) plus ``rot_dim`` dims that form the rotated key part of every
    head; unrotated keys and values are ``W_uk c`` and ``W_uv c``.  Only the latent and the rotated key
    part are cached.  ``window``: keys p-window+1..p (None: all).  ``sink``: a learned logit per head
    that joins the softmax's denominator, unscaled, with no key or value."""
    kind: str = "latent_attention"
    hidden_size: int = 0
    num_heads: int = 0
    head_dim: int = 0                 # unrotated dims of a head's query and key
    rot_dim: int = 0                  # rotated dims of a head's query; the shared key part
    v_head_dim: int = 0
    q_rank: int = 0
    kv_rank: int = 0
    scale: float = 1.0
    window: Optional[int] = None
    sink: bool = False
    position: Optional[Any] = None    # RotarySpec over (at most) rot_dim dims, split-half pairing
    norm_eps: float = 1e-6


@dataclass(frozen=True)
class RetentionSpec:
    """Linear attention with one fixed decay per head: ``S <- decay S + k v^T``, ``o = S^T q``, no
    softmax or denominator.  q and k are rotated (``position``), k is scaled by ``head_dim ** -0.5``
    after the rotation; each head's ``o`` is divided by its root mean square (no weight), multiplied
    by ``silu(gate)`` and projected."""
    kind: str = "retention"
    hidden_size: int = 0
    num_heads: int = 0
    head_dim: int = 0
    v_head_dim: int = 0
    decays: tuple = ()                # one per head
    position: Optional[Any] = None    # RotarySpec, split-half pairing
    norm_eps: float = 1e-6


@dataclass(frozen=True)
class MoESpec:
    """Routed SwiGLU experts."""
    kind: str = "moe"
    hidden_size: int = 0
    num_experts: int = 0
    top_k: int = 0
    intermediate_size: int = 0
    # "sigmoid" | "softmax": scores over all experts.  "top_softmax": the bias is part of the logit, the
    # largest logits are chosen and their weights are the softmax among the chosen logits.
    score_fn: str = "sigmoid"
    selection_bias: bool = True       # bias added for selection only ("top_softmax": part of the logit)
    renormalize: bool = True
    routed_scale: float = 1.0
    # "silu": silu(gate) * up.  "clamped_swiglu": g * sigmoid(activation_alpha * g) * (u + 1) with
    # g = min(gate, activation_limit) and u = clamp(up, -activation_limit, activation_limit).
    activation: str = "silu"
    activation_limit: float = 0.0
    activation_alpha: float = 1.702
    # groups > 1: the experts form that many equal groups of neighbours; a group's score is the sum of
    # its two largest selection scores, and only experts of the keep_groups best groups can be chosen
    groups: int = 1
    keep_groups: int = 1
    # a DenseMLPSpec: an expert of its own sizes that every token runs; its output is added
    shared: Optional[Any] = None
    # the router has this many more outputs after the experts': "experts" without weights whose output is
    # their input; they take part in scores and selection like the others
    identity_experts: int = 0


@dataclass(frozen=True)
class DenseMLPSpec:
    """A dense gated feed-forward (one always-selected expert); activations as :class:`MoESpec`'s."""
    kind: str = "dense_mlp"
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "silu"
    activation_limit: float = 0.0
    activation_alpha: float = 1.702


@dataclass(frozen=True)
class PlainMLPSpec:
    """An ungated feed-forward: down(act(up(x)))."""
    kind: str = "plain_mlp"
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "relu2"         # "relu2" (squared relu) | "gelu_tanh" | "silu" | "relu"


@dataclass(frozen=True)
class LayerSpec:
    """One layer: its parts and the name of their arrangement in a block.

    The built-in arrangement ``pre_norm`` takes a mixer and a feed-forward between two norms.
    An arrangement with further parts (a norm after each sublayer, a second feed-forward beside
    the first, ...) finds their specs under ``extra`` by the names it gives them, builds them with
    the same registries, and lists them in its ``parts()``; their checkpoint tensors go into
    ``sources`` under "<part name>.<parameter>" like everyone's."""
    mixer: Any
    feed_forward: Any
    mixer_norm: Any
    feed_forward_norm: Any
    arrangement: str = "pre_norm"
    # "pre_norm_stream": x <- x + mixer(norm(x)), x <- x + ff(norm(x)) over a 32-bit stream; the
    # feed-forward (with its norm) may be None.
    # "post_norm": x <- norm(residual_scale * x + sublayer(x)) for each sublayer; the feed-forward
    # (with its norm) may be None
    # "stream_mix": pre-norm over several 32-bit streams; extra["mixer_streams"] and extra["feed_forward_streams"]
    # (StreamMixSpec) say how each sublayer reads and writes them; the feed-forward may be None.
    # "sublayer_norm": x <- x + norm(mixer(x)), x <- x + norm(ff(x)) over a 32-bit stream: the norms
    # sit on the sublayers' outputs and the sublayers read x itself; the feed-forward (with its
    # norm) may be None
    residual_scale: float = 1.0
    extra: dict = field(default_factory=dict)       # part name -> spec, for arrangements with more parts
    # part-local parameter name -> tuple[Source, ...]; keys are "<part>.<param>" with
    # part in {"mixer", "feed_forward", "mixer_norm", "feed_forward_norm"}.
    sources: dict = field(default_factory=dict)


@dataclass(frozen=True)
class ScheduleEntry:
    """One visit of the execution order.

    ``layer`` indexes ``ModelSpec.layers`` (weights).  ``cache`` names the cache layer
    this visit attends over, ``None`` for "a cache layer of its own".  With
    ``write_cache=False`` the visit writes nothing and only reads what the entry that
    owns ``cache`` wrote earlier in the same step (key/value sharing between layers).
    """
    layer: int
    cache: Optional[int] = None
    write_cache: bool = True
    # Before this visit the stream becomes W [x; x0], x0 being the embedding output and W the
    # model's ``reinject_source`` tensor [width, 2 width] (a looped stack takes the embedding in
    # again at the start of every pass).
    reinject: bool = False


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position: int
    layers: Sequence[LayerSpec]
    order: Sequence[ScheduleEntry]
    final_norm: Any
    final_norm_source: str = "model.norm.weight"
    final_norm_sources: Optional[dict] = None       # parameter name -> checkpoint name, for a final norm with several
    embed_source: str = "model.embed_tokens.weight"
    head_source: Optional[str] = "lm_head.weight"   # None = tied to the embedding
    embed_scale: float = 1.0                        # the embedded tokens are multiplied by this (in the activation type)
    logit_scale: float = 1.0                        # the logits are multiplied by this
    logit_softcap: Optional[float] = None           # c: logits become c * tanh(logits / c), in 32-bit
    ignored_prefixes: tuple = ()                    # checkpoint names skipped at load
    ignored_rule: Optional[Any] = None              # name -> bool: further names skipped at load
    stored_dtype: str = "bfloat16"
    # "activation": blocks carry (hidden, residual) in the activation type.  "float32": the residual
    # stream is 32-bit whatever the activation type; blocks carry (its copy in the activation type,
    # the stream), the embedding is scaled in 32-bit and the final norm reads the stream.
    residual_stream: str = "activation"
    reinject_source: Optional[str] = None           # checkpoint name of the [width, 2 width] matrix of ScheduleEntry.reinject
    streams: int = 1                                # copies of the residual stream ("stream_mix" blocks); the last norm reads their sum
