"""A model assembled from a :class:`ModelSpec`: embedding, blocks in their execution
order, final norm, LM head.  Architecture-agnostic.

The loop mirrors src/sparseengine/models/qwen3.py:291-328 (embed → layers → final fused
add+norm) and src/sparseengine/layers/embed_head.py:75-84 (LM head on selected rows
only); here the rows are whatever the caller asks for, and the final norm also runs on
those rows only.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..config.specs import ModelSpec, ParamSpec, Source
from ..csrc import ops
from ..parts.base import KVRequest, StateRequest, StepContext, make_norm
from ..parts.block import (PostNormBlock, PreNormBlock, PreNormStreamBlock, StreamMixBlock, SublayerNormBlock,
                           make_block)
from ..parts.linear import linear, linear32
from ..parts.norm import RMSNorm


@dataclass
class Param:
    """A parameter with its owner and the checkpoint tensors that fill it."""
    owner: object
    name: str            # attribute on the owner
    qualified: str       # unique name for messages, e.g. "layers.3.mixer.qkv"
    spec: ParamSpec
    sources: tuple       # tuple[Source, ...]
    tensor: Optional[torch.Tensor] = None


@dataclass(frozen=True)
class EntryCache:
    """Where a schedule entry keeps keys/values and state."""
    group: Optional[int]         # index into CacheLayout.groups
    cache_layer: Optional[int]   # layer index inside the group's storage
    write: bool
    state: Optional[int]         # index into CacheLayout.states


@dataclass(frozen=True)
class CacheLayout:
    groups: tuple        # tuple[(KVRequest, number of cache layers)]
    states: tuple        # tuple[StateRequest], one per schedule entry that has state
    entries: tuple       # tuple[EntryCache], one per schedule entry


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise TypeError(f"engine dtype must be float32 or bfloat16, got {dtype}")
        self.spec = spec
        self.dtype = dtype
        self.blocks = [make_block(ls, dtype) for ls in spec.layers]
        self.final_norm = make_norm(spec.final_norm, dtype)
        self.embed = None
        self.head = None
        self.profile = None     # a dict: CUDA-event pairs per part are collected in it (a debugging aid)
        self.stream_taps = None  # a list: receives a copy of the residual stream after every schedule entry (a debugging aid)
        if spec.residual_stream not in ("activation", "float32"):
            raise ValueError(f"residual_stream {spec.residual_stream!r} is not known ('activation' or 'float32')")
        # blocks over the 32-bit stream that carry (output not yet added, stream)
        self.pending_stream = any(isinstance(b, PreNormStreamBlock) for b in self.blocks)
        if self.pending_stream and not (all(isinstance(b, PreNormStreamBlock) for b in self.blocks)
                                        and spec.residual_stream == "float32"
                                        and hasattr(self.final_norm, "forward_stream")):
            raise ValueError("pre_norm_stream blocks need residual_stream='float32', a final norm with forward_stream, "
                             "and no other arrangement beside them")
        # blocks over several 32-bit streams that carry (result not yet written, streams)
        self.multi_stream = any(isinstance(b, StreamMixBlock) for b in self.blocks)
        if self.multi_stream and not (all(isinstance(b, StreamMixBlock) for b in self.blocks)
                                      and spec.residual_stream == "float32" and isinstance(self.final_norm, RMSNorm)
                                      and spec.streams >= 1
                                      and all(b.mixer_streams.spec.streams == spec.streams for b in self.blocks)):
            raise ValueError("stream_mix blocks need residual_stream='float32', ModelSpec.streams equal to every block's, "
                             "an RMS final norm with a 32-bit weight, and no other arrangement beside them")
        self.reinject = None
        if any(e.reinject for e in spec.order) and not (self.pending_stream and spec.reinject_source):
            raise ValueError("ScheduleEntry.reinject needs pre_norm_stream blocks and ModelSpec.reinject_source")
        for i, e in enumerate(spec.order):
            if not 0 <= e.layer < len(self.blocks):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, the model has {len(self.blocks)}")
            if e.cache is not None and not 0 <= e.cache < i:
                raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache}, which is not earlier")
        self.layout = self._cache_layout()

    # ---- parameters --------------------------------------------------------------------
    def params(self) -> list[Param]:
        s = self.spec
        out = [Param(self, "embed", "embed", ParamSpec((s.vocab_size, s.hidden_size)), (Source(s.embed_source),))]
        if s.head_source is not None:
            out.append(Param(self, "head", "head", ParamSpec((s.vocab_size, s.hidden_size)),
                             (Source(s.head_source),)))
        if s.reinject_source is not None:
            out.append(Param(self, "reinject", "reinject", ParamSpec((s.hidden_size, 2 * s.hidden_size)),
                             (Source(s.reinject_source),)))
        for name, p in self.final_norm.parameters().items():
            source = (s.final_norm_sources or {}).get(name, s.final_norm_source)
            out.append(Param(self.final_norm, name, f"final_norm.{name}", p, (Source(source),)))
        for i, (block, ls) in enumerate(zip(self.blocks, s.layers)):
            for part_name, part in block.parts().items():
                for name, p in part.parameters().items():
                    key = f"{part_name}.{name}"
                    if key not in ls.sources:
                        raise ValueError(f"layer {i}: no checkpoint source given for parameter {key!r}")
                    out.append(Param(part, name, f"layers.{i}.{key}", p, tuple(ls.sources[key])))
        return out

    def bind(self, params: list[Param]) -> None:
        by_owner: dict = {}
        for p in params:
            if p.tensor is None:
                raise ValueError(f"parameter {p.qualified} was not loaded")
            by_owner.setdefault(id(p.owner), (p.owner, {}))[1][p.name] = p.tensor
        for owner, tensors in by_owner.values():
            if owner is self:
                for n, t in tensors.items():
                    setattr(self, n, t)
            else:
                owner.bind(tensors)
        if self.spec.head_source is None:
            self.head = self.embed
        if self.reinject is not None:       # W [x; x0] = W_x x + W_0 x0: the second term is the same for every pass of a step
            width = self.spec.hidden_size
            self._reinject_x = self.reinject[:, :width].contiguous()
            self._reinject_0 = self.reinject[:, width:].contiguous()

    def param_dtype(self, p: ParamSpec) -> torch.dtype:
        return torch.float32 if p.dtype == "float32" else self.dtype

    # ---- cache needs -------------------------------------------------------------------
    def _cache_layout(self) -> CacheLayout:
        groups: list = []          # [KVRequest, count]
        states: list = []
        entries: list = []
        for e in self.spec.order:
            mixer = self.blocks[e.layer].mixer
            kv = mixer.kv_request()
            st = mixer.state_request()
            group = layer = None
            if kv is not None:
                if e.cache is not None:
                    owner = entries[e.cache]
                    if owner.group is None or groups[owner.group][0] != kv:
                        raise ValueError("a schedule entry can only share a cache of the same shape and window")
                    group, layer = owner.group, owner.cache_layer
                else:
                    for gi, (req, _) in enumerate(groups):
                        if req == kv:
                            group = gi
                            break
                    else:
                        groups.append([kv, 0])
                        group = len(groups) - 1
                    layer = groups[group][1]
                    groups[group][1] += 1
            state = None
            if st is not None:
                states.append(st)
                state = len(states) - 1
            write = e.write_cache and e.cache is None
            entries.append(EntryCache(group, layer, write if kv is not None else False, state))
        return CacheLayout(tuple((g[0], g[1]) for g in groups), tuple(states), tuple(entries))

    def _timed_block(self, block, hidden, residual, step, slot):
        """The pre-norm block part by part with a CUDA event pair around each part."""
        def timed(name, fn, *a):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn(*a)
            e1.record()
            self.profile.setdefault(name, []).append((e0, e1))
            return out
        if isinstance(block, StreamMixBlock):
            return block.forward(hidden, residual, step, slot, timed=timed)
        if isinstance(block, PostNormBlock):
            y = timed("mixer." + block.mixer.spec.kind, block.mixer.forward, hidden, step, slot)
            hidden, residual = timed("mixer_norm", block.mixer_norm.forward_stream, residual, y, block.alpha)
            if block.feed_forward_norm is not None:
                y = timed("feed_forward", block.feed_forward.forward, hidden, step) if block.feed_forward is not None else None
                hidden, residual = timed("feed_forward_norm", block.feed_forward_norm.forward_stream, residual, y, block.alpha)
            return hidden, residual
        if isinstance(block, SublayerNormBlock):
            y = timed("mixer." + block.mixer.spec.kind, block.mixer.forward, hidden, step, slot)
            hidden, residual = timed("mixer_norm", block.mixer_norm.forward_into_stream, residual, y)
            if block.feed_forward is not None:
                y = timed("feed_forward." + block.feed_forward.spec.kind, block.feed_forward.forward, hidden, step)
                hidden, residual = timed("feed_forward_norm", block.feed_forward_norm.forward_into_stream, residual, y)
            return hidden, residual
        if isinstance(block, PreNormStreamBlock):
            x, residual = timed("mixer_norm", block.mixer_norm.forward_stream, residual, hidden)
            hidden = timed("mixer." + block.mixer.spec.kind, block.mixer.forward, x, step, slot)
            if block.feed_forward is not None:
                x, residual = timed("feed_forward_norm", block.feed_forward_norm.forward_stream, residual, hidden)
                hidden = timed("feed_forward." + block.feed_forward.spec.kind, block.feed_forward.forward, x, step)
            return hidden, residual
        if not isinstance(block, PreNormBlock):
            return timed("block", block.forward, hidden, residual, step, slot)
        x, residual = timed("mixer_norm", block.mixer_norm.forward, hidden, residual)
        hidden = timed("mixer", block.mixer.forward, x, step, slot)
        x, residual = timed("feed_forward_norm", block.feed_forward_norm.forward, hidden, residual)
        hidden = timed("feed_forward", block.feed_forward.forward, x, step)
        return hidden, residual

    # ---- forward -----------------------------------------------------------------------
    def forward(self, step: StepContext, slots: list, want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Run the step's tokens through every schedule entry; return logits
        ``[len(want_rows), vocab]`` in the activation dtype, or ``None`` if no row is wanted."""
        s = self.spec
        stream32 = s.residual_stream == "float32"
        hidden = torch.empty(step.num_tokens, s.hidden_size, dtype=self.dtype, device=step.token_ids.device)
        pending_stream = self.pending_stream
        x0 = x0_term = None
        if self.multi_stream:
            # (result not yet written, streams [tokens, S, width]): every stream starts as the scaled embedding
            residual = torch.empty(step.num_tokens, s.streams, s.hidden_size, dtype=torch.float32, device=hidden.device)
            ops.stream_embed(self.embed, step.token_ids, residual, scale=s.embed_scale)
            hidden = None
        elif pending_stream:
            # (output not yet added, 32-bit stream); `hidden` keeps the embedding output for the re-injections
            residual = torch.empty(hidden.shape, dtype=torch.float32, device=hidden.device)
            ops.embed_stream(self.embed, step.token_ids, residual, hidden if self.dtype != torch.float32 else None,
                             scale=s.embed_scale)
            if self.reinject is not None:
                x0 = hidden if self.dtype != torch.float32 else residual.clone()
            hidden = None
        elif stream32:
            # the stream is 32-bit whatever the activation type; `hidden` is its copy for the matrix products
            residual = hidden if self.dtype == torch.float32 else torch.empty(hidden.shape, dtype=torch.float32,
                                                                              device=hidden.device)
            ops.embed_stream(self.embed, step.token_ids, residual, None if residual is hidden else hidden,
                             scale=s.embed_scale)
        else:
            ops.embed_gather(self.embed, step.token_ids, hidden)
            if s.embed_scale != 1.0:
                hidden.mul_(s.embed_scale)
            residual = None
        for entry, slot in zip(s.order, slots):
            block = self.blocks[entry.layer]
            if entry.reinject:
                # the stream becomes W_x x + W_0 x0 (32-bit sums; x rounded to the activation type for the product)
                x = torch.empty(residual.shape, dtype=self.dtype, device=residual.device)
                ops.add_rmsnorm_stream(residual, hidden, None, 0.0, out_act=x)
                if x0_term is None:
                    x0_term = linear32(x0, self._reinject_0)
                residual = linear32(x, self._reinject_x).add_(x0_term)
                hidden = None
            if self.profile is None:
                hidden, residual = block.forward(hidden, residual, step, slot)
            else:
                hidden, residual = self._timed_block(block, hidden, residual, step, slot)
            if self.stream_taps is not None and self.multi_stream:
                both = residual.clone()          # the streams with the result they have not taken in yet, as one
                ops.stream_mix(both, write=hidden[0].write_args(hidden[1], hidden[2]), dtype=self.dtype)
                self.stream_taps.append(ops.stream_sum(both, torch.empty(both.shape[0], both.shape[2], dtype=torch.float32,
                                                                         device=both.device)))
            elif self.stream_taps is not None:
                tap = (residual if stream32 else hidden).float().clone()
                if pending_stream and hidden is not None:
                    tap += hidden.float()
                self.stream_taps.append(tap)
        if want_rows is None or want_rows.numel() == 0:
            return None
        n = want_rows.numel()
        if self.multi_stream:
            # the wanted rows of the streams and of what they have not taken in yet; the last norm reads their sum
            r = torch.empty(n, s.streams * s.hidden_size, dtype=torch.float32, device=residual.device)
            ops.gather_rows(residual.view(step.num_tokens, -1), want_rows, r)
            mix, y, gate = hidden
            yr = torch.empty(n, s.hidden_size, dtype=self.dtype, device=r.device)
            ops.gather_rows(y, want_rows, yr)
            gr = None
            if gate is not None:
                gr = torch.empty(n, s.hidden_size, dtype=self.dtype, device=r.device)
                ops.gather_rows(gate, want_rows, gr)
            h = torch.empty(n, s.hidden_size, dtype=self.dtype, device=r.device)
            ops.stream_mix(r.view(n, s.streams, s.hidden_size), write=mix.write_args(yr, gr),
                           read=(None, self.final_norm.weight, self.final_norm.spec.eps, h), dtype=self.dtype, store=False)
        elif pending_stream:  # the wanted rows of the stream and of what it has not taken in yet
            r = torch.empty(n, s.hidden_size, dtype=torch.float32, device=residual.device)
            ops.gather_rows(residual, want_rows, r)
            p = None
            if hidden is not None:
                p = torch.empty(n, s.hidden_size, dtype=self.dtype, device=residual.device)
                ops.gather_rows(hidden, want_rows, p)
            h, _ = self.final_norm.forward_stream(r, p)
        elif stream32:      # the final norm reads the wanted rows of the stream
            r = torch.empty(n, s.hidden_size, dtype=torch.float32, device=hidden.device)
            ops.gather_rows(residual, want_rows, r)
            # a norm that reads the 32-bit stream and answers in the activation type
            h, _ = self.final_norm.forward_stream(r) if isinstance(self.final_norm, RMSNorm) else self.final_norm.forward(r)
        else:
            h = torch.empty(n, s.hidden_size, dtype=self.dtype, device=hidden.device)
            ops.gather_rows(hidden, want_rows, h)
            if residual is not None:
                r = torch.empty_like(h)
                ops.gather_rows(residual, want_rows, r)
                h, _ = self.final_norm.forward(h, r)
            else:
                h, _ = self.final_norm.forward(h)
        logits = linear(h, self.head)
        if s.logit_scale != 1.0:
            logits.mul_(float(s.logit_scale))
        if s.logit_softcap is not None:
            ops.softcap_(logits, float(s.logit_softcap))
        return logits
