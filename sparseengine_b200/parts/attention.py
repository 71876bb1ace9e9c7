"""Grouped-query attention over the paged cache.

qkv projection → (optional) whole-projection QK RMSNorm → position encoding → K/V into
their page → attention over the request's pages → output projection.  Order of effects
as in the reference (src/sparseengine/models/minimax_m2.py:334-359): this step's keys are
written before attention reads the cache.

The general preparation (``prep="general"``) adds, each by a field of the spec: values of a head
size of their own, a query temperature, layers without keys of their own, a cap on the scores,
a sink of score 0 or of a learned score per head in the softmax, an output gate, values blended with
those of an earlier layer, norms per head, biases on the projections, and first positions that stay
visible beside a window.  The blended values are what is cached; the earlier layer's values of this step's tokens
travel from layer to layer in the step's scratch (``StepContext.extras``), so nothing of them
is kept between steps.
"""
from __future__ import annotations

import torch

from ..config.specs import ParamSpec
from ..csrc import ops
from .base import KVRequest, Mixer, make_position, register_mixer
from .linear import linear
from .position import RotaryArgs, as_rotary_args


class PagedAttention(Mixer):
    graph_safe = True
    # a step's entries are a grid dimension of the prompt-portion kernels
    max_step_entries = ops.LIMITS["grid_dim_yz"]

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        s = spec
        if s.num_heads <= 0 or s.num_kv_heads <= 0 or s.num_heads % s.num_kv_heads:
            raise ValueError("num_heads must be a positive multiple of num_kv_heads")
        if s.prep not in ("rotary", "general"):
            raise ValueError(f"attention prep {s.prep!r} is not known ('rotary' or 'general')")
        self.general = s.prep == "general"
        # the parameter that projects the mixer's input (a mixer of mixers may stack it with its neighbours' and
        # hand `forward` the product's columns as `proj`); the rotary preparation reads a matrix of its own
        self.input_projection = "qkv" if self.general else None
        if self.general:
            # no rotation; any head sizes the plain kernels take
            if not (0 < s.head_dim <= ops.LIMITS["attention_max_head_dim"]
                    and 0 < s.value_dim <= ops.LIMITS["attention_max_head_dim"]):
                raise ValueError(f"head sizes {s.head_dim} / {s.value_dim} are not supported (1 to "
                                 f"{ops.LIMITS['attention_max_head_dim']})")
            if s.position is not None and getattr(s.position, "pairing", "split_half") != "split_half":
                raise ValueError("the general preparation rotates split halves only")
            if s.q_temperature is not None and not (len(s.q_temperature) == 2 and int(s.q_temperature[1]) > 0):
                raise ValueError("q_temperature is (coef, every) with every > 0")
        elif (s.v_head_dim not in (None, s.head_dim) or s.q_temperature is not None or not s.own_kv
              or s.score_softcap is not None or s.sink is not None or s.output_gate or s.value_mix is not None
              or s.bias or s.keep_first or s.qk_norm == "per_head"):
            raise ValueError("v_head_dim, q_temperature, own_kv=False, score_softcap, sink, output_gate, value_mix, "
                             "bias, keep_first and per-head norms need prep='general'")
        elif s.head_dim <= 0 or s.head_dim % 16 or s.head_dim > ops.LIMITS["attention_max_head_dim"]:
            raise ValueError(f"head_dim {s.head_dim} is not supported (multiples of 16 up to "
                             f"{ops.LIMITS['attention_max_head_dim']})")
        if s.num_heads > ops.LIMITS["grid_dim_yz"]:
            raise ValueError(f"{s.num_heads} query heads are not supported (at most {ops.LIMITS['grid_dim_yz']}: "
                             "heads are a grid dimension of the attention kernels)")
        if s.qk_norm not in (None, "whole_projection", "per_head"):
            raise ValueError(f"qk_norm {s.qk_norm!r} is not supported (None, 'whole_projection' or 'per_head')")
        if s.keep_first < 0 or (s.keep_first and s.window is None):
            raise ValueError("keep_first is a count of first positions that stay visible beside a window")
        if s.bias and (s.output_gate or not s.own_kv):
            raise ValueError("biases go with projections of q, k and v alone")
        if s.window is not None and s.window <= 0:
            raise ValueError("window must be positive (None: all keys)")
        if s.score_softcap is not None and not s.score_softcap > 0:
            raise ValueError("score_softcap must be positive (None: no cap)")
        if s.sink not in (None, "zero", "learned"):
            raise ValueError(f"sink {s.sink!r} is not known (None, 'zero' or 'learned')")
        if s.value_mix not in (None, "first", "blend"):
            raise ValueError(f"value_mix {s.value_mix!r} is not known (None, 'first' or 'blend')")
        if s.value_mix is not None and not s.own_kv:
            raise ValueError("value_mix needs values of the layer's own")
        self.position = make_position(s.position, dtype) if s.position is not None else None
        rot = getattr(s.position, "rotary_dim", 0) if s.position is not None else 0
        if rot > s.head_dim:
            raise ValueError(f"the position encoding rotates {rot} dims, a head has {s.head_dim}")
        self.q_norm = self.k_norm = self.v_mix = self.qkv_bias = self.o_bias = self.sink = None
        # True: whoever combines this mixer's output with others adds `o_bias` (see `output_bias`)
        self.defer_output_bias = False

    def parameters(self):
        s = self.spec
        q, kv = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        rows = q + (kv + s.num_kv_heads * s.value_dim if s.own_kv else 0)
        if s.output_gate:
            rows += s.num_heads * s.value_dim
        out = {"qkv": ParamSpec((rows, s.hidden_size)), "o": ParamSpec((s.hidden_size, s.num_heads * s.value_dim))}
        if s.value_mix is not None:
            out["v_mix"] = ParamSpec((), "float32", "unit")
        if s.qk_norm is not None:
            per_head = s.qk_norm == "per_head"      # one weight of head_dim elements for all heads
            out["q_norm"] = ParamSpec((s.head_dim if per_head else q,), "act", "norm")
            if s.own_kv:
                out["k_norm"] = ParamSpec((s.head_dim if per_head else kv,), "act", "norm")
        if s.bias:
            out["qkv_bias"] = ParamSpec((rows,), "float32", "bias")
            out["o_bias"] = ParamSpec((s.hidden_size,), "float32", "bias")
        if s.sink == "learned":
            out["sink"] = ParamSpec((s.num_heads,), "float32", "bias")
        return out

    def kv_request(self):
        s = self.spec
        return KVRequest(s.num_kv_heads, s.head_dim, s.window, None if s.value_dim == s.head_dim else s.value_dim,
                         keep_first=int(s.keep_first) if s.window is not None else 0)

    def output_bias(self):
        """The output projection's bias (32-bit), for a caller that has set ``defer_output_bias``."""
        return self.o_bias

    VALUE_MIX_KEY = "attention.value_mix.first"     # in StepContext.extras: the kept values [tokens, kv heads * value_dim]

    def forward_general(self, x, step, slot, proj=None):
        """Whole-projection norms, rotation, query temperature, value blending and the page writes in
        one kernel (32-bit, rounded once); a layer without keys of its own only prepares its queries.
        ``proj``: the input's projection if the caller has computed it (a view with a row pitch)."""
        s = self.spec
        tokens = x.shape[0]
        if proj is None:
            proj = linear(x, self.qkv)
        q_cols, kv_cols = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        v_cols = s.num_kv_heads * s.value_dim
        inv_freq, rotary_dim = None, 0
        if self.position is not None:
            rope = as_rotary_args(self.position.kernel_args(x.device))
            if rope.scale != 1.0 or rope.pairing != "split_half":
                raise ValueError("the general preparation rotates split halves without a factor on cos and sin")
            inv_freq, rotary_dim = rope.inv_freq, rope.rotary_dim
        v_first = None
        if s.value_mix is not None:
            kept = step.extras.get(self.VALUE_MIX_KEY)
            if s.value_mix == "first" or kept is None:
                # the view keeps the projection alive for the layers that follow in this step
                step.extras[self.VALUE_MIX_KEY] = proj[:, q_cols + kv_cols:q_cols + kv_cols + v_cols]
            else:
                v_first = kept
        q = torch.empty(tokens, q_cols, dtype=x.dtype, device=x.device)
        writes = s.own_kv and slot.write_cache
        ops.qk_prep_general(proj, self.q_norm, self.k_norm if s.own_kv else None, step.positions, step.token_seq,
                            step.seq_rows, slot.table, slot.kv, q, num_heads=s.num_heads, num_kv_heads=s.num_kv_heads,
                            head_dim=s.head_dim, v_head_dim=s.value_dim, eps=s.qk_norm_eps, page_size=slot.page_size,
                            has_kv=writes, temperature=s.q_temperature, inv_freq=inv_freq, rotary_dim=rotary_dim,
                            v_first=v_first, v_mix=self.v_mix if v_first is not None else None, bias=self.qkv_bias,
                            per_head=s.qk_norm == "per_head")
        attn = torch.empty(tokens, s.num_heads * s.value_dim, dtype=x.dtype, device=x.device)
        gate = None
        if s.output_gate:
            g0 = q_cols + (kv_cols + v_cols if s.own_kv else 0)
            gate = proj[:, g0:g0 + s.num_heads * s.value_dim]
        # the kernel before the attention is the one that wrote q and this step's keys; it waited for the
        # projection (whose columns the gate is), and the step's inputs are older than both
        self.attend(q, attn, step, slot, after_qk_prep=True, gate=gate)
        y = linear(attn, self.o)
        if self.o_bias is not None and not self.defer_output_bias:
            y += self.o_bias.to(y.dtype) if y.dtype != torch.float32 else self.o_bias
        return y

    def forward(self, x, step, slot, proj=None):
        if self.general:
            return self.forward_general(x, step, slot, proj)
        if proj is not None:
            raise ValueError("a projection computed by the caller needs prep='general'")
        s = self.spec
        tokens = x.shape[0]
        # the position part first: whatever it launches to make its table then lies before the
        # projection, and q/k preparation, which starts as the projection's dependent, may read the
        # table while the projection still runs
        rope = (as_rotary_args(self.position.kernel_args(x.device)) if self.position is not None
                else RotaryArgs(None, 0))
        qkv = linear(x, self.qkv)
        q = torch.empty(tokens, s.num_heads * s.head_dim, dtype=x.dtype, device=x.device)
        ops.qk_prep(qkv, self.q_norm, self.k_norm, rope.inv_freq, step.positions, step.token_seq, step.seq_rows,
                    slot.table, slot.kv, q, num_heads=s.num_heads, num_kv_heads=s.num_kv_heads,
                    head_dim=s.head_dim, rotary_dim=rope.rotary_dim, eps=s.qk_norm_eps, rope_scale=rope.scale,
                    page_size=slot.page_size, write_cache=slot.write_cache, pairing=rope.pairing,
                    step_inputs_settled=True)       # the projection before it does not write the positions
        attn = torch.empty_like(q)
        self.attend(q, attn, step, slot, after_qk_prep=True)
        return linear(attn, self.o)

    # The split-key kernel (one CTA per token, KV head and key split) reads a request's keys once
    # per token, the prompt-portion kernels once per 256 (token, head) rows but without splitting
    # the keys.  So portions go to the latter: steps of more than `decode_kernel_max_tokens`
    # tokens, and smaller steps whose longest entry has at least `portion_min_tokens` tokens and
    # that average at least `portion_min_average` tokens per entry (measured at M2 sizes: a
    # 512-token portion after an 8,192-token prefix takes 1.39 ms per layer instead of 3.79, a
    # 32-token one 0.87 instead of 1.08; eight decoding requests beside a 64-token portion 0.86
    # instead of 0.91).  The three numbers are defaults measured at those sizes on a B200; the
    # engine option ``kernel_tuning`` sets them per engine (results do not depend on them).
    decode_kernel_max_tokens = 512
    portion_min_tokens = 16
    portion_min_average = 8

    def takes_portion_kernel(self, step) -> bool:
        if step.num_tokens > self.decode_kernel_max_tokens:
            return True
        return (step.max_q_len >= self.portion_min_tokens
                and step.num_tokens >= self.portion_min_average * step.num_seqs)
    use_tensor_cores = None      # False: always the plain kernel

    def attend(self, q, out, step, slot, after_qk_prep=False, gate=None):
        """``after_qk_prep``: the kernel launched last is the one that wrote this step's keys and
        ``q``; the split-key kernel then looks its place in the block table up while it still runs.
        ``gate``: the output gate's projection (a view with a row pitch), or None."""
        s = self.spec
        sink = self.sink if s.sink == "learned" else s.sink == "zero"
        options = dict(v_head_dim=s.value_dim, softcap=s.score_softcap, sink=sink, gate=gate, keep_first=s.keep_first)
        if (self.use_tensor_cores is not False and q.dtype == torch.bfloat16
                and ops.attn_decode_supported(s.head_dim, s.num_heads, s.num_kv_heads)
                and ops.attn_decode_value_dim_supported(s.value_dim)):
            if not self.takes_portion_kernel(step):
                max_keys = step.max_kv_len if s.window is None else min(step.max_kv_len, s.window + s.keep_first)
                ops.attn_decode(q, slot.kv, slot.table, step.seq_rows, step.token_seq, step.positions, out,
                                num_heads=s.num_heads, num_kv_heads=s.num_kv_heads, head_dim=s.head_dim,
                                page_size=slot.page_size, scale=s.scale, window=s.window, max_keys=max_keys,
                                step_inputs_settled=after_qk_prep, **options)
            else:
                # prompt portions: tcgen05 + tensor memory for head size 128 (values as wide), m16n8k16 tiles otherwise
                fn = (ops.attn_prefill_tc if s.value_dim == s.head_dim
                      and ops.attn_prefill_tc_supported(s.head_dim, s.num_heads, s.num_kv_heads) else ops.attn_prefill)
                fn(q, slot.kv, slot.table, step.seq_rows, step.cu_q, step.kv_len, out, entries=step.num_seqs,
                   max_q_len=step.max_q_len, num_heads=s.num_heads, num_kv_heads=s.num_kv_heads,
                   head_dim=s.head_dim, page_size=slot.page_size, scale=s.scale, window=s.window, **options)
            return
        ops.paged_attention_plain(q, slot.kv, slot.table, step.seq_rows, step.token_seq, step.positions, out,
                                  num_heads=s.num_heads, num_kv_heads=s.num_kv_heads, head_dim=s.head_dim,
                                  page_size=slot.page_size, scale=s.scale, window=s.window, **options)


register_mixer("attention", PagedAttention)
