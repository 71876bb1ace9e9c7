"""Mixers that keep a state of fixed size per request instead of keys and values: a selective
state-space mixer and a gated delta rule (kernels: csrc/recurrent.cu).

Both ask the cache manager for one 32-bit state row per request (zeroed at admission): the
recurrence's matrices, then the last ``taps - 1`` inputs of the short causal convolution.  A step
brings any mix of prompt portions and single tokens; the kernels find each request's tokens and
state row through the step's device arrays, so the parts run inside replayed CUDA graphs.
Projections are matrix products in the activation type; what enters a recurrence (step sizes,
decays, gates of the recurrence, unit norms, the state) is 32-bit.
"""
from __future__ import annotations

import torch

from ..config.specs import ParamSpec
from ..csrc import ops
from .base import Mixer, StateRequest, make_position, register_mixer
from .linear import linear
from .position import as_rotary_args


def _check_state_rows(rows: int, what: str) -> None:
    if not 0 < rows <= ops.LIMITS["recurrent_max_state_rows"]:
        raise ValueError(f"{what} {rows} is not supported (1 to {ops.LIMITS['recurrent_max_state_rows']}: a state "
                         "column's rows live in the registers of one warp's lanes)")


class StateSpaceMixer(Mixer):
    """``[z | x | B | C | dt] = in_proj(h)``; x, B, C through a causal convolution (bias) and silu;
    ``dt = softplus(dt + dt_bias)``; per head ``S <- exp(-exp(A_log) dt) S + dt B x^T``,
    ``y = S^T C + D x``; ``y * silu(z)`` RMS-normed in ``norm_groups`` parts, times a weight; out
    projection."""
    graph_safe = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        s = spec
        if min(s.num_heads, s.head_dim, s.groups, s.conv_taps, s.norm_groups, s.hidden_size) <= 0:
            raise ValueError("the sizes of a state-space mixer must be positive")
        if s.num_heads % s.groups:
            raise ValueError("num_heads must be a multiple of groups")
        if (s.num_heads * s.head_dim) % s.norm_groups:
            raise ValueError("norm_groups must divide num_heads * head_dim")
        if s.num_heads > ops.LIMITS["grid_dim_yz"] or s.norm_groups > ops.LIMITS["grid_dim_yz"]:
            raise ValueError("heads and norm groups are grid dimensions of the kernels (at most 65,535)")
        _check_state_rows(s.state_size, "state_size")
        self.inner = s.num_heads * s.head_dim
        self.conv_channels = self.inner + 2 * s.groups * s.state_size
        self.conv_off = s.num_heads * s.head_dim * s.state_size

    def parameters(self):
        s = self.spec
        return {"in_proj": ParamSpec((2 * self.inner + 2 * s.groups * s.state_size + s.num_heads, s.hidden_size)),
                "conv_w": ParamSpec((self.conv_channels, s.conv_taps), "float32"),
                "conv_b": ParamSpec((self.conv_channels,), "float32", "bias"),
                "dt_bias": ParamSpec((s.num_heads,), "float32", "bias"),
                "a_log": ParamSpec((s.num_heads,), "float32", "bias"),
                "d_skip": ParamSpec((s.num_heads,), "float32", "norm"),
                "norm_w": ParamSpec((self.inner,), "float32", "norm"),
                "o": ParamSpec((s.hidden_size, self.inner))}

    def state_request(self):
        return StateRequest((self.conv_off + (self.spec.conv_taps - 1) * self.conv_channels,), torch.float32)

    def forward(self, x, step, slot):
        s = self.spec
        tokens = x.shape[0]
        proj = linear(x, self.in_proj)
        xbc = torch.empty(tokens, self.conv_channels, dtype=torch.float32, device=x.device)
        ops.causal_conv(proj, self.inner, self.conv_w, self.conv_b, slot.state, self.conv_off, step, xbc)
        y = torch.empty(tokens, self.inner, dtype=torch.float32, device=x.device)
        ops.ssm_scan(xbc, proj, self.inner + self.conv_channels, self.dt_bias, self.a_log, self.d_skip, slot.state, step, y,
                     heads=s.num_heads, head_dim=s.head_dim, state_size=s.state_size, groups=s.groups)
        gated = torch.empty(tokens, self.inner, dtype=x.dtype, device=x.device)
        ops.gated_group_norm(y, proj, 0, self.norm_w, gated, parts=s.norm_groups, eps=s.norm_eps)
        return linear(gated, self.o)


class GatedDeltaMixer(Mixer):
    """``[q | k | v | b | a | g] = in_proj(h)``; q, k, v through causal convolutions and silu; q and
    k unit vectors per head (q times ``head_dim ** -0.5``); ``beta = sigmoid(b)``; decay per head and key
    channel ``exp(-exp(A_log) softplus(a2(a) + dt_bias))``; per head ``S <- diag(decay) S``,
    ``u = beta (v - S^T k)``, ``S <- S + k u^T``, ``o = S^T q``; each head's ``o`` over its root
    mean square, times a weight shared by the heads, times ``sigmoid(g2(g))``; out projection.
    With ``decay_per="head"`` the decay is one number per head, ``exp(-exp(A_log) softplus(a + dt_bias))``
    with ``a`` a column of the input projection, and the gate ``gate_activation(g)`` with ``g`` columns of
    the input projection (no low ranks)."""
    graph_safe = True
    chunk_min_tokens = 16        # (one decay per head) the longest entry of a step from which the chunked kernel runs; None: never

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        s = spec
        if s.decay_per not in ("channel", "head") or s.gate_activation not in ("sigmoid", "silu"):
            raise ValueError("decay_per is 'channel' or 'head', gate_activation 'sigmoid' or 'silu'")
        self.per_head = s.decay_per == "head"
        ranks = () if self.per_head else (s.decay_rank, s.gate_rank)
        if min(s.num_heads, s.num_kv_heads, s.head_dim, s.v_head_dim, s.conv_taps, s.hidden_size, *ranks) <= 0:
            raise ValueError("the sizes of a gated-delta mixer must be positive")
        if s.num_heads % s.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if s.num_heads > ops.LIMITS["grid_dim_yz"]:
            raise ValueError("heads are a grid dimension of the kernels (at most 65,535)")
        _check_state_rows(s.head_dim, "head_dim")
        self.qk = s.num_kv_heads * s.head_dim
        self.vv = s.num_heads * s.v_head_dim
        self.conv_channels = 2 * self.qk + self.vv
        self.conv_off = s.num_heads * s.v_head_dim * s.head_dim
        self.b_off = self.conv_channels
        self.a_off = self.b_off + s.num_heads
        # one decay per head: the decay's and the gate's columns come straight from the input projection
        self.a_cols = s.num_heads if self.per_head else s.decay_rank
        self.g_off = self.a_off + self.a_cols
        self.g_cols = self.vv if self.per_head else s.gate_rank

    def parameters(self):
        s = self.spec
        out = {"in_proj": ParamSpec((self.g_off + self.g_cols, s.hidden_size)),
               "conv_w": ParamSpec((self.conv_channels, s.conv_taps), "float32"),
               "dt_bias": ParamSpec((s.num_heads * (1 if self.per_head else s.head_dim),), "float32", "bias"),
               "a_log": ParamSpec((s.num_heads,), "float32", "bias"),
               "norm_w": ParamSpec((s.v_head_dim,), "float32", "norm"),
               "o": ParamSpec((s.hidden_size, self.vv))}
        if not self.per_head:
            out["a2"] = ParamSpec((s.num_heads * s.head_dim, s.decay_rank))
            out["g2"] = ParamSpec((self.vv, s.gate_rank))
        return out

    def state_request(self):
        return StateRequest((self.conv_off + (self.spec.conv_taps - 1) * self.conv_channels,), torch.float32)

    def forward(self, x, step, slot):
        s = self.spec
        tokens, dev = x.shape[0], x.device
        proj = linear(x, self.in_proj)
        qkv = torch.empty(tokens, self.conv_channels, dtype=torch.float32, device=dev)
        ops.causal_conv(proj, 0, self.conv_w, None, slot.state, self.conv_off, step, qkv)
        a, gate = proj[:, self.a_off:self.a_off + self.a_cols], proj[:, self.g_off:self.g_off + self.g_cols]
        if not self.per_head:       # through the low ranks
            a, gate = linear(a, self.a2), linear(gate, self.g2)
        dec = torch.empty(tokens, s.num_heads * s.head_dim, dtype=torch.float32, device=dev)
        beta = torch.empty(tokens, s.num_heads, dtype=torch.float32, device=dev)
        # One decay per head: a step with a prompt portion whose (entry, head, 32 columns) blocks do not fill the device
        # takes the recurrence in chunks of 64 tokens.  The chunked form does about twice the 32-bit multiply-adds of the
        # walk token by token (the keys' products with one another, the triangular system, the products with the state at
        # the chunk's start), so it is ahead only while the walk leaves SMs idle (measured at 16 heads of 128 x 128: one
        # 2,048-token prompt 930 against 1,010 us; four of them about 1,500 against 1,220 us).
        chunked = (self.per_head and self.chunk_min_tokens is not None and step.max_q_len >= self.chunk_min_tokens
                   and s.head_dim <= ops.LIMITS["delta_chunk_max_head_dim"]
                   and step.num_seqs * s.num_heads * (-(-s.v_head_dim // 32)) <= ops.sm_count(dev))
        log_dec = torch.empty(tokens, s.num_heads, dtype=torch.float32, device=dev) if chunked else None
        ops.delta_prep(qkv, a, proj, self.b_off, self.dt_bias, self.a_log, dec, beta, heads=s.num_heads,
                       kv_heads=s.num_kv_heads, head_dim=s.head_dim, v_head_dim=s.v_head_dim, unit_eps=s.unit_eps,
                       q_scale=s.head_dim ** -0.5, per_head=self.per_head, log_dec=log_dec)
        o = torch.empty(tokens, self.vv, dtype=torch.float32, device=dev)
        if chunked:
            ops.delta_chunk(qkv, log_dec, beta, slot.state, step, o, heads=s.num_heads, kv_heads=s.num_kv_heads,
                            head_dim=s.head_dim, v_head_dim=s.v_head_dim)
        else:
            ops.delta_scan(qkv, dec, beta, slot.state, step, o, heads=s.num_heads, kv_heads=s.num_kv_heads,
                           head_dim=s.head_dim, v_head_dim=s.v_head_dim)
        out = torch.empty(tokens, self.vv, dtype=x.dtype, device=dev)
        ops.delta_out(o, gate, self.norm_w, out, heads=s.num_heads, v_head_dim=s.v_head_dim, eps=s.norm_eps,
                      silu=s.gate_activation == "silu")
        return linear(out, self.o)


class RetentionMixer(Mixer):
    """``[q | k | v | g] = in_proj(h)``; q and k rotated by position, k times ``head_dim ** -0.5``; per
    head ``S <- decay S + k v^T``, ``o = S^T q`` with a fixed decay; each head's ``o`` over its root
    mean square, times ``silu(g)``; out projection (kernels: csrc/retention.cu).  The state is one
    32-bit ``[heads, head_dim, v_head_dim]`` row per request."""
    graph_safe = True
    chunk_min_tokens = 16        # the longest entry of a step from which the chunked kernel runs; None: never

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        s = spec
        if min(s.num_heads, s.head_dim, s.v_head_dim, s.hidden_size) <= 0:
            raise ValueError("the sizes of a retention mixer must be positive")
        if len(s.decays) != s.num_heads:
            raise ValueError(f"a retention mixer needs one decay per head ({s.num_heads}), got {len(s.decays)}")
        if s.head_dim > ops.LIMITS["retention_max_head_dim"]:
            raise ValueError(f"head_dim {s.head_dim} is not supported (at most {ops.LIMITS['retention_max_head_dim']}: "
                             "a state column's rows live in the registers of eight warps)")
        if s.num_heads > ops.LIMITS["grid_dim_yz"]:
            raise ValueError("heads are a grid dimension of the kernels (at most 65,535)")
        self.position = make_position(s.position, dtype) if s.position is not None else None
        if self.position is not None:
            if s.position.pairing != "split_half":
                raise ValueError("the retention kernels rotate split halves only")
            if s.position.rotary_dim > s.head_dim:
                raise ValueError(f"the position encoding rotates {s.position.rotary_dim} dims, a head has {s.head_dim}")
        self.qk = s.num_heads * s.head_dim
        self.vv = s.num_heads * s.v_head_dim
        self._decay = None

    def parameters(self):
        s = self.spec
        return {"in_proj": ParamSpec((2 * self.qk + 2 * self.vv, s.hidden_size)),
                "o": ParamSpec((s.hidden_size, self.vv))}

    def state_request(self):
        s = self.spec
        return StateRequest((s.num_heads * s.head_dim * s.v_head_dim,), torch.float32)

    def forward(self, x, step, slot):
        s = self.spec
        tokens, dev = x.shape[0], x.device
        if self._decay is None or self._decay.device != dev:
            self._decay = torch.tensor([float(g) for g in s.decays], dtype=torch.float32, device=dev)
        inv_freq, rotary_dim = None, 0
        if self.position is not None:
            rope = as_rotary_args(self.position.kernel_args(dev))
            if rope.scale != 1.0:
                raise ValueError("the retention kernels take no factor on cos and sin")
            inv_freq, rotary_dim = rope.inv_freq, rope.rotary_dim
        proj = linear(x, self.in_proj)
        q32 = torch.empty(tokens, self.qk, dtype=torch.float32, device=dev)
        k32 = torch.empty(tokens, self.qk, dtype=torch.float32, device=dev)
        ops.retention_prep(proj, 0, self.qk, inv_freq, step.positions, q32, k32, heads=s.num_heads, head_dim=s.head_dim,
                           rotary_dim=rotary_dim, k_scale=s.head_dim ** -0.5)
        o = torch.empty(tokens, self.vv, dtype=torch.float32, device=dev)
        # a step with a prompt portion takes the recurrence in chunks of 64 tokens (closed form per chunk);
        # steps of single tokens and of short pieces walk it token by token
        chunked = self.chunk_min_tokens is not None and step.max_q_len >= self.chunk_min_tokens
        (ops.retention_chunk if chunked else ops.retention_scan)(
            q32, k32, proj, 2 * self.qk, self._decay, slot.state, step, o, heads=s.num_heads, head_dim=s.head_dim,
            v_head_dim=s.v_head_dim)
        gated = torch.empty(tokens, self.vv, dtype=x.dtype, device=dev)
        ops.retention_out(o, proj, 2 * self.qk + self.vv, gated, heads=s.num_heads, v_head_dim=s.v_head_dim, eps=s.norm_eps)
        return linear(gated, self.o)


class MatrixMemoryMixer(Mixer):
    """``[q | k | v | g | i | f] = in_proj(h)``; per head a matrix memory with exponential gates held stable
    by a running maximum (``config.specs.MatrixMemorySpec``; kernels: csrc/matrix_memory.cu).  The state is
    one 32-bit row per request: ``[heads, head_dim, v_head_dim + 1]`` (the normaliser is the last column),
    then the maximum per head."""
    graph_safe = True
    chunk_min_tokens = 16        # the longest entry of a step from which the chunked kernel runs; None: never

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        s = spec
        if min(s.num_heads, s.head_dim, s.v_head_dim, s.hidden_size) <= 0 or not s.gate_cap > 0:
            raise ValueError("the sizes and the gate cap of a matrix memory must be positive")
        if s.head_dim > ops.LIMITS["memory_max_head_dim"]:
            raise ValueError(f"head_dim {s.head_dim} is not supported (at most {ops.LIMITS['memory_max_head_dim']}: "
                             "a state column's rows live in the registers of eight warps)")
        if s.num_heads > ops.LIMITS["grid_dim_yz"]:
            raise ValueError("heads are a grid dimension of the kernels (at most 65,535)")
        self.qk = s.num_heads * s.head_dim
        self.vv = s.num_heads * s.v_head_dim
        self.g_off = 2 * self.qk + self.vv
        self.i_off = self.g_off + self.vv
        self.f_off = self.i_off + s.num_heads
        self.m_off = s.num_heads * s.head_dim * (s.v_head_dim + 1)

    def parameters(self):
        s = self.spec
        return {"in_proj": ParamSpec((self.f_off + s.num_heads, s.hidden_size)),
                "gate_bias": ParamSpec((2 * s.num_heads,), "float32", "bias"),       # input gates, then forget gates
                "norm_w": ParamSpec((self.vv,), "float32", "norm"),
                "o": ParamSpec((s.hidden_size, self.vv))}

    def state_request(self):
        return StateRequest((self.m_off + self.spec.num_heads,), torch.float32)

    # the parameter that projects the mixer's input (a mixer of mixers may stack it with its neighbours' and
    # hand `forward` the product's columns as `proj`)
    input_projection = "in_proj"

    def forward(self, x, step, slot, proj=None):
        s = self.spec
        tokens, dev = x.shape[0], x.device
        if proj is None:
            proj = linear(x, self.in_proj)
        gates = torch.empty(tokens, s.num_heads, 3, dtype=torch.float32, device=dev)
        ops.memory_gates(proj, self.i_off, self.f_off, self.gate_bias, s.gate_cap, slot.state, self.m_off, step, gates,
                         heads=s.num_heads)
        o = torch.empty(tokens, s.num_heads, s.v_head_dim + 1, dtype=torch.float32, device=dev)
        # a step with a prompt portion takes the recurrence in chunks of 64 tokens (closed form per chunk);
        # steps of single tokens and of short pieces walk it token by token
        chunked = self.chunk_min_tokens is not None and step.max_q_len >= self.chunk_min_tokens
        (ops.memory_chunk if chunked else ops.memory_scan)(
            proj, 0, self.qk, 2 * self.qk, gates, s.head_dim ** -0.5, slot.state, step, o, heads=s.num_heads,
            head_dim=s.head_dim, v_head_dim=s.v_head_dim)
        gated = torch.empty(tokens, self.vv, dtype=x.dtype, device=dev)
        ops.memory_out(o, gates, proj, self.g_off, self.norm_w, gated, heads=s.num_heads, v_head_dim=s.v_head_dim,
                       eps=s.norm_eps, den_eps=s.den_eps)
        return linear(gated, self.o)


register_mixer("matrix_memory", MatrixMemoryMixer)
register_mixer("retention", RetentionMixer)
register_mixer("mamba2", StateSpaceMixer)
register_mixer("channel_delta", GatedDeltaMixer)
