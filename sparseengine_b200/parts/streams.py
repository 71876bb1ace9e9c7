"""Several copies of the residual stream (hyper-connections), and a gate on what a sublayer returns
(kernel: csrc/stream_mix.cu).

A token carries ``streams`` 32-bit copies ``x_1 .. x_S`` of the residual stream, equal at the start.
A sublayer reads ``u = sum_s in[s] x_s`` (then normed) and writes ``x_t <- sum_s mix[s, t] x_s +
out[t] y`` for all ``t`` at once; with ``gated`` the sublayer's result ``y`` is first multiplied by
``sigmoid(W h + b)``, ``h`` being the normed input the sublayer itself read.  With one stream and
nothing learned this is ``x <- x + y``.  :class:`StreamMix` owns one sublayer's numbers;
``parts.block.StreamMixBlock`` strings the sublayers of a layer together so that one kernel does a
sublayer's write and the next one's read.
"""
from __future__ import annotations

import torch

from ..config.specs import ParamSpec
from ..csrc import ops
from .base import Part
from .linear import linear


class StreamMix(Part):
    graph_safe = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        if not 0 < spec.streams <= ops.LIMITS["stream_mix_max_streams"]:
            raise ValueError(f"{spec.streams} residual streams are not supported (1 to "
                             f"{ops.LIMITS['stream_mix_max_streams']}: a column's stream values live in registers)")
        if not 0 < spec.hidden_size <= ops.LIMITS["rmsnorm_max_width"]:
            raise ValueError(f"stream width {spec.hidden_size} is not supported (1 to {ops.LIMITS['rmsnorm_max_width']})")
        if not spec.learned and spec.streams != 1:
            raise ValueError("several residual streams need learned read, write and mixing weights")
        self.in_w = self.out_w = self.mix = self.gate = self.gate_bias = None

    def parameters(self):
        s = self.spec
        out = {}
        if s.learned:
            out.update({"in_w": ParamSpec((s.streams,), "float32", "norm"), "out_w": ParamSpec((s.streams,), "float32", "norm"),
                        "mix": ParamSpec((s.streams, s.streams), "float32", "matrix")})
        if s.gated:
            out.update({"gate": ParamSpec((s.hidden_size, s.hidden_size)),
                        "gate_bias": ParamSpec((s.hidden_size,), "float32", "bias")})
        return out

    def constants(self, device):
        """in, out and mix of a sublayer that has learned none (one stream): ones."""
        if self.mix is None or self.mix.device != torch.device(device):
            self.in_w = torch.ones(1, dtype=torch.float32, device=device)
            self.out_w = torch.ones(1, dtype=torch.float32, device=device)
            self.mix = torch.ones(1, 1, dtype=torch.float32, device=device)

    def gate_logits(self, h):
        """``W h`` of the gate on the sublayer's result (None without a gate); the bias and the sigmoid
        are the write kernel's."""
        return linear(h, self.gate) if self.spec.gated else None

    def write_args(self, y, gate):
        if not self.spec.learned:
            self.constants(y.device)
        return (y, gate, self.gate_bias if gate is not None else None, self.mix, self.out_w)

    def read_weights(self, device):
        if not self.spec.learned:
            self.constants(device)
        return self.in_w
