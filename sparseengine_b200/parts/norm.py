"""RMSNorm with an optional fused residual add (kernel: csrc/elementwise.cu).

Reference: src/sparseengine/layers/layernorm.py:120-159.
"""
from __future__ import annotations

import torch

from ..config.specs import ParamSpec
from ..csrc import ops
from .base import Norm, register_norm


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        if not 0 < spec.size <= ops.LIMITS["rmsnorm_max_width"]:
            raise ValueError(f"RMSNorm width {spec.size} is not supported: the kernel takes rows of 1 to "
                             f"{ops.LIMITS['rmsnorm_max_width']} elements")
        if not spec.eps > 0:
            raise ValueError("RMSNorm eps must be positive")

    def parameters(self):
        if self.spec.offset:        # kept in 32-bit: offset + w would lose the stored digits in a 16-bit type
            return {"weight": ParamSpec((self.spec.size,), "float32", "bias")}
        return {"weight": ParamSpec((self.spec.size,), "act", "norm")}

    def bind(self, tensors):
        super().bind(tensors)
        if self.spec.offset:
            self.weight = self.weight + float(self.spec.offset)     # what the kernels multiply by

    def forward(self, x, residual=None):
        out = torch.empty_like(x)
        if residual is None:
            ops.rmsnorm(x, self.weight, self.spec.eps, out)
            return out, x
        new_residual = torch.empty_like(x)
        ops.rmsnorm(x, self.weight, self.spec.eps, out, residual=residual, residual_out=new_residual)
        return out, new_residual

    def forward_stream(self, stream, y=None):
        """Over a 32-bit residual stream (kernel: csrc/stream32.cu): ``stream += y`` in place (``y``:
        the last sublayer's output in the activation type, or None), then the norm of the sum in the
        activation type.  Returns ``(normed, stream)``."""
        out = torch.empty(stream.shape, dtype=self.dtype, device=stream.device)
        ops.add_rmsnorm_stream(stream, y, self.weight, self.spec.eps, out32=stream if y is not None else None, out_act=out)
        return out, stream

    def forward_into_stream(self, stream, y):
        """A norm on a sublayer's output (kernel: csrc/stream32.cu): ``stream += norm(y)`` in place
        (32-bit).  Returns ``(the new stream in the activation type, stream)``; in a 32-bit engine the
        first is the stream itself."""
        if self.dtype == torch.float32:
            ops.rmsnorm_add_stream(stream, y, self.weight, self.spec.eps)
            return stream, stream
        out = torch.empty(stream.shape, dtype=self.dtype, device=stream.device)
        ops.rmsnorm_add_stream(stream, y, self.weight, self.spec.eps, out_act=out)
        return out, stream


register_norm("rms", RMSNorm)


class LayerNorm(Norm):
    """Layer norm with weight and bias over a 32-bit residual stream (kernel: csrc/stream32.cu).

    ``forward_stream(stream, y, alpha)`` normalises ``alpha * stream + y`` and returns the result
    twice: in the activation type (what the next matrix product reads) and in 32-bit (the new
    stream).  ``forward(x)`` is the plain form for a model's final norm: it reads the 32-bit
    stream and returns the activation type."""
    graph_safe = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        if not 0 < spec.size <= ops.LIMITS["layernorm_max_width"]:
            raise ValueError(f"LayerNorm width {spec.size} is not supported: the kernel takes rows of 1 to "
                             f"{ops.LIMITS['layernorm_max_width']} elements")
        if not spec.eps > 0:
            raise ValueError("LayerNorm eps must be positive")
        self.bias = None

    def parameters(self):
        out = {"weight": ParamSpec((self.spec.size,), "act", "norm")}
        if self.spec.bias:
            out["bias"] = ParamSpec((self.spec.size,), "act", "bias")
        return out

    def forward_stream(self, stream, y=None, alpha: float = 1.0):
        out32 = torch.empty_like(stream)
        if self.dtype == torch.float32:
            ops.add_layernorm(stream, y, alpha, self.weight, self.bias, self.spec.eps, out32=out32)
            return out32, out32
        act = torch.empty(stream.shape, dtype=self.dtype, device=stream.device)
        ops.add_layernorm(stream, y, alpha, self.weight, self.bias, self.spec.eps, out32=out32, out_act=act)
        return act, out32

    def forward(self, x, residual=None):
        if residual is not None:
            raise ValueError("LayerNorm.forward takes the stream alone; blocks use forward_stream")
        x32 = x if x.dtype == torch.float32 else x.float()
        out = torch.empty(x.shape, dtype=self.dtype, device=x.device)
        if self.dtype == torch.float32:
            ops.add_layernorm(x32, None, 1.0, self.weight, self.bias, self.spec.eps, out32=out)
        else:
            ops.add_layernorm(x32, None, 1.0, self.weight, self.bias, self.spec.eps, out_act=out)
        return out, x


register_norm("layer_norm", LayerNorm)
