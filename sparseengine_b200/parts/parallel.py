"""Mixers side by side: every branch reads the same input, the result is the weighted sum of what
they return (``config.specs.ParallelMixerSpec``).

A branch is any registered mixer.  The cache manager sees one mixer: the pages are the branch's that
asks for pages, the state slot the branch's that asks for one (at most one each).  A branch that
has a bias on its output projection leaves it to the sum (one kernel: csrc/stream_mix.cu,
``scaled_sum``), where it is weighed like the branch.  Branches that name the parameter that
projects their input (``input_projection``) get one product for all of them: their matrices are
stacked (the branches' own parameters become views of the stack) and each branch is handed its
columns of the result.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, make_mixer, register_mixer
from .linear import linear


class ParallelMixer(Mixer):
    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        if len(spec.branches) != 2 or len(spec.scales) != 2 or len(spec.names) != 2 or len(set(spec.names)) != 2:
            raise ValueError("a parallel mixer has two branches, each with a scale and a name of its own")
        self.branches = [make_mixer(b, dtype) for b in spec.branches]
        self.scales = [float(a) for a in spec.scales]
        if sum(b.kv_request() is not None for b in self.branches) > 1 or \
                sum(b.state_request() is not None for b in self.branches) > 1:
            raise ValueError("at most one branch of a parallel mixer may ask for pages, and one for a state slot")
        self.graph_safe = all(b.graph_safe for b in self.branches)
        limits = [b.max_step_entries for b in self.branches if b.max_step_entries is not None]
        self.max_step_entries = min(limits) if limits else None
        for b in self.branches:
            if hasattr(b, "defer_output_bias"):
                b.defer_output_bias = True
        self._bias = None
        self._stacked = None         # the branches' input projections as one matrix, and where each one's rows start

    def parameters(self):
        return {f"{name}_{k}": p for name, b in zip(self.spec.names, self.branches) for k, p in b.parameters().items()}

    def bind(self, tensors):
        for name, b in zip(self.spec.names, self.branches):
            b.bind({k[len(name) + 1:]: v for k, v in tensors.items() if k.startswith(name + "_")})
        # the branches' output biases, weighed like the branches
        self._bias = None
        for a, b in zip(self.scales, self.branches):
            bias = b.output_bias() if hasattr(b, "output_bias") else None
            if bias is not None:
                self._bias = a * bias.float() if self._bias is None else self._bias + a * bias.float()
        # one product for the branches' input projections
        self._stacked = None
        names = [getattr(b, "input_projection", None) for b in self.branches]
        if all(n is not None and getattr(b, n, None) is not None for n, b in zip(names, self.branches)):
            parts = [getattr(b, n) for n, b in zip(names, self.branches)]
            if all(p.dim() == 2 and p.shape[1] == parts[0].shape[1] and p.dtype == parts[0].dtype for p in parts):
                stack = torch.cat(parts, 0)
                starts, at = [], 0
                for n, b, p in zip(names, self.branches, parts):
                    setattr(b, n, stack[at:at + p.shape[0]])       # the branch's own parameter: a view of the stack
                    starts.append((at, p.shape[0]))
                    at += p.shape[0]
                self._stacked = (stack, starts)

    def kv_request(self):
        return next((r for r in (b.kv_request() for b in self.branches) if r is not None), None)

    def state_request(self):
        return next((r for r in (b.state_request() for b in self.branches) if r is not None), None)

    def forward(self, x, step, slot):
        if self._stacked is not None:
            stack, starts = self._stacked
            proj = linear(x, stack)
            y0, y1 = (b.forward(x, step, slot, proj=proj[:, at:at + n]) for b, (at, n) in zip(self.branches, starts))
        else:
            y0 = self.branches[0].forward(x, step, slot)
            y1 = self.branches[1].forward(x, step, slot)
        return ops.scaled_sum(y0, y1, self.scales[0], self.scales[1], torch.empty_like(y0), bias=self._bias)


register_mixer("parallel", ParallelMixer)
