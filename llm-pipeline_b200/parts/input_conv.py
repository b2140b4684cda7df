"""A short causal convolution beside the identity, in front of a sublayer: what the sublayer reads, h, becomes

    h_t + sum_{j = 0 .. K-1} w[:, j] * h_(t - K + 1 + j)         per channel, zeros before the request's first token

(no bias, no activation). One part serves all sublayers of a layer that have one: their inputs lie side by side as the
channels of one convolution (``names``: one tensor ``[width, K]`` per sublayer), so a layer needs one launch and one
piece of state. Between steps a request keeps its last K - 1 inputs per channel in its state slot (float32, two copies
that take turns by the parity of the last position written, so a step of one token never overwrites what it read and
a captured decode step can be replayed). Inputs and arithmetic are float32; the result leaves in the compute type, one
matrix per sublayer."""

from __future__ import annotations

from typing import Dict, Sequence

import torch

from ..ops import kernels
from ..weights.source import ParamSpec
from .base import Part, TensorGetter


class InputConv(Part):
    graph_safe = True

    def __init__(self, size: int, taps: int, names: Sequence[str], unused: Sequence[str] = ()):
        """``unused``: names of filters a checkpoint may hold although no sublayer of this layer reads them."""
        self.size, self.taps, self.names, self.unused = int(size), int(taps), tuple(names), tuple(unused)
        if not 1 <= self.taps <= kernels.SHORT_CONV_MAX_TAPS:
            raise ValueError(f"the convolution kernel takes 1 to {kernels.SHORT_CONV_MAX_TAPS} taps, got {self.taps}")
        self.weight = None

    def state_entries(self) -> int:
        return 2 * (self.taps - 1) * self.size * len(self.names)

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {name: ParamSpec((self.size, self.taps), role="vector", init="small") for name in self.names}
        specs.update({name: ParamSpec((self.size, self.taps), role="vector", optional=True, init="small") for name in self.unused})
        return specs

    def load(self, get: TensorGetter) -> None:
        self.weight = torch.cat([get(name, "vector").float() for name in self.names], dim=0).contiguous()

    def forward(self, normed: torch.Tensor, ctx, state: torch.Tensor, state_offset: int) -> torch.Tensor:
        """``normed``: float32 [tokens, k size], the sublayers' inputs side by side; returns [k, tokens, size] in the compute type."""
        N, k = normed.shape[0], len(self.names)
        out = torch.empty((k, N, self.size), dtype=ctx.dtype, device=normed.device)
        if state is None:                       # one tap: nothing is carried between steps
            if self.taps != 1:
                raise RuntimeError("the input convolution needs its state slots")
            state, state_offset = torch.zeros((1, 1), dtype=torch.float32, device=normed.device), 0
        kernels.short_conv(normed, self.weight, None, state, state_offset, ctx.q_start, ctx.slots, ctx.positions, ctx.token_request,
                           None, ctx.max_q_len, silu=False, add_input=True, out_typed=out)
        return out
