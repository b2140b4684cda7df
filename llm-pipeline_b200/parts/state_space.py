"""State-space mixers: a matrix state per head that decays by one scalar per head and token.

``ssd`` (the selective state-space recurrence in its scalar-decay form). With h the mixer's input, H heads of P value
channels, G groups of N state channels (head i reads group i // (H / G)) and inner = H P, one product gives
``[z | x | B | C | dt]`` of widths inner, inner, G N, G N, H. Then::

    (x, B, C) <- silu(conv(x | B | C) + conv_bias)     a causal convolution over time per channel, K taps
    dt <- softplus(dt + dt_bias),   a = exp(-exp(A_log) dt)                          per head
    S_t = a S_(t-1) + dt B_t x_t^T   (S is N x P, zero before the first token),   y_t = S_t^T C_t + D x_t
    y <- y * silu(z), then an RMS norm in ``norm_groups`` equal parts of the row, times ``norm``;  out = Wo y

The product leaves float32; convolution, step sizes, decays, state, read-out, gate and norm are float32
(``csrc/short_conv.cu``, ``csrc/state_space.cu``); the normed rows are rounded once to the compute type for the output
product, whose result is float32 again.

State of a request: one float32 vector in its slot, ``[conv piece | state piece]``. Each piece holds two copies that take
turns by the parity of the last position written, so a step of one token never overwrites what it read and a captured
decode step can be replayed. A mixer that is one of several in a layer gets a column range of the layer's vector."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.spec import StateSpec
from ..ops import kernels
from ..ops.linear import linear
from ..weights.source import ParamSpec
from .base import LayerCache, Mixer, TensorGetter
from .registry import register_mixer


@register_mixer("ssd")
class StateSpaceDuality(Mixer):
    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, heads: int, vdim: int, state: int, groups: int = 1, conv: int = 4,
                 norm_groups: int = 1, eps: float = 1e-6, names: Optional[Dict[str, str]] = None):
        """``names``: the tensors' names below ``prefix`` where they differ from the keys ``in``, ``conv``, ``conv.b``,
        ``dt_bias``, ``A_log``, ``D``, ``norm``, ``o``."""
        self.prefix, self.hidden_size = prefix, int(hidden_size)
        self.heads, self.vdim, self.state, self.groups = int(heads), int(vdim), int(state), int(groups)
        self.taps, self.norm_groups, self.eps = int(conv), int(norm_groups), float(eps)
        if self.heads <= 0 or self.groups <= 0 or self.heads % self.groups:
            raise ValueError(f"{self.heads} heads cannot share {self.groups} groups of state channels")
        self.inner = self.heads * self.vdim
        if self.norm_groups <= 0 or self.inner % self.norm_groups:
            raise ValueError(f"a row of {self.inner} entries cannot be normed in {self.norm_groups} equal parts")
        if not 1 <= self.taps <= kernels.SHORT_CONV_MAX_TAPS:
            raise ValueError(f"the convolution kernel takes 1 to {kernels.SHORT_CONV_MAX_TAPS} taps, got {self.taps}")
        self.channels = self.inner + 2 * self.groups * self.state
        self.conv_entries = 2 * (self.taps - 1) * self.channels
        self.scan_entries = 2 * self.heads * self.state * self.vdim
        self.names = {n: n for n in ("in", "conv", "conv.b", "dt_bias", "A_log", "D", "norm", "o")}
        self.names.update(names or {})
        self.w_in = self.w_out = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.d_skip = self.norm_w = None

    def state_entries(self) -> int:
        return self.conv_entries + self.scan_entries

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.state_entries(),), torch.float32)

    def graph_key_group(self):
        return "ssd"                          # launches of a step of single tokens depend on the number of requests alone

    def _name(self, key: str) -> str:
        return f"{self.prefix}.{self.names[key]}"

    def param_specs(self) -> Dict[str, ParamSpec]:
        D, H = self.hidden_size, self.heads
        return {self._name("in"): ParamSpec((self.inner + self.channels + H, D)),
                self._name("conv"): ParamSpec((self.channels, self.taps), role="vector", init="normal"),
                self._name("conv.b"): ParamSpec((self.channels,), role="vector", init="small"),
                self._name("dt_bias"): ParamSpec((H,), role="vector", init="small"),
                self._name("A_log"): ParamSpec((H,), role="vector", init="small"),
                self._name("D"): ParamSpec((H,), role="vector", init="unit"),
                self._name("norm"): ParamSpec((self.inner,), role="vector", init="norm"),
                self._name("o"): ParamSpec((D, self.inner))}

    def load(self, get: TensorGetter) -> None:
        self.w_in = get(self._name("in"), "matrix").contiguous()
        self.w_out = get(self._name("o"), "matrix").contiguous()
        self.conv_w = get(self._name("conv"), "vector").float().contiguous()
        self.conv_b = get(self._name("conv.b"), "vector").float().contiguous()
        self.dt_bias, self.a_log, self.d_skip, self.norm_w = (get(self._name(n), "vector").float().contiguous()
                                                              for n in ("dt_bias", "A_log", "D", "norm"))

    def forward(self, x, ctx, cache: LayerCache):
        if cache.state is None:
            raise RuntimeError("the state-space mixer needs its state slots")
        N, inner, C = ctx.num_tokens, self.inner, self.channels
        proj = linear(x, self.w_in, out_dtype=torch.float32)
        z, xbc, dt = proj[:, :inner], proj[:, inner:inner + C], proj[:, inner + C:]
        mixed = torch.empty((N, C), dtype=torch.float32, device=x.device)
        kernels.short_conv(xbc, self.conv_w, self.conv_b, cache.state, 0, ctx.q_start, ctx.slots, ctx.positions, ctx.token_request,
                           mixed, ctx.max_q_len, silu=True)
        y = torch.empty((N, inner), dtype=torch.float32, device=x.device)
        kernels.ssd_scan(mixed, dt, self.dt_bias, self.a_log, self.d_skip, cache.state, self.conv_entries, ctx.q_start, ctx.slots,
                         ctx.positions, y, self.heads, self.groups, self.state, self.vdim)
        normed = torch.empty((N, inner), dtype=x.dtype, device=x.device)
        kernels.gated_group_norm(y, z, self.norm_w, normed, inner // self.norm_groups, self.eps, gate_first=True)
        return linear(normed, self.w_out, out_dtype=torch.float32), None
