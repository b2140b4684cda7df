"""The selective state-space mixer with a decay per channel and state entry (``selective_scan``).

With h the mixer's input, ``inner`` channels, ``state`` entries per channel and a step-size latent of ``dt_rank``::

    [x | z] = W_in h                                            inner entries each
    x <- silu(conv(x) + conv_bias)                              a causal convolution over time per channel, K taps
    [d | B | C] = W_x x                                         dt_rank, state, state entries
    dt = softplus(W_dt d + dt_bias)                             one step size per channel
    S_t[c, n] = exp(dt_c A[c, n]) S_(t-1)[c, n] + dt_c x_c B_n  A = -exp(A_log); S is zero before the first token
    y_c = sum_n S_t[c, n] C_n + D_c x_c;   out = W_o (y * silu(z))

The projections take operands of the compute type and leave float32; the convolution with its activation, step sizes,
decays, the state, the read-out and the gate are float32 (``csrc/short_conv.cu``, ``csrc/selective_scan.cu``); the gated
read-out is rounded once to the compute type for the output product, whose result is float32 again.

State of a request: one float32 vector in its slot, ``[conv piece | state piece]``: the convolution's last K - 1 inputs
and S. Each piece holds two copies that take turns by the parity of the last position written, so a step of one token
never overwrites what it read and a captured decode step can be replayed."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.spec import StateSpec
from ..ops import kernels
from ..ops.linear import linear
from ..weights.source import ParamSpec
from .base import LayerCache, Mixer, TensorGetter
from .registry import register_mixer


@register_mixer("selective_scan")
class SelectiveScan(Mixer):
    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, inner: int, state: int, dt_rank: int, conv: int = 4,
                 names: Optional[Dict[str, str]] = None):
        """``names``: the tensors' names below ``prefix`` where they differ from the keys ``in``, ``conv``, ``conv.b``,
        ``x``, ``dt``, ``dt.b``, ``A_log``, ``D``, ``o``."""
        self.prefix, self.hidden_size = prefix, int(hidden_size)
        self.inner, self.state, self.dt_rank, self.taps = int(inner), int(state), int(dt_rank), int(conv)
        if min(self.inner, self.state, self.dt_rank) <= 0:
            raise ValueError("the selective scan needs positive sizes")
        if self.state > kernels.SELECTIVE_SCAN_MAX_STATES:
            raise ValueError(f"the scan kernel keeps up to {kernels.SELECTIVE_SCAN_MAX_STATES} state entries a channel, got {self.state}")
        if not 1 <= self.taps <= kernels.SHORT_CONV_MAX_TAPS:
            raise ValueError(f"the convolution kernel takes 1 to {kernels.SHORT_CONV_MAX_TAPS} taps, got {self.taps}")
        self.conv_entries = 2 * (self.taps - 1) * self.inner
        self.scan_entries = 2 * self.inner * self.state
        self.names = {n: n for n in ("in", "conv", "conv.b", "x", "dt", "dt.b", "A_log", "D", "o")}
        self.names.update(names or {})
        self.w_in = self.w_x = self.w_dt = self.w_out = self.conv_w = self.conv_b = self.dt_bias = self.a = self.d_skip = None

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.conv_entries + self.scan_entries,), torch.float32)

    def graph_key_group(self):
        return "selective_scan"                # launches of a step of single tokens depend on the number of requests alone

    def _name(self, key: str) -> str:
        return f"{self.prefix}.{self.names[key]}"

    def param_specs(self) -> Dict[str, ParamSpec]:
        D, I, N, R = self.hidden_size, self.inner, self.state, self.dt_rank
        return {self._name("in"): ParamSpec((2 * I, D)),
                self._name("conv"): ParamSpec((I, self.taps), role="vector", init="normal"),
                self._name("conv.b"): ParamSpec((I,), role="vector", init="small"),
                self._name("x"): ParamSpec((R + 2 * N, I)),
                self._name("dt"): ParamSpec((I, R)),
                self._name("dt.b"): ParamSpec((I,), role="vector", init="small"),
                self._name("A_log"): ParamSpec((I, N), role="vector", init="small"),
                self._name("D"): ParamSpec((I,), role="vector", init="unit"),
                self._name("o"): ParamSpec((D, I))}

    def load(self, get: TensorGetter) -> None:
        self.w_in = get(self._name("in"), "matrix").contiguous()
        self.w_x = get(self._name("x"), "matrix").contiguous()
        self.w_dt = get(self._name("dt"), "matrix").contiguous()
        self.w_out = get(self._name("o"), "matrix").contiguous()
        self.conv_w = get(self._name("conv"), "vector").float().contiguous()
        self.conv_b = get(self._name("conv.b"), "vector").float().contiguous()
        self.dt_bias = get(self._name("dt.b"), "vector").float().contiguous()
        self.d_skip = get(self._name("D"), "vector").float().contiguous()
        self.a = (-torch.exp(get(self._name("A_log"), "vector").float())).contiguous()       # float32, once

    def forward(self, x, ctx, cache: LayerCache):
        if cache.state is None:
            raise RuntimeError("the selective scan mixer needs its state slots")
        N, I, S, R = ctx.num_tokens, self.inner, self.state, self.dt_rank
        xz = linear(x, self.w_in, out_dtype=torch.float32)                       # [N, x | z]
        xc = torch.empty((N, I), dtype=torch.float32, device=x.device)
        xc_typed = torch.empty((N, I), dtype=x.dtype, device=x.device)
        kernels.short_conv(xz[:, :I], self.conv_w, self.conv_b, cache.state, 0, ctx.q_start, ctx.slots, ctx.positions, ctx.token_request,
                           xc, ctx.max_q_len, silu=True, out_typed=xc_typed)
        dbc = linear(xc_typed, self.w_x, out_dtype=torch.float32)                # [N, d | B | C]
        d_typed = torch.empty((N, R), dtype=x.dtype, device=x.device)
        kernels.convert_rows(dbc[:, :R], d_typed)
        dt = linear(d_typed, self.w_dt, out_dtype=torch.float32)                 # [N, inner], before bias and softplus
        gated = torch.empty((N, I), dtype=x.dtype, device=x.device)
        kernels.selective_scan(xc, dt, self.dt_bias, dbc[:, R:R + S], dbc[:, R + S:], self.a, self.d_skip, xz[:, I:], cache.state,
                               self.conv_entries, ctx.q_start, ctx.slots, ctx.positions, gated)
        return linear(gated, self.w_out, out_dtype=torch.float32), None
