"""The gated delta rule: a matrix state per head that forgets channel by channel and is corrected along the current key.

With h the mixer's input, H value heads of ``vdim`` channels, G query/key heads of ``dim`` channels (head i reads
query/key head i // (H / G))::

    q, k, v <- silu(conv(Wq h)), silu(conv(Wk h)), silu(conv(Wv h))     a causal convolution over time per channel, no bias
    q <- q / sqrt(sum(q^2) + 1e-6) * dim^(-1/2),  k <- k / sqrt(sum(k^2) + 1e-6)            per head
    beta = sigmoid(Wb h)                                                       one per value head
    g = exp(-exp(A_log) softplus(Wa2 (Wa1 h) + dt_bias))                       per value head and key channel
    S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q         S is dim x vdim, zero before the first token
    o <- o / sqrt(mean(o^2) + eps) * norm * sigmoid(Wg2 (Wg1 h))               per head; norm has vdim entries
    out = Wo o

The six products that read h are one product against [Wq; Wk; Wv; Wb; Wa1; Wg1] with a float32 result; the inner sizes of
the two-step projections are whatever the tensors have. Convolutions, unit norms, step sizes, decays, state and read-out
are float32 (``csrc/short_conv.cu``, ``csrc/delta_rule.cu``); the gated rows are rounded once to the compute type for the
output product.

State of a request: one float32 vector ``[conv piece | state piece]``, each piece two copies that take turns by the parity
of the last position written (see ``state_space.py``)."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.spec import StateSpec
from ..ops import kernels
from ..ops.linear import linear
from ..weights.source import ParamSpec
from .base import LayerCache, Mixer, TensorGetter
from .registry import register_mixer


@register_mixer("gated_delta_rule")
class GatedDeltaRule(Mixer):
    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, heads: int, qk_heads: int, dim: int, vdim: int, conv: int = 4,
                 eps: float = 1e-6, decay_rank: Optional[int] = None, gate_rank: Optional[int] = None,
                 names: Optional[Dict[str, str]] = None):
        """``decay_rank`` / ``gate_rank``: the inner sizes of the two-step projections; None: the tensors give them."""
        self.prefix, self.hidden_size = prefix, int(hidden_size)
        self.heads, self.qk_heads, self.dim, self.vdim = int(heads), int(qk_heads), int(dim), int(vdim)
        self.taps, self.eps = int(conv), float(eps)
        if self.heads <= 0 or self.qk_heads <= 0 or self.heads % self.qk_heads:
            raise ValueError(f"{self.heads} value heads cannot share {self.qk_heads} query/key heads")
        if not 1 <= self.taps <= kernels.SHORT_CONV_MAX_TAPS:
            raise ValueError(f"the convolution kernel takes 1 to {kernels.SHORT_CONV_MAX_TAPS} taps, got {self.taps}")
        self.decay_rank = int(decay_rank) if decay_rank else None
        self.gate_rank = int(gate_rank) if gate_rank else None
        self.qk_size, self.v_size = self.qk_heads * self.dim, self.heads * self.vdim
        self.channels = 2 * self.qk_size + self.v_size
        self.conv_entries = 2 * (self.taps - 1) * self.channels
        self.scan_entries = 2 * self.heads * self.dim * self.vdim
        self.names = {n: n for n in ("q", "k", "v", "q.conv", "k.conv", "v.conv", "b", "A_log", "dt_bias", "a1", "a2", "g1", "g2",
                                     "norm", "o")}
        self.names.update(names or {})
        self.w_in = self.w_a2 = self.w_g2 = self.w_out = self.conv_w = self.a_log = self.dt_bias = self.norm_w = None

    def state_entries(self) -> int:
        return self.conv_entries + self.scan_entries

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.state_entries(),), torch.float32)

    def graph_key_group(self):
        return "gated_delta_rule"

    def _name(self, key: str) -> str:
        return f"{self.prefix}.{self.names[key]}"

    def param_specs(self) -> Dict[str, ParamSpec]:
        D, H, K = self.hidden_size, self.heads, self.taps
        return {self._name("q"): ParamSpec((self.qk_size, D)), self._name("k"): ParamSpec((self.qk_size, D)),
                self._name("v"): ParamSpec((self.v_size, D)),
                self._name("q.conv"): ParamSpec((self.qk_size, K), role="vector", init="unit"),
                self._name("k.conv"): ParamSpec((self.qk_size, K), role="vector", init="unit"),
                self._name("v.conv"): ParamSpec((self.v_size, K), role="vector", init="unit"),
                self._name("b"): ParamSpec((H, D)),
                self._name("A_log"): ParamSpec((H,), role="vector", init="small"),
                self._name("dt_bias"): ParamSpec((H * self.dim,), role="vector", init="small"),
                self._name("a1"): ParamSpec((self.decay_rank, D)), self._name("a2"): ParamSpec((H * self.dim, self.decay_rank)),
                self._name("g1"): ParamSpec((self.gate_rank, D)), self._name("g2"): ParamSpec((self.v_size, self.gate_rank)),
                self._name("norm"): ParamSpec((self.vdim,), role="vector", init="norm"),
                self._name("o"): ParamSpec((D, self.v_size))}

    def load(self, get: TensorGetter) -> None:
        parts = [get(self._name(n), "matrix") for n in ("q", "k", "v", "b", "a1", "g1")]
        self.w_a2 = get(self._name("a2"), "matrix").contiguous()
        self.w_g2 = get(self._name("g2"), "matrix").contiguous()
        if parts[4].shape[0] != self.w_a2.shape[1] or parts[5].shape[0] != self.w_g2.shape[1]:
            raise ValueError(f"{self.prefix}: the two steps of a projection disagree on their inner size")
        self.decay_rank, self.gate_rank = int(parts[4].shape[0]), int(parts[5].shape[0])
        self.w_in = torch.cat(parts, dim=0).contiguous()
        self.w_out = get(self._name("o"), "matrix").contiguous()
        self.conv_w = torch.cat([get(self._name(n), "vector").float() for n in ("q.conv", "k.conv", "v.conv")], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm_w = (get(self._name(n), "vector").float().contiguous() for n in ("A_log", "dt_bias", "norm"))

    def forward(self, x, ctx, cache: LayerCache):
        if cache.state is None:
            raise RuntimeError("the delta-rule mixer needs its state slots")
        N, C, H = ctx.num_tokens, self.channels, self.heads
        proj = linear(x, self.w_in, out_dtype=torch.float32)
        beta = proj[:, C:C + H]
        low_a = proj[:, C + H:C + H + self.decay_rank]
        low_g = proj[:, C + H + self.decay_rank:]
        if x.dtype != torch.float32:
            low_a, low_g = low_a.to(x.dtype), low_g.to(x.dtype)
        decay = linear(low_a, self.w_a2, out_dtype=torch.float32)
        gate = linear(low_g, self.w_g2, out_dtype=torch.float32)
        mixed = torch.empty((N, C), dtype=torch.float32, device=x.device)
        kernels.short_conv(proj[:, :C], self.conv_w, None, cache.state, 0, ctx.q_start, ctx.slots, ctx.positions, ctx.token_request,
                           mixed, ctx.max_q_len, silu=True)
        q, k, v = mixed[:, :self.qk_size], mixed[:, self.qk_size:2 * self.qk_size], mixed[:, 2 * self.qk_size:]
        kernels.delta_prep(q, k, decay, beta, self.a_log, self.dt_bias, H, self.qk_heads, self.dim)
        o = torch.empty((N, self.v_size), dtype=torch.float32, device=x.device)
        kernels.delta_scan(q, k, v, decay, beta, cache.state, self.conv_entries, ctx.q_start, ctx.slots, ctx.positions, o,
                           H, self.qk_heads, self.dim, self.vdim)
        normed = torch.empty((N, self.v_size), dtype=x.dtype, device=x.device)
        kernels.gated_group_norm(o, gate, self.norm_w, normed, self.vdim, self.eps, gate_first=False)
        return linear(normed, self.w_out, out_dtype=torch.float32), None
