"""SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))`` without biases
(src/llm_pipeline/models/qwen3/custom_builder.py:193-207; the activation is SiLU whatever
``hidden_act`` says, :204). Gate and up are one matrix product against [gate; up].
Beside it: ``poly_norm_mlp`` and ``relu_squared_mlp``, feed-forwards without a gate."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import kernels
from ..ops.linear import PendingProduct, gate_up_swiglu, linear, pending_product
from ..weights.source import ParamSpec
from .base import FeedForward, TensorGetter
from .registry import register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, names: Optional[Dict[str, str]] = None):
        """``names``: the three matrices' names below ``prefix`` where they are not ``gate_proj.weight``, ``up_proj.weight``
        and ``down_proj.weight`` (keys ``gate``, ``up``, ``down``)."""
        self.prefix, self.hidden_size, self.intermediate_size = prefix, int(hidden_size), int(intermediate_size)
        self.names = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        self.names.update(names or {})
        self.w_gate_up = self.w_down = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        p, H, I, n = self.prefix, self.hidden_size, self.intermediate_size, self.names
        return {f"{p}.{n['gate']}": ParamSpec((I, H)), f"{p}.{n['up']}": ParamSpec((I, H)), f"{p}.{n['down']}": ParamSpec((H, I))}

    def load(self, get: TensorGetter) -> None:
        p, n = self.prefix, self.names
        self.w_gate_up = torch.cat([get(f"{p}.{n['gate']}", "matrix"), get(f"{p}.{n['up']}", "matrix")], dim=0).contiguous()
        self.w_down = get(f"{p}.{n['down']}", "matrix").contiguous()

    takes_scaled_rows = True             # x goes straight into gate_up_swiglu() or linear()

    def forward(self, x, ctx):
        out, bias = self.forward_deferred(x, ctx)
        return (out.value() if isinstance(out, PendingProduct) else out), bias

    def forward_deferred(self, x, ctx):
        act = gate_up_swiglu(x, self.w_gate_up)          # the few rows of a decode step: product and activation in one kernel
        if act is None:
            gate_up = linear(x, self.w_gate_up)
            act = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
            kernels.swiglu(gate_up, act)
        return pending_product(act, self.w_down), None


@register_feed_forward("poly_norm_mlp")
class PolyNormMLP(FeedForward):
    """``down(act(up(x)))`` without gate and biases, with the PolyNorm activation: for a token's vector z of ``ff``
    values, ``act(z) = a N(z) + b N(z^2) + c N(z^3) + e`` with powers taken element by element, N(v) = v / sqrt(mean(v^2)
    + eps) over the token's ff values, and the four learned numbers (a, b, c, e) in one tensor. The up product's result
    and the three mean squares are float32; the activation is rounded once to the compute type for the down product,
    whose result is float32."""

    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, eps: float):
        self.prefix, self.hidden_size, self.intermediate_size, self.eps = prefix, int(hidden_size), int(intermediate_size), float(eps)
        self.w_up = self.w_down = self.act = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        p, H, I = self.prefix, self.hidden_size, self.intermediate_size
        return {f"{p}.up": ParamSpec((I, H)), f"{p}.down": ParamSpec((H, I)), f"{p}.act": ParamSpec((4,), role="vector", init="unit")}

    def load(self, get: TensorGetter) -> None:
        p = self.prefix
        self.w_up = get(f"{p}.up", "matrix").contiguous()
        self.w_down = get(f"{p}.down", "matrix").contiguous()
        self.act = get(f"{p}.act", "vector").float().contiguous()

    def forward(self, x, ctx):
        z = linear(x, self.w_up, out_dtype=torch.float32)
        act = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
        kernels.poly_norm(z, self.act, self.eps, act)
        return linear(act, self.w_down, out_dtype=torch.float32), None


@register_feed_forward("relu_squared_mlp")
class ReluSquaredMLP(FeedForward):
    """``down(max(up(x), 0)^2)`` without gate and biases; the result is float32."""

    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int):
        self.prefix, self.hidden_size, self.intermediate_size = prefix, int(hidden_size), int(intermediate_size)
        self.w_up = self.w_down = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        p, H, I = self.prefix, self.hidden_size, self.intermediate_size
        return {f"{p}.up": ParamSpec((I, H)), f"{p}.down": ParamSpec((H, I))}

    def load(self, get: TensorGetter) -> None:
        p = self.prefix
        self.w_up = get(f"{p}.up", "matrix").contiguous()
        self.w_down = get(f"{p}.down", "matrix").contiguous()

    def forward(self, x, ctx):
        z = linear(x, self.w_up)
        kernels.relu_squared(z, z)
        return linear(z, self.w_down, out_dtype=torch.float32), None


@register_feed_forward("xielu_mlp")
class XieluMLP(FeedForward):
    """``down(f(up(x) + b_up)) + b_down`` without gate, with the piecewise activation

        f(z) = a_pos z^2 + z / 2                       for z > 0
        f(z) = a_neg (exp(z) - 1 - z) + z / 2          for z <= 0

    whose two coefficients are learned as ``act = (p, q)``: a_pos = softplus(p), a_neg = 1/2 + softplus(q) (both
    branches have slope 1/2 at zero). The first product leaves float32, bias and activation are float32
    (``csrc/activations.cu``), the activation is rounded once to the compute type for the down product, whose result is
    float32. ``bias``: whether the two projections have biases (``<name>.b``)."""

    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, bias: bool = True):
        self.prefix, self.hidden_size, self.intermediate_size, self.bias = prefix, int(hidden_size), int(intermediate_size), bool(bias)
        self.w_up = self.w_down = self.b_up = self.b_down = None
        self.a_pos = self.a_neg = 0.0

    def param_specs(self) -> Dict[str, ParamSpec]:
        p, H, I = self.prefix, self.hidden_size, self.intermediate_size
        specs = {f"{p}.up": ParamSpec((I, H)), f"{p}.down": ParamSpec((H, I)), f"{p}.act": ParamSpec((2,), role="vector", init="unit")}
        if self.bias:
            specs.update({f"{p}.up.b": ParamSpec((I,), role="vector", init="small"),
                          f"{p}.down.b": ParamSpec((H,), role="vector", init="small")})
        return specs

    def load(self, get: TensorGetter) -> None:
        p = self.prefix
        self.w_up = get(f"{p}.up", "matrix").contiguous()
        self.w_down = get(f"{p}.down", "matrix").contiguous()
        if self.bias:
            self.b_up = get(f"{p}.up.b", "vector").float().contiguous()
            self.b_down = get(f"{p}.down.b", "vector").float().contiguous()
        # softplus in float64 on the host: the two numbers are constants of the layer from here on
        act = torch.nn.functional.softplus(get(f"{p}.act", "vector").double().cpu())
        self.a_pos, self.a_neg = float(act[0]), 0.5 + float(act[1])

    def forward(self, x, ctx):
        z = linear(x, self.w_up, out_dtype=torch.float32)
        act = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
        kernels.xielu(z, self.b_up, self.a_pos, self.a_neg, act)
        return linear(act, self.w_down, out_dtype=torch.float32), self.b_down


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    """``down(act(gate(x)) * up(x))`` without biases, with the activation as a parameter: ``gelu_tanh``, the tanh form of GELU
    ``0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))``, or ``silu``. Gate and up are one product against [gate; up] that
    leaves float32; activation and product are float32 (``csrc/activations.cu``) and rounded once to the compute type for
    the down product, whose result is float32. ``names``: the three matrices' names below ``prefix`` (keys ``gate``,
    ``up``, ``down``)."""

    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, activation: str = "gelu_tanh",
                 names: Optional[Dict[str, str]] = None):
        if activation not in ("gelu_tanh", "silu"):
            raise ValueError(f"unknown activation {activation!r} (known: gelu_tanh, silu)")
        self.prefix, self.hidden_size, self.intermediate_size, self.activation = prefix, int(hidden_size), int(intermediate_size), activation
        self.names = {"gate": "gate", "up": "up", "down": "down"}
        self.names.update(names or {})
        self.w_gate_up = self.w_down = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        p, H, I, n = self.prefix, self.hidden_size, self.intermediate_size, self.names
        return {f"{p}.{n['gate']}": ParamSpec((I, H)), f"{p}.{n['up']}": ParamSpec((I, H)), f"{p}.{n['down']}": ParamSpec((H, I))}

    def load(self, get: TensorGetter) -> None:
        p, n = self.prefix, self.names
        self.w_gate_up = torch.cat([get(f"{p}.{n['gate']}", "matrix"), get(f"{p}.{n['up']}", "matrix")], dim=0).contiguous()
        self.w_down = get(f"{p}.{n['down']}", "matrix").contiguous()

    def forward(self, x, ctx):
        gate_up = linear(x, self.w_gate_up, out_dtype=torch.float32)
        act = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
        kernels.gated_act(gate_up, act, self.activation)
        return linear(act, self.w_down, out_dtype=torch.float32), None
