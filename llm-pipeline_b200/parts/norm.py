"""Norms fused with the residual add: RMSNorm, and layer norm with weight and bias.

Formula of src/llm_pipeline/models/qwen3/custom_builder.py:53-58: in float32,
``weight * (x * rsqrt(mean(x^2) + eps))``, rounded once to the compute type. The residual adds of
custom_builder.py:244,250 are folded in: the addend left by the previous part is summed into the
float32 residual by the same kernel that normalises it."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import kernels
from ..ops.linear import residual_product
from ..weights.source import ParamSpec
from .base import Norm, ResidualStream, TensorGetter
from .registry import register_norm


@register_norm("rms_norm")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, prefix: str, size: int, eps: float, offset: float = 0.0, name: Optional[str] = None, gain: float = 1.0):
        """``offset``: the stored weight w stands for ``offset + w`` (1.0 for weights kept around zero); ``name``: the
        tensor's full name where it is not ``<prefix>.weight``; ``gain``: a constant factor on the normed rows (a layer
        that adds ``m * norm(sublayer)`` to its residual gives that norm the gain m)."""
        self.prefix, self.size, self.eps, self.offset, self.gain = prefix, int(size), float(eps), float(offset), float(gain)
        self.name = name or f"{prefix}.weight"
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.size,), role="vector", init="small" if self.offset else "norm")}

    def load(self, get: TensorGetter) -> None:
        self.weight = get(self.name, "vector").contiguous()
        if self.offset or self.gain != 1.0:
            self.weight = ((self.weight.float() + self.offset) * self.gain).contiguous()      # the factor itself, float32

    def add_norm(self, stream: ResidualStream, ctx, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        count = rows.numel() if rows is not None else stream.residual.shape[0]
        out = torch.empty((count, self.size), dtype=ctx.dtype, device=stream.residual.device)
        if not stream.plain or (stream.pending is not None and stream.pending.dtype != ctx.dtype):
            # the addend has a norm of its own or another type, or the layers' results are mixed: the general kernel
            return stream.fold(self.weight, self.eps, out, rows)
        kernels.add_rmsnorm(stream.residual, stream.pending, self.weight, self.eps, out,
                            delta_bias=stream.pending_bias, rows=rows)
        if rows is None:
            stream.pending, stream.pending_bias = None, None
        return out

    def add_norm_deferred(self, stream: ResidualStream, ctx):
        """As ``add_norm`` for all rows, but a pending product of a decode step's few rows is added into the residual by
        its own kernel, which leaves the rows normalised but for their factors (``ScaledRows``) to the product after."""
        product = stream.take_pending_product() if stream.plain else None
        if product is None:
            return self.add_norm(stream, ctx)
        residual = stream.residual
        if product.accumulate:
            # many rows: the library's product adds itself into the residual, the norm kernel only reads it
            if not kernels.library_add_product(residual, product.x, product.weight):
                stream.add(product.value())
            return self.add_norm(stream, ctx)

        def finished() -> torch.Tensor:
            # for a consumer that cannot apply the factors: the norm of the residual as it now is
            out = torch.empty((residual.shape[0], self.size), dtype=ctx.dtype, device=residual.device)
            return kernels.add_rmsnorm(residual, None, self.weight, self.eps, out)

        return residual_product(product, residual, self.weight, self.eps, finished)


@register_norm("layer_norm")
class LayerNorm(Norm):
    """``(x - mean) / sqrt(var + eps) * w + b`` with var the mean of the squared deviations, in float32, rounded once to
    the compute type. The kernel first adds what is pending on the stream into the float32 residual: one addend, or the
    two of a block whose sublayers ran side by side. ``name`` / ``bias_name``: the tensors' full names where they are not
    ``<prefix>.weight`` / ``<prefix>.bias``."""

    graph_safe = True

    def __init__(self, prefix: str, size: int, eps: float, name: Optional[str] = None, bias_name: Optional[str] = None):
        self.prefix, self.size, self.eps = prefix, int(size), float(eps)
        self.name = name or f"{prefix}.weight"
        self.bias_name = bias_name or f"{prefix}.bias"
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.size,), role="vector", init="norm"),
                self.bias_name: ParamSpec((self.size,), role="vector", init="small")}

    def load(self, get: TensorGetter) -> None:
        self.weight = get(self.name, "vector").contiguous()
        self.bias = get(self.bias_name, "vector").contiguous()
        if self.weight.dtype != self.bias.dtype:
            self.weight, self.bias = self.weight.float(), self.bias.float()

    def add_norm(self, stream: ResidualStream, ctx, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        count = rows.numel() if rows is not None else stream.residual.shape[0]
        out = torch.empty((count, self.size), dtype=ctx.dtype, device=stream.residual.device)
        if not stream.plain:
            stream.fold()                               # a normed addend or a mix over depth: the general kernel first
        first, second = stream.take_addends()
        if first is not None and stream.pending_bias is not None:
            first, second = stream.pending, None        # a bias on the addend: summed by the stream
            first = first.float() + stream.pending_bias.float()
        kernels.add_layernorm(stream.residual, first, second, self.weight, self.bias, self.eps, out, rows=rows)
        if rows is None:
            stream.clear_addends()
        return out


@register_norm("rms_norm_multi")
class RMSNormMulti(Norm):
    """Several RMS norms of the same rows that differ in their weights only (the sublayers of a layer that run side by
    side, each behind a norm of its own): ``x / sqrt(mean(x^2) + eps) * w_j`` for every name in ``names``, from one pass
    over the row. The kernel first adds what is pending on the stream into the float32 residual: one addend (with its
    bias) or the two of sublayers that ran side by side. ``add_norm`` gives the first weight's rows in the compute type
    (so the part also serves as a plain norm, with ``rows`` for a model's last norm); ``add_norm_all`` gives all of them
    side by side as float32 ``[tokens, k size]`` for a reader that goes on in 32-bit."""

    graph_safe = True

    def __init__(self, prefix: str, size: int, eps: float, names, unused=()):
        """``unused``: names of weights a checkpoint may hold although no sublayer of this layer reads them."""
        self.prefix, self.size, self.eps = prefix, int(size), float(eps)
        self.names, self.unused = tuple(names), tuple(unused)
        if not self.names:
            raise ValueError("a norm needs at least one weight")
        self.weights: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {name: ParamSpec((self.size,), role="vector", init="norm") for name in self.names}
        specs.update({name: ParamSpec((self.size,), role="vector", optional=True, init="norm") for name in self.unused})
        return specs

    def load(self, get: TensorGetter) -> None:
        self.weights = torch.stack([get(name, "vector").float() for name in self.names]).contiguous()

    def _run(self, stream: ResidualStream, weights: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor]) -> torch.Tensor:
        if not stream.plain:
            stream.fold()                               # a normed addend or a mix over depth: the general kernel first
        first, second = stream.take_addends()
        kernels.add_rmsnorm_multi(stream.residual, first, second, stream.pending_bias if first is not None else None, weights,
                                  self.eps, out, rows=rows)
        if rows is None:
            stream.clear_addends()
        return out

    def add_norm(self, stream: ResidualStream, ctx, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        count = rows.numel() if rows is not None else stream.residual.shape[0]
        out = torch.empty((count, self.size), dtype=ctx.dtype, device=stream.residual.device)
        return self._run(stream, self.weights[:1], out, rows)

    def add_norm_all(self, stream: ResidualStream, ctx) -> torch.Tensor:
        out = torch.empty((stream.residual.shape[0], len(self.names) * self.size), dtype=torch.float32, device=stream.residual.device)
        return self._run(stream, self.weights, out, None)
