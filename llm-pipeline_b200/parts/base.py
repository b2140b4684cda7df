"""Interfaces of the parts a model is put together from.

Every part takes its sizes and constants as constructor parameters, declares the tensors it
expects (``param_specs``: full tensor name -> ``ParamSpec``), receives them through ``load`` and
works on the tensors of one step. No part knows which model it is in.

* ``Norm.add_norm(stream, rows=None)``: folds the stream's pending sum into the float32 residual
  and returns the normalised rows in the compute type.
* ``PositionEncoding.tables(ctx)``: per-step tensors derived from the token positions (for the
  rotary kind: float32 cos/sin ``[tokens, rotary_dim / 2]``).
* ``Mixer.forward(x, ctx, cache) -> (out, bias)``: mixes tokens of the same request; ``cache`` is
  the ``LayerCache`` of this execution (pages and/or a state tensor). ``cache_spec()`` and
  ``state_spec()`` tell the cache manager what it needs.
* ``FeedForward.forward(x, ctx) -> (out, bias)``: works on each token alone.
* ``Block.forward(stream, ctx, cache)``: the arrangement of the above around the residual stream.
* ``DepthMix``: optional per layer; weights with which the results of all layers so far are summed into what goes on.

Optional, for the few rows of a decode step (``ops/linear.py``: a norm between two streaming products folded into
them): a mixer or feed-forward with ``forward_deferred(...)`` may return its last product as a ``PendingProduct``; a
norm with ``add_norm_deferred(stream, ctx)`` may take such a product from the stream and return ``ScaledRows``; a part
that sets ``takes_scaled_rows`` accepts those as its ``x`` (``linear()`` does). A block uses these only where both
sides offer them; parts without them see tensors only.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Hashable, Optional, Tuple

import torch

from ..cache.spec import KVPagesSpec, PagesSpec, StateSpec
from ..ops.linear import PendingProduct
from ..weights.source import ParamSpec

TensorGetter = Callable[[str, str], torch.Tensor]   # (full tensor name, role) -> tensor on the device


@dataclass
class LayerCache:
    """What one execution of a layer may touch: the pages of its cache id (``writes`` is False when
    an earlier execution owns them), the index of their group (for block tables and slot
    mappings in the step context), and the state tensor ``[slots, ...]`` of its cache id."""

    pages: Optional[torch.Tensor] = None
    group: Optional[int] = None
    state: Optional[torch.Tensor] = None
    writes: bool = True


class ResidualStream:
    """The hidden state between parts: a float32 residual ``[tokens, hidden]`` and a pending
    addend (with an optional bias vector) that the next norm folds in.

    Two more things may be pending, for blocks that ask for them: a norm of the addend itself (``add(..., norm=)``: the
    addend is normed before it is added), and a mix over depth (``mix(weights, index)``: once the addend is in, the
    residual is this layer's result; it is kept as ``history[index]`` and replaced by ``sum_j weights[j] history[j]``,
    j = 0 .. index). ``history`` is float32 ``[results, tokens, hidden]`` with the embedding's output at 0; only models
    with such a mix have one. The next norm kernel does all of it in one pass over the row.

    A block whose sublayers run side by side leaves two addends (``add``, then ``add_beside``); a norm that knows of it
    (``layer_norm``) adds both in its kernel, everybody else sees their sum as the one pending addend."""

    def __init__(self, residual: torch.Tensor, history: Optional[torch.Tensor] = None):
        self.residual = residual
        self._pending = None
        self._beside = None                           # a second addend, of a sublayer that ran beside the first
        self.pending_bias: Optional[torch.Tensor] = None
        self.pending_norm = None                      # a Norm part with ``weight`` and ``eps``: norms the addend
        self.pending_mix: Optional[Tuple[torch.Tensor, int]] = None
        self.history = history

    def add(self, delta, bias: Optional[torch.Tensor] = None, norm=None) -> None:
        """``delta``: a tensor, or a product not yet taken (``ops.linear.PendingProduct``) that the next norm may
        fold into its own work. ``norm``: the addend passes through this norm first."""
        if self._pending is not None or self.pending_mix is not None:
            raise RuntimeError("the residual stream already holds a pending addend")
        self._pending, self.pending_bias, self.pending_norm = delta, bias, norm

    def add_beside(self, delta: torch.Tensor) -> None:
        """A second addend beside the pending one (the other sublayer of a block whose sublayers read the same input);
        without bias or norm of its own."""
        if self._pending is None or self._beside is not None or self.pending_norm is not None or self.pending_mix is not None:
            raise RuntimeError("a second addend needs a plain first one and no other second one")
        self._beside = delta.value() if isinstance(delta, PendingProduct) else delta

    def take_addends(self):
        """(first, second) pending addends as tensors, for a norm whose kernel adds both; only for a plain stream without a
        pending bias. The caller clears them (``clear_addends``) once they are in the residual."""
        return self.pending_raw(), self._beside

    def pending_raw(self) -> Optional[torch.Tensor]:
        if isinstance(self._pending, PendingProduct):
            self._pending = self._pending.value()
        return self._pending

    def clear_addends(self) -> None:
        self._pending, self._beside, self.pending_bias = None, None, None

    def mix(self, weights: torch.Tensor, index: int) -> None:
        """What the stream holds once the pending addend is in is result ``index``; what goes on is the weighted sum of
        the results 0 .. index (``weights``: float32, one per result)."""
        if self.history is None:
            raise RuntimeError("this stream keeps no history of layer results; the model's specification names no depth mix")
        if self.pending_mix is not None:
            raise RuntimeError("the residual stream already holds a pending mix")
        self.pending_mix = (weights, int(index))

    @property
    def plain(self) -> bool:
        """Nothing is pending but, at most, an addend with its bias."""
        return self.pending_norm is None and self.pending_mix is None

    @property
    def pending(self) -> Optional[torch.Tensor]:
        """The pending addend as a tensor (a product not yet taken is taken now; two addends become their float32 sum)."""
        if isinstance(self._pending, PendingProduct):
            self._pending = self._pending.value()
        if self._beside is not None:
            self._pending, self._beside = self._pending.float() + self._beside.float(), None
        return self._pending

    @pending.setter
    def pending(self, delta) -> None:
        self._pending = delta

    def fold(self, weight: Optional[torch.Tensor] = None, eps: float = 0.0, out: Optional[torch.Tensor] = None,
             rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Everything pending in one kernel, and the RMS norm of the result by ``weight`` into ``out`` if given. With
        ``rows`` only those rows are computed and the stream stays as it is."""
        from ..ops import kernels

        delta = self.pending
        if delta is not None and self.pending_bias is not None:
            delta = delta.float() + self.pending_bias.float()
        norm, mixing = self.pending_norm, self.pending_mix
        kernels.add_norm_mix(self.residual, delta=delta,
                             delta_weight=norm.weight if norm is not None and delta is not None else None,
                             delta_eps=norm.eps if norm is not None else 0.0,
                             history=self.history if mixing is not None else None,
                             mix=mixing[0] if mixing is not None else None, index=mixing[1] if mixing is not None else 0,
                             weight=weight, eps=eps, out=out, rows=rows)
        if rows is None:
            self._pending, self.pending_bias, self.pending_norm, self.pending_mix = None, None, None, None
        return out

    def settle(self) -> torch.Tensor:
        """Add what is pending into the residual and return it: the whole state of the stream in one float32 tensor
        (between pieces of a step that are captured apart; the norms fold the addend in on their own otherwise)."""
        if not self.plain:
            self.fold()
            return self.residual
        pending = self.pending
        if pending is not None:
            self.residual = self.residual + pending.float()
            if self.pending_bias is not None:
                self.residual = self.residual + self.pending_bias.float()
            self._pending, self.pending_bias = None, None
        return self.residual

    def take_pending_product(self) -> Optional[PendingProduct]:
        """The pending addend if it is a product not yet taken and without bias, which is then the caller's to add;
        else None, and nothing changes."""
        if isinstance(self._pending, PendingProduct) and self.pending_bias is None and self.plain and self._beside is None:
            product, self._pending = self._pending, None
            return product
        return None


class Part:
    prefix: str = ""
    # True when the part's work for a step can be captured in a CUDA graph and replayed: fixed launch
    # shapes for fixed step shapes, no host synchronisation, and running the step twice leaves the same
    # state. The built-in parts are; a part that does not say so keeps the whole model on eager steps.
    graph_safe: bool = False

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def copies(self) -> Dict[str, str]:
        """Names of optional tensors of this part that, where a checkpoint holds them, must repeat
        another tensor: {own name: the name it repeats}. The loader compares the two."""
        return {}

    def load(self, get: TensorGetter) -> None:
        pass


class Norm(Part):
    def add_norm(self, stream: ResidualStream, ctx, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    # Streams of position ids the encoding reads for every token: ``ctx.position_ids`` is [streams of the model, N].
    # With one stream (the default) that is each token's place in its request; an encoding with more (a place along
    # several axes) gets what the request brought (``StepEntry.positions``), or the place in every stream.
    streams: int = 1

    def tables(self, ctx):
        raise NotImplementedError


class Mixer(Part):
    def cache_spec(self) -> Optional[PagesSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def graph_key(self, shape) -> Hashable:
        """For a mixer whose launches for a step of single tokens depend on more than the number of requests: what they
        depend on, as a hashable value (``shape``: ``engine.StepShape``). It becomes part of the key under which the step
        function captures and replays such steps. None: nothing."""
        return None

    def captured_context_limit(self) -> Optional[int]:
        """The longest context (keys a request sees) for which the mixer's kernels can be sized in a captured step of
        single tokens; None: any. Mixers of one ``graph_key_group`` answer alike."""
        return None

    def graph_key_group(self) -> Hashable:
        """Mixers that return equal values here give equal ``graph_key`` for every step; the model then asks one of
        them. The default keeps every mixer apart."""
        return id(self)

    def forward(self, x: torch.Tensor, ctx, cache: LayerCache) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        raise NotImplementedError


class DepthMix(Part):
    """How a layer's result is combined with the results of the layers before it (and the embedding's output) into
    what the next layer reads. ``weights`` (float32, on the device after ``load``) holds one weight per result so far;
    ``index`` is the place of this layer's result among them. A block that has one calls
    ``stream.mix(self.depth_mix.weights, self.depth_mix.index)`` at its end."""

    weights: Optional[torch.Tensor] = None
    index: int = 0


class Embedding(Part):
    def forward(self, ctx) -> torch.Tensor:
        """float32 residual [tokens, hidden] of ctx.token_ids"""
        raise NotImplementedError


class Head(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        """float32 logits [rows, vocab]"""
        raise NotImplementedError


class Block:
    """An arrangement of a mixer, a feed-forward and named norms around the residual stream. ``norms`` maps the
    names of ``LayerSpec.named_norms()`` to the built norms; the two of a pre-norm block may also come as the third
    and fourth argument. ``NORMS`` lists the names a block kind needs; building a layer without one of them fails."""

    NORMS: Tuple[str, ...] = ()

    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], mixer_norm: Optional[Norm] = None,
                 feed_forward_norm: Optional[Norm] = None, norms: Optional[Dict[str, Norm]] = None,
                 depth_mix: Optional["DepthMix"] = None):
        self.mixer, self.feed_forward, self.depth_mix = mixer, feed_forward, depth_mix
        self.norms: Dict[str, Norm] = {}
        if mixer_norm is not None:
            self.norms["mixer"] = mixer_norm
        if feed_forward_norm is not None:
            self.norms["feed_forward"] = feed_forward_norm
        self.norms.update(norms or {})
        missing = [name for name in self.needed_norms() if name not in self.norms]
        if missing:
            raise ValueError(f"a {type(self).__name__} needs the norms {list(self.NORMS)}; the layer lacks {missing}")

    def needed_norms(self) -> Tuple[str, ...]:
        """The norms this layer cannot be built without (``NORMS``, unless the kind says otherwise for a layer
        without a feed-forward)."""
        return self.NORMS

    @property
    def mixer_norm(self) -> Optional[Norm]:
        return self.norms.get("mixer")

    @property
    def feed_forward_norm(self) -> Optional[Norm]:
        return self.norms.get("feed_forward")

    def parts(self):
        return tuple(self.norms.values()) + tuple(
            part for part in (self.mixer, self.feed_forward, self.depth_mix) if part is not None)

    def state_spec(self) -> Optional[StateSpec]:
        """What the layer keeps per request beside pages: the mixer's state, unless the block kind keeps more."""
        return self.mixer.state_spec()

    def forward(self, stream: ResidualStream, ctx, cache: LayerCache) -> None:
        raise NotImplementedError
