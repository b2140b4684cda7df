"""Arrangements of a mixer, a feed-forward and their norms around the residual stream.

``pre_norm_residual`` is the decoder layer of
src/llm_pipeline/models/qwen3/custom_builder.py:222-255: ``x += mixer(norm1(x))`` then
``x += feed_forward(norm2(x))``. The sums are not taken here: each part's output is left pending
on the stream and the next norm kernel adds it into the float32 residual."""

from __future__ import annotations

import torch

from ..cache.spec import StateSpec
from ..ops import kernels
from .base import Block, LayerCache, ResidualStream
from .input_conv import InputConv
from .registry import register_block


@register_block("pre_norm_residual")
class PreNormResidualBlock(Block):
    NORMS = ("mixer", "feed_forward")

    def forward(self, stream: ResidualStream, ctx, cache: LayerCache) -> None:
        h = self._norm(self.mixer_norm, self.mixer, stream, ctx)
        out, bias = getattr(self.mixer, "forward_deferred", self.mixer.forward)(h, ctx, cache)
        stream.add(out, bias)
        h = self._norm(self.feed_forward_norm, self.feed_forward, stream, ctx)
        out, bias = getattr(self.feed_forward, "forward_deferred", self.feed_forward.forward)(h, ctx)
        stream.add(out, bias)

    @staticmethod
    def _norm(norm, consumer, stream: ResidualStream, ctx):
        """The norm's rows for ``consumer``: with their factors still to be applied where the norm can leave them so
        and the consumer takes them so."""
        deferred = getattr(norm, "add_norm_deferred", None)
        if deferred is not None and getattr(consumer, "takes_scaled_rows", False):
            return deferred(stream, ctx)
        return norm.add_norm(stream, ctx)


@register_block("sandwich_norm_residual")
class SandwichNormResidualBlock(Block):
    """A norm before and after each sublayer: ``x += norm_out(mixer(norm_in(x)))``, then the same around the
    feed-forward if the layer has one. Neither the outer norms nor the sums are taken here: a sublayer's output is left
    pending on the stream together with the norm it has to pass, and the next norm kernel norms it, adds it into the
    float32 residual and norms the sum for its own reader in one pass. A layer with a depth mix asks the stream for it
    at its end (``ResidualStream.mix``), which the same kernel does."""

    NORMS = ("mixer", "mixer_out", "feed_forward", "feed_forward_out")

    def needed_norms(self):
        return self.NORMS if self.feed_forward is not None else ("mixer", "mixer_out")

    def forward(self, stream: ResidualStream, ctx, cache: LayerCache) -> None:
        h = self.norms["mixer"].add_norm(stream, ctx)
        out, bias = self.mixer.forward(h, ctx, cache)
        stream.add(out, bias, norm=self.norms["mixer_out"])
        if self.feed_forward is not None:
            h = self.norms["feed_forward"].add_norm(stream, ctx)
            out, bias = self.feed_forward.forward(h, ctx)
            stream.add(out, bias, norm=self.norms["feed_forward_out"])
        if self.depth_mix is not None:
            stream.mix(self.depth_mix.weights, self.depth_mix.index)


@register_block("parallel_residual")
class ParallelResidualBlock(Block):
    """Both sublayers read the same residual: ``x += mixer(norm(x)) + feed_forward(norm(x))`` (a layer without a
    feed-forward adds the mixer's output alone). Neither sum is taken here: the two outputs are left pending on the
    stream side by side, and the next norm kernel adds both into the float32 residual before it norms the row.

    A norm that offers ``add_norm_all`` (``rms_norm_multi``) gives each sublayer its own weighting of the normed row, in the
    order mixer, feed-forward. ``input_conv`` = {"taps": K, "names": [one tensor per sublayer]} puts a short causal
    convolution beside the identity in front of each sublayer (``parts/input_conv.py``); its carried inputs lie at the
    front of the layer's state vector, the mixer's state (if it has one) behind them."""

    NORMS = ("mixer",)

    def __init__(self, mixer, feed_forward, mixer_norm=None, feed_forward_norm=None, norms=None, depth_mix=None, input_conv=None):
        super().__init__(mixer, feed_forward, mixer_norm, feed_forward_norm, norms, depth_mix)
        self.sublayers = 1 if feed_forward is None else 2
        self.input_conv = None
        norm = self.norms["mixer"]
        if input_conv is not None:
            if not hasattr(norm, "add_norm_all"):
                raise ValueError("a convolution in front of the sublayers reads float32 rows: the layer's norm must offer add_norm_all")
            names = list(input_conv["names"])
            if len(names) != self.sublayers:
                raise ValueError(f"a layer of {self.sublayers} sublayers needs as many input convolutions, got {names}")
            self.input_conv = InputConv(norm.size, int(input_conv["taps"]), names, input_conv.get("unused", ()))
        if hasattr(norm, "add_norm_all") and len(norm.names) != self.sublayers:
            raise ValueError(f"a layer of {self.sublayers} sublayers needs as many norm weights, got {list(norm.names)}")
        self._own_state = self.input_conv.state_entries() if self.input_conv is not None else 0
        inner = mixer.state_spec()
        if self._own_state and inner is not None and (inner.dtype != torch.float32 or len(inner.shape) != 1):
            raise ValueError("behind an input convolution a mixer keeps its state as a float32 vector")
        self._mixer_state = inner

    def parts(self):
        return super().parts() + ((self.input_conv,) if self.input_conv is not None else ())

    def state_spec(self):
        if not self._own_state:
            return self._mixer_state
        return StateSpec((self._own_state + (self._mixer_state.shape[0] if self._mixer_state is not None else 0),), torch.float32)

    def _inputs(self, stream: ResidualStream, ctx, cache: LayerCache):
        """What the mixer and the feed-forward read."""
        norm = self.norms["mixer"]
        if not hasattr(norm, "add_norm_all"):
            h = norm.add_norm(stream, ctx)
            return h, h
        normed = norm.add_norm_all(stream, ctx)                       # float32 [tokens, sublayers * size]
        if self.input_conv is not None:
            hs = self.input_conv.forward(normed, ctx, cache.state if self._own_state else None, 0)
        else:
            hs = torch.empty((self.sublayers, normed.shape[0], norm.size), dtype=ctx.dtype, device=normed.device)
            for j in range(self.sublayers):
                kernels.convert_rows(normed[:, j * norm.size:(j + 1) * norm.size], hs[j])
        return hs[0], hs[self.sublayers - 1]

    def forward(self, stream: ResidualStream, ctx, cache: LayerCache) -> None:
        h_mixer, h_ff = self._inputs(stream, ctx, cache)
        if self._own_state:
            state = cache.state[:, self._own_state:] if self._mixer_state is not None else None
            cache = LayerCache(pages=cache.pages, group=cache.group, state=state, writes=cache.writes)
        out, bias = self.mixer.forward(h_mixer, ctx, cache)
        stream.add(out, bias)
        if self.feed_forward is not None:
            out, bias = self.feed_forward.forward(h_ff, ctx)
            if bias is not None:
                out = out.float() + bias.float()
            stream.add_beside(out)
