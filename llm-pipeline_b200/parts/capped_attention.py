"""Softmax attention with grouped key/value heads, capped scores, a distance bias, a sliding window that keeps the first
tokens, a sink in the denominator and a gate on the output (``capped_attention``).

With h the mixer's input, H query heads, G key/value heads (head i uses key/value head i // (H / G)), queries and keys
of ``dim`` entries and values of ``vdim``::

    q, k, v = Wq h + bq, Wk h + bk, Wv h + bv
    v <- v / sqrt(mean(v^2) + eps)  per head, where ``value_norm_eps`` is given (cached so)
    s(i, j) = (q(i) . k(j)) * scale;   s <- cap * tanh(s / cap)  where ``softcap`` is given
    s(i, j) <- s(i, j) - slope_h (i - j),   slope_h = 2^(-8 (h + 1) / H)                  where ``distance_bias`` is set
    seen(i, j) = j <= i and (i - j < window or j < keep_first)                            (no window: every j <= i)
    p(i, j) = exp(s(i, j)) / (exp(sink_h) + sum_seen exp(s))       sink_h: a constant (``sink`` = 0.0: one is added to the
                                                                   denominator), a tensor per head (``sink`` = "learned"), or none
    o_h(i) = sum_j p(i, j) v(j);   o <- o * sigmoid(Wg h)  where ``gate`` is set;   out = Wo o + bo

No rotation: positions enter through the distance bias and the mask alone; kept tokens keep their true positions.
The projections that read h are one product against [Wq; Wk; Wv; Wg] with a float32 result; one kernel adds the biases,
norms the values, writes the queries in the compute type and the token's [k | v] rows into its page slot; the attention
kernel reads all keys and values from pages, this step's included, and applies the gate as it stores. Scores, cap, bias,
softmax and weighted sums are float32 (``csrc/capped_attention.cu``: any sizes, both types; ``csrc/capped_attention_mma.cu``:
bfloat16 on the tensor cores for key and value sizes of 16, 32, 64 and 128, the probabilities rounded to bfloat16 for the
product with the values). The pages of a windowed layer go back to the pool
as the window passes them, but for those of the kept tokens (``HeadRowPagesSpec(window, keep_first)``)."""

from __future__ import annotations

from typing import Dict, Optional, Union

import torch

from ..cache.spec import HeadRowPagesSpec
from ..ops import kernels
from ..ops.linear import linear
from ..weights.source import ParamSpec
from .attention import AttentionPolicy
from .base import LayerCache, Mixer, TensorGetter
from .registry import register_mixer


@register_mixer("capped_attention")
class CappedAttention(Mixer):
    graph_safe = True      # a step only writes this step's keys and values: repeating it changes nothing

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float,
                 softcap: Optional[float] = None, window: Optional[int] = None, keep_first: int = 0, distance_bias: bool = False,
                 sink: Union[None, float, str] = None, value_norm_eps: Optional[float] = None, gate: bool = False, bias: bool = True,
                 names: Optional[Dict[str, str]] = None):
        """``names``: the tensors' names below ``prefix`` where they differ from ``q``, ``k``, ``v``, ``o``, ``g``, ``sink``
        (biases add ``.b``)."""
        self.prefix, self.hidden_size = prefix, int(hidden_size)
        self.num_heads, self.num_kv_heads, self.dim, self.vdim = int(num_heads), int(num_kv_heads), int(dim), int(vdim)
        if self.num_heads <= 0 or self.num_kv_heads <= 0 or self.num_heads % self.num_kv_heads:
            raise ValueError(f"{self.num_heads} query heads cannot share {self.num_kv_heads} key/value heads")
        if not 0 < self.vdim <= 512:
            raise ValueError(f"the capped attention kernel takes value sizes up to 512, got {self.vdim}")
        self.scale, self.softcap = float(scale), float(softcap) if softcap else 0.0
        self.window = int(window) if window else None
        self.keep_first = int(keep_first or 0) if self.window else 0
        self.distance_bias, self.gate, self.bias = bool(distance_bias), bool(gate), bool(bias)
        if sink is not None and sink != "learned" and not isinstance(sink, (int, float)):
            raise ValueError(f"a sink is a number, 'learned' or None, got {sink!r}")
        self.sink = sink
        self.value_norm_eps = None if value_norm_eps is None else float(value_norm_eps)
        self.q_size, self.k_size, self.v_size = self.num_heads * self.dim, self.num_kv_heads * self.dim, self.num_kv_heads * self.vdim
        self.o_size = self.num_heads * self.vdim
        self.names = {n: n for n in ("q", "k", "v", "o", "g", "sink")}
        self.names.update(names or {})
        self.w_in = self.b_qkv = self.w_o = self.b_o = self.slopes = self.sinks = None

    def cache_spec(self) -> HeadRowPagesSpec:
        return HeadRowPagesSpec(self.num_kv_heads, self.dim + self.vdim, self.window, self.keep_first)

    def graph_key_group(self):
        return ("capped_attention", self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.window, self.keep_first)

    def _name(self, key: str) -> str:
        return f"{self.prefix}.{self.names[key]}"

    def _tiles(self, ctx, per_tile: int):
        key = ("capped_attention_tiles", per_tile)
        tiles = ctx.memo.get(key)
        if tiles is None:
            if ctx.max_q_len == 1:
                # one token a request: tile r is request r (made on the device, so that a captured step holds no copy from the host)
                tiles = (torch.arange(ctx.num_requests, dtype=torch.int32, device=ctx.device),
                         torch.zeros(ctx.num_requests, dtype=torch.int32, device=ctx.device))
            else:
                req, tok0, _seg, _slot, _places = AttentionPolicy.plan_items(ctx.starts, ctx.q_lens, per_tile, 0, 1, 1, kernels.sm_count())
                host = torch.tensor([req, tok0], dtype=torch.int32).pin_memory()
                dev = host.to(ctx.device, non_blocking=True)
                tiles = (dev[0].contiguous(), dev[1].contiguous())
            ctx.memo[key] = tiles
        return tiles

    def param_specs(self) -> Dict[str, ParamSpec]:
        D = self.hidden_size
        sizes = {"q": self.q_size, "k": self.k_size, "v": self.v_size}
        specs = {self._name(n): ParamSpec((sizes[n], D)) for n in ("q", "k", "v")}
        specs[self._name("o")] = ParamSpec((D, self.o_size))
        if self.bias:
            specs.update({self._name(n) + ".b": ParamSpec((sizes[n],), role="vector", init="small") for n in ("q", "k", "v")})
            specs[self._name("o") + ".b"] = ParamSpec((D,), role="vector", init="small")
        if self.gate:
            specs[self._name("g")] = ParamSpec((self.o_size, D))
        if self.sink == "learned":
            specs[self._name("sink")] = ParamSpec((self.num_heads,), role="vector", init="small")
        return specs

    def load(self, get: TensorGetter) -> None:
        parts = [get(self._name(n), "matrix") for n in ("q", "k", "v")]
        if self.gate:
            parts.append(get(self._name("g"), "matrix"))
        self.w_in = torch.cat(parts, dim=0).contiguous()
        self.w_o = get(self._name("o"), "matrix").contiguous()
        device = self.w_o.device
        if self.bias:
            self.b_qkv = torch.cat([get(self._name(n) + ".b", "vector").float() for n in ("q", "k", "v")]).contiguous()
            self.b_o = get(self._name("o") + ".b", "vector").float().contiguous()
        H = self.num_heads
        self.slopes = (torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=torch.float64).float().to(device)
                       if self.distance_bias else None)
        if self.sink == "learned":
            self.sinks = get(self._name("sink"), "vector").float().contiguous()
        elif self.sink is not None:
            self.sinks = torch.full((H,), float(self.sink), dtype=torch.float32, device=device)

    def forward(self, x, ctx, cache: LayerCache):
        if cache.pages is None or cache.group is None:
            raise RuntimeError("the capped attention mixer needs the pages of its cache")
        N = ctx.num_tokens
        proj = linear(x, self.w_in, out_dtype=torch.float32)               # [N, q | k | v | gate]
        width = self.q_size + self.k_size + self.v_size
        q = torch.empty((N, self.q_size), dtype=x.dtype, device=x.device)
        kernels.capped_qkv_post(proj[:, :width], self.b_qkv, self.value_norm_eps, q, ctx.slot_mapping[cache.group] if cache.writes else None,
                                cache.pages if cache.writes else None, self.num_heads, self.num_kv_heads, self.dim, self.vdim)
        out = torch.empty((N, self.o_size), dtype=x.dtype, device=x.device)
        gate = proj[:, width:] if self.gate else None
        if kernels.capped_mma_supports(x.dtype, self.dim, self.vdim) and (width % 2 == 0 or not self.gate):
            # bfloat16 and sizes the tensor-core kernel has instances of: prompts in tiles of 64 rows (token, head of a group),
            # single tokens with the four warps of a block sharing the keys
            tile_req, tile_tok0 = self._tiles(ctx, kernels.capped_mma_tokens_per_tile(self.num_heads, self.num_kv_heads))
            kernels.capped_attention_mma(q, cache.pages, ctx.block_tables[cache.group], ctx.q_start, ctx.ctx_len, tile_req, tile_tok0, out,
                                         self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.window or 0, self.keep_first,
                                         self.scale, self.softcap, slopes=self.slopes, sink=self.sinks, gate=gate, split=ctx.max_q_len == 1)
            return linear(out, self.w_o, out_dtype=torch.float32), self.b_o
        kernels.capped_attention(q, cache.pages, ctx.block_tables[cache.group], ctx.token_request, ctx.positions, out, self.num_heads,
                                 self.num_kv_heads, self.dim, self.vdim, self.window or 0, self.keep_first, self.scale, self.softcap,
                                 slopes=self.slopes, sink=self.sinks, gate=proj[:, width:] if self.gate else None)
        return linear(out, self.w_o, out_dtype=torch.float32), self.b_o
