"""Causal attention without softmax, with the heads' weights mixed before they meet the values.

With h the mixer's input, H query heads, G key/value heads (head i uses key/value head i // (H / G)), queries and keys
of ``dim`` entries and values of ``vdim``::

    q, k, v = Wq h + bq, Wk h + bk, Wv h + bv;   the first ``rotary_dim`` entries of every q and k head are rotated
    s_g(i, j) = (q_g(i) . k(j)) * scale;   s <- cap * tanh(s / cap)  where a cap is given
    w_g(i, j) = sigmoid(s_g(i, j) + head_bias[g])  for j <= i, else 0        not normalised over keys
    m_h(i, j) = sum_g talk[h, g] w_g(i, j)                                   the heads' weights, mixed
    o_h(i) = sum_j m_h(i, j) v(j);   out = Wo [o_0 .. o_(H-1)]

The three projections are one product against [Wq; Wk; Wv] with a float32 result; one kernel adds the biases, rotates,
writes the queries in the compute type and the token's [k | v] rows into its page slot; the attention kernel reads all
keys and values from pages, this step's included. Scores, weights, their mix and the weighted sums are float32
(``csrc/sigmoid_attention.cu``). Because no sum over keys normalises anything, ranges of keys add up: steps with few
tokens over long contexts give every fixed range of keys a block of its own. In bfloat16, for the head counts and sizes
it has instances of, the tensor-core kernel (``csrc/sigmoid_attention_mma.cu``) takes prompts and single tokens alike:
tiles of up to 16 new tokens of a request, scores and values on mma.sync, the weights and their mix in float32, the mixed
weights rounded to bfloat16 for the product with the values."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.spec import HeadRowPagesSpec
from ..ops import kernels
from ..ops.linear import linear
from ..weights.source import ParamSpec
from .attention import AttentionPolicy
from .base import LayerCache, Mixer, TensorGetter
from .registry import register_mixer


@register_mixer("sigmoid_attention")
class SigmoidAttention(Mixer):
    graph_safe = True      # a step only writes this step's keys and values: repeating it changes nothing

    # Blocks per SM below which a step's tokens are too few to fill the GPU and the keys are cut into segments.
    SEGMENTS_BELOW_BLOCKS_PER_SM = 2.0
    MMA_SEGMENTS_BELOW_BLOCKS_PER_SM = 0.5      # the same for the tensor-core kernel, a block of which fills an SM
    MMA_LONG_SEGMENTS_BELOW_BLOCKS_PER_SM = 2.0 # below this, long prompts are cut into long key ranges
    SEGMENTS_MAX_BYTES = 256 << 20              # the float32 partial sums of all segments never take more than this

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float,
                 softcap: Optional[float] = None, bias: bool = True, head_mix: bool = True, head_bias: bool = True,
                 position: Optional[str] = None, rotary_dim: int = 0, names: Optional[Dict[str, str]] = None):
        """``head_mix`` / ``head_bias``: whether the design has the matrix that mixes the heads' weights and the number
        per head that is added to the score (without: the identity and zeros). ``names``: the tensors' names below
        ``prefix`` where they differ from ``q``, ``k``, ``v``, ``o``, ``talk``, ``pb`` (biases add ``.b``)."""
        self.prefix, self.hidden_size = prefix, int(hidden_size)
        self.num_heads, self.num_kv_heads, self.dim, self.vdim = int(num_heads), int(num_kv_heads), int(dim), int(vdim)
        if self.num_heads <= 0 or self.num_kv_heads <= 0 or self.num_heads % self.num_kv_heads:
            raise ValueError(f"{self.num_heads} query heads cannot share {self.num_kv_heads} key/value heads")
        if self.num_heads > kernels.SIGMOID_MAX_HEADS:
            raise ValueError(f"the sigmoid attention kernel mixes up to {kernels.SIGMOID_MAX_HEADS} heads, got {self.num_heads}")
        self.scale, self.softcap = float(scale), float(softcap) if softcap else 0.0
        self.bias, self.head_mix, self.head_bias = bool(bias), bool(head_mix), bool(head_bias)
        self.position = position
        self.rotary_dim = int(rotary_dim) if position else 0
        if self.rotary_dim > self.dim or self.rotary_dim % 2:
            raise ValueError(f"{self.rotary_dim} rotated entries do not fit heads of {self.dim}")
        self.q_size, self.k_size, self.v_size = self.num_heads * self.dim, self.num_kv_heads * self.dim, self.num_kv_heads * self.vdim
        self.names = {n: n for n in ("q", "k", "v", "o", "talk", "pb")}
        self.names.update(names or {})
        self.w_qkv = self.b_qkv = self.w_o = self.talk = self.pb = None
        self.compute_dtype = None      # the type of the queries and pages, known once the weights are loaded
        self._mma = None               # whether the tensor-core kernel takes this mixer's sizes in that type

    def cache_spec(self) -> HeadRowPagesSpec:
        return HeadRowPagesSpec(self.num_kv_heads, self.dim + self.vdim, None)

    def graph_key_group(self):
        return ("sigmoid_attention", self.num_heads)

    def graph_key(self, shape) -> int:
        """The key ranges a step of single tokens takes (their number and size): a captured step holds the grid it was
        captured with."""
        segments, keys = self._segments(shape.num_requests, shape.longest)
        return segments | keys << 20

    def _segments(self, tokens: int, longest: int):
        """(number of key ranges, keys of a range) for a step of ``tokens`` new tokens whose longest context is ``longest``."""
        if self._mma is None:
            self._mma = kernels.sigmoid_attention_mma_supports(self.compute_dtype, self.num_heads, self.num_kv_heads, self.dim, self.vdim)
        sms = kernels.sm_count()
        if not self._mma:
            keys = kernels.SIGMOID_SEGMENT_KEYS
            if tokens >= self.SEGMENTS_BELOW_BLOCKS_PER_SM * sms or longest <= keys:
                return 1, keys
        else:
            # tiles of the tensor-core kernel, a block of which fills an SM (a lower bound: a request's last tile may be
            # short). Very few: short ranges, so that every SM gets a block. Fewer than two rounds of blocks over long
            # prompts: long ranges, so that the tiles that see most keys do not take twice the average.
            blocks = -(-tokens // kernels.SIGMOID_MMA_ROWS)
            if blocks < self.MMA_SEGMENTS_BELOW_BLOCKS_PER_SM * sms:
                keys = kernels.SIGMOID_MMA_SEGMENT_KEYS
            elif blocks < self.MMA_LONG_SEGMENTS_BELOW_BLOCKS_PER_SM * sms:
                keys = kernels.SIGMOID_MMA_LONG_SEGMENT_KEYS
            else:
                return 1, kernels.SIGMOID_MMA_SEGMENT_KEYS
            if longest <= keys:
                return 1, keys
        segments = -(-longest // keys)
        if tokens * segments * self.num_heads * self.vdim * 4 > self.SEGMENTS_MAX_BYTES:
            return 1, keys
        return segments, keys

    def _tiles(self, ctx):
        key = ("sigmoid_attention_tiles", kernels.SIGMOID_MMA_ROWS)
        tiles = ctx.memo.get(key)
        if tiles is None:
            if ctx.max_q_len == 1:
                # one token a request: tile r is request r (made on the device, so that a captured step holds no copy from the host)
                tiles = (torch.arange(ctx.num_requests, dtype=torch.int32, device=ctx.device),
                         torch.zeros(ctx.num_requests, dtype=torch.int32, device=ctx.device))
            else:
                req, tok0, _seg, _slot, _places = AttentionPolicy.plan_items(ctx.starts, ctx.q_lens, kernels.SIGMOID_MMA_ROWS, 0, 1, 1,
                                                                             kernels.sm_count())
                host = torch.tensor([req, tok0], dtype=torch.int32).pin_memory()
                dev = host.to(ctx.device, non_blocking=True)
                tiles = (dev[0].contiguous(), dev[1].contiguous())
            ctx.memo[key] = tiles
        return tiles

    def _name(self, key: str) -> str:
        return f"{self.prefix}.{self.names[key]}"

    def param_specs(self) -> Dict[str, ParamSpec]:
        D, H = self.hidden_size, self.num_heads
        sizes = {"q": self.q_size, "k": self.k_size, "v": self.v_size}
        specs = {self._name(n): ParamSpec((sizes[n], D)) for n in ("q", "k", "v")}
        if self.bias:
            specs.update({self._name(n) + ".b": ParamSpec((sizes[n],), role="vector", init="small") for n in ("q", "k", "v")})
        if self.head_mix:
            specs[self._name("talk")] = ParamSpec((H, H), role="vector", init="unit")
        if self.head_bias:
            specs[self._name("pb")] = ParamSpec((H,), role="vector", init="small")
        specs[self._name("o")] = ParamSpec((D, H * self.vdim))
        return specs

    def load(self, get: TensorGetter) -> None:
        self.w_qkv = torch.cat([get(self._name(n), "matrix") for n in ("q", "k", "v")], dim=0).contiguous()
        self.w_o = get(self._name("o"), "matrix").contiguous()
        device = self.w_o.device
        self.compute_dtype, self._mma = self.w_o.dtype, None
        if self.bias:
            self.b_qkv = torch.cat([get(self._name(n) + ".b", "vector").float() for n in ("q", "k", "v")]).contiguous()
        self.talk = (get(self._name("talk"), "vector").float().contiguous() if self.head_mix
                     else torch.eye(self.num_heads, dtype=torch.float32, device=device))
        self.pb = (get(self._name("pb"), "vector").float().contiguous() if self.head_bias
                   else torch.zeros(self.num_heads, dtype=torch.float32, device=device))

    def forward(self, x, ctx, cache: LayerCache):
        if cache.pages is None or cache.group is None:
            raise RuntimeError("the sigmoid attention mixer needs the pages of its cache")
        N = ctx.num_tokens
        qkv = linear(x, self.w_qkv, out_dtype=torch.float32)
        cos = sin = None
        if self.rotary_dim:
            cos, sin = ctx.position_tables[self.position]
        q = torch.empty((N, self.q_size), dtype=x.dtype, device=x.device)
        kernels.sig_qkv_post(qkv, self.b_qkv, cos, sin, self.rotary_dim, q, ctx.slot_mapping[cache.group] if cache.writes else None,
                             cache.pages if cache.writes else None, self.num_heads, self.num_kv_heads, self.dim, self.vdim)
        out = torch.empty((N, self.num_heads * self.vdim), dtype=x.dtype, device=x.device)
        segments, segment_keys = self._segments(N, ctx.decode_ctx_bound or ctx.max_ctx_len)
        sizes = (self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.scale, self.softcap, segments)
        if self._mma and q.dtype == torch.bfloat16:
            tile_req, tile_tok0 = self._tiles(ctx)
            kernels.sigmoid_attention_mma(q, cache.pages, ctx.block_tables[cache.group], ctx.q_start, ctx.ctx_len, ctx.positions,
                                          tile_req, tile_tok0, self.talk, self.pb, out, *sizes, segment_keys=segment_keys)
        else:
            kernels.sigmoid_attention(q, cache.pages, ctx.block_tables[cache.group], ctx.token_request, ctx.positions, self.talk,
                                      self.pb, out, *sizes)
        return linear(out, self.w_o, out_dtype=torch.float32), None
