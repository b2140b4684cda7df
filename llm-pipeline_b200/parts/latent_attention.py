"""Causal attention whose cache holds one small latent vector per token instead of keys and values per head.

With h the mixer's input, H heads, per head ``dim`` unrotated and ``rot_dim`` rotated query/key entries, values of
``vdim`` and a latent of ``kv_rank`` entries::

    q = Wq h                                  per head [dim | rot_dim]; the rot_dim part is rotated by the position
    [l | k_r] = Wdkv h                        kv_rank + rot_dim entries
    c = rms_norm(l) * w_c                     the latent; k_r is rotated by the position and shared by all heads
    k_h = Wuk_h c,  v_h = Wuv_h c             never formed: see below
    score_h(i, j) = (q_h,plain(i) . k_h(j) + q_h,rot(i) . k_r(j)) * scale,  j <= i,  softmax over j
    out = Wo concat_h(sum_j p_h(i, j) v_h(j))

Only ``[c | k_r]`` is cached (``TokenPagesSpec``: one row of kv_rank + rot_dim entries per token). Both up-projections
are linear, so they move to the query's side: ``q_h,plain . (Wuk_h c) = (Wuk_h^T q_h,plain) . c`` and
``sum_j p_j (Wuv_h c_j) = Wuv_h (sum_j p_j c_j)``. Every head then attends over the same cached rows, with a query of
kv_rank + rot_dim entries and the rows' first kv_rank entries as values, in prompts and in decoding alike; the two maps
are one batched product over the heads before and after the attention kernel. Scores, softmax, norm and angles are
float32. ``rot_dims`` (<= rot_dim) entries of the rotated parts take the rotation, the rest pass unchanged.

Options that other designs of this family use (all off by default): the queries through a normed latent of their own
(``q_rank``: ``c_q = rms_norm(Wdq h) * w_q``, ``q = Wuq c_q``), a learned sink per head in the softmax's denominator, a
sigmoid gate ``sigmoid(Wg h)`` on the heads' outputs before ``Wo``, the interleaved pairing of rotated entries, and a
layer without rows of its own that attends over the rows another layer cached (its queries, up-projections, sink and
gate are its own). With any of them the products that read h leave float32 and one kernel norms, rotates and rounds
once (``latent_rows_post``)."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.spec import TokenPagesSpec
from ..ops import kernels
from ..ops.linear import batched_linear, linear
from ..weights.source import ParamSpec
from .attention import AttentionPolicy
from .base import LayerCache, Mixer, TensorGetter
from .registry import register_mixer


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    graph_safe = True      # a step only writes this step's cache rows: repeating it changes nothing

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int,
                 scale: float, norm_eps: float, position: Optional[str] = None, rot_dims: Optional[int] = None,
                 q_rank: Optional[int] = None, sink: bool = False, gate: bool = False, own_rows: bool = True,
                 interleaved: bool = False):
        """``q_rank``: the queries go through a normed latent of that size (``dq``, ``dq.norm``, ``uq`` instead of ``q``);
        ``sink``: a learned number per head whose exponential joins the softmax's denominator (``sink``); ``gate``: the heads'
        outputs are multiplied by sigmoid(Wg h) (``g``); ``own_rows`` False: the layer has no ``dkv`` and reads the rows
        another layer cached; ``interleaved``: the rotation pairs entry 2i with 2i + 1 instead of i with i + rot_dims / 2."""
        self.prefix, self.hidden_size, self.num_heads = prefix, int(hidden_size), int(num_heads)
        self.dim, self.rot_dim, self.vdim, self.kv_rank = int(dim), int(rot_dim), int(vdim), int(kv_rank)
        self.scale, self.norm_eps, self.position = float(scale), float(norm_eps), position
        self.rot_dims = (self.rot_dim if rot_dims is None else int(rot_dims)) if position else 0
        if self.rot_dims > self.rot_dim or self.rot_dims % 2:
            raise ValueError(f"{self.rot_dims} rotated entries do not fit a rotated part of {self.rot_dim}")
        if self.kv_rank > 1024:
            raise ValueError(f"the latent attention kernels take latents of at most 1024 entries, got {self.kv_rank}")
        self.q_rank = int(q_rank) if q_rank else None
        self.sink, self.gate, self.own_rows, self.interleaved = bool(sink), bool(gate), bool(own_rows), bool(interleaved)
        # the float32 path: products that read the input leave float32 and one kernel norms, rotates and rounds once
        self.split = bool(self.q_rank or self.gate or not self.own_rows or self.interleaved)
        self.q_size = self.num_heads * (self.dim + self.rot_dim)
        self.w_in = self.w_uk_t = self.w_uv = self.w_o = self.c_norm = None
        self.w_dq = self.q_norm = self.w_uq = self.w_rest = self.sinks = None

    def cache_spec(self) -> Optional[TokenPagesSpec]:
        return TokenPagesSpec((self.kv_rank + self.rot_dim,), None) if self.own_rows else None

    def graph_key_group(self):
        return ("latent_attention", self.num_heads, self.kv_rank, self.rot_dim)

    def param_specs(self) -> Dict[str, ParamSpec]:
        p, Hd, H = self.prefix, self.hidden_size, self.num_heads
        specs = {f"{p}.uk": ParamSpec((H * self.dim, self.kv_rank)), f"{p}.uv": ParamSpec((H * self.vdim, self.kv_rank)),
                 f"{p}.o": ParamSpec((Hd, H * self.vdim))}
        if self.q_rank:
            specs.update({f"{p}.dq": ParamSpec((self.q_rank, Hd)), f"{p}.dq.norm": ParamSpec((self.q_rank,), role="vector", init="norm"),
                          f"{p}.uq": ParamSpec((self.q_size, self.q_rank))})
        else:
            specs[f"{p}.q"] = ParamSpec((self.q_size, Hd))
        if self.own_rows:
            specs.update({f"{p}.dkv": ParamSpec((self.kv_rank + self.rot_dim, Hd)),
                          f"{p}.dkv.norm": ParamSpec((self.kv_rank,), role="vector", init="norm")})
        if self.sink:
            specs[f"{p}.sink"] = ParamSpec((H,), role="vector", init="small")
        if self.gate:
            specs[f"{p}.g"] = ParamSpec((H * self.vdim, Hd))
        return specs

    def load(self, get: TensorGetter) -> None:
        p, H = self.prefix, self.num_heads
        # per head: Wuk_h^T [kv_rank, dim] (the map of the query into the latent space) and Wuv_h [vdim, kv_rank]
        self.w_uk_t = get(f"{p}.uk", "matrix").view(H, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = get(f"{p}.uv", "matrix").view(H, self.vdim, self.kv_rank).contiguous()
        self.w_o = get(f"{p}.o", "matrix").contiguous()
        if self.own_rows:
            self.c_norm = get(f"{p}.dkv.norm", "vector").contiguous()
        if self.sink:
            self.sinks = get(f"{p}.sink", "vector").float().contiguous()
        if not self.split:
            self.w_in = torch.cat([get(f"{p}.q", "matrix"), get(f"{p}.dkv", "matrix")], dim=0).contiguous()
            return
        if self.q_rank:
            self.w_dq = get(f"{p}.dq", "matrix").contiguous()
            self.q_norm = get(f"{p}.dq.norm", "vector").float().view(1, -1).contiguous()
            self.w_uq = get(f"{p}.uq", "matrix").contiguous()
        else:
            self.w_uq = get(f"{p}.q", "matrix").contiguous()
        rest = ([get(f"{p}.dkv", "matrix")] if self.own_rows else []) + ([get(f"{p}.g", "matrix")] if self.gate else [])
        self.w_rest = torch.cat(rest, dim=0).contiguous() if rest else None

    # Blocks per SM below which a step's tiles are too few and the keys are cut into segments with blocks of their own
    # (decode steps, short portions over long contexts); and the context from which that is worth a second kernel.
    SEGMENTS_BELOW_BLOCKS_PER_SM = 2.0
    SEGMENTS_MIN_CONTEXT = 2 * kernels.LATENT_SEGMENT_KEYS

    def attend(self, ctx, q_lat, q_rot, out, cache: LayerCache) -> None:
        """Attention of the step's rows over the cache: the tensor-core kernel for bfloat16 where it serves the sizes,
        else the general kernel (float32, sizes that are no multiples of 16)."""
        tables = ctx.block_tables[cache.group]
        if not kernels.latent_mma_supports(q_lat.dtype, self.kv_rank, self.rot_dim, cache.pages.shape[1]) or self.dim % 8 or self.rot_dim % 8:
            kernels.latent_attention(q_lat, q_rot, cache.pages, tables, ctx.token_request, ctx.positions, out, self.scale, sink=self.sinks)
            return
        per_tile = kernels.latent_mma_tokens_per_tile(self.num_heads)
        key = ("latent_attention_tiles", per_tile)
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
        longest = ctx.decode_ctx_bound or ctx.max_ctx_len
        blocks = tiles[0].numel() * -(-self.num_heads // 16) * -(-self.kv_rank // 128)
        segments = 0
        if blocks < self.SEGMENTS_BELOW_BLOCKS_PER_SM * kernels.sm_count() and longest >= self.SEGMENTS_MIN_CONTEXT:
            segments = -(-longest // kernels.LATENT_SEGMENT_KEYS)
        kernels.latent_attention_mma(q_lat, q_rot, cache.pages, tables, ctx.q_start, ctx.ctx_len, ctx.positions, tiles[0], tiles[1],
                                     out, self.scale, segments, sink=self.sinks)

    def forward(self, x, ctx, cache: LayerCache):
        if cache.pages is None or cache.group is None:
            raise RuntimeError("the latent attention mixer needs the pages of its cache")
        N, H, rank, rot = ctx.num_tokens, self.num_heads, self.kv_rank, self.rot_dim
        cos = sin = None
        if self.rot_dims:
            cos, sin = ctx.position_tables[self.position]
        gate = None
        if not self.split:
            qd = linear(x, self.w_in)                                        # [N, H (dim + rot) | rank + rot]
            kernels.latent_kv_post(qd, H, self.dim, rot, rank, self.c_norm, self.norm_eps, cos, sin, self.rot_dims,
                                   ctx.slot_mapping[cache.group] if cache.writes else None, cache.pages if cache.writes else None)
            q = qd[:, :self.q_size].view(N, H, self.dim + rot)
        else:
            if self.q_rank:
                latent = linear(x, self.w_dq, out_dtype=torch.float32)
                normed = torch.empty((N, self.q_rank), dtype=x.dtype, device=x.device)
                kernels.add_rmsnorm_multi(latent, None, None, None, self.q_norm, self.norm_eps, normed)
                q32 = linear(normed, self.w_uq, out_dtype=torch.float32)
            else:
                q32 = linear(x, self.w_uq, out_dtype=torch.float32)
            rest = linear(x, self.w_rest, out_dtype=torch.float32) if self.w_rest is not None else None
            writes = self.own_rows and cache.writes
            dkv = rest[:, :rank + rot] if self.own_rows else None
            if self.gate:
                gate = rest[:, rank + rot:] if self.own_rows else rest
            q = torch.empty((N, self.q_size), dtype=x.dtype, device=x.device)
            kernels.latent_rows_post(q32, dkv if writes else None, H, self.dim, rot, rank, self.c_norm, self.norm_eps, cos, sin,
                                     self.rot_dims, self.interleaved, q, ctx.slot_mapping[cache.group] if writes else None,
                                     cache.pages if writes else None)
            q = q.view(N, H, self.dim + rot)
        q_lat = torch.empty((N, H, rank), dtype=x.dtype, device=x.device)
        batched_linear(q[:, :, :self.dim].transpose(0, 1), self.w_uk_t, q_lat.transpose(0, 1))
        mixed = torch.empty((N, H, rank), dtype=x.dtype, device=x.device)
        self.attend(ctx, q_lat, q[:, :, self.dim:], mixed, cache)
        values = torch.empty((N, H, self.vdim), dtype=x.dtype, device=x.device)
        batched_linear(mixed.transpose(0, 1), self.w_uv, values.transpose(0, 1))
        values = values.view(N, H * self.vdim)
        if gate is not None:
            kernels.sigmoid_gate(values, gate)
        return linear(values, self.w_o, out_dtype=torch.float32), None
