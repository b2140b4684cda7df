"""A plain, slow implementation of the Tupidra decoder for the tests: whole sequences, no cache, float64, one function
per mechanism, written from the design's equations. It shares no code with the engine.

A model is ``(config, weights)``: ``config`` the dictionary of ``config.json``, ``weights`` a dictionary from tensor
names to tensors. Positions count from 0. Linear weights are ``[out, in]``."""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def rms(x: torch.Tensor, eps: float, w: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def causal_conv(h: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h [T, C], w [C, K]: out_t = sum_j w[:, j] h_(t - K + 1 + j), zeros before the start."""
    T, K = h.shape[0], w.shape[1]
    out = torch.zeros_like(h)
    for j in range(K):
        shift = K - 1 - j
        if shift < T:
            out[shift:] += h[:T - shift] * w[:, j]
    return out if b is None else out + b


def input_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return h + causal_conv(h, w)


def yarn_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(frequencies [dims / 2], magnitude)"""
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def where(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    i = torch.arange(dims // 2, dtype=F)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float, scaling: Optional[dict]) -> torch.Tensor:
    """x [T, ..., n]: the first ``dims`` entries of the last axis are rotated, entry 2i with entry 2i + 1."""
    f, mag = yarn_frequencies(dims, base, scaling)
    angle = positions.to(F)[:, None] * f[None, :]
    cos, sin = torch.cos(angle) * mag, torch.sin(angle) * mag
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def latent_rows(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    """The cached part of a latent attention layer: (latent c [T, rank], rotated shared key part [T, rot_dim])."""
    rank, rot_dim, rot = int(m["kv_rank"]), int(m["rot_dim"]), m["rot"]
    T = h.shape[0]
    dkv = h @ W[f"{p}.dkv"].T
    c = rms(dkv[:, :rank], eps, W[f"{p}.dkv.norm"])
    k_rot = rotate_interleaved(dkv[:, rank:], torch.arange(T), int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
    return c, k_rot


def latent_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float, shared=None):
    """``shared``: (c, k_rot) of the layer whose cache this one reads, or None for a layer with rows of its own.
    Returns (output, (c, k_rot))."""
    H, dim, rot_dim, vdim, rank = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
    rot, T = m["rot"], h.shape[0]
    cq = rms(h @ W[f"{p}.dq"].T, eps, W[f"{p}.dq.norm"])
    q = (cq @ W[f"{p}.uq"].T).view(T, H, dim + rot_dim)
    q_plain = q[..., :dim]
    q_rot = rotate_interleaved(q[..., dim:], torch.arange(T), int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
    c, k_rot = shared if shared is not None else latent_rows(h, W, p, m, eps)
    k = (c @ W[f"{p}.uk"].T).view(T, H, dim)
    v = (c @ W[f"{p}.uv"].T).view(T, H, vdim)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * float(m["scale"])
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    scores = scores.masked_fill(~mask, -math.inf)
    sink = W[f"{p}.sink"].to(F)
    top = torch.maximum(scores.max(dim=-1).values, sink[:, None])
    e = torch.exp(scores - top[..., None])
    prob = e / (e.sum(dim=-1) + torch.exp(sink[:, None] - top))[..., None]
    heads = torch.einsum("hij,jhd->ihd", prob, v).reshape(T, H * vdim)
    heads = heads * torch.sigmoid(h @ W[f"{p}.g"].T)
    return heads @ W[f"{p}.o"].T, (c, k_rot)


def window_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    H, G, dim, vdim = (int(m[k]) for k in ("heads", "kv_heads", "dim", "vdim"))
    T = h.shape[0]
    q = (h @ W[f"{p}.q"].T + W[f"{p}.q.b"]).view(T, H, dim)
    k = (h @ W[f"{p}.k"].T + W[f"{p}.k.b"]).view(T, G, dim)
    v = rms((h @ W[f"{p}.v"].T + W[f"{p}.v.b"]).view(T, G, vdim), eps)
    group = torch.arange(H) // (H // G)
    s = torch.einsum("ihd,jhd->hij", q, k[:, group]) * float(m["scale"])
    cap = m.get("softcap")
    if cap:
        s = float(cap) * torch.tanh(s / float(cap))
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    slopes = torch.tensor([2.0 ** (-8.0 * (n + 1) / H) for n in range(H)], dtype=F)
    s = s - slopes[:, None, None] * (i - j).to(F)
    mask = m.get("mask") or {}
    size, keep = mask.get("size"), int(mask.get("keep_first") or 0)
    seen = j <= i
    if size is not None:
        seen = seen & ((i - j < int(size)) | (j < keep))
    s = s.masked_fill(~seen, -math.inf)
    top = s.max(dim=-1).values.clamp(min=0.0)
    e = torch.exp(s - top[..., None])
    prob = e / (torch.exp(-top) + e.sum(dim=-1))[..., None]
    heads = torch.einsum("hij,jhd->ihd", prob, v[:, group]).reshape(T, H * vdim)
    heads = heads * torch.sigmoid(h @ W[f"{p}.g"].T)
    return heads @ W[f"{p}.o"].T + W[f"{p}.o.b"]


def selective_scan(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
    inner, N, R = int(m["inner"]), int(m["state"]), int(m["dt_rank"])
    T = h.shape[0]
    xz = h @ W[f"{p}.in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, W[f"{p}.conv"], W[f"{p}.conv.b"]))
    dbc = x @ W[f"{p}.x"].T
    dt = torch.nn.functional.softplus(dbc[:, :R] @ W[f"{p}.dt"].T + W[f"{p}.dt.b"])
    B, C = dbc[:, R:R + N], dbc[:, R + N:R + 2 * N]
    A = -torch.exp(W[f"{p}.A_log"])
    S = torch.zeros(inner, N, dtype=F)
    y = torch.zeros(T, inner, dtype=F)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + W[f"{p}.D"] * x[t]
    return (y * silu(z)) @ W[f"{p}.o"].T


def dense_ff(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (gelu_tanh(h @ W[f"{p}.gate"].T) * (h @ W[f"{p}.up"].T)) @ W[f"{p}.down"].T


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: List[int], return_layers: bool = False):
    """Logits [T, vocab] of one sequence (and, on request, the residual after every layer, [layers, T, width])."""
    W = {k: (v.to(F) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)]
    kept = {}
    after = []
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}", layer["mixer"]
        h = input_conv(rms(x, eps, W[f"{p}.norm1"]), W[f"{p}.canon1"])
        if layer["type"] == "mamba1":
            out = selective_scan(h, W, f"{p}.mix", m)
        elif layer["type"] == "attention":
            out = window_attention(h, W, f"{p}.mix", m, eps)
        elif layer["type"] == "latent_attention":
            source = m.get("kv_from")
            out, kept[i] = latent_attention(h, W, f"{p}.mix", m, eps, kept[int(source)] if source is not None else None)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            out = out + dense_ff(input_conv(rms(x, eps, W[f"{p}.norm2"]), W[f"{p}.canon2"]), W, f"{p}.mlp")
        x = x + out
        after.append(x)
    logits = rms(x, eps, W["final.norm"]) @ W["head"].T
    return (logits, torch.stack(after)) if return_layers else logits
