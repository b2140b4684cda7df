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


def attend_latent(q_plain, q_rot, k, k_rot, v, scale: float, sink: torch.Tensor) -> torch.Tensor:
    """q_plain [T, H, dim], q_rot [T, H, rot] (rotated), k [T, H, dim], k_rot [T, rot] (rotated, shared by the heads), v [T, H,
    vdim]; causal softmax whose denominator also holds exp(sink_h). Returns [T, H, vdim]."""
    T = q_plain.shape[0]
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * scale
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    scores = scores.masked_fill(~mask, -math.inf)
    top = torch.maximum(scores.max(dim=-1).values, sink[:, None])
    e = torch.exp(scores - top[..., None])
    prob = e / (e.sum(dim=-1) + torch.exp(sink[:, None] - top))[..., None]
    return torch.einsum("hij,jhd->ihd", prob, v)


def latent_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float, shared=None):
    """``shared``: (c, k_rot) of the layer whose cache this one reads, or None for a layer with rows of its own.
    Returns (output, (c, k_rot))."""
    H, dim, rot_dim, vdim, rank = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
    rot, T = m["rot"], h.shape[0]
    cq = rms(h @ W[f"{p}.dq"].T, eps, W[f"{p}.dq.norm"])
    q = (cq @ W[f"{p}.uq"].T).view(T, H, dim + rot_dim)
    q_rot = rotate_interleaved(q[..., dim:], torch.arange(T), int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
    c, k_rot = shared if shared is not None else latent_rows(h, W, p, m, eps)
    k = (c @ W[f"{p}.uk"].T).view(T, H, dim)
    v = (c @ W[f"{p}.uv"].T).view(T, H, vdim)
    heads = attend_latent(q[..., :dim], q_rot, k, k_rot, v, float(m["scale"]), W[f"{p}.sink"].to(F)).reshape(T, H * vdim)
    heads = heads * torch.sigmoid(h @ W[f"{p}.g"].T)
    return heads @ W[f"{p}.o"].T, (c, k_rot)


def attend_window(q, k, v, scale: float, cap, size, keep: int) -> torch.Tensor:
    """q [T, H, dim], k [T, G, dim], v [T, G, vdim] (already normed); capped scores minus the distance bias, the window with
    its kept first tokens, and one added to the softmax's denominator. Returns [T, H, vdim]."""
    T, H, G = q.shape[0], q.shape[1], k.shape[1]
    group = torch.arange(H) // (H // G)
    s = torch.einsum("ihd,jhd->hij", q, k[:, group]) * scale
    if cap:
        s = float(cap) * torch.tanh(s / float(cap))
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    slopes = torch.tensor([2.0 ** (-8.0 * (n + 1) / H) for n in range(H)], dtype=F)
    s = s - slopes[:, None, None] * (i - j).to(F)
    seen = j <= i
    if size is not None:
        seen = seen & ((i - j < int(size)) | (j < int(keep)))
    s = s.masked_fill(~seen, -math.inf)
    top = s.max(dim=-1).values.clamp(min=0.0)
    e = torch.exp(s - top[..., None])
    prob = e / (torch.exp(-top) + e.sum(dim=-1))[..., None]
    return torch.einsum("hij,jhd->ihd", prob, v[:, group])


def window_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    H, G, dim, vdim = (int(m[k]) for k in ("heads", "kv_heads", "dim", "vdim"))
    T = h.shape[0]
    q = (h @ W[f"{p}.q"].T + W[f"{p}.q.b"]).view(T, H, dim)
    k = (h @ W[f"{p}.k"].T + W[f"{p}.k.b"]).view(T, G, dim)
    v = rms((h @ W[f"{p}.v"].T + W[f"{p}.v.b"]).view(T, G, vdim), eps)
    mask = m.get("mask") or {}
    heads = attend_window(q, k, v, float(m["scale"]), m.get("softcap"), mask.get("size"), int(mask.get("keep_first") or 0))
    heads = heads.reshape(T, H * vdim) * torch.sigmoid(h @ W[f"{p}.g"].T)
    return heads @ W[f"{p}.o"].T + W[f"{p}.o.b"]


def scan(x, dt, A, B, C, D, S=None):
    """The recurrence itself on given rows: x, dt [T, inner], A [inner, N], B, C [T, N]; returns (y [T, inner], last state)."""
    T, inner = x.shape
    S = torch.zeros(inner, A.shape[1], dtype=F) if S is None else S
    y = torch.zeros(T, inner, dtype=F)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + D * x[t]
    return y, S


def selective_scan(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
    inner, N, R = int(m["inner"]), int(m["state"]), int(m["dt_rank"])
    xz = h @ W[f"{p}.in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, W[f"{p}.conv"], W[f"{p}.conv.b"]))
    dbc = x @ W[f"{p}.x"].T
    dt = torch.nn.functional.softplus(dbc[:, :R] @ W[f"{p}.dt"].T + W[f"{p}.dt.b"])
    y, _ = scan(x, dt, -torch.exp(W[f"{p}.A_log"]), dbc[:, R:R + N], dbc[:, R + N:R + 2 * N], W[f"{p}.D"])
    return (y * silu(z)) @ W[f"{p}.o"].T


def dense_ff(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (gelu_tanh(h @ W[f"{p}.gate"].T) * (h @ W[f"{p}.up"].T)) @ W[f"{p}.down"].T


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: List[int], return_layers: bool = False):
    """Logits [T, vocab] of one sequence (and, on request, the residual after every layer, [layers, T, width])."""
    W = {k: (v.to(F) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    taps = int((config.get("canon") or {}).get("taps") or 0)
    filtered = (lambda h, name: input_conv(h, W[name])) if taps else (lambda h, name: h)
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)]
    kept = {}
    after = []
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}", layer["mixer"]
        h = filtered(rms(x, eps, W[f"{p}.norm1"]), f"{p}.canon1")
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
            out = out + dense_ff(filtered(rms(x, eps, W[f"{p}.norm2"]), f"{p}.canon2"), W, f"{p}.mlp")
        x = x + out
        after.append(x)
    logits = rms(x, eps, W["final.norm"]) @ W["head"].T
    return (logits, torch.stack(after)) if return_layers else logits


def expected_tensors(config: dict) -> Dict[str, tuple]:
    """Every tensor a model of this configuration has, with its shape."""
    D, V = int(config["width"]), int(config["vocab"])
    taps = int((config.get("canon") or {}).get("taps") or 0)
    out = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}", layer["mixer"]
        out[f"{p}.norm1"] = (D,)
        if taps:
            out[f"{p}.canon1"] = (D, taps)
        if layer.get("mlp") is not None:
            ff = int(layer["mlp"]["ff"])
            out.update({f"{p}.norm2": (D,), f"{p}.mlp.gate": (ff, D), f"{p}.mlp.up": (ff, D), f"{p}.mlp.down": (D, ff)})
            if taps:
                out[f"{p}.canon2"] = (D, taps)
        x = f"{p}.mix"
        if layer["type"] == "mamba1":
            I, N, R, K = (int(m[k]) for k in ("inner", "state", "dt_rank", "conv"))
            out.update({f"{x}.in": (2 * I, D), f"{x}.conv": (I, K), f"{x}.conv.b": (I,), f"{x}.x": (R + 2 * N, I), f"{x}.dt": (I, R),
                        f"{x}.dt.b": (I,), f"{x}.A_log": (I, N), f"{x}.D": (I,), f"{x}.o": (D, I)})
        elif layer["type"] == "attention":
            H, G, d, dv = (int(m[k]) for k in ("heads", "kv_heads", "dim", "vdim"))
            out.update({f"{x}.q": (H * d, D), f"{x}.q.b": (H * d,), f"{x}.k": (G * d, D), f"{x}.k.b": (G * d,), f"{x}.v": (G * dv, D),
                        f"{x}.v.b": (G * dv,), f"{x}.g": (H * dv, D), f"{x}.o": (D, H * dv), f"{x}.o.b": (D,)})
        else:
            H, d, r, dv, rank, qr = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"))
            out.update({f"{x}.dq": (qr, D), f"{x}.dq.norm": (qr,), f"{x}.uq": (H * (d + r), qr), f"{x}.uk": (H * d, rank),
                        f"{x}.uv": (H * dv, rank), f"{x}.sink": (H,), f"{x}.g": (H * dv, D), f"{x}.o": (D, H * dv)})
            if m.get("kv_from") is None:
                out.update({f"{x}.dkv": (rank + r, D), f"{x}.dkv.norm": (rank,)})
    return out
