"""A plain, slow implementation of the Nufolix decoder: whole sequences, no cache, no batching, one function per
mechanism, written from the design's equations with plain tensor arithmetic. It shares no code with the engine and is
the oracle of its tests. All functions work in the type of the tensors they are given (float64 in the tests).

Notation: ``n`` tokens of one sequence, positions 0 .. n - 1; ``x`` is ``[n, width]``; a linear weight is ``[out, in]``
and applied as ``x @ W.T``; ``W`` maps tensor names to tensors.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) along the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def weighted_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(x, eps) * w


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.logaddexp(x, torch.zeros_like(x))


def short_convolution(x: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal convolution over time, channel by channel: ``x`` [n, channels], ``taps`` [channels, k] whose last column
    multiplies the current token and whose first the token k - 1 places back; zeros before the sequence."""
    n, k = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros((k - 1, x.shape[1]), dtype=x.dtype), x], dim=0)
    out = torch.zeros_like(x)
    for j in range(k):
        out = out + padded[j:j + n] * taps[:, j]
    return out if bias is None else out + bias


def rotate_half(v: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """Rotary encoding of the first ``dims`` entries of the last axis of ``v`` [n, heads, d]: entry i is paired with
    entry i + dims / 2, angle = position * base^(-2 i / dims); entries from ``dims`` on pass unchanged."""
    half = dims // 2
    i = torch.arange(half, dtype=v.dtype)
    freq = base ** (-2.0 * i / dims)
    angle = positions.to(v.dtype)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, v[..., dims:]], dim=-1)


def state_space(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, cfg: dict, eps: float) -> torch.Tensor:
    """The ``mamba2`` mixer: a selective state-space recurrence with one scalar decay per head and token."""
    n = h.shape[0]
    H, P, N, G = cfg["heads"], cfg["vdim"], cfg["state"], cfg["groups"]
    inner = H * P
    proj = h @ W[f"{p}.in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_convolution(xbc, W[f"{p}.conv"], W[f"{p}.conv.b"]))
    x = xbc[:, :inner].view(n, H, P)
    B = xbc[:, inner:inner + G * N].view(n, G, N)
    C = xbc[:, inner + G * N:].view(n, G, N)
    dt = softplus(dt + W[f"{p}.dt_bias"])                               # [n, H]
    decay = torch.exp(-torch.exp(W[f"{p}.A_log"]) * dt)                 # [n, H]
    per_group = H // G
    y = torch.zeros((n, H, P), dtype=h.dtype)
    for head in range(H):
        g = head // per_group
        S = torch.zeros((N, P), dtype=h.dtype)
        for t in range(n):
            S = decay[t, head] * S + dt[t, head] * torch.outer(B[t, g], x[t, head])
            y[t, head] = S.T @ C[t, g] + W[f"{p}.D"][head] * x[t, head]
    y = y.reshape(n, inner) * silu(z)
    parts = cfg["norm_groups"]
    y = rms(y.view(n, parts, inner // parts), eps).reshape(n, inner) * W[f"{p}.norm"]
    return y @ W[f"{p}.o"].T


def sigmoid_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, cfg: dict) -> torch.Tensor:
    """The left half of the ``parallel`` mixer: causal attention whose weights are sigmoids of capped scores plus a
    number per head, not normalised over keys, and mixed across heads before they meet the values."""
    n = h.shape[0]
    H, G, d, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    pos = torch.arange(n)
    q = (h @ W[f"{p}.q"].T + W[f"{p}.q.b"]).view(n, H, d)
    k = (h @ W[f"{p}.k"].T + W[f"{p}.k.b"]).view(n, G, d)
    v = (h @ W[f"{p}.v"].T + W[f"{p}.v.b"]).view(n, G, dv)
    rot = cfg.get("rot")
    if rot and rot.get("dims"):
        q = rotate_half(q, pos, rot["dims"], rot["base"])
        k = rotate_half(k, pos, rot["dims"], rot["base"])
    per_kv = H // G
    kv_of = torch.arange(H) // per_kv
    scores = torch.einsum("ihd,jhd->hij", q, k[:, kv_of]) * cfg["scale"]
    cap = cfg.get("softcap")
    if cap:
        scores = cap * torch.tanh(scores / cap)
    weights = torch.sigmoid(scores + W[f"{p}.pb"][:, None, None])
    visible = pos[None, :] <= pos[:, None]
    weights = weights * visible[None].to(h.dtype)
    mixed = torch.einsum("hg,gij->hij", W[f"{p}.talk"], weights)
    out = torch.einsum("hij,jhv->ihv", mixed, v[:, kv_of]).reshape(n, H * dv)
    return out @ W[f"{p}.o"].T


def gated_delta_rule(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, cfg: dict, eps: float) -> torch.Tensor:
    """The right half of the ``parallel`` mixer: a matrix state per head that decays channel by channel and is
    corrected towards the current value along the current key."""
    n = h.shape[0]
    H, G, d, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    q = silu(short_convolution(h @ W[f"{p}.q"].T, W[f"{p}.q.conv"])).view(n, G, d)
    k = silu(short_convolution(h @ W[f"{p}.k"].T, W[f"{p}.k.conv"])).view(n, G, d)
    v = silu(short_convolution(h @ W[f"{p}.v"].T, W[f"{p}.v.conv"])).view(n, H, dv)
    q = q / torch.sqrt((q * q).sum(dim=-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[f"{p}.b"].T)                                          # [n, H]
    step = softplus((h @ W[f"{p}.a1"].T) @ W[f"{p}.a2"].T + W[f"{p}.dt_bias"]).view(n, H, d)
    decay = torch.exp(-torch.exp(W[f"{p}.A_log"])[None, :, None] * step)             # [n, H, d]
    per_qk = H // G
    o = torch.zeros((n, H, dv), dtype=h.dtype)
    for head in range(H):
        g = head // per_qk
        S = torch.zeros((d, dv), dtype=h.dtype)
        for t in range(n):
            S = decay[t, head][:, None] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            o[t, head] = S.T @ q[t, g]
    gate = torch.sigmoid((h @ W[f"{p}.g1"].T) @ W[f"{p}.g2"].T).view(n, H, dv)
    o = rms(o, eps) * W[f"{p}.norm"] * gate
    return o.reshape(n, H * dv) @ W[f"{p}.o"].T


def parallel_mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, cfg: dict, eps: float) -> torch.Tensor:
    left = sigmoid_attention(h, W, f"{p}.left", cfg["left"])
    right = gated_delta_rule(h, W, f"{p}.right", cfg["right"], eps)
    return cfg["left_scale"] * left + cfg["right_scale"] * right


def xielu(z: torch.Tensor, act: torch.Tensor) -> torch.Tensor:
    """z > 0: softplus(p) z^2 + z / 2; z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2, with act = (p, q)."""
    a_pos = softplus(act[0])
    a_neg = 0.5 + softplus(act[1])
    return torch.where(z > 0, a_pos * z * z + 0.5 * z, a_neg * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z)


def dense_mlp(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    z = h @ W[f"{p}.up"].T + W[f"{p}.up.b"]
    return xielu(z, W[f"{p}.act"]) @ W[f"{p}.down"].T + W[f"{p}.down.b"]


def forward(config: dict, W: Dict[str, torch.Tensor], tokens: List[int], return_layers: bool = False):
    """Logits [n, vocab] of one sequence; with ``return_layers`` also the residual stream after every layer."""
    eps = config["norm"]["eps"]
    m = config["residual_mult"]
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]
    after = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}"
        h = weighted_norm(x, W[f"{p}.norm1"], eps)
        if layer["type"] == "mamba2":
            out = state_space(h, W, f"{p}.mix", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            out = parallel_mixer(h, W, f"{p}.mix", layer["mixer"], eps)
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        x = x + m * weighted_norm(out, W[f"{p}.norm1b"], eps)
        if layer.get("mlp") is not None:
            h = weighted_norm(x, W[f"{p}.norm2"], eps)
            x = x + m * weighted_norm(dense_mlp(h, W, f"{p}.mlp"), W[f"{p}.norm2b"], eps)
        after.append(x)
    logits = weighted_norm(x, W["final.norm"], eps) @ W["embed"].T
    return (logits, torch.stack(after)) if return_layers else logits


def expected_tensors(config: dict, decay_rank: int = 8, gate_rank: int = 8) -> Dict[str, tuple]:
    """Names and shapes of a model's tensors. The inner sizes of the two-step projections of the delta rule's decay and
    gate are no configuration keys: the tensors' shapes give them."""
    D, V = config["width"], config["vocab"]
    out: Dict[str, tuple] = {"embed": (V, D), "final.norm": (D,)}
    for i, layer in enumerate(config["layers"]):
        p, c = f"l{i}", layer["mixer"]
        out[f"{p}.norm1"] = (D,)
        out[f"{p}.norm1b"] = (D,)
        if layer["type"] == "mamba2":
            inner = c["heads"] * c["vdim"]
            channels = inner + 2 * c["groups"] * c["state"]
            out.update({f"{p}.mix.in": (inner + channels + c["heads"], D), f"{p}.mix.conv": (channels, c["conv"]),
                        f"{p}.mix.conv.b": (channels,), f"{p}.mix.dt_bias": (c["heads"],), f"{p}.mix.A_log": (c["heads"],),
                        f"{p}.mix.D": (c["heads"],), f"{p}.mix.norm": (inner,), f"{p}.mix.o": (D, inner)})
        else:
            l, r = c["left"], c["right"]
            lp, rp = f"{p}.mix.left", f"{p}.mix.right"
            out.update({f"{lp}.q": (l["heads"] * l["dim"], D), f"{lp}.q.b": (l["heads"] * l["dim"],),
                        f"{lp}.k": (l["kv_heads"] * l["dim"], D), f"{lp}.k.b": (l["kv_heads"] * l["dim"],),
                        f"{lp}.v": (l["kv_heads"] * l["vdim"], D), f"{lp}.v.b": (l["kv_heads"] * l["vdim"],),
                        f"{lp}.talk": (l["heads"], l["heads"]), f"{lp}.pb": (l["heads"],), f"{lp}.o": (D, l["heads"] * l["vdim"])})
            qk, vv = r["kv_heads"] * r["dim"], r["heads"] * r["vdim"]
            rank_a, rank_g = decay_rank, gate_rank
            out.update({f"{rp}.q": (qk, D), f"{rp}.q.conv": (qk, r["conv"]), f"{rp}.k": (qk, D), f"{rp}.k.conv": (qk, r["conv"]),
                        f"{rp}.v": (vv, D), f"{rp}.v.conv": (vv, r["conv"]), f"{rp}.b": (r["heads"], D), f"{rp}.A_log": (r["heads"],),
                        f"{rp}.norm": (r["vdim"],), f"{rp}.a1": (rank_a, D), f"{rp}.a2": (r["heads"] * r["dim"], rank_a),
                        f"{rp}.dt_bias": (r["heads"] * r["dim"],), f"{rp}.g1": (rank_g, D), f"{rp}.g2": (vv, rank_g),
                        f"{rp}.o": (D, vv)})
        if layer.get("mlp") is not None:
            out[f"{p}.norm2"] = (D,)
            out[f"{p}.norm2b"] = (D,)
            F = layer["mlp"]["ff"]
            out.update({f"{p}.mlp.up": (F, D), f"{p}.mlp.up.b": (F,), f"{p}.mlp.down": (D, F), f"{p}.mlp.down.b": (D,),
                        f"{p}.mlp.act": (2,)})
    return out
