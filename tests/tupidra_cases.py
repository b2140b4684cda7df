"""Small Tupidra configurations with weights made for the tests, and the comparison with the plain implementation.

The weights are drawn so that every mechanism carries weight in the logits: projections of unit gain, norm weights,
biases, sinks, convolution taps and input filters well away from their neutral values, decays per channel and state entry
between "forgets within a few tokens" and "keeps hundreds". They are rounded to bfloat16 once, so the engine in either
type and the float64 oracle read the same numbers. ``sharpen`` raises the score scales so that a softmax sits on one or
two keys anywhere in what a token sees, and a key that is lost, shifted by one or read from another page changes the
result by its whole value."""

from __future__ import annotations

import copy
import math
from typing import Dict, List, Optional

import torch

import plain_tupidra as plain
from razelorn_cases import assert_matches, row_errors, write_model, TOL  # noqa: F401  (shared test helpers)


def dense(ff: int) -> dict:
    return {"kind": "dense", "ff": ff}


def mamba(inner: int, state: int, dt_rank: int, conv: int = 4, mlp: Optional[dict] = None) -> dict:
    return {"type": "mamba1", "mlp": mlp, "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}}


def attention(heads: int, kv_heads: int, dim: int, vdim: int, size: Optional[int] = None, keep: int = 0, softcap: Optional[float] = 15.0,
              mlp: Optional[dict] = None) -> dict:
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": 1.0 / math.sqrt(dim)}
    if softcap is not None:
        mixer["softcap"] = softcap
    if size is not None:
        mixer["mask"] = {"size": size, "keep_first": keep}
    return {"type": "attention", "mlp": mlp, "mixer": mixer}


def latent(heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, q_rank: int, base: float = 100.0, scaling: Optional[dict] = None,
           kv_from: Optional[int] = None, mlp: Optional[dict] = None) -> dict:
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = scaling
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
             "scale": 1.0 / math.sqrt(dim + rot_dim), "rot": rot}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mlp": mlp, "mixer": mixer}


def config(layers: List[dict], width: int = 64, vocab: int = 131, eps: float = 1e-5, taps: int = 4) -> dict:
    return {"architecture": "Tupidra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps}, "layers": layers}


RAMP = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}       # with base 100 and 8 entries: ramp 0, 1/2, 1, 1

# Several shapes. Key/value heads that are one, several or as many as the heads; values wider than, as wide as and narrower
# than keys; windows shorter and longer than a page, none, and shorter than the kept tokens; latents that are and are not
# multiples of 16; layers that read another layer's rows, also two of them; layers without a feed-forward; input filters of
# one tap (nothing carried), two and five; state sizes that take one lane and several; sizes that are no multiples of 4.
CONFIGS: Dict[str, dict] = {
    "mixed": config([
        mamba(96, 12, 5, conv=3, mlp=dense(72)),
        attention(4, 2, 16, 24, size=40, keep=3, mlp=dense(48)),
        latent(3, 16, 8, 24, 32, 20, scaling=RAMP, mlp=dense(40)),
        mamba(80, 24, 3, conv=4),
        attention(3, 3, 32, 16, size=None, softcap=None, mlp=dense(56)),
        latent(2, 24, 8, 16, 32, 12, scaling=RAMP, kv_from=2),
    ]),
    "attention_first": config([
        attention(6, 1, 16, 16, size=9, keep=20, softcap=6.0, mlp=dense(40)),
        latent(4, 16, 16, 32, 48, 24, base=10000.0, mlp=dense(64)),
        latent(1, 32, 16, 8, 48, 40, base=10000.0, kv_from=1, mlp=dense(24)),
        attention(2, 2, 64, 32, size=17, keep=0, softcap=30.0),
        latent(8, 8, 16, 16, 48, 16, base=10000.0, kv_from=1),
        mamba(64, 40, 8, conv=2, mlp=dense(100)),
    ], width=48, vocab=97, eps=3e-6, taps=2),
    "odd_sizes": config([
        mamba(30, 7, 1, conv=1, mlp=None),
        attention(3, 1, 10, 14, size=7, keep=1, softcap=25.0, mlp=dense(30)),
        latent(3, 10, 6, 14, 20, 9, base=37.0, scaling={"factor": 3.0, "original": 20, "fast": 4.0, "slow": 1.0}, mlp=dense(22)),
        mamba(22, 5, 6, conv=5, mlp=dense(18)),
    ], width=54, vocab=61, taps=1),
    "scan_only": config([mamba(64, 16, 4, conv=4, mlp=dense(64)), mamba(40, 200, 2, conv=4)], width=32, vocab=80, taps=5),
    "wide_heads": config([
        attention(16, 2, 64, 128, size=50, keep=2, mlp=dense(64)),
        latent(16, 32, 32, 64, 128, 48, base=50000.0, scaling={"factor": 4.0, "original": 128, "fast": 8.0, "slow": 1.0}, mlp=dense(32)),
        attention(2, 1, 128, 64, size=33, keep=5, softcap=50.0),
        latent(20, 16, 32, 16, 128, 32, base=50000.0, scaling={"factor": 4.0, "original": 128, "fast": 8.0, "slow": 1.0}, kv_from=1),
    ], width=96, vocab=150, taps=3),
}


def sharpen(cfg: dict, sharp: float) -> dict:
    """Scores of spread ``sharp`` (the test's weights give queries and keys of unit entries)."""
    cfg = copy.deepcopy(cfg)
    for layer in cfg["layers"]:
        m = layer["mixer"]
        if layer["type"] == "attention":
            m["scale"] = sharp / math.sqrt(m["dim"])
            if m.get("softcap"):
                m["softcap"] = max(m["softcap"], 4.0 * sharp)
        elif layer["type"] == "latent_attention":
            m["scale"] = sharp / math.sqrt(m["dim"] + m["rot_dim"])
    return cfg


def weights_for(cfg: dict, seed: int, slow: bool = False) -> Dict[str, torch.Tensor]:
    """``slow``: decays close to one, so that the scans' states keep what the first tokens wrote for hundreds of tokens."""
    gen = torch.Generator().manual_seed(seed)
    W: Dict[str, torch.Tensor] = {}

    def normal(*shape, std=1.0, mean=0.0):
        return torch.randn(*shape, generator=gen, dtype=torch.float32) * std + mean

    def uniform(*shape, low=0.0, high=1.0):
        return torch.rand(*shape, generator=gen, dtype=torch.float32) * (high - low) + low

    for name, shape in plain.expected_tensors(cfg).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and "." in name else name
        if name in ("embed", "head"):
            W[name] = normal(*shape, std=1.0 if name == "embed" else 4.0 / math.sqrt(shape[1]))      # logits of a spread that leaves few near ties
        elif leaf.startswith("norm") or name == "final.norm" or leaf.endswith(".norm"):
            W[name] = normal(*shape, std=0.25, mean=1.0)
        elif leaf.startswith("canon"):
            W[name] = normal(*shape, std=0.4)
        elif leaf.endswith(".conv"):
            W[name] = normal(*shape, std=0.6) + torch.tensor([0.0] * (shape[1] - 1) + [0.8])
        elif leaf.endswith("A_log"):
            W[name] = uniform(*shape, low=-6.5, high=-5.0) if slow else uniform(*shape, low=-5.0, high=0.5)
        elif leaf.endswith("dt.b"):
            W[name] = normal(*shape, std=0.7, mean=-1.5 if slow else -0.5)
        elif leaf.endswith(".D"):
            W[name] = normal(*shape, std=0.5, mean=0.7)
        elif leaf.endswith(".sink"):
            W[name] = normal(*shape, std=1.0, mean=0.5)
        elif len(shape) == 1:                                  # biases
            W[name] = normal(*shape, std=0.3)
        elif len(shape) == 2:
            W[name] = normal(*shape, std=1.0 / math.sqrt(shape[1]))
        else:
            raise AssertionError(f"no rule for {name} {shape}")
    return {name: t.to(torch.bfloat16).float() for name, t in W.items()}


def oracle(cfg: dict, W: Dict[str, torch.Tensor], requests: Dict[str, List[int]]) -> Dict[str, torch.Tensor]:
    W64 = {k: v.double() for k, v in W.items()}
    return {rid: plain.forward(cfg, W64, toks).float() for rid, toks in requests.items()}
