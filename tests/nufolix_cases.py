"""Small Nufolix configurations with weights made for the tests, and the comparison with the plain implementation.

The weights are drawn so that every mechanism carries weight in the logits: projections of unit gain, norm weights,
biases and convolution taps well away from their neutral values, a head mix that is far from the identity, decays that
differ from head to head between "forgets within a few tokens" and "keeps hundreds", and two-step projections of
visible size. They are rounded to bfloat16 once, so the engine in either type and the float64 oracle read the same
numbers. ``sharpen`` makes the attention sparse: scores of a wide spread under a strongly negative number per head, so
that a handful of keys, wherever they are, hold nearly all the weight of a query and a key that is lost, shifted by one
or read from another page changes the result by its whole value.
"""

from __future__ import annotations

import copy
import math
from typing import Dict, List, Optional

import torch

import plain_nufolix as plain
from razelorn_cases import assert_matches, row_errors, write_model, TOL  # noqa: F401  (shared test helpers)

DECAY_RANK, GATE_RANK = 6, 10          # inner sizes of the delta rule's two-step projections: the tensors give them


def dense(ff: int) -> dict:
    return {"kind": "dense", "ff": ff}


def mamba2(heads: int, vdim: int, state: int, groups: int = 1, conv: int = 4, norm_groups: int = 1, mlp: Optional[dict] = None) -> dict:
    return {"type": "mamba2", "mlp": mlp,
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}}


def left(heads: int, kv_heads: int, dim: int, vdim: int, rot_dims: Optional[int] = None, base: float = 10000.0,
         softcap: Optional[float] = 12.0, sharp: float = 1.0) -> dict:
    part = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": sharp / math.sqrt(dim)}
    if softcap is not None:
        part["softcap"] = softcap
    if rot_dims:
        part["rot"] = {"base": base, "dims": rot_dims}
    return part


def right(heads: int, kv_heads: int, dim: int, vdim: int, conv: int = 4) -> dict:
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def parallel(left_part: dict, right_part: dict, left_scale: float = 0.8, right_scale: float = 1.3, mlp: Optional[dict] = None) -> dict:
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": left_part, "right": right_part, "left_scale": left_scale, "right_scale": right_scale}}


def config(layers: List[dict], width: int = 64, vocab: int = 131, eps: float = 1e-5, mult: float = 0.6, scale: float = 3.0) -> dict:
    return {"architecture": "Nufolix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
            "embedding": {"scale": scale}, "layers": layers}


# Several shapes. Key/value (and query/key) heads that are one, several or as many as the heads; values wider than, as
# wide as and narrower than keys; state channels more and fewer than value channels; one and several groups of state
# channels and of the norm; convolutions of one tap (no carried inputs), two and up to six; a rotation of all, part
# and none of a key; with and without a cap on the scores; layers with and without a feed-forward in either kind; two
# layers of one kind in a row; sizes that are no multiples of 16 or of 4; residual factors above and below one.
CONFIGS: Dict[str, dict] = {
    "mixed": config([
        mamba2(4, 16, 24, groups=2, conv=4, norm_groups=2, mlp=dense(72)),
        parallel(left(4, 2, 16, 24, rot_dims=8), right(4, 2, 16, 24, conv=3)),
        mamba2(3, 32, 8, groups=1, conv=2, norm_groups=3),
        parallel(left(3, 3, 32, 16, rot_dims=None, softcap=None), right(2, 2, 24, 40, conv=4), 1.1, 0.4, mlp=dense(48)),
    ]),
    "attention_first": config([
        parallel(left(6, 1, 16, 16, rot_dims=16, base=500.0, softcap=5.0), right(6, 1, 8, 16, conv=2), 1.0, 1.0, mlp=dense(40)),
        parallel(left(2, 2, 64, 32, rot_dims=32), right(1, 1, 32, 64, conv=6), 0.5, 2.0),
        mamba2(2, 24, 40, groups=2, conv=3, norm_groups=1, mlp=dense(100)),
    ], width=48, vocab=97, eps=3e-6, mult=1.25, scale=1.0),
    "odd_sizes": config([
        mamba2(5, 6, 7, groups=5, conv=1, norm_groups=2, mlp=None),
        parallel(left(3, 1, 10, 14, rot_dims=6, softcap=30.0), right(3, 3, 12, 5, conv=1), 1.5, 0.7, mlp=dense(30)),
        mamba2(1, 20, 12, groups=1, conv=5, norm_groups=4, mlp=dense(22)),
        parallel(left(1, 1, 24, 8, rot_dims=24), right(4, 1, 6, 9, conv=5), 0.3, 0.9),
    ], width=54, vocab=61, mult=0.9, scale=0.5),
    "state_space_only": config([mamba2(8, 8, 16, groups=4, conv=4, norm_groups=1, mlp=dense(64)),
                                mamba2(2, 64, 32, groups=1, conv=4, norm_groups=2)], width=32, vocab=80),
    "wide_heads": config([
        parallel(left(2, 1, 128, 128, rot_dims=64, softcap=50.0), right(2, 1, 128, 128, conv=4), 1.0, 1.0, mlp=dense(64)),
        parallel(left(16, 4, 16, 32, rot_dims=16), right(8, 4, 32, 16, conv=4), 1.0, 1.0),
    ], width=96, vocab=150),
}


def sharpen(cfg: dict, sharp: float) -> dict:
    """Scores of spread ``sharp`` (the test's weights give queries and keys of unit entries); see ``weights_for``."""
    cfg = copy.deepcopy(cfg)
    for layer in cfg["layers"]:
        if layer["type"] == "parallel":
            part = layer["mixer"]["left"]
            part["scale"] = sharp / math.sqrt(part["dim"])
            if part.get("softcap"):
                part["softcap"] = max(part["softcap"], 4.0 * sharp)
    return cfg


def weights_for(cfg: dict, seed: int, head_bias: float = -1.0) -> Dict[str, torch.Tensor]:
    """``head_bias``: the mean of the number per head that is added to a score; with sharpened scores a value of about
    minus twice their spread leaves a few keys in a hundred with a weight worth speaking of."""
    gen = torch.Generator().manual_seed(seed)
    D = cfg["width"]
    W: Dict[str, torch.Tensor] = {}

    def normal(*shape, std=1.0, mean=0.0):
        return torch.randn(*shape, generator=gen, dtype=torch.float32) * std + mean

    def uniform(*shape, low=0.0, high=1.0):
        return torch.rand(*shape, generator=gen, dtype=torch.float32) * (high - low) + low

    for name, shape in plain.expected_tensors(cfg, DECAY_RANK, GATE_RANK).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and "." in name else name
        if name == "embed":
            W[name] = normal(*shape)
        elif leaf.startswith("norm") or name == "final.norm" or leaf.endswith(".norm"):
            W[name] = normal(*shape, std=0.25, mean=1.0)
        elif leaf.endswith(".conv"):
            W[name] = normal(*shape, std=0.6) + torch.tensor([0.0] * (shape[1] - 1) + [0.8])
        elif leaf.endswith("conv.b") or leaf.endswith(".b") and len(shape) == 1:
            W[name] = normal(*shape, std=0.3)
        elif leaf.endswith("A_log"):
            W[name] = uniform(*shape, low=-5.0, high=0.5)          # decays per unit step between 0.99 and 0.2
        elif leaf.endswith("dt_bias"):
            W[name] = normal(*shape, std=0.7, mean=-0.5)
        elif leaf.endswith(".D"):
            W[name] = normal(*shape, std=0.5, mean=0.7)
        elif leaf.endswith(".talk"):
            W[name] = torch.eye(shape[0]) * 0.7 + normal(*shape, std=0.4)
        elif leaf.endswith(".pb"):
            W[name] = normal(*shape, std=0.5, mean=head_bias)
        elif leaf.endswith(".act"):
            W[name] = normal(*shape, std=0.8)
        elif leaf.endswith(".a2") or leaf.endswith(".g2"):
            W[name] = normal(*shape, std=2.0 / math.sqrt(shape[1]))
        elif len(shape) == 2:
            W[name] = normal(*shape, std=1.0 / math.sqrt(shape[1]))
        else:
            raise AssertionError(f"no rule for {name} {shape}")
    return {name: t.to(torch.bfloat16).float() for name, t in W.items()}


def oracle(cfg: dict, W: Dict[str, torch.Tensor], requests: Dict[str, List[int]]) -> Dict[str, torch.Tensor]:
    W64 = {k: v.double() for k, v in W.items()}
    return {rid: plain.forward(cfg, W64, toks).float() for rid, toks in requests.items()}
