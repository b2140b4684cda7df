"""Typed configuration of the Tupidra decoder, read from its ``config.json``.

A small hybrid decoder. Every layer runs its mixer and its feed-forward side by side on the same residual, each behind
an RMS norm of its own and a short causal convolution beside the identity (``canon.taps`` taps):
``x += mixer(f1(norm1(x))) + mlp(f2(norm2(x)))`` with ``f(h) = h + conv(h)``. A layer names its mixer by ``type``:

* ``mamba1``: the selective state-space recurrence with a decay per channel and state entry;
* ``attention``: softmax attention with grouped key/value heads and biases, values divided by their root mean square,
  capped scores, a distance bias with a slope per head, a sliding window that keeps the first tokens, one added to the
  softmax's denominator, and a sigmoid gate on the heads' outputs; no rotation;
* ``latent_attention``: attention over one cached latent vector per token, queries through a normed latent of their own,
  a part of every key rotated (entry 2i with 2i + 1, frequencies blended by a ramp over the entries, cos and sin scaled), a
  learned sink per head in the denominator and a sigmoid gate on the heads' outputs; with ``kv_from: j`` the layer has no
  cache rows of its own and attends over those of layer j.

The feed-forward is dense and gated with the tanh form of GELU, or absent (``mlp`` null). Keys::

    {"architecture": "Tupidra", "vocab": V, "width": D, "norm": {"eps": e}, "canon": {"taps": K},
     "layers": [{"type": "mamba1", "mlp": {"kind": "dense", "ff": F},
                 "mixer": {"inner": I, "state": N, "dt_rank": R, "conv": K}},
                {"type": "attention", "mlp": ...,
                 "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": v, "scale": s, "softcap": c,
                           "mask": {"size": w, "keep_first": k}}},
                {"type": "latent_attention", "mlp": ...,
                 "mixer": {"heads": H, "dim": d, "rot_dim": r, "vdim": v, "kv_rank": c, "q_rank": q, "scale": s,
                           "rot": {"base": b, "dims": r, "scaling": {"factor": f, "original": L, "fast": a, "slow": b}},
                           "kv_from": j}}]}

Tensor names: ``embed``, ``final.norm``, ``head``; per layer i ``l<i>.norm1``, ``.norm2``, ``.canon1``, ``.canon2``
(``norm2`` and ``canon2`` only with a feed-forward), ``.mix.*`` and ``.mlp.*``."""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Tuple

from .base import LayerSpec, ModelConfig, ModelSpec, PartSpec, ScheduleEntry
from .registry import register_architecture

_MIXERS = ("mamba1", "attention", "latent_attention")
_MLPS = ("dense",)
_NEEDS = {"mamba1": ("inner", "state", "dt_rank", "conv"),
          "attention": ("heads", "kv_heads", "dim", "vdim", "scale"),
          "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale")}


@dataclass(frozen=True)
class TupidraConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    canon_taps: int = 0
    layers: Tuple[Dict[str, Any], ...] = field(default_factory=tuple)
    max_position_embeddings: int = 1 << 20

    architecture = "Tupidra"
    model_type = "tupidra"

    # the names other parts of the engine read from any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_json(cls, data: Dict[str, Any]) -> "TupidraConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm") if data.get(k) is None]
        if missing:
            raise ValueError(f"Tupidra config.json lacks required keys: {missing}")
        if "eps" not in data["norm"]:
            raise ValueError("Tupidra config.json lacks norm.eps")
        taps = (data.get("canon") or {}).get("taps", 0)
        config = cls(vocab=int(data["vocab"]), width=int(data["width"]), norm_eps=float(data["norm"]["eps"]),
                     canon_taps=int(taps or 0), layers=tuple(copy.deepcopy(list(data["layers"]))),
                     max_position_embeddings=int(data.get("max_position_embeddings", 1 << 20)))
        config.validate()
        return config

    def validate(self) -> None:
        problems: List[str] = []
        if self.vocab <= 0 or self.width <= 0:
            problems.append(f"vocab and width must be positive, got {self.vocab} and {self.width}")
        if not self.norm_eps > 0:
            problems.append(f"norm.eps must be positive, got {self.norm_eps}")
        if self.canon_taps < 0:
            problems.append(f"canon.taps cannot be negative, got {self.canon_taps}")
        if not self.layers:
            problems.append("the model has no layers")
        for i, layer in enumerate(self.layers):
            kind, mixer, mlp = layer.get("type"), layer.get("mixer") or {}, layer.get("mlp")
            if kind not in _MIXERS:
                problems.append(f"layer {i}: unknown type {kind!r} (known: {list(_MIXERS)})")
                continue
            lacking = [k for k in _NEEDS[kind] if mixer.get(k) is None]
            if lacking:
                problems.append(f"layer {i}: the {kind} mixer lacks {lacking}")
                continue
            if kind == "attention" and int(mixer["heads"]) % int(mixer["kv_heads"]):
                problems.append(f"layer {i}: {mixer['heads']} heads cannot share {mixer['kv_heads']} key/value heads")
            if kind == "latent_attention":
                rot = mixer.get("rot")
                if int(mixer["rot_dim"]) > 0 and (not rot or rot.get("base") is None):
                    problems.append(f"layer {i}: a rotated key part needs rot.base")
                elif rot and (int(rot.get("dims", mixer["rot_dim"])) > int(mixer["rot_dim"]) or int(rot.get("dims", mixer["rot_dim"])) % 2):
                    problems.append(f"layer {i}: rot.dims must be even and at most rot_dim")
                source = mixer.get("kv_from")
                if source is not None:
                    j = int(source)
                    other = self.layers[j] if 0 <= j < i else None
                    if other is None or other.get("type") != "latent_attention" or (other.get("mixer") or {}).get("kv_from") is not None:
                        problems.append(f"layer {i}: kv_from must name an earlier latent attention layer with rows of its own, got {source}")
                    elif any(other["mixer"].get(k) != mixer.get(k) for k in ("kv_rank", "rot_dim")):
                        problems.append(f"layer {i}: kv_rank and rot_dim must equal those of layer {j}")
            if mlp is not None:
                if mlp.get("kind") not in _MLPS:
                    problems.append(f"layer {i}: unknown mlp kind {mlp.get('kind')!r} (known: {list(_MLPS)})")
                elif mlp.get("ff") is None:
                    problems.append(f"layer {i}: a dense mlp needs ff")
        if problems:
            raise ValueError("invalid Tupidra configuration: " + "; ".join(problems))

    def to_json(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "canon": {"taps": self.canon_taps}, "layers": copy.deepcopy(list(self.layers))}

    def eos_token_ids(self) -> List[int]:
        return []

    def parameter_counts(self) -> Dict[str, int]:
        from ..models import expected_params

        total = 0
        for spec in expected_params(self.model_spec()).values():
            count = 1
            for n in spec.shape:
                count *= n if n is not None else 0
            total += count
        return {"total_parameters": total}

    def model_spec(self) -> ModelSpec:
        D = self.width
        positions: Dict[str, PartSpec] = {}
        layers: List[LayerSpec] = []
        schedule: List[ScheduleEntry] = []
        for i, layer in enumerate(self.layers):
            p, m, mlp = f"l{i}", layer["mixer"], layer.get("mlp")
            pages_from = None
            if layer["type"] == "mamba1":
                mixer = PartSpec("selective_scan", {"hidden_size": D, "inner": int(m["inner"]), "state": int(m["state"]),
                                                    "dt_rank": int(m["dt_rank"]), "conv": int(m["conv"])}, f"{p}.mix")
            elif layer["type"] == "attention":
                mask = m.get("mask") or {}
                size = mask.get("size")
                mixer = PartSpec("capped_attention", {
                    "hidden_size": D, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]), "dim": int(m["dim"]),
                    "vdim": int(m["vdim"]), "scale": float(m["scale"]), "softcap": float(m["softcap"]) if m.get("softcap") else None,
                    "window": int(size) if size else None, "keep_first": int(mask.get("keep_first") or 0), "distance_bias": True,
                    "sink": 0.0, "value_norm_eps": self.norm_eps, "gate": True, "bias": True}, f"{p}.mix")
            else:
                rot_dim = int(m["rot_dim"])
                rot = m.get("rot") or {}
                position, rot_dims = None, 0
                if rot_dim > 0 and int(rot.get("dims", rot_dim)) > 0:
                    rot_dims = int(rot.get("dims", rot_dim))
                    scaling = rot.get("scaling")
                    args: Dict[str, Any] = {"rotary_dim": rot_dims, "theta": float(rot["base"]), "scaling": 1.0}
                    tag = ""
                    if scaling:
                        rule = {"kind": "ramp", "factor": float(scaling["factor"]), "original": float(scaling["original"]),
                                "fast": float(scaling["fast"]), "slow": float(scaling["slow"])}
                        args["frequency_scaling"] = rule
                        args["scaling"] = 0.1 * math.log(rule["factor"]) + 1.0          # cos and sin carry this factor
                        tag = "_ramp_" + "_".join(repr(rule[k]) for k in ("factor", "original", "fast", "slow"))
                    position = f"rotary_{rot_dims}_{float(rot['base'])!r}{tag}"
                    positions.setdefault(position, PartSpec("rotary", args))
                source = m.get("kv_from")
                pages_from = int(source) if source is not None else None
                mixer = PartSpec("latent_attention", {
                    "hidden_size": D, "num_heads": int(m["heads"]), "dim": int(m["dim"]), "rot_dim": rot_dim, "vdim": int(m["vdim"]),
                    "kv_rank": int(m["kv_rank"]), "scale": float(m["scale"]), "norm_eps": self.norm_eps, "position": position,
                    "rot_dims": rot_dims, "q_rank": int(m["q_rank"]), "sink": True, "gate": True, "own_rows": pages_from is None,
                    "interleaved": True}, f"{p}.mix")
            names = [f"{p}.norm1"] + ([f"{p}.norm2"] if mlp is not None else [])
            spare = [] if mlp is not None else [f"{p}.norm2"]            # a checkpoint may hold them for a layer without a feed-forward
            feed_forward = None
            if mlp is not None:
                feed_forward = PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": int(mlp["ff"]), "activation": "gelu_tanh"},
                                        f"{p}.mlp")
            block_args: Dict[str, Any] = {}
            if self.canon_taps > 0:
                block_args["input_conv"] = {"taps": self.canon_taps, "unused": [] if mlp is not None else [f"{p}.canon2"],
                                            "names": [f"{p}.canon1"] + ([f"{p}.canon2"] if mlp is not None else [])}
            layers.append(LayerSpec(block="parallel_residual", mixer=mixer, feed_forward=feed_forward,
                                    norms={"mixer": PartSpec("rms_norm_multi", {"size": D, "eps": self.norm_eps, "names": names, "unused": spare})},
                                    block_args=block_args))
            schedule.append(ScheduleEntry(i, i, pages_from))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=D,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": D, "name": "embed"}, "embed"),
            positions=positions, layers=tuple(layers), schedule=tuple(schedule),
            final_norm=PartSpec("rms_norm_multi", {"size": D, "eps": self.norm_eps, "names": ["final.norm"]}),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": D, "name": "head"}, "head"),
            max_position=self.max_position_embeddings,
        )
        spec.validate()
        return spec


register_architecture("Tupidra", TupidraConfig)
