"""Typed configuration of the Nufolix decoder, read from its ``config.json``.

A small hybrid decoder. Every layer names its mixer by ``type``: ``mamba2``, a selective state-space recurrence with a
scalar decay per head, or ``parallel``, two mixers side by side that read the same input (left: causal attention whose
weights are sigmoids of capped scores, mixed across heads; right: a gated delta rule with a decay per key channel).
A layer has a dense feed-forward with the xIELU activation and biases, or none (``mlp`` null). Every sublayer has an RMS
norm before and after it and enters the residual with the factor ``residual_mult``; the embedding is scaled; the head is
the embedding table. Keys::

    {"architecture": "Nufolix", "vocab": V, "width": D, "norm": {"eps": e}, "residual_mult": m, "embedding": {"scale": s},
     "layers": [{"type": "mamba2", "mlp": null,
                 "mixer": {"heads": H, "vdim": P, "state": N, "groups": G, "conv": K, "norm_groups": n}},
                {"type": "parallel", "mlp": {"kind": "dense", "ff": F},
                 "mixer": {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": v, "scale": s, "softcap": c,
                                    "rot": {"base": b, "dims": r}},
                           "right": {"heads": H, "kv_heads": G, "dim": d, "vdim": v, "conv": K},
                           "left_scale": a, "right_scale": b}}]}

Tensor names: ``embed``, ``final.norm``; per layer i ``l<i>.norm1``, ``.norm1b`` (around the mixer), ``.norm2``,
``.norm2b`` (around the feed-forward), ``.mix.*`` (``.mix.left.*`` and ``.mix.right.*`` in a parallel layer) and
``.mlp.*``. The inner sizes of the delta rule's two-step projections (``a1``/``a2``, ``g1``/``g2``) are no keys: the
tensors give them."""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Tuple

from .base import LayerSpec, ModelConfig, ModelSpec, PartSpec, ScheduleEntry
from .registry import register_architecture

_MIXERS = ("mamba2", "parallel")
_MLPS = ("dense",)


@dataclass(frozen=True)
class NufolixConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float = 1.0
    embedding_scale: float = 1.0
    layers: Tuple[Dict[str, Any], ...] = field(default_factory=tuple)
    max_position_embeddings: int = 1 << 20

    architecture = "Nufolix"
    model_type = "nufolix"

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
    def from_json(cls, data: Dict[str, Any]) -> "NufolixConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm") if data.get(k) is None]
        if missing:
            raise ValueError(f"Nufolix config.json lacks required keys: {missing}")
        if "eps" not in data["norm"]:
            raise ValueError("Nufolix config.json lacks norm.eps")
        scale = (data.get("embedding") or {}).get("scale", 1.0)
        mult = data.get("residual_mult", 1.0)
        config = cls(vocab=int(data["vocab"]), width=int(data["width"]), norm_eps=float(data["norm"]["eps"]),
                     residual_mult=float(1.0 if mult is None else mult), embedding_scale=float(1.0 if scale is None else scale),
                     layers=tuple(copy.deepcopy(list(data["layers"]))),
                     max_position_embeddings=int(data.get("max_position_embeddings", 1 << 20)))
        config.validate()
        return config

    def validate(self) -> None:
        problems: List[str] = []
        if self.vocab <= 0 or self.width <= 0:
            problems.append(f"vocab and width must be positive, got {self.vocab} and {self.width}")
        if not self.norm_eps > 0:
            problems.append(f"norm.eps must be positive, got {self.norm_eps}")
        if not self.layers:
            problems.append("the model has no layers")
        for i, layer in enumerate(self.layers):
            kind, mixer, mlp = layer.get("type"), layer.get("mixer") or {}, layer.get("mlp")
            if kind not in _MIXERS:
                problems.append(f"layer {i}: unknown type {kind!r} (known: {list(_MIXERS)})")
                continue
            if kind == "mamba2":
                lacking = [k for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups") if mixer.get(k) is None]
                if lacking:
                    problems.append(f"layer {i}: the mamba2 mixer lacks {lacking}")
                else:
                    if int(mixer["heads"]) % int(mixer["groups"]):
                        problems.append(f"layer {i}: {mixer['heads']} heads cannot share {mixer['groups']} groups")
                    if (int(mixer["heads"]) * int(mixer["vdim"])) % int(mixer["norm_groups"]):
                        problems.append(f"layer {i}: norm_groups must divide heads * vdim")
            else:
                left, right = mixer.get("left") or {}, mixer.get("right") or {}
                lacking = [f"left.{k}" for k in ("heads", "kv_heads", "dim", "vdim", "scale") if left.get(k) is None]
                lacking += [f"right.{k}" for k in ("heads", "kv_heads", "dim", "vdim", "conv") if right.get(k) is None]
                lacking += [k for k in ("left_scale", "right_scale") if mixer.get(k) is None]
                if lacking:
                    problems.append(f"layer {i}: the parallel mixer lacks {lacking}")
                else:
                    for side, part in (("left", left), ("right", right)):
                        if int(part["heads"]) % int(part["kv_heads"]):
                            problems.append(f"layer {i}: {side}: {part['heads']} heads cannot share {part['kv_heads']} key heads")
                    rot = left.get("rot")
                    if rot and int(rot.get("dims", 0) or 0) > 0:
                        if rot.get("base") is None:
                            problems.append(f"layer {i}: a rotation needs rot.base")
                        if int(rot["dims"]) > int(left["dim"]) or int(rot["dims"]) % 2:
                            problems.append(f"layer {i}: rot.dims must be even and at most dim")
            if mlp is not None:
                if mlp.get("kind") not in _MLPS:
                    problems.append(f"layer {i}: unknown mlp kind {mlp.get('kind')!r} (known: {list(_MLPS)})")
                elif mlp.get("ff") is None:
                    problems.append(f"layer {i}: a dense mlp needs ff")
        if problems:
            raise ValueError("invalid Nufolix configuration: " + "; ".join(problems))

    def to_json(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "residual_mult": self.residual_mult, "embedding": {"scale": self.embedding_scale},
                "layers": copy.deepcopy(list(self.layers))}

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

        def norm(name: str, gain: float = 1.0) -> PartSpec:
            return PartSpec("rms_norm", {"size": D, "eps": self.norm_eps, "name": name, "gain": gain})

        positions: Dict[str, PartSpec] = {}
        layers: List[LayerSpec] = []
        for i, layer in enumerate(self.layers):
            p, m, mlp = f"l{i}", layer["mixer"], layer.get("mlp")
            if layer["type"] == "mamba2":
                mixer = PartSpec("ssd", {"hidden_size": D, "heads": int(m["heads"]), "vdim": int(m["vdim"]), "state": int(m["state"]),
                                         "groups": int(m["groups"]), "conv": int(m["conv"]), "norm_groups": int(m["norm_groups"]),
                                         "eps": self.norm_eps}, f"{p}.mix")
            else:
                left, right = m["left"], m["right"]
                position, rot_dims = None, 0
                rot = left.get("rot")
                if rot and int(rot.get("dims", 0) or 0) > 0:
                    rot_dims = int(rot["dims"])
                    position = f"rotary_{rot_dims}_{float(rot['base'])!r}"
                    positions.setdefault(position, PartSpec("rotary", {"rotary_dim": rot_dims, "theta": float(rot["base"]), "scaling": 1.0}))
                cap = left.get("softcap")
                mixer = PartSpec("side_by_side", {
                    "left": {"kind": "sigmoid_attention", "prefix": "left", "args": {
                        "hidden_size": D, "num_heads": int(left["heads"]), "num_kv_heads": int(left["kv_heads"]), "dim": int(left["dim"]),
                        "vdim": int(left["vdim"]), "scale": float(left["scale"]), "softcap": float(cap) if cap else None,
                        "bias": True, "position": position, "rotary_dim": rot_dims}},
                    "right": {"kind": "gated_delta_rule", "prefix": "right", "args": {
                        "hidden_size": D, "heads": int(right["heads"]), "qk_heads": int(right["kv_heads"]), "dim": int(right["dim"]),
                        "vdim": int(right["vdim"]), "conv": int(right["conv"]), "eps": self.norm_eps}},
                    "left_scale": float(m["left_scale"]), "right_scale": float(m["right_scale"])}, f"{p}.mix")
            norms = {"mixer": norm(f"{p}.norm1"), "mixer_out": norm(f"{p}.norm1b", self.residual_mult)}
            feed_forward = None
            if mlp is not None:
                norms.update({"feed_forward": norm(f"{p}.norm2"), "feed_forward_out": norm(f"{p}.norm2b", self.residual_mult)})
                feed_forward = PartSpec("xielu_mlp", {"hidden_size": D, "intermediate_size": int(mlp["ff"]), "bias": True}, f"{p}.mlp")
            layers.append(LayerSpec(block="sandwich_norm_residual", mixer=mixer, feed_forward=feed_forward, norms=norms))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=D,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": D, "name": "embed",
                                                   "scale": self.embedding_scale}, "embed"),
            positions=positions, layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i, i) for i in range(len(layers))),
            final_norm=norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": D, "tied_to": "embed", "tied_name": "embed"}, "head"),
            max_position=self.max_position_embeddings,
        )
        spec.validate()
        return spec


register_architecture("Nufolix", NufolixConfig)
