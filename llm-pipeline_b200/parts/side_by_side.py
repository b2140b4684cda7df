"""Two mixers side by side: both read the same input, and the result is a weighted sum of theirs.

``side_by_side`` builds its two members from part specifications (kind, sizes, tensor-name prefix below its own), so
any two registered mixers can stand beside each other. What they ask of the cache manager is put together: at most one
member may keep pages (the layer has one page group), and the members' states lie one after the other in the request's
state vector, each member seeing its own column range. The sum ``left_scale * left + right_scale * right`` is float32."""

from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from ..cache.spec import StateSpec
from ..ops import kernels
from .base import LayerCache, Mixer, TensorGetter
from .registry import lookup, register_mixer


@register_mixer("side_by_side")
class SideBySide(Mixer):
    def __init__(self, prefix: str, left: Dict[str, Any], right: Dict[str, Any], left_scale: float = 1.0, right_scale: float = 1.0):
        """``left`` / ``right``: {"kind": a registered mixer, "args": its sizes, "prefix": its tensors' prefix below this one's}."""
        self.prefix = prefix
        self.scales = (float(left_scale), float(right_scale))
        self.members = tuple(lookup("mixer", m["kind"])(f"{prefix}.{m['prefix']}" if m.get("prefix") else prefix, **m["args"])
                             for m in (left, right))
        if sum(m.cache_spec() is not None for m in self.members) > 1:
            raise ValueError("mixers side by side share one page group: only one of them may keep pages")
        self.graph_safe = all(getattr(m, "graph_safe", False) for m in self.members)
        self._state_at = []
        at = 0
        for m in self.members:
            spec = m.state_spec()
            if spec is None:
                self._state_at.append(None)
                continue
            if spec.dtype != torch.float32 or len(spec.shape) != 1:
                raise ValueError("mixers side by side keep their states as float32 vectors")
            self._state_at.append((at, at + spec.shape[0]))
            at += spec.shape[0]
        self._state_entries = at

    def cache_spec(self):
        for m in self.members:
            if m.cache_spec() is not None:
                return m.cache_spec()
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self._state_entries,), torch.float32) if self._state_entries else None

    def graph_key_group(self):
        return ("side_by_side",) + tuple(m.graph_key_group() for m in self.members)

    def graph_key(self, shape):
        return tuple(m.graph_key(shape) for m in self.members)

    def captured_context_limit(self):
        limits = [n for n in (m.captured_context_limit() for m in self.members) if n is not None]
        return min(limits) if limits else None

    def param_specs(self):
        out = {}
        for m in self.members:
            out.update(m.param_specs())
        return out

    def copies(self):
        out = {}
        for m in self.members:
            out.update(m.copies())
        return out

    def load(self, get: TensorGetter) -> None:
        for m in self.members:
            m.load(get)

    def forward(self, x, ctx, cache: LayerCache):
        results = []
        for m, span in zip(self.members, self._state_at):
            state = cache.state[:, span[0]:span[1]] if span is not None and cache.state is not None else None
            view = LayerCache(pages=cache.pages if m.cache_spec() is not None else None, group=cache.group, state=state,
                              writes=cache.writes)
            out, bias = m.forward(x, ctx, view)
            out = out.float() if out.dtype != torch.float32 else out
            if bias is not None:
                out = out + bias.float()
            results.append(out.contiguous())
        total = torch.empty_like(results[0])
        kernels.scaled_sum(results[0], self.scales[0], results[1], self.scales[1], total)
        return total, None
