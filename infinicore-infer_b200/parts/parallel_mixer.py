"""Two mixers side by side on the same input: left_scale * left(h) + right_scale * right(h).

Each side is any registered mixer that can add its output into the stream times a factor (``plan`` with a residual scale):
the left one's records, then the right one's; both read the activations that the norm before the block left.  What the
two keep between steps is handed out side by side: pages for the one that asks for them (at most one may), and every state
of fixed size (a recurrence's, a convolution's tails, a shifted input's last row) as one ``StateSlots`` need whose tensors
each side finds again in its order.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from ..cache import StateSlot, StateSlots
from ..cache.manager import StateView
from ..weights import TensorDecl
from .base import part_class, register


def _sides(spec) -> List[Tuple[object, str, float]]:
    return [(spec.left, spec.left_prefix, spec.left_scale), (spec.right, spec.right_prefix, spec.right_scale)]


def _needs(sub) -> Tuple[object, object]:
    """(what the side's cache asks for, what it keeps beside it)."""
    cls = part_class("mixer", sub)
    ask = getattr(cls, "state_need", None)
    return cls.cache_need(sub), (ask(sub, True) if ask is not None else None)


@register("mixer", "parallel")
class ParallelMixer:
    @staticmethod
    def tensor_decls(spec) -> Dict[str, TensorDecl]:
        out = {}
        for sub, prefix, _ in _sides(spec):
            for name, decl in part_class("mixer", sub).tensor_decls(sub).items():
                out[prefix + name] = decl
        return out

    @staticmethod
    def cache_need(spec):
        """The pages of the side that keeps some (None: neither does)."""
        paged = [need for need, _ in (_needs(sub) for sub, _, _ in _sides(spec)) if need is not None and need.group_key() is not None]
        if len(paged) > 1:
            raise ValueError("both sides of a parallel mixer keep pages; a run-order entry has one paged cache")
        return paged[0] if paged else None

    @staticmethod
    def _states(spec) -> List[Tuple[int, str, StateSlot]]:
        """(side, "cache" or "state", the need) of every state of fixed size, in the order of the ``StateSlots`` tensors."""
        out = []
        for i, (sub, _, _) in enumerate(_sides(spec)):
            cache, state = _needs(sub)
            if cache is not None and cache.group_key() is None:
                out.append((i, "cache", cache))
            if state is not None:
                out.append((i, "state", state))
        for _, _, need in out:
            if not isinstance(need, StateSlot):
                raise TypeError(f"a side of a parallel mixer asks for {need!r}; states of fixed size are what it can keep beside pages")
        return out

    @staticmethod
    def state_need(spec, writes_cache: bool = True):
        states = ParallelMixer._states(spec)
        return StateSlots(tuple(need for _, _, need in states)) if states else None

    def __init__(self, spec, weights, prefix: str, runtime):
        self.spec, self.runtime = spec, runtime
        self.sides = [part_class("mixer", sub)(sub, weights, prefix + p, runtime) for sub, p, _ in _sides(spec)]
        for side in self.sides:
            if not hasattr(side, "plan"):
                raise TypeError(f"{type(side).__name__} cannot add its output into the stream (no plan)")

    def weight_bytes(self) -> int:
        return sum(side.weight_bytes() for side in self.sides if hasattr(side, "weight_bytes"))

    def plan(self, program, view, writes_cache: bool = True, residual_scale: float = 1.0, state_view=None) -> None:
        states = self._states(self.spec)
        if states and (state_view is None or len(state_view) != len(states)):
            raise ValueError("a parallel mixer whose sides keep state needs the views of all of it")
        for i, (side, (sub, _, scale)) in enumerate(zip(self.sides, _sides(self.spec))):
            cache, _ = _needs(sub)
            side_view = view if cache is not None and cache.group_key() is not None else None
            side_state = None
            for j, (owner, what, _) in enumerate(states):
                if owner == i and what == "cache":
                    side_view = state_view[j]
                elif owner == i and what == "state":
                    side_state = state_view[j]
            if side_state is not None or hasattr(type(side), "state_need"):
                side.plan(program, side_view, writes_cache, residual_scale * scale, state_view=side_state)
            else:
                side.plan(program, side_view, writes_cache, residual_scale * scale)
