"""Gated feed-forward with a choice of activation: down(act(gate(h)) * up(h)), act silu, relu or the tanh form of gelu; or
the clamped unit g' sigmoid(1.702 g') (u' + 1) with g' = min(gate h, limit), u' = clamp(up h, -limit, limit).

One fused gate | up product, the gated unit, the down product into the slot of products that wait for the stream (the
block decides how it is added: plainly, or through a norm).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..weights import MATRIX, TensorDecl
from .base import register
from .program import ACT, record


@register("feed_forward", "glu")
class GLU:
    @staticmethod
    def tensor_decls(spec) -> Dict[str, TensorDecl]:
        d, di = spec.hidden_size, spec.intermediate_size
        return {spec.gate_name: TensorDecl((di, d)), spec.up_name: TensorDecl((di, d)), spec.down_name: TensorDecl((d, di))}

    def __init__(self, spec, weights, prefix: str, runtime):
        self.spec, self.runtime = spec, runtime
        if spec.act not in ("silu", "gelu_tanh", "relu", "swish_clamp"):
            raise ValueError(f"a gated feed-forward with activation {spec.act!r} is not built")
        if spec.act == "swish_clamp" and not spec.limit > 0:
            raise ValueError("a clamped unit needs a positive limit")
        self.w_gate_up = weights.get_rows([prefix + spec.gate_name, prefix + spec.up_name], MATRIX)
        self.w_down = weights.get(prefix + spec.down_name, MATRIX)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    def plan_delta(self, program) -> None:
        """Two records: gate | up with the activation (h -> act), down into the delta slot."""
        s = self.spec
        program.emit_records([
            record("gate_up", "h", "act", n=s.intermediate_size, k=s.hidden_size, w=self.w_gate_up, act=ACT[s.act], limit=float(s.limit)),
            record("linear", "act", "delta", n=s.hidden_size, k=s.intermediate_size, w=self.w_down),
        ], keep=(self.w_gate_up, self.w_down))

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        """The part alone: its own records over ``h``; float32 ``[T, hidden]``."""
        from .program import run_part_alone
        return run_part_alone(self.runtime, self.plan_delta, ctx, h, self.spec.hidden_size, result_slot="delta")
