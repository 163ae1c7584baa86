"""A feed-forward without a gate: down(act(up(h))).

The up product into float32 rows, the activation (which rounds to the activation type once), the down product into the
slot of products that wait for the stream, or added into the stream where the block asks for that.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..weights import MATRIX, TensorDecl
from .base import register
from .program import ACT, record


@register("feed_forward", "mlp")
class MLP:
    @staticmethod
    def tensor_decls(spec) -> Dict[str, TensorDecl]:
        d, di = spec.hidden_size, spec.intermediate_size
        return {spec.up_name: TensorDecl((di, d)), spec.down_name: TensorDecl((d, di))}

    def __init__(self, spec, weights, prefix: str, runtime):
        self.spec, self.runtime = spec, runtime
        if spec.act not in ("gelu_erf", "gelu_tanh", "silu", "relu"):
            raise ValueError(f"a feed-forward with activation {spec.act!r} is not built")
        self.w_up = weights.get(prefix + spec.up_name, MATRIX)
        self.w_down = weights.get(prefix + spec.down_name, MATRIX)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_up, self.w_down))

    def plan(self, program, residual_scale: float = 1.0) -> None:
        """The feed-forward in a block that adds its output to the stream itself."""
        self.plan_delta(program, into_stream=residual_scale)

    def plan_delta(self, program, into_stream=None) -> None:
        """Three records: up (h -> float32 rows), the activation (-> act), down into the delta slot or the stream."""
        s = self.spec
        program.emit_records([
            record("linear", "h", "tmp", n=s.intermediate_size, k=s.hidden_size, w=self.w_up),
            record("activate", "tmp", "act", n=s.intermediate_size, act=ACT[s.act]),
            record("linear", "act", "delta", n=s.hidden_size, k=s.intermediate_size, w=self.w_down) if into_stream is None else
            record("residual", "act", "x", n=s.hidden_size, k=s.intermediate_size, w=self.w_down, scale=float(into_stream)),
        ], keep=(self.w_up, self.w_down))

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        """The part alone: its own records over ``h``; float32 ``[T, hidden]``."""
        from .program import run_part_alone
        return run_part_alone(self.runtime, self.plan_delta, ctx, h, self.spec.hidden_size, result_slot="delta")
