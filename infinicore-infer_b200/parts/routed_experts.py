"""A feed-forward of small gated units (experts) of which each row uses a few, chosen by a router.

Scores are sigmoid(router h) in float32; a row goes to the ``top`` experts of largest score; an expert sees score * h;
the results add up without renormalising.  A shared gated unit, if the layer has one, runs for every row first (the
feed-forward's usual two records) and the experts' sum is added to it.  The rows of each expert are listed on the
device, so a step never waits for the host; the experts' products run over those lists (csrc/blocks.cu).

The other form of scores (``score_form`` "softmax_renorm"): softmax over all experts, the chosen ones' scores divided by
their sum, multiplying the units' outputs; and the other unit (``act`` "swish_clamp"): clamped sums,
g sigmoid(1.702 g) (u + 1).  The router may have a bias, and the shared unit's output a gate per row, sigmoid(w . h), which
the kernel that adds the experts' sum applies to what it adds to.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..weights import MATRIX, VECTOR, TensorDecl
from .base import part_class, register
from .program import ACT, record


@register("feed_forward", "routed_experts")
class RoutedExperts:
    @staticmethod
    def tensor_decls(spec) -> Dict[str, TensorDecl]:
        d, f = spec.hidden_size, spec.expert_size
        decls = {spec.router_name: TensorDecl((spec.num_experts, d), VECTOR)}
        if spec.router_bias:
            decls[spec.router_name + spec.bias_suffix] = TensorDecl((spec.num_experts,), VECTOR, init="zeros")
        if spec.shared_gate_name:
            decls[spec.shared_prefix + spec.shared_gate_name] = TensorDecl((1, d), VECTOR)
        for e in range(spec.num_experts):
            p = spec.expert_prefix.format(e)
            decls[p + spec.gate_name] = TensorDecl((f, d))
            decls[p + spec.up_name] = TensorDecl((f, d))
            decls[p + spec.down_name] = TensorDecl((d, f))
        if spec.shared is not None:
            for name, decl in part_class("feed_forward", spec.shared).tensor_decls(spec.shared).items():
                decls[spec.shared_prefix + name] = decl
        return decls

    def __init__(self, spec, weights, prefix: str, runtime):
        self.spec, self.runtime = spec, runtime
        if spec.score_form not in ("sigmoid", "softmax_renorm"):
            raise ValueError(f"routed experts with scores of form {spec.score_form!r} are not built")
        if spec.scale_input != (spec.score_form == "sigmoid"):
            raise ValueError("built are sigmoid scores on a unit's input and renormalised softmax scores on its output")
        if spec.act == "swish_clamp" and not spec.limit > 0:
            raise ValueError("a clamped unit needs a positive limit")
        if not 1 <= spec.top <= spec.num_experts:
            raise ValueError(f"{spec.top} of {spec.num_experts} experts")
        self.router = weights.get(prefix + spec.router_name, VECTOR)
        self.router_bias = weights.get(prefix + spec.router_name + spec.bias_suffix, VECTOR) if spec.router_bias else None
        if spec.shared_gate_name and spec.shared is None:
            raise ValueError("a gate on a shared unit that the layer does not have")
        self.shared_gate = weights.get(prefix + spec.shared_prefix + spec.shared_gate_name, VECTOR) if spec.shared_gate_name else None
        names = [prefix + spec.expert_prefix.format(e) for e in range(spec.num_experts)]
        self.w_gate_up = weights.get_rows([p + n for p in names for n in (spec.gate_name, spec.up_name)], MATRIX)
        self.w_down = weights.get_rows([p + spec.down_name for p in names], MATRIX)
        self.shared = None
        if spec.shared is not None:
            self.shared = part_class("feed_forward", spec.shared)(spec.shared, weights, prefix + spec.shared_prefix, runtime)
            if not hasattr(self.shared, "plan_delta"):
                raise TypeError(f"{type(self.shared).__name__} cannot leave its output for the experts to add to (no plan_delta)")

    def weight_bytes(self) -> int:
        """What a step of few rows reads: the router, the shared unit, ``top`` experts a row at most (here: one row's)."""
        s = self.spec
        one = (self.w_gate_up.numel() + self.w_down.numel()) * self.w_gate_up.element_size() // s.num_experts
        return 4 * self.router.numel() + s.top * one + (self.shared.weight_bytes() if self.shared is not None else 0)

    def plan(self, program, residual_scale: float = 1.0) -> None:
        """The feed-forward in a block that adds its output to the stream as it is: the sum waits for the next norm to add it."""
        if residual_scale != 1.0:
            raise ValueError("routed experts add their sum to the stream unscaled")
        self.plan_delta(program, into_stream=True)

    def plan_delta(self, program, into_stream: bool = False) -> None:
        s = self.spec
        if self.shared is not None:
            self.shared.plan_delta(program)
        program.emit_records([
            record("experts", "h", "delta", n=s.hidden_size, experts=s.num_experts, top=s.top, ff=s.expert_size, vec=self.router,
                   w=self.w_gate_up, w3=self.w_down, add=self.shared is not None, act=ACT[s.act], limit=float(s.limit),
                   score_form=1 if s.score_form == "softmax_renorm" else 0, into_stream=into_stream, router_bias=self.router_bias,
                   gate_w=self.shared_gate),
        ], keep=(self.router, self.w_gate_up, self.w_down, self.router_bias, self.shared_gate))

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        """The part alone: its own records over ``h``; float32 ``[T, hidden]``."""
        from .program import run_part_alone
        return run_part_alone(self.runtime, self.plan_delta, ctx, h, self.spec.hidden_size, result_slot="delta")
