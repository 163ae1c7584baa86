"""The gated delta rule: a recurrence per head whose state is corrected toward each new value instead of only added to.

    S <- g_t S;   w_t = beta_t (v_t - S^T k_t);   S <- S + k_t w_t^T;   o_t = S^T q_t          S [head_dim, v_head_dim]

One fused product [q | k | v | beta | decay | gate] of the mixer's input into float32 rows; a short causal convolution
over time with its activation on the q, k and v columns (``causal_conv``: the last taps - 1 inputs of every channel are
kept per request); the recurrence from and into the request's state slot, which makes q and k unit vectors and forms
beta = sigmoid(.) and g = exp(-exp(A_log) softplus(. + dt_bias)) in float32 (csrc/mixers.cu: ``delta_rule``); an RMS
norm per head with a shared weight, times the gate's activation (``norm_gate``); the output product.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..cache import StateSlot
from ..weights import MATRIX, VECTOR, TensorDecl
from .base import register
from .program import ACT, record


@register("mixer", "delta_rule")
class DeltaRule:
    @staticmethod
    def _widths(spec):
        return spec.num_kv_heads * spec.head_dim, spec.num_heads * spec.v_head_dim

    @staticmethod
    def tensor_decls(spec) -> Dict[str, TensorDecl]:
        d, H = spec.hidden_size, spec.num_heads
        nk, nv = DeltaRule._widths(spec)
        decls = {spec.q_name: TensorDecl((nk, d)), spec.k_name: TensorDecl((nk, d)), spec.v_name: TensorDecl((nv, d)),
                 spec.beta_name: TensorDecl((H, d)), spec.decay_name: TensorDecl((H, d)), spec.gate_name: TensorDecl((nv, d)),
                 spec.a_log_name: TensorDecl((H,), VECTOR, init="zeros"), spec.dt_bias_name: TensorDecl((H,), VECTOR, init="zeros"),
                 spec.norm_name: TensorDecl((spec.v_head_dim,), VECTOR, init="ones"), spec.o_name: TensorDecl((d, nv))}
        for name, n in ((spec.q_name, nk), (spec.k_name, nk), (spec.v_name, nv)):
            decls[name + spec.conv_suffix] = TensorDecl((n, spec.conv_taps), VECTOR, init="taps")
        return decls

    @staticmethod
    def cache_need(spec):
        return StateSlot((spec.num_heads, spec.head_dim, spec.v_head_dim), "float32")

    @staticmethod
    def state_need(spec, writes_cache: bool = True):
        """The convolutions' tails: the last taps - 1 projected rows of q, k and v."""
        if spec.conv_taps <= 1:
            return None
        nk, nv = DeltaRule._widths(spec)
        return StateSlot((spec.conv_taps - 1, 2 * nk + nv), "float32")

    def __init__(self, spec, weights, prefix: str, runtime):
        self.spec, self.runtime = spec, runtime
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} heads are no multiple of {spec.num_kv_heads} key heads")
        if spec.conv_taps < 1 or spec.conv_act not in ACT or spec.gate_act not in ACT:
            raise ValueError(f"a delta rule with {spec.conv_taps} taps, activations {spec.conv_act!r} and {spec.gate_act!r} is not built")
        names = [spec.q_name, spec.k_name, spec.v_name, spec.beta_name, spec.decay_name, spec.gate_name]
        self.w_in = weights.get_rows([prefix + n for n in names], MATRIX)
        self.w_o = weights.get(prefix + spec.o_name, MATRIX)
        vec = lambda name: weights.get(prefix + name, VECTOR)
        # the three convolutions as one: their channels lie side by side in the fused product's rows
        self.taps = torch.cat([vec(n + spec.conv_suffix) for n in (spec.q_name, spec.k_name, spec.v_name)], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm = vec(spec.a_log_name), vec(spec.dt_bias_name), vec(spec.norm_name)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o))

    def plan(self, program, view, writes_cache: bool = True, residual_scale: float = 1.0, state_view=None) -> None:
        """The mixer in a block that adds its output to the stream itself."""
        self.plan_delta(program, view, writes_cache, state_view=state_view, into_stream=residual_scale)

    def plan_delta(self, program, view, writes_cache: bool = True, state_view=None, into_stream=None) -> None:
        """Four records: the fused product (h -> float32 rows), the convolutions (-> float32 rows of q, k, v), the recurrence
        with norm and gate (-> o), the output product into the delta slot (``into_stream`` s: added into the stream times s)."""
        s = self.spec
        nk, nv = self._widths(s)
        H, C, ld = s.num_heads, 2 * nk + nv, self.w_in.shape[0]
        tails = state_view.state if state_view is not None else None
        if s.conv_taps > 1 and tails is None:
            raise ValueError("a convolution of more than one tap needs its tails' state")
        q_scale = float(s.q_scale) if s.q_scale is not None else float(s.head_dim) ** -0.5
        program.emit_records([
            record("linear", "h", "tmp", n=ld, k=s.hidden_size, w=self.w_in),
            record("causal_conv", "tmp", None, out2_slot="mix", n=C, ld=ld, q_off=0, taps=s.conv_taps, conv_q=self.taps,
                   act=ACT[s.conv_act], state=tails),
            record("delta_rule", "mix", "o", heads=H, groups=s.num_kv_heads, head_dim=s.head_dim, v_head_dim=s.v_head_dim, ld=C,
                   q_off=0, k_off=nk, v_off=2 * nk, r_off=ld, b_off=C, a_off=C + H, g_off=C + 2 * H, a_log=self.a_log,
                   dt_bias=self.dt_bias, q_scale=q_scale, unit_eps=float(s.unit_eps), state=view.state, vec=self.norm, eps=s.norm_eps,
                   per_head_norm=1, gate_act=ACT[s.gate_act]),
            record("linear", "o", "delta", n=s.hidden_size, k=nv, w=self.w_o) if into_stream is None else
            record("residual", "o", "x", n=s.hidden_size, k=nv, w=self.w_o, scale=float(into_stream)),
        ], keep=(self.w_in, self.w_o, self.taps, self.a_log, self.dt_bias, self.norm, tails, view.state))

    def forward(self, h: torch.Tensor, ctx, view, writes_cache: bool = True, state_view=None) -> torch.Tensor:
        """The part alone: its own records over ``h``; float32 ``[T, hidden]``."""
        from .program import run_part_alone
        return run_part_alone(self.runtime, lambda program: self.plan_delta(program, view, writes_cache, state_view), ctx, h,
                              self.spec.hidden_size, result_slot="delta")
