"""Linear attention as a recurrence with a float32 state per request and head.

    S_t = diag(a_t) S_(t-1) + k_t v_t^T        o_t = S_t^T q_t

One fused product [q | k | v | gate (| decay projection)] of the mixer's input in float32; the recurrence over each
request's rows, from and into the request's state slot (csrc/mixers.cu: ``linear_scan``); an RMS norm of the output,
times an activation of the gate (``norm_gate``); the output product.  The decay is a constant per head or
sigmoid(W2 (W1 h) + b2) ** (1 / tau) per key channel; both, like the state, in float32.  ``LinearAttentionSpec`` names
every choice.

With ``token_shift`` every projection reads its own mixture of a row and the row before it (``token_shift`` record: the
mixtures side by side, the request's last row kept as state), so the fused product becomes one product per projection
into column ranges of the same float32 rows; with a bonus a row reads the state before its own decay:
    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T q_t        S_t = diag(a_t) S_(t-1) + k_t v_t^T
"""
from __future__ import annotations

from typing import Dict

import torch

from ..cache import StateSlot, StateSlots
from ..weights import MATRIX, VECTOR, TensorDecl
from .base import register
from .program import ACT, record


@register("mixer", "linear_attention")
class LinearAttention:
    @staticmethod
    def _widths(spec):
        return spec.num_heads * spec.head_dim, spec.num_heads * spec.v_head_dim

    @staticmethod
    def tensor_decls(spec) -> Dict[str, TensorDecl]:
        d = spec.hidden_size
        nk, nv = LinearAttention._widths(spec)
        shared_norm = spec.norm_per_head and spec.norm_per_head != "unit"
        decls = {spec.q_name: TensorDecl((nk, d)), spec.k_name: TensorDecl((nk, d)), spec.v_name: TensorDecl((nv, d)),
                 spec.gate_name: TensorDecl((nv, d)), spec.o_name: TensorDecl((d, nv)),
                 spec.norm_name: TensorDecl((spec.v_head_dim if shared_norm else nv,), VECTOR, init="ones")}
        if spec.decay is None:
            decls[spec.decay_down_name] = TensorDecl((spec.decay_rank, d))
            decls[spec.decay_up_name] = TensorDecl((nk, spec.decay_rank))
            decls[LinearAttention._decay_bias(spec)] = TensorDecl((nk,), VECTOR, init="zeros")
        if spec.token_shift:
            for name in LinearAttention._shifted(spec):
                decls[spec.shift_prefix + name[0]] = TensorDecl((d,), VECTOR, init="half")
        if spec.bonus_name:
            decls[spec.bonus_name] = TensorDecl((spec.num_heads, spec.head_dim), VECTOR, init="taps")
        return decls

    @staticmethod
    def _decay_bias(spec) -> str:
        return spec.decay_bias_name or spec.decay_up_name + spec.bias_suffix

    @staticmethod
    def _shifted(spec):
        """(name of the mixing vector, name of the projection) of every projection that reads a shifted mixture, in the
        order of their columns."""
        out = [(n, n) for n in (spec.q_name, spec.k_name, spec.v_name, spec.gate_name)]
        if spec.decay is None:
            out.append((spec.decay_shift_name, spec.decay_down_name))
        return out

    @staticmethod
    def cache_need(spec):
        return StateSlot((spec.num_heads, spec.head_dim, spec.v_head_dim), "float32")

    @staticmethod
    def state_need(spec, writes_cache: bool = True):
        """The last row of the mixer's input, for the first row of the next step."""
        return StateSlot((spec.hidden_size,), "float32") if spec.token_shift else None

    def __init__(self, spec, weights, prefix: str, runtime):
        self.spec, self.runtime = spec, runtime
        if spec.decay is None and spec.decay_rank <= 0:
            raise ValueError("a linear attention needs constant decays or a decay projection")
        if spec.decay is not None and len(spec.decay) != spec.num_heads:
            raise ValueError(f"{len(spec.decay)} decays for {spec.num_heads} heads")
        if spec.decay_form not in ("sigmoid_pow", "exp_neg_exp") or spec.decay_act not in ACT:
            raise ValueError(f"a decay of form {spec.decay_form!r} with activation {spec.decay_act!r} is not built")
        names = [spec.q_name, spec.k_name, spec.v_name, spec.gate_name] + ([spec.decay_down_name] if spec.decay is None else [])
        self.w_in = weights.get_rows([prefix + n for n in names], MATRIX)
        self.w_o = weights.get(prefix + spec.o_name, MATRIX)
        self.norm = weights.get(prefix + spec.norm_name, VECTOR)
        self.decay = self.w2 = self.b2 = self.mu = self.bonus = None
        if spec.token_shift:        # the mixing vectors, one row per projection in the order of their columns
            self.mu = torch.stack([weights.get(prefix + spec.shift_prefix + mu, VECTOR) for mu, _ in self._shifted(spec)]).contiguous()
        if spec.bonus_name:
            self.bonus = weights.get(prefix + spec.bonus_name, VECTOR).contiguous()
        if spec.decay is None:
            self.w2 = weights.get(prefix + spec.decay_up_name, MATRIX)
            self.b2 = weights.get(prefix + self._decay_bias(spec), VECTOR)
        else:
            self.decay = torch.tensor(spec.decay, dtype=torch.float64).to(torch.float32).to(runtime.device)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o, self.w2) if t is not None)

    # ---- work lists: what this mixer asks every step to carry --------------------------------------------------------
    # A request that brings at most ``scan_piece()`` rows runs its recurrence in one go from its state slot; the rows of a
    # longer portion are cut into pieces that run side by side and are then joined (csrc/mixers.cu).  The lists: the requests
    # of the first kind, (first row, rows) of every piece, and (request, first piece, pieces) of every request that has some.
    LISTS = ("direct", "pieces", "piece_reqs")

    @staticmethod
    def step_list_capacity(T: int, B: int) -> Dict[str, int]:
        from ..kernels import host
        return {"direct": B, "pieces": 2 * (T // host.scan_piece() + B), "piece_reqs": 3 * B}

    @staticmethod
    def fill_step_lists(B: int, pad_B: int, lens, starts, arrays) -> Dict[str, tuple]:
        from ..kernels import host
        piece = host.scan_piece()
        direct, pieces, piece_reqs = arrays["direct"], arrays["pieces"], arrays["piece_reqs"]
        row = n_direct = n_pieces = n_reqs = 0
        for i in range(B):
            n = lens[i]
            if n <= piece:
                direct[n_direct] = i
                n_direct += 1
            else:
                first = n_pieces
                for r0 in range(0, n, piece):
                    pieces[2 * n_pieces], pieces[2 * n_pieces + 1] = row + r0, min(piece, n - r0)
                    n_pieces += 1
                piece_reqs[3 * n_reqs: 3 * n_reqs + 3] = (i, first, n_pieces - first)
                n_reqs += 1
            row += n
        for i in range(B, pad_B):
            direct[n_direct] = i
            n_direct += 1
        return {"direct": (n_direct, n_direct == pad_B), "pieces": (n_pieces, False), "piece_reqs": (n_reqs, False)}

    def plan(self, program, view, writes_cache: bool = True, residual_scale: float = 1.0, state_view=None) -> None:
        """The mixer in a block that adds its output to the stream itself."""
        self.plan_delta(program, view, writes_cache, state_view=state_view, into_stream=residual_scale)

    def plan_delta(self, program, view, writes_cache: bool = True, state_view=None, into_stream=None) -> None:
        """Three records: the fused product (h -> float32 rows), the recurrence with norm and gate (-> o), the output product
        into the delta slot (``into_stream`` s: added into the stream times s).  With a token shift the first is the shift
        and one product per projection."""
        s = self.spec
        nk, nv = self._widths(s)
        ld = self.w_in.shape[0]
        direct, pieces, piece_reqs = program.work_lists(LinearAttention, self.LISTS)
        widths = [nk, nk, nv, nv] + ([s.decay_rank] if s.decay is None else [])
        offs = [sum(widths[:i]) for i in range(len(widths))]
        if s.token_shift:
            if state_view is None or state_view.state is None:
                raise ValueError("a token shift needs the state that keeps a request's last row")
            records = [record("token_shift", "h", "shift", n=s.hidden_size, heads=len(widths), vec=self.mu, state=state_view.state)]
            row = 0
            for part, (width, off) in enumerate(zip(widths, offs)):
                records.append(record("linear", "shift", "tmp", n=width, k=s.hidden_size, w=self.w_in[row: row + width], in_part=part,
                                      ld=ld, out_off=off))
                row += width
        else:
            records = [record("linear", "h", "tmp", n=ld, k=s.hidden_size, w=self.w_in)]
        per_head = 2 if s.norm_per_head == "unit" else (1 if s.norm_per_head else 0)
        records += [
            record("linear_attention", "tmp", "o", list_short=direct, list_tiles=pieces, list_aux=piece_reqs, heads=s.num_heads, head_dim=s.head_dim, v_head_dim=s.v_head_dim, ld=ld,
                   q_off=0, k_off=nk, v_off=2 * nk, g_off=2 * nk + nv, r_off=2 * nk + 2 * nv, act=ACT[s.qkv_act], q_scale=s.q_scale,
                   gate_act=ACT[s.gate_act], per_head_norm=per_head, eps=s.norm_eps, vec=self.norm, decay=self.decay,
                   w2=self.w2, b2=self.b2, rank=s.decay_rank if s.decay is None else 0, tau=s.decay_tau, state=view.state,
                   bonus=self.bonus, decay_form=1 if s.decay_form == "exp_neg_exp" else 0, rank_act=ACT[s.decay_act]),
            record("linear", "o", "delta", n=s.hidden_size, k=nv, w=self.w_o) if into_stream is None else
            record("residual", "o", "x", n=s.hidden_size, k=nv, w=self.w_o, scale=float(into_stream)),
        ]
        program.emit_records(records, keep=(self.w_in, self.w_o, self.norm, self.decay, self.w2, self.b2, view.state, self.mu, self.bonus,
                                            state_view.state if state_view is not None else None))

    def forward(self, h: torch.Tensor, ctx, view, writes_cache: bool = True, state_view=None) -> torch.Tensor:
        """The part alone: its own records over ``h``; float32 ``[T, hidden]``."""
        from .program import run_part_alone
        return run_part_alone(self.runtime, lambda program: self.plan_delta(program, view, writes_cache, state_view), ctx, h,
                              self.spec.hidden_size, result_slot="delta")
