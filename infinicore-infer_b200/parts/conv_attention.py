"""Softmax attention with a short convolution on its projections, whole-projection norms, partial rotation, a window,
a sink and a gate per head, over the paged cache; optionally on another layer's keys and values.  Further options of the
same records: a rotation that pairs the halves of a head's leading elements, with stretched frequencies; a division of
every head of q and k by its root mean square after the rotation; capped scores; first positions that the window keeps.

One fused product [q | k | v | gate] (or [q | gate] for a layer that borrows its keys) of the mixer's input in float32;
``conv_qkv`` (csrc/mixers.cu) convolves every channel over time (the taps - 1 projected rows before a portion come from
the request's tail, which then moves on), norms q and k over all their heads at once, rotates the leading elements of
each head in pairs by float32 angles, and writes the queries and, into the pages at the rows' positions, the keys
(after all of that) and the values (after the convolution only); the attention over the pages with its sink, each
head's output times the sigmoid of its gate; the output product.  What the cache holds is therefore what a borrowing
layer needs: it makes queries only and reads the writer's pages under its own mask.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..cache import PagedKV, StateSlot
from ..weights import MATRIX, VECTOR, TensorDecl
from .attention import Attention
from .base import register
from .program import record


@register("mixer", "conv_attention")
class ConvAttention:
    @staticmethod
    def _widths(spec):
        return spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim, spec.num_kv_heads * spec.v_head_dim

    @staticmethod
    def _projections(spec):
        """(name, channels, is normed) of the projections that pass the convolution."""
        nq, nk, nv = ConvAttention._widths(spec)
        out = [(spec.q_name, nq, True)]
        if not spec.shares_kv:
            out += [(spec.k_name, nk, True), (spec.v_name, nv, False)]
        return out

    @staticmethod
    def tensor_decls(spec) -> Dict[str, TensorDecl]:
        d = spec.hidden_size
        decls = {}
        for name, n, normed in ConvAttention._projections(spec):
            decls[name] = TensorDecl((n, d))
            if spec.conv_taps:
                decls[name + spec.conv_suffix] = TensorDecl((n, spec.conv_taps), VECTOR, init="taps")
            if normed and spec.qk_norm:
                decls[name + spec.norm_suffix] = TensorDecl((n,), VECTOR, init="ones")
            elif normed and spec.head_norm == "before_rotation":
                decls[name + spec.norm_suffix] = TensorDecl((spec.head_dim,), VECTOR, init="ones")
            if spec.bias:
                decls[name + spec.bias_suffix] = TensorDecl((n,), VECTOR, init="zeros")
        if spec.head_gate:
            decls[spec.gate_name] = TensorDecl((spec.num_heads, d))
        decls[spec.o_name] = TensorDecl((d, spec.num_heads * spec.v_head_dim))
        return decls

    @staticmethod
    def cache_need(spec):
        # a chunked mask never looks further back than one chunk: the pages behind that are given back as for a window
        return PagedKV(spec.num_kv_heads, spec.head_dim, spec.window or spec.chunk,
                       None if spec.v_head_dim == spec.head_dim else spec.v_head_dim,
                       keep_first=spec.keep_first if spec.window else 0)

    @staticmethod
    def state_need(spec, writes_cache: bool = True):
        """The convolution's tails: the last taps - 1 projected rows of every convolved projection of this layer."""
        if spec.conv_taps <= 1:
            return None
        return StateSlot((spec.conv_taps - 1, sum(n for _, n, _ in ConvAttention._projections(spec))), "float32")

    def __init__(self, spec, weights, prefix: str, runtime):
        self.spec, self.runtime = spec, runtime
        proj = self._projections(spec)
        names = [n for n, _, _ in proj] + ([spec.gate_name] if spec.head_gate else [])
        self.w_in = weights.get_rows([prefix + n for n in names], MATRIX)
        self.w_o = weights.get(prefix + spec.o_name, MATRIX)
        get = lambda name: weights.get(prefix + name, VECTOR)
        self.conv = {n: get(n + spec.conv_suffix) for n, _, _ in proj} if spec.conv_taps else {}
        if spec.window and spec.chunk:
            raise ValueError("an attention has a sliding window or chunks, not both")
        if spec.head_norm == "before_rotation" and spec.qk_norm:
            raise ValueError("a norm over the whole projection and one per head ahead of the rotation are not built together")
        if spec.bias and (spec.conv_taps or spec.head_gate):
            raise ValueError("biases beside a convolution or a gate per head are not built")
        per_head = spec.qk_norm or spec.head_norm == "before_rotation"
        self.norms = {n: get(n + spec.norm_suffix) for n, _, normed in proj if normed} if per_head else {}
        self.bias = torch.cat([get(n + spec.bias_suffix) for n, _, _ in proj]).contiguous() if spec.bias else None
        self.freq, self.rot_mag = None, 1.0
        if spec.position is not None and spec.position.dims:
            p = spec.position
            if p.layout not in ("pairs", "halves"):
                raise ValueError(f"a rotation pairs neighbours (\"pairs\") or halves (\"halves\"), not {p.layout!r}")
            freq, self.rot_mag = p.frequencies()          # float64, rounded once
            self.freq = torch.tensor(freq, dtype=torch.float64).to(torch.float32).to(runtime.device)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o))

    # the rows of requests that bring few rows and the tiles of the others: the lists of the softmax attention
    LISTS = Attention.LISTS
    step_list_capacity = Attention.step_list_capacity
    fill_step_lists = Attention.fill_step_lists

    def plan(self, program, view, writes_cache: bool = True, residual_scale: float = 1.0, state_view=None) -> None:
        """The mixer in a block that adds its output to the stream itself: the output product adds ``residual_scale`` times
        itself."""
        self.plan_delta(program, view, writes_cache, state_view=state_view, into_stream=residual_scale)

    def plan_delta(self, program, view, writes_cache: bool = True, state_view=None, into_stream=None) -> None:
        """Four records: the fused product (h -> float32 rows), convolution / norm / rotation / cache write (-> q), the
        attention (-> o), the output product into the delta slot (``into_stream`` s: added into the stream times s)."""
        s = self.spec
        if writes_cache == s.shares_kv:
            raise ValueError("a layer that borrows its keys writes no cache, and one that has keys writes its own")
        nq, nk, nv = self._widths(s)
        ld = self.w_in.shape[0]
        k_off, v_off = (nq, nq + nk) if not s.shares_kv else (0, 0)
        g_off = nq + (0 if s.shares_kv else nk + nv)
        short, tiles = program.work_lists(Attention, self.LISTS)
        state = state_view.state if state_view is not None else None
        if s.conv_taps > 1 and state is None:
            raise ValueError("a convolution of more than one tap needs its tails' state")
        rot = s.position.dims if self.freq is not None else 0
        program.emit_records([
            record("linear", "h", "tmp", n=ld, k=s.hidden_size, w=self.w_in),
            record("conv_qkv", "tmp", "q", heads=s.num_heads, kv_heads=s.num_kv_heads, head_dim=s.head_dim, v_head_dim=s.v_head_dim,
                   ld=ld, q_off=0, k_off=k_off, v_off=v_off, has_kv=not s.shares_kv, taps=s.conv_taps,
                   conv_q=self.conv.get(s.q_name), conv_k=self.conv.get(s.k_name), conv_v=self.conv.get(s.v_name),
                   norm_q=self.norms.get(s.q_name), norm_k=self.norms.get(s.k_name), eps=s.qk_norm_eps, freq=self.freq, rot_dims=rot,
                   state=state, cache_group=view.group_index, k_pages=view.k_pages, v_pages=view.v_pages,
                   num_pages=view.k_pages.shape[0], writes_cache=writes_cache, rot_mag=self.rot_mag, bias=self.bias,
                   head_norm=2 if s.head_norm == "before_rotation" else int(bool(s.head_norm)),
                   rot_half=self.freq is not None and s.position.layout == "halves"),
            record("attention", "q", "o", heads=s.num_heads, kv_heads=s.num_kv_heads, head_dim=s.head_dim, v_head_dim=s.v_head_dim,
                   window=-int(s.chunk) if s.chunk else (s.window or 0), softmax_scale=s.softmax_scale, cache_group=view.group_index, list_short=short,
                   list_tiles=tiles, max_positions=program.max_blocks * program.page_size, k_pages=view.k_pages,
                   v_pages=view.v_pages, num_pages=view.k_pages.shape[0], sink=s.sink, gated=s.head_gate, ld=ld, g_off=g_off,
                   cap=float(s.score_cap or 0.0), keep_first=s.keep_first if s.window else 0),
            record("linear", "o", "delta", n=s.hidden_size, k=s.num_heads * s.v_head_dim, w=self.w_o) if into_stream is None else
            record("residual", "o", "x", n=s.hidden_size, k=s.num_heads * s.v_head_dim, w=self.w_o, scale=float(into_stream)),
        ], keep=(self.w_in, self.w_o, self.conv, self.norms, self.freq, state, view.k_pages, view.v_pages, self.bias))

    def forward(self, h: torch.Tensor, ctx, view, writes_cache: bool = True, state_view=None) -> torch.Tensor:
        """The part alone: its own records over ``h``; float32 ``[T, hidden]``."""
        from .program import run_part_alone
        return run_part_alone(self.runtime, lambda program: self.plan_delta(program, view, writes_cache, state_view), ctx, h,
                              self.spec.hidden_size, page_size=view.page_size, result_slot="delta")
