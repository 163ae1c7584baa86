"""Causal softmax attention whose keys and values are maps of one latent vector per position.

What is cached per position is the latent vector c (RMS-normed) and one rotated key part r that all heads share; head
h's key is [W_uk[h] c | r] and its value W_uv[h] c.  The maps are moved to the other side of the products, so that the
attention itself runs over the cached rows and nothing is made per cached position in a step:

    score(t, j, h) = ((W_uk[h]^T q_plain[t, h]) . c_j + q_rot[t, h] . r_j) * scale
    out(t, h)      = W_uv[h] (sum_j softmax_j c_j)

One fused product [q | latent and shared key part | gate] of the mixer's input in float32; ``latent_qkv`` splits the
queries, norms the latent vector, rotates (float32 angles) and writes the cache row; a product per head brings the plain
query parts into the latent space; the attention over the paged rows (float32 scores and weights); a product per head
back to value heads, times the sigmoid of the gate; the output product.  Kernels: csrc/blocks.cu.

Options of the same records: queries through a latent of their own (``q_rank``: the fused product is [query latent | key
and value latent], ``latent_qkv`` norms both, a product makes the heads' queries from the normed one and a cast hands
them to the per-head product), a sliding window (the cache gives back the pages it has passed), no rotated part, no gate.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..cache import PagedKV
from ..weights import MATRIX, VECTOR, TensorDecl
from .base import register
from .program import record


@register("mixer", "latent_attention")
class LatentAttention:
    @staticmethod
    def tensor_decls(spec) -> Dict[str, TensorDecl]:
        d, H = spec.hidden_size, spec.num_heads
        decls = {spec.kv_down_name: TensorDecl((spec.latent_size + spec.rot_dim, d)),
                 spec.kv_down_name + spec.norm_suffix: TensorDecl((spec.latent_size,), VECTOR, init="ones"),
                 spec.k_up_name: TensorDecl((H * spec.head_dim, spec.latent_size)),
                 spec.v_up_name: TensorDecl((H * spec.v_head_dim, spec.latent_size)),
                 spec.o_name: TensorDecl((d, H * spec.v_head_dim))}
        if spec.q_rank:
            decls[spec.q_down_name] = TensorDecl((spec.q_rank, d))
            decls[spec.q_down_name + spec.norm_suffix] = TensorDecl((spec.q_rank,), VECTOR, init="ones")
            decls[spec.q_up_name] = TensorDecl((H * (spec.head_dim + spec.rot_dim), spec.q_rank))
        else:
            decls[spec.q_name] = TensorDecl((H * (spec.head_dim + spec.rot_dim), d))
        if spec.output_gate:
            decls[spec.gate_name] = TensorDecl((H * spec.v_head_dim, d))
        return decls

    @staticmethod
    def cache_need(spec):
        """One row [latent | rotated key part] per position; the values are the row's leading elements."""
        return PagedKV(1, spec.latent_size + spec.rot_dim, spec.window or None, spec.latent_size, values_in_keys=True)

    def __init__(self, spec, weights, prefix: str, runtime):
        self.spec, self.runtime = spec, runtime
        H, dn, R = spec.num_heads, spec.head_dim, spec.latent_size
        if spec.q_rank and spec.rot_dim:
            raise ValueError("queries through a latent beside a rotated part are not built")
        names = [spec.q_down_name if spec.q_rank else spec.q_name, spec.kv_down_name] + ([spec.gate_name] if spec.output_gate else [])
        self.w_in = weights.get_rows([prefix + n for n in names], MATRIX)
        self.q_norm = self.w_q_up = None
        if spec.q_rank:
            self.q_norm = weights.get(prefix + spec.q_down_name + spec.norm_suffix, VECTOR)
            self.w_q_up = weights.get(prefix + spec.q_up_name, MATRIX)
        self.norm = weights.get(prefix + spec.kv_down_name + spec.norm_suffix, VECTOR)
        # head h's key map [dn, R], transposed: the matrix that takes the head's plain query part into the latent space
        self.w_q_latent = weights.get(prefix + spec.k_up_name, MATRIX).view(H, dn, R).transpose(1, 2).contiguous()
        self.w_v = weights.get(prefix + spec.v_up_name, MATRIX)         # [H, dv, R] as stored
        self.w_o = weights.get(prefix + spec.o_name, MATRIX)
        self.freq, self.magnitude, self.rot_dims = None, 1.0, 0
        if spec.position is not None and spec.position.dims:
            if spec.position.dims > spec.rot_dim or spec.position.dims % 2:
                raise ValueError(f"a rotation of {spec.position.dims} elements does not fit a rotated part of {spec.rot_dim}")
            f, self.magnitude = spec.position.frequencies()
            self.freq = torch.tensor(f, dtype=torch.float64).to(torch.float32).to(runtime.device)
            self.rot_dims = spec.position.dims

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_q_latent, self.w_v, self.w_o, self.w_q_up) if t is not None)

    def plan_delta(self, program, view, writes_cache: bool = True, state_view=None) -> None:
        """Six records: the fused product (h -> float32 rows), queries and cache row, the plain query parts into the latent
        space, the attention, the value maps with the gate, the output product into the delta slot."""
        s = self.spec
        if not writes_cache:
            raise ValueError("a latent attention writes the cache it reads")
        H, dn, dr, dv, R = s.num_heads, s.head_dim, s.rot_dim, s.v_head_dim, s.latent_size
        ld = self.w_in.shape[0]
        kv_off = s.q_rank if s.q_rank else H * (dn + dr)
        g_off = kv_off + R + dr
        if s.q_rank:
            # the queries' latent, normed, into "o"; the heads' queries by a product of it (float32 rows in "tmp", which the
            # norms have read by then), cast into "act" as the per-head product's operand
            head = [record("latent_qkv", "tmp", "q", out2_slot="o", heads=H, head_dim=dn, rot_width=0, rank=R, rot_dims=0,
                           norm_k=self.norm, eps=s.norm_eps, ld=ld, q_off=0, k_off=kv_off, q_rank=s.q_rank, norm_q=self.q_norm,
                           cache_group=view.group_index, k_pages=view.k_pages, num_pages=view.k_pages.shape[0]),
                    record("linear", "o", "tmp", n=H * dn, k=s.q_rank, w=self.w_q_up),
                    record("activate", "tmp", "act", n=H * dn, ld=H * dn, act=0),
                    record("head_linear", "act", "q", heads=H, n=R, k=dn, out_hs=R, w=self.w_q_latent)]
        else:
            head = [record("latent_qkv", "tmp", "q", out2_slot="o", heads=H, head_dim=dn, rot_width=dr, rank=R, rot_dims=self.rot_dims,
                           freq=self.freq, rot_mag=self.magnitude, norm_k=self.norm, eps=s.norm_eps, ld=ld, q_off=0, k_off=kv_off,
                           cache_group=view.group_index, k_pages=view.k_pages, num_pages=view.k_pages.shape[0]),
                    record("head_linear", "o", "q", heads=H, n=R, k=dn, out_hs=R + dr, w=self.w_q_latent)]
        program.emit_records([
            record("linear", "h", "tmp", n=ld, k=s.hidden_size, w=self.w_in)] + head + [
            record("latent_attention", "q", "o", heads=H, rank=R, rot_width=dr, softmax_scale=s.softmax_scale, window=s.window or 0,
                   cache_group=view.group_index, k_pages=view.k_pages, num_pages=view.k_pages.shape[0],
                   max_positions=program.max_blocks * program.page_size),
            record("head_linear", "o", "act", heads=H, n=dv, k=R, out_hs=dv, w=self.w_v, gated=s.output_gate, g_off=g_off, ld=ld),
            record("linear", "act", "delta", n=s.hidden_size, k=H * dv, w=self.w_o),
        ], keep=(self.w_in, self.norm, self.w_q_latent, self.w_v, self.w_o, self.freq, view.k_pages, self.q_norm, self.w_q_up))

    def forward(self, h: torch.Tensor, ctx, view, writes_cache: bool = True, state_view=None) -> torch.Tensor:
        """The part alone: its own records over ``h``; float32 ``[T, hidden]``."""
        from .program import run_part_alone
        return run_part_alone(self.runtime, lambda program: self.plan_delta(program, view, writes_cache, state_view), ctx, h,
                              self.spec.hidden_size, page_size=view.page_size, result_slot="delta")
