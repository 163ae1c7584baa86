"""The model: embedding, the layers in their run order, final norm, output product.

Built from a ``ModelSpec`` alone.  ``forward`` runs the rows of one step and returns the
float32 logits of the wanted rows.  Reference: src/models/jiuge/jiuge.cpp:114-298
(``inferDeviceBatch``); the embedding scale, the residual scale and the logit scale are
MiniCPM's (scripts/jiuge.py:97-114) and arrive here as plain numbers of the specification.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..weights import MATRIX, TensorDecl
from .base import ResidualStream, Runtime, StepContext, part_class
from .program import Program


def model_manifest(spec) -> Dict[str, TensorDecl]:
    """Every tensor the model reads, by checkpoint name.  The output matrix is optional: when
    the checkpoint has none the embedding is used (scripts/jiuge.py:182-191)."""
    out = {spec.embed_name: TensorDecl((spec.vocab_size, spec.hidden_size)),
           spec.lm_head_name: TensorDecl((spec.vocab_size, spec.hidden_size), optional=True)}
    if spec.position_table_name:
        out[spec.position_table_name] = TensorDecl((spec.position_rows, spec.hidden_size))
    for name, decl in part_class("norm", spec.final_norm).tensor_decls(spec.final_norm).items():
        out[spec.final_norm_prefix + name] = decl
    for i, layer in enumerate(spec.layers):
        prefix = spec.layer_prefix.format(i)
        for name, decl in part_class("block", layer).tensor_decls(layer).items():
            out[prefix + name] = decl
    for e in spec.order:          # steps between layers name their tensors without a layer's prefix
        if e.before is not None:
            out.update(part_class("stream", e.before).tensor_decls(e.before))
    return out


def cache_needs(spec) -> List[object]:
    """What each cache of the run order asks of the cache manager."""
    needs: List[object] = [None] * spec.num_caches
    for e in spec.order:
        if e.writes_cache:
            layer = spec.layers[e.layer]
            needs[e.cache] = part_class("block", layer).cache_need(layer)
    for e in spec.order:
        if not e.writes_cache:
            layer = spec.layers[e.layer]
            mine = part_class("block", layer).cache_need(layer)
            if mine != needs[e.cache]:
                # a reader with a mask of its own: the pages are kept for the widest window among the cache's users
                both = needs[e.cache].shared_with(mine) if hasattr(needs[e.cache], "shared_with") else None
                if both is None:
                    raise ValueError(f"layer {e.layer} reads cache {e.cache}, which holds {needs[e.cache]}, "
                                     f"but needs {mine}")
                needs[e.cache] = both
    return needs


def state_needs(spec) -> List[object]:
    """What each entry of the run order keeps for itself beside its cache (``StateSlot`` or None), asked of the block
    class's ``state_need(spec, writes_cache)`` where it has one."""
    out: List[object] = []
    for e in spec.order:
        layer = spec.layers[e.layer]
        ask = getattr(part_class("block", layer), "state_need", None)
        out.append(ask(layer, e.writes_cache) if ask is not None else None)
    return out


class Model:
    def __init__(self, spec, weights, runtime: Runtime):
        self.spec, self.runtime = spec, runtime
        self.embedding = weights.get(spec.embed_name, MATRIX)
        if weights.has(spec.lm_head_name):
            self.lm_head = weights.get(spec.lm_head_name, MATRIX)
        else:
            self.lm_head = self.embedding       # tied: one copy serves both ends
        self.position_table = None
        if spec.position_table_name:          # a learned vector per position, added to the embedding's output
            self.position_table = weights.get(spec.position_table_name, MATRIX)
            if spec.max_positions > self.position_table.shape[0]:
                raise ValueError(f"sequences of up to {spec.max_positions} positions, but {spec.position_table_name} holds {self.position_table.shape[0]}")
        self.final_norm = part_class("norm", spec.final_norm)(spec.final_norm, weights,
                                                              spec.final_norm_prefix, runtime)
        self.layers = [part_class("block", layer)(layer, weights, spec.layer_prefix.format(i), runtime)
                       for i, layer in enumerate(spec.layers)]
        shared: dict = {}          # tensors that several steps between layers use are loaded once
        self.before = [None if e.before is None else part_class("stream", e.before)(e.before, weights, "", runtime, shared=shared)
                       for e in spec.order]

    @property
    def graph_safe(self) -> bool:
        return all(getattr(layer, "graph_safe", True) for layer in self.layers)

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights one decode step reads: every matrix of every run entry, the output matrix."""
        total = self.lm_head.numel() * self.lm_head.element_size()
        if self.position_table is not None:
            total += self.spec.hidden_size * self.position_table.element_size()
        for e in self.spec.order:
            total += getattr(self.layers[e.layer], "weight_bytes", lambda: 0)()
        total += sum(b.weight_bytes() for b in self.before if b is not None and hasattr(b, "weight_bytes"))
        return total

    def plan(self, views, page_size: int, max_blocks: int, state_views=None) -> Program:
        """The whole model as a program: the embedding, the layers in their run order, the final norm over the wanted
        rows with the logit scale riding on it (as in the reference, scripts/jiuge.py:198-201), the output product."""
        import ctypes
        from .. import kernels
        spec = self.spec
        program = Program(self.runtime, spec.hidden_size, page_size, max_blocks, capacity=8 * len(spec.order) + 8)
        program.emit("jk_emit_embedding", ctypes.c_void_p(self.embedding.data_ptr()), ctypes.c_int(kernels.dtype_code(self.embedding.dtype)),
                     ctypes.c_int(spec.hidden_size), ctypes.c_float(spec.embed_scale), keep=(self.embedding,))
        hidden = spec.hidden_size
        if self.position_table is not None:
            from .program import record
            program.emit_records([record("add_rows", "x", "x", n=hidden, k=self.position_table.shape[0], w=self.position_table,
                                         w_dtype=kernels.dtype_code(self.position_table.dtype), fixed_row=-1)], keep=(self.position_table,))
        if any(getattr(b, "needs_embedding_output", False) for b in self.before):
            from .program import record
            program.emit_records([record("embed", None, "x0", n=hidden, w=self.embedding, w_dtype=kernels.dtype_code(self.embedding.dtype),
                                         scale=spec.embed_scale)], keep=(self.embedding,))
        for index, e in enumerate(spec.order):
            layer, view = self.layers[e.layer], views[e.cache]
            if self.before[index] is not None:
                self.before[index].plan(program)
            own = state_views[index] if state_views else None
            if hasattr(layer, "plan"):
                if own is not None or hasattr(type(layer), "state_need"):
                    layer.plan(program, view, e.writes_cache, state_view=own)
                else:
                    layer.plan(program, view, e.writes_cache)
            else:
                program.host(_host_block(layer, view, e.writes_cache, hidden))
        if hasattr(self.final_norm, "plan"):
            self.final_norm.plan(program, out_scale=spec.logit_scale, wanted_rows=True)
        else:
            program.host(_host_final_norm(self.final_norm, spec.logit_scale, hidden))
        program.emit("jk_emit_output", ctypes.c_void_p(self.lm_head.data_ptr()), ctypes.c_int(spec.vocab_size),
                     ctypes.c_int(spec.hidden_size), keep=(self.lm_head,))
        if spec.logit_softcap:
            from .program import record
            program.emit_records([record("softcap", "logits", None, n=spec.vocab_size, cap=float(spec.logit_softcap), wanted_rows=True)])
        return program


def _host_block(layer, view, writes_cache: bool, hidden: int):
    def run_block(ctx, io):
        stream = ResidualStream(io.view("x", hidden))
        layer.forward(stream, ctx, view, writes_cache)
        stream.value()
    run_block.__qualname__ = type(layer).__name__ + ".forward"
    return run_block


def _host_final_norm(norm, logit_scale: float, hidden: int):
    def run_final_norm(ctx, io):
        out = norm.forward(ResidualStream(io.view("x", hidden)), ctx, out_scale=logit_scale, rows=ctx.want_rows)
        io.view("hw", hidden, rows=out.shape[0]).copy_(out)
    run_final_norm.__qualname__ = type(norm).__name__ + ".forward"
    return run_final_norm
