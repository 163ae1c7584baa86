"""A step between two layers that adds one row of a table to the whole stream: x <- x + table[index].

The table holds one vector per pass of a repeated span of layers; the specification says which row this step adds.
One record (``add_rows`` with a fixed row); the table is kept in float32 and loaded once for all passes.
"""
from __future__ import annotations

from typing import Dict

from ..weights import VECTOR, TensorDecl
from .base import register
from .program import record


@register("stream", "step_vector")
class StepVector:
    @staticmethod
    def tensor_decls(spec) -> Dict[str, TensorDecl]:
        return {spec.table_name: TensorDecl((spec.steps, spec.hidden_size), VECTOR, init="zeros")}

    def __init__(self, spec, weights, prefix: str, runtime, shared=None):
        self.spec = spec
        shared = shared if shared is not None else {}
        name = spec.table_name
        self.table = shared[name] if name in shared else shared.setdefault(name, weights.get(prefix + name, VECTOR))
        if not 0 <= spec.index < self.table.shape[0]:
            raise ValueError(f"row {spec.index} of a table of {self.table.shape[0]}")

    def weight_bytes(self) -> int:
        return self.spec.hidden_size * self.table.element_size()

    def plan(self, program) -> None:
        from .. import kernels
        s = self.spec
        program.emit_records([record("add_rows", "x", "x", n=s.hidden_size, k=self.table.shape[0], w=self.table,
                                     w_dtype=kernels.dtype_code(self.table.dtype), fixed_row=s.index)], keep=(self.table,))
