"""RMSNorm: y = x * w / sqrt(mean(x^2) + eps), computed in float32.

Reference: ``rmsnorm`` at src/models/jiuge/jiuge.cpp:198, :246, :262 with a float32 weight
(scripts/jiuge.py:145-146).  The pending residual addition is done by the same kernel.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..weights import VECTOR, TensorDecl
from .base import ResidualStream, register


@register("norm", "rmsnorm")
class RMSNorm:
    @staticmethod
    def tensor_decls(spec) -> Dict[str, TensorDecl]:
        return {spec.weight_name: TensorDecl((spec.size,), VECTOR, init="zeros" if getattr(spec, "one_plus", False) else "ones")}

    def __init__(self, spec, weights, prefix: str, runtime):
        self.spec, self.runtime = spec, runtime
        self.weight = weights.get(prefix + spec.weight_name, VECTOR)
        if getattr(spec, "one_plus", False):          # stored around zero: the factor is 1 + w, formed once in float32
            self.weight = (self.weight.to(torch.float32) + 1.0).contiguous()

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def plan(self, program, out_scale: float = 1.0, wanted_rows: bool = False) -> None:
        """One record: add what waits for the stream, normalise every row (or the wanted rows) into the next product's
        activations."""
        import ctypes
        program.emit("jk_emit_rmsnorm", ctypes.c_void_p(self.weight.data_ptr()), ctypes.c_int(self.spec.size),
                     ctypes.c_float(self.spec.eps), ctypes.c_float(out_scale), ctypes.c_int(1 if wanted_rows else 0),
                     keep=(self.weight,))

    def plan_add(self, program) -> None:
        """One record: stream += rmsnorm(the product that waits in the delta slot) * weight.  The norm of the sublayer that
        follows may join the record (``plan_after_add``)."""
        from .program import record
        program.emit_records([record("norm_add", "delta", None, n=self.spec.size, eps=self.spec.eps, vec=self.weight)], keep=(self.weight,))

    def plan_after_add(self, program) -> None:
        """This norm over every row, right after a ``plan_add``: it joins that record (the kernel holds the new stream's row
        in shared memory), else it is a record of its own."""
        if not program.amend_last("norm_add", out_slot="h", vec2=self.weight, eps2=self.spec.eps):
            self.plan(program)
        else:
            program.keep.append(self.weight)

    def forward(self, residual: ResidualStream, ctx, out_scale: float = 1.0,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Normalise every row, or only ``rows`` (int32 indices) of the residual stream."""
        from .. import kernels
        n = rows.numel() if rows is not None else residual.x.shape[0]
        out = self.runtime.empty(n, self.spec.size)
        delta, scale = residual.take_pending()
        kernels.add_rmsnorm(residual.x, delta, scale, self.weight, self.spec.eps, out, out_scale, rows)
        return out
