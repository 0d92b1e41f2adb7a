"""RMSNorm with the residual add fused in front of it."""
from __future__ import annotations

from .. import ops
from ..weights.loader import TensorDecl
from .base import Norm, as_delta, register_norm, vector_f32


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """y = x * rsqrt(mean(x^2) + eps) * w: eps inside the root, plain x*w, mean over the whole width,
    all in float32 (crates/mach-model/src/kernels.rs:63-80 of gqf2008/machserve).

    params: tensor (name of the weight), size, eps.
    """

    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        self.name, self.size, self.eps = spec["tensor"], int(spec["size"]), float(spec["eps"])

    def tensors(self):
        return [TensorDecl(self.name, (self.size,), init="scale")]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = vector_f32(tensors[self.name])

    def forward(self, residual, delta, out, rows=None):
        return ops.add_rmsnorm(residual, as_delta(delta), self.weight, out, self.eps, rows)

    def fold_into(self, matrix):
        """W[n][k] *= g[k], in float32 and rounded once; g becomes 1 ((x / rms * g) . W^T = (x . (W g)^T) / rms)."""
        matrix.copy_((matrix.float() * self.weight[None, :]).to(matrix.dtype))
        self.weight.fill_(1.0)
        return True
