"""The dense gated feed-forward (SwiGLU)."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorDecl
from .base import FeedForward, RowStats, as_delta, matrix, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    """delta = down(silu(gate(x)) * up(x)); SiLU on the gate, no biases
    (crates/mach-model/src/batched.rs:4424-4453 of gqf2008/machserve).  gate and up are one
    matrix product over the concatenated weights.

    params: prefix, hidden_size, intermediate_size; tensor names `{prefix}gate_proj.weight`,
    `{prefix}up_proj.weight`, `{prefix}down_proj.weight`.
    """

    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        self.prefix = spec["prefix"]
        self.hidden, self.inter = int(spec["hidden_size"]), int(spec["intermediate_size"])

    def tensors(self):
        p = self.prefix
        return [
            TensorDecl(p + "gate_proj.weight", (self.inter, self.hidden)),
            TensorDecl(p + "up_proj.weight", (self.inter, self.hidden)),
            TensorDecl(p + "down_proj.weight", (self.hidden, self.inter)),
        ]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        p = self.prefix
        self.w_gate_up = matrix(torch.cat([tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]], dim=0), rt)
        self.w_down = matrix(tensors[p + "down_proj.weight"], rt)

    # With few rows in bfloat16 the norm in front and the add behind need no kernels of their own: the gate/up
    # product reads the residual's bfloat16 copy and divides its output rows by the rows' rms (the norm's weight is
    # folded into the matrix's columns), and the down product adds into the float32 residual and leaves each row's
    # sums of squares and a bfloat16 copy for the part that follows.
    fused_rows = 16

    def fuse_norm(self, norm):
        import torch

        rt = self.rt
        ok = (rt.dtype == torch.bfloat16 and self.hidden % 8 == 0 and self.inter % 8 == 0
              # matrices that the small-row products stream faster than the library does (measured: up to about
              # 64 MB; a 7B model's gate/up and down matrices go through the library at twice the speed)
              and all(w.numel() * w.element_size() <= ops.SMALL_M_MAX_WEIGHT_BYTES for w in (self.w_gate_up, self.w_down)))
        return ok and norm.fold_into(self.w_gate_up)

    def forward_fused(self, ctx, residual, pending, norm, cache=None, owns_cache=True):
        import torch

        rt, ws = self.rt, self.rt.workspace
        t, d = residual.shape
        nb = ops.gemm_small_m_stats_blocks(d)
        h = ws.get("ffn.h", (t, self.inter), rt.dtype)
        xcopy = ws.get("block.residual_copy", (t, d), rt.dtype)
        if isinstance(pending, RowStats) and pending.copy is not None:
            ops.gemm_small_m_scaled(pending.copy, pending.stats, pending.blocks, norm.eps, self.w_gate_up[: self.inter],
                                    self.w_gate_up[self.inter :], h)
        else:  # after a part that returned a delta
            xn = ws.get("block.normed", (t, d), rt.dtype)
            norm.forward(residual, as_delta(pending), xn)
            ops.gemm_small_m_silu_mul(xn, self.w_gate_up[: self.inter], self.w_gate_up[self.inter :], h)
        stats = ws.get("block.stats_ffn", (t, nb), torch.float32)
        ops.gemm_small_m_resadd(h, self.w_down, residual, stats, xcopy)
        return RowStats(stats, nb, xcopy)

    def forward(self, ctx, x):
        rt, t = self.rt, x.shape[0]
        ws = rt.workspace
        h = ws.get("ffn.h", (t, self.inter), rt.dtype)
        if rt.dtype == torch.bfloat16 and ops.gemm_small_m_preferred(t, self.inter, self.hidden):
            # few rows: gate, up and the gating in one pass over the weights
            ops.gemm_small_m_silu_mul(x, self.w_gate_up[: self.inter], self.w_gate_up[self.inter :], h)
        elif rt.dtype == torch.bfloat16 and ops.gemm_pair_tc_silu_preferred(t, self.inter, self.hidden):
            # many rows of a wide model: the gating in the epilogue of this repository's tcgen05 product
            ops.gemm_pair_tc_silu_mul(x, self.w_gate_up, h)
        else:
            gate_up = ws.get("ffn.gate_up", (t, 2 * self.inter), rt.dtype)
            ops.linear(x, self.w_gate_up, None, gate_up)
            ops.silu_mul(gate_up, h)
        delta = ws.get("ffn.delta", (t, self.hidden), rt.dtype)
        return ops.linear(h, self.w_down, None, delta)
