"""RMSNorm on the residual stream.

y = x * rsqrt(mean(x^2) + eps) * gain with the sum, the root and the scaling in
float32 (kernel/LayerNorm/RMSNorm.h:13-30,40-42 of the reference).  The stream's
pending term is added to the residual in the same pass
(kernel/residual/Residual.h:17-19 is a separate kernel there).
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import ParamInfo, Part, ResidualStream, register_part


class RMSNorm(Part):
    role = "norm"

    def __init__(self, size: int, eps: float, weight_name: str = "weight", prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        self.size = size
        self.eps = float(eps)
        self.weight_name = weight_name        # "": the gain is the tensor named like the part
        self.gain = None

    def parameters(self):
        return {self.name(self.weight_name): ParamInfo((self.size,), kind="gain", init="ones_normal")}

    def bind(self, tensors):
        self.gain = tensors[self.name(self.weight_name)]

    def forward(self, stream: ResidualStream, ctx, tag: str = "normed") -> torch.Tensor:
        out = ctx.workspace.get(tag, stream.rows, self.size, self.dtype)
        ops.add_rmsnorm(stream.resid, stream.pending, self.gain, out, stream.rows, self.eps)
        stream.pending = None
        return out

    def forward_rows(self, rows_f32: torch.Tensor, n_rows: int, out: torch.Tensor) -> torch.Tensor:
        """Norm of float32 rows that are not a stream (the gathered rows before the head)."""
        ops.add_rmsnorm(rows_f32, None, self.gain, out, n_rows, self.eps)
        return out


register_part("norm", "rmsnorm", RMSNorm)


class DynamicTanh(Part):
    """y = tanh(alpha * x) * w + b: a norm that takes no mean and no variance, so every element
    stands alone.  alpha is a scalar, w and b vectors; the tensors are `<prefix>` (w),
    `<prefix>.b` and `<prefix>.alpha` unless other names are given.  The arithmetic is float32 on
    the float32 residual, and the stream's pending term is added in the same pass."""

    role = "norm"

    def __init__(self, size: int, weight_name: str = "", bias_name: str = "b", alpha_name: str = "alpha",
                 prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        self.size = size
        self.names = (self.name(weight_name), self.name(bias_name), self.name(alpha_name))
        self.w = self.b = None
        self.alpha = 1.0

    def parameters(self):
        w, b, a = self.names
        return {w: ParamInfo((self.size,), kind="gain", init="ones_normal"),
                b: ParamInfo((self.size,), kind="gain", init="normal"),
                a: ParamInfo((), kind="gain", init="ones_normal")}

    def bind(self, tensors):
        w, b, a = self.names
        self.w, self.b = tensors[w].contiguous(), tensors[b].contiguous()
        self.alpha = float(tensors[a].item())

    def forward(self, stream: ResidualStream, ctx, tag: str = "normed") -> torch.Tensor:
        out = ctx.workspace.get(tag, stream.rows, self.size, self.dtype)
        ops.add_dyt(stream.resid, stream.pending, self.w, self.b, self.alpha, out, stream.rows)
        stream.pending = None
        return out

    def forward_rows(self, rows_f32: torch.Tensor, n_rows: int, out: torch.Tensor) -> torch.Tensor:
        ops.add_dyt(rows_f32, None, self.w, self.b, self.alpha, out, n_rows)
        return out


register_part("norm", "dyt", DynamicTanh)


class LayerNorm(Part):
    """y = (x - mean(x)) / sqrt(var(x) + eps) * w with a weight and no bias, the variance taken from the
    deviations, everything in float32.  The part serves on both sides of a residual sum: `forward` norms
    the stream for the next sublayer (adding first what is pending, like the other norms), and `attach`
    leaves a sublayer's output pending on the stream as a term that is still to be normed by this part
    and scaled by `mult` before it joins the residual: x += mult * ln(y).  The norm that comes next (or
    `fold`) does both in one pass over the row.  The tensor is `<prefix>` unless a name is given."""

    role = "norm"

    def __init__(self, size: int, eps: float, weight_name: str = "", prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        self.size, self.eps = size, float(eps)
        self.weight_name = weight_name
        self.gain = None

    def parameters(self):
        return {self.name(self.weight_name): ParamInfo((self.size,), kind="gain", init="ones_normal")}

    def bind(self, tensors):
        self.gain = tensors[self.name(self.weight_name)].contiguous()

    def _post(self, stream: ResidualStream):
        """(post-norm weight, multiplier) of the stream's pending term."""
        if stream.pending is None or stream.pending_post is None:
            return None, 1.0
        part, mult = stream.pending_post
        if not isinstance(part, LayerNorm) or part.eps != self.eps:
            raise ValueError("a pending term that another kind of norm is to treat cannot be folded by this one")
        return part.gain, float(mult)

    def forward(self, stream: ResidualStream, ctx, tag: str = "normed") -> torch.Tensor:
        out = ctx.workspace.get(tag, stream.rows, self.size, self.dtype)
        post, mult = self._post(stream)
        ops.add_layernorm(stream.resid, stream.pending, post, mult, self.gain, out, stream.rows, self.eps)
        stream.pending = stream.pending_post = None
        return out

    def attach(self, stream: ResidualStream, y, mult: float = 1.0) -> None:
        stream.pending, stream.pending_post = y, (self, float(mult))

    def fold(self, stream: ResidualStream, ctx) -> None:
        """resid += mult * ln(pending): the stream made whole without a norm after it."""
        post, mult = self._post(stream)
        ops.add_layernorm(stream.resid, stream.pending, post, mult, None, None, stream.rows, self.eps)
        stream.pending = stream.pending_post = None

    def forward_rows(self, rows_f32: torch.Tensor, n_rows: int, out: torch.Tensor) -> torch.Tensor:
        ops.add_layernorm(rows_f32, None, None, 1.0, self.gain, out, n_rows, self.eps)
        return out


register_part("norm", "layernorm", LayerNorm)
