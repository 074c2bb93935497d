"""Hyper-connections: the residual stream kept as several copies, mixed anew around every sublayer.

Instead of one x a token carries S streams x_1 .. x_S (all equal to the embedding at the start; the model's
output is their sum).  A sublayer reads one mix of them and writes back into all of them:

    u    = sum_s a[s] x_s                       a  [S]       what the sublayer's norm sees
    y    = sublayer(norm(u))
    x_t <- sum_s M[s, t] x_s + b[t] y           M  [S, S] indexed (from, to), b [S]; all streams at once from the old ones

With S = 1, a = b = 1 and M = 1 this is the plain residual sum.  The streams of a token lie side by side in one
float32 row of the engine's residual buffer (ModelSpec.stream_copies = S).  As with the single stream, a sublayer's
output stays pending until the next norm: `HyperNorm.forward` first applies the write of the sublayer before it,
then forms u and norms it, in one pass over the row (csrc/hyper.cu).

The norm of this part is an RMS norm whose gain is one number for all coordinates; `ScalarRMSNorm` is the same norm
on a plain stream (the rows before the head).
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import ParamInfo, Part, ResidualStream, build_part, register_part


class HyperNorm(Part):
    """The read, the norm and the write of one sublayer.  Tensors: `<prefix>.<gain_name>` (one number) and
    `<prefix>.<hc_name>.in|out|mix`."""

    role = "norm"

    def __init__(self, size: int, streams: int, eps: float, gain_name: str = "norm", hc_name: str = "hc",
                 prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        if size <= 0 or not (1 <= streams <= 8):
            raise ValueError(f"hyper-connections: width {size} must be positive and streams {streams} 1 to 8")
        self.size, self.streams, self.eps = int(size), int(streams), float(eps)
        self.gain_name, self.hc_name = gain_name, hc_name
        self.gain = self.w_in = self.w_out = self.w_mix = None

    def _names(self):
        hc = self.name(self.hc_name)
        return self.name(self.gain_name), hc + ".in", hc + ".out", hc + ".mix"

    def parameters(self):
        g, a, b, m = self._names()
        S = self.streams
        return {g: ParamInfo((), kind="gain", init="ones_normal"), a: ParamInfo((S,), kind="gain", init="ones_normal"),
                b: ParamInfo((S,), kind="gain", init="ones_normal"), m: ParamInfo((S, S), kind="gain", init="eye_normal")}

    def bind(self, tensors):
        g, a, b, m = self._names()
        self.gain = tensors[g].reshape(1).contiguous()
        self.w_in, self.w_out, self.w_mix = tensors[a].contiguous(), tensors[b].contiguous(), tensors[m].contiguous()

    def _pending(self, stream: ResidualStream):
        """(y, M, b) of the write that is still to be done, or three Nones."""
        if stream.pending is None:
            return None, None, None
        post = stream.pending_post
        if post is None or not isinstance(post[0], HyperNorm) or post[0].streams != self.streams:
            raise ValueError("hyper-connections: a pending term must come from a sublayer of the same streams")
        return stream.pending, post[0].w_mix, post[0].w_out

    def forward(self, stream: ResidualStream, ctx, tag: str = "normed") -> torch.Tensor:
        out = ctx.workspace.get(tag, stream.rows, self.size, self.dtype)
        y, mix, wout = self._pending(stream)
        ops.hc_norm(stream.resid, y, mix, wout, self.w_in, self.gain, out, stream.rows, self.size, self.streams, self.eps,
                    self.dtype)
        stream.pending = stream.pending_post = None
        return out

    def attach(self, stream: ResidualStream, y, mult: float = 1.0) -> None:
        """Leave the sublayer's output pending: this part's M and b are applied by the next norm (or by fold)."""
        stream.pending, stream.pending_post = y, (self, 1.0)

    def fold(self, stream: ResidualStream, ctx) -> None:
        y, mix, wout = self._pending(stream)
        ops.hc_norm(stream.resid, y, mix, wout, None, None, None, stream.rows, self.size, self.streams, self.eps, self.dtype)
        stream.pending = stream.pending_post = None


register_part("norm", "hyper_rmsnorm", HyperNorm)


class ScalarRMSNorm(Part):
    """x / sqrt(mean(x^2) + eps) * g with one number g (the tensor named like the part unless a name is given), float32."""

    role = "norm"

    def __init__(self, size: int, eps: float, weight_name: str = "", prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        self.size, self.eps, self.weight_name = int(size), float(eps), weight_name
        self.gain = None

    def parameters(self):
        return {self.name(self.weight_name): ParamInfo((), kind="gain", init="ones_normal")}

    def bind(self, tensors):
        self.gain = tensors[self.name(self.weight_name)].reshape(1).contiguous()

    def forward(self, stream: ResidualStream, ctx, tag: str = "normed") -> torch.Tensor:
        stream.fold(ctx)
        out = ctx.workspace.get(tag, stream.rows, self.size, self.dtype)
        ops.scalar_rmsnorm_rows(out, stream.resid, self.gain, stream.rows, self.eps)
        return out

    def forward_rows(self, rows_f32: torch.Tensor, n_rows: int, out: torch.Tensor) -> torch.Tensor:
        ops.scalar_rmsnorm_rows(out, rows_f32, self.gain, n_rows, self.eps)
        return out


register_part("norm", "scalar_rmsnorm", ScalarRMSNorm)


class HyperBlock:
    """u = read1(x); x <- write1(x, mixer(norm1(u))); the same around the feed-forward with the second set of weights.
    A layer without a feed-forward has only the first sublayer.  norm1 and norm2 are HyperNorm parts (they hold the
    read and write weights of their sublayer)."""

    role = "block"
    roles = {"norm1": "norm", "mixer": "mixer", "norm2": "norm", "ffn": "ffn"}

    def __init__(self, part_specs, dtype, device):
        optional = ("norm2", "ffn") if part_specs.get("ffn") is None else ()
        missing = [r for r in self.roles if part_specs.get(r) is None and r not in optional]
        if missing:
            raise ValueError(f"hyper block lacks parts {missing}")
        self.parts = {r: build_part(self.roles[r], part_specs[r], dtype, device) if part_specs.get(r) is not None else None
                      for r in self.roles}
        for r in ("norm1", "norm2"):
            if self.parts[r] is not None and not hasattr(self.parts[r], "attach"):
                raise ValueError(f"hyper block: the norm '{part_specs[r].kind}' holds no write weights (no attach)")
        self.mixer, self.ffn = self.parts["mixer"], self.parts["ffn"]

    def forward(self, stream: ResidualStream, ctx, view) -> None:
        p = self.parts
        p["norm1"].attach(stream, self.mixer.forward(p["norm1"].forward(stream, ctx), ctx, view))
        if self.ffn is not None:
            p["norm2"].attach(stream, self.ffn.forward(p["norm2"].forward(stream, ctx), ctx))


register_part("block", "hyper", HyperBlock)
