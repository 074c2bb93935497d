"""How a layer's parts are arranged on the residual stream.

"prenorm": x += mixer(norm1(x)); x += ffn(norm2(x)), the arrangement of the
reference's block (model/llm/tiny_llama.cpp:29-34).  Each sum is left pending on
the stream and folded in by the next norm.  A layer without a feed-forward leaves
out norm2 and ffn: it is x += mixer(norm1(x)) alone.
"""
from __future__ import annotations

import dataclasses

import torch

from .base import ResidualStream, StateNeed, build_part, register_part


class PreNormBlock:
    role = "block"
    roles = {"norm1": "norm", "mixer": "mixer", "norm2": "norm", "ffn": "ffn"}

    def __init__(self, part_specs, dtype, device):
        optional = ("norm2", "ffn") if part_specs.get("ffn") is None else ()
        missing = [r for r in self.roles if part_specs.get(r) is None and r not in optional]
        if missing:
            raise ValueError(f"prenorm block lacks parts {missing}")
        self.parts = {r: build_part(self.roles[r], part_specs[r], dtype, device) if part_specs.get(r) is not None else None
                      for r in self.roles}
        self.norm1, self.mixer = self.parts["norm1"], self.parts["mixer"]
        self.norm2, self.ffn = self.parts["norm2"], self.parts["ffn"]
        # a feed-forward that keeps something per request (the inputs of a convolution over time) says so with state_need();
        # the layer's state row is then the mixer's numbers followed by the feed-forward's
        self.ffn_state = self.ffn.state_need() if self.ffn is not None and hasattr(self.ffn, "state_need") else None
        self.mixer_cols = 0
        if self.ffn_state is not None:
            need = self.mixer.state_need()
            n = 1
            for d in (need.shape if need is not None else (0,)):
                n *= int(d)
            self.mixer_cols = (n + 3) // 4 * 4
            if need is not None and need.dtype != torch.float32 or self.ffn_state.dtype != torch.float32 or len(self.ffn_state.shape) != 1:
                raise ValueError("prenorm block: the states of a mixer and a feed-forward that share a row are flat float32")

    def state_need(self):
        """What the layer keeps per request: the mixer's state, followed by the feed-forward's where it has one."""
        if self.ffn_state is None:
            return self.mixer.state_need()
        return StateNeed((self.mixer_cols + int(self.ffn_state.shape[0]),), torch.float32)

    def forward(self, stream: ResidualStream, ctx, view) -> None:
        if self.ffn_state is None:
            stream.pending = self.mixer.forward(self.norm1.forward(stream, ctx), ctx, view)
            if self.ffn is not None:
                stream.pending = self.ffn.forward(self.norm2.forward(stream, ctx), ctx)
            return
        rows = view.state.view(view.state.shape[0], -1)
        mixer_view = dataclasses.replace(view, state=rows[:, :self.mixer_cols] if self.mixer_cols else None)
        stream.pending = self.mixer.forward(self.norm1.forward(stream, ctx), ctx, mixer_view)
        stream.pending = self.ffn.forward(self.norm2.forward(stream, ctx), ctx, state=rows[:, self.mixer_cols:])


register_part("block", "prenorm", PreNormBlock)


class SandwichBlock:
    """x += m * post1(mixer(norm1(x))); x += m * post2(ffn(norm2(x))): every sublayer has a norm before it
    and a norm on its output, and the normed output joins the residual scaled by m.  The output is left
    pending on the stream with its norm still to do (norm.attach), so that the next norm adds and norms
    in one pass.  A layer without a feed-forward leaves out norm2, ffn and post2."""

    role = "block"
    roles = {"norm1": "norm", "mixer": "mixer", "post1": "norm", "norm2": "norm", "ffn": "ffn", "post2": "norm"}

    def __init__(self, part_specs, dtype, device, residual_mult: float = 1.0):
        self.mult = float(residual_mult)
        optional = ("norm2", "ffn", "post2") if part_specs.get("ffn") is None else ()
        missing = [r for r in self.roles if part_specs.get(r) is None and r not in optional]
        if missing:
            raise ValueError(f"sandwich block lacks parts {missing}")
        self.parts = {r: build_part(self.roles[r], part_specs[r], dtype, device) if part_specs.get(r) is not None else None
                      for r in self.roles}
        for r in ("post1", "post2"):
            if self.parts[r] is not None and not hasattr(self.parts[r], "attach"):
                raise ValueError(f"sandwich block: the norm '{part_specs[r].kind}' cannot stand behind a sublayer (no attach)")
        self.mixer, self.ffn = self.parts["mixer"], self.parts["ffn"]

    def forward(self, stream: ResidualStream, ctx, view) -> None:
        p = self.parts
        p["post1"].attach(stream, self.mixer.forward(p["norm1"].forward(stream, ctx), ctx, view), self.mult)
        if self.ffn is not None:
            p["post2"].attach(stream, self.ffn.forward(p["norm2"].forward(stream, ctx), ctx), self.mult)


register_part("block", "sandwich", SandwichBlock)


class StreamBlock:
    """A place in the layer order that holds no layer but one transform of the whole stream (role "stream")."""

    role = "block"

    def __init__(self, part_specs, dtype, device):
        self.parts = {"stream": build_part("stream", part_specs["stream"], dtype, device)}
        self.mixer = None

    def forward(self, stream: ResidualStream, ctx, view) -> None:
        self.parts["stream"].forward(stream, ctx)


register_part("block", "stream", StreamBlock)
