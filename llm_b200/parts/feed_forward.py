"""SwiGLU feed-forward: down( silu(gate(x)) * up(x) ).

The reference runs gate and up as two products and the activation as a third kernel
(model/modules/MLP.h:10-13, kernel/activation/SwiGLU.h:31-33); here gate and up are
one product over a stacked weight, and with many rows (prompts) the product's epilogue applies
the activation itself, so that the stacked product never reaches memory.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import ParamInfo, Part, register_part
from .linear import FUSE_PARTIALS, linear, linear_act, linear_swiglu


_GLU_NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight",
              "gate_bias": "gate_proj.bias", "up_bias": "up_proj.bias", "down_bias": "down_proj.bias"}


class SwiGLU(Part):
    """down( act(gate(x)) * up(x) ) with act silu (the default) or relu; other tensor names through `names`."""

    role = "ffn"

    def __init__(self, hidden_size: int, intermediate_size: int, bias: bool = False, activation: str = "silu", names=None,
                 prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        if activation not in ops.GLU_ACTIVATIONS:
            raise ValueError(f"gated feed-forward: unknown activation '{activation}'; known: {sorted(ops.GLU_ACTIVATIONS)}")
        self.activation = activation
        self.names = dict(_GLU_NAMES, **(names or {}))
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.bias = bool(bias)        # the three projections carry bias vectors (model/modules/MLP.h:9-13)
        self.w_gate_up = None
        self.w_down = None
        self.b_gate_up = None
        self.b_down = None

    def parameters(self):
        n = lambda k: self.name(self.names[k])
        p = {
            n("gate"): ParamInfo((self.intermediate_size, self.hidden_size)),
            n("up"): ParamInfo((self.intermediate_size, self.hidden_size)),
            n("down"): ParamInfo((self.hidden_size, self.intermediate_size)),
        }
        if self.bias:
            p[n("gate_bias")] = ParamInfo((self.intermediate_size,), kind="gain", init="normal")
            p[n("up_bias")] = ParamInfo((self.intermediate_size,), kind="gain", init="normal")
            p[n("down_bias")] = ParamInfo((self.hidden_size,), kind="gain", init="normal")
        return p

    def bind(self, tensors):
        n = lambda k: tensors[self.name(self.names[k])]
        self.w_gate_up = torch.cat([n("gate"), n("up")], dim=0).contiguous()
        self.w_down = n("down").contiguous()
        if self.bias:
            self.b_gate_up = torch.cat([n("gate_bias"), n("up_bias")]).contiguous()
            self.b_down = n("down_bias").contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        T, ws = ctx.n_tokens, ctx.workspace
        act = ws.get("ffn_act", T, self.intermediate_size, self.dtype)
        # with many rows the product's epilogue makes the activation; with few rows, or biases, the row kernel
        if self.bias or not linear_swiglu(x, self.w_gate_up, act, T, self.activation):
            gate_up = linear(x, self.w_gate_up, ws.get("gate_up", T, 2 * self.intermediate_size, self.dtype), T,
                             allow_partial=FUSE_PARTIALS, bias=self.b_gate_up)
            ops.silu_mul(act, gate_up, T, self.activation)
        return linear(act, self.w_down, ws.get("ffn_out", T, self.hidden_size, self.dtype), T, allow_partial=FUSE_PARTIALS,
                      bias=self.b_down)


register_part("ffn", "swiglu", SwiGLU)


class ActMLP(Part):
    """down(act(up(x))): a feed-forward with one up-projection and an element-wise activation
    ("relu2": the square of relu, "gelu": erf, "gelu_tanh", "silu").  Tensors `<prefix>.up` and
    `<prefix>.down` unless other names are given."""

    role = "ffn"

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "relu2", up_name: str = "up",
                 down_name: str = "down", prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"feed-forward: unknown activation '{activation}'; known: {sorted(ops.ACTIVATIONS)}")
        self.hidden_size, self.intermediate_size, self.activation = hidden_size, intermediate_size, activation
        self.up_name, self.down_name = up_name, down_name
        self.w_up = self.w_down = None

    def parameters(self):
        return {self.name(self.up_name): ParamInfo((self.intermediate_size, self.hidden_size)),
                self.name(self.down_name): ParamInfo((self.hidden_size, self.intermediate_size))}

    def bind(self, tensors):
        self.w_up = tensors[self.name(self.up_name)].contiguous()
        self.w_down = tensors[self.name(self.down_name)].contiguous()

    def forward(self, x: torch.Tensor, ctx, tag: str = "ffn") -> torch.Tensor:
        T, ws = ctx.n_tokens, ctx.workspace
        act = ws.get(tag + "_act", T, self.intermediate_size, self.dtype)
        if not linear_act(x, self.w_up, act, T, self.activation):      # many rows: the activation in the product's epilogue
            up = linear(x, self.w_up, ws.get(tag + "_up", T, self.intermediate_size, self.dtype), T, allow_partial=FUSE_PARTIALS)
            ops.act_rows(act, up, T, self.activation)
        return linear(act, self.w_down, ws.get(tag + "_out", T, self.hidden_size, self.dtype), T, allow_partial=FUSE_PARTIALS)


register_part("ffn", "mlp", ActMLP)


class ClampedGLU(Part):
    """down( g * sigmoid(alpha g) * (u + 1) ) with g = min(gate(x), limit) and u = clamp(up(x), -limit, limit): a gated
    unit whose gate is cut off above, whose linear branch is cut off on both sides and shifted by one.  All three
    projections carry biases unless bias is off.  Tensors `<prefix>.gate|up|down` and `<name>.b`; limit and alpha
    are parameters."""

    role = "ffn"

    def __init__(self, hidden_size: int, intermediate_size: int, limit: float, alpha: float = 1.702, bias: bool = True,
                 prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        if min(hidden_size, intermediate_size) <= 0 or not limit > 0:
            raise ValueError("clamped gated unit: sizes and limit must be positive")
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.limit, self.alpha, self.bias = float(limit), float(alpha), bool(bias)
        self.w_gate_up = self.w_down = self.b_gate_up = self.b_down = None

    def parameters(self):
        n, W, I = self.name, self.hidden_size, self.intermediate_size
        p = {n("gate"): ParamInfo((I, W)), n("up"): ParamInfo((I, W)), n("down"): ParamInfo((W, I))}
        if self.bias:
            p.update({n("gate.b"): ParamInfo((I,), kind="gain", init="normal"), n("up.b"): ParamInfo((I,), kind="gain", init="normal"),
                      n("down.b"): ParamInfo((W,), kind="gain", init="normal")})
        return p

    def bind(self, tensors):
        t = lambda local: tensors[self.name(local)]
        self.w_gate_up = torch.cat([t("gate"), t("up")], dim=0).contiguous()
        self.w_down = t("down").contiguous()
        if self.bias:
            self.b_gate_up = torch.cat([t("gate.b"), t("up.b")]).contiguous()
            self.b_down = t("down.b").contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        T, ws = ctx.n_tokens, ctx.workspace
        I = self.intermediate_size
        # one product for gate and up; its split-K partial results go unsummed to the activation kernel, which
        # adds the biases, clamps and multiplies in float32
        gate_up = linear(x, self.w_gate_up, ws.get("gate_up", T, 2 * I, self.dtype), T, allow_partial=FUSE_PARTIALS)
        act = ws.get("ffn_act", T, I, self.dtype)
        ops.clamped_glu(act, gate_up, self.b_gate_up, T, self.limit, self.alpha)
        return linear(act, self.w_down, ws.get("ffn_out", T, self.hidden_size, self.dtype), T, allow_partial=FUSE_PARTIALS,
                      bias=self.b_down)


register_part("ffn", "clamped_glu", ClampedGLU)
