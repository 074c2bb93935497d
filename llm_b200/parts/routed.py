"""Routed feed-forward (mixture of experts) with an optional shared expert.

  z      = Wr h + b                      float32
  S      = the `top` experts with the largest z
  w_e    = softmax over { z_e : e in S } (the chosen logits alone)
  out    = sum_{e in S} w_e * down_e(act(up_e(h)))  +  down_s(act_s(up_s(h)))   (shared, if any)

Further forms, all parameters: router "softmax_all", where w_e is expert e's share of the softmax over all experts (so
the chosen weights do not sum to one); router "sigmoid_groups", where the scores are s = sigmoid(z), the choice is made on
s + correction (a learned vector, `<prefix>.correction`), the experts form `groups` equal runs of neighbours of which only the
`keep_groups` best (by the sum of their two largest choice scores) can be chosen from, and the weights are the chosen s,
not renormalised; gated experts, down_e(act(gate_e(h)) * up_e(h)), with act silu or the clamped unit
g sigmoid(alpha g) (u + 1), g = min(gate, limit), u = clamp(up, -limit, limit) (activation "clamped").

On the device: the router kernel writes each token's choices and weights; the (token, choice)
pairs are sorted by expert into tiles of one expert each; the experts' up-projections run as
one grouped product that gathers the tokens' rows and applies the activation; the
down-projections as a second grouped product into float32; the last kernel sums a token's
choices with their weights, in the order of the choices, and adds the shared expert.  Nothing
on the host looks at the routing: every launch is sized by the numbers of tokens, choices and
experts, so a step stays replayable from a CUDA graph.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import ParamInfo, Part, register_part
from .feed_forward import ActMLP


# Gated experts on the tensor cores: from this width on the grouped product applies silu(gate) * up in its epilogue;
# below it the product leaves [gate, up] and a row kernel makes the activation.  Measured on B200 (2,048-token prompt,
# decode at batch 8 / 64): width 4096 (experts of 2752): 7.35 ms, 1.39 / 2.19 ms fused against 8.28, 1.47 / 2.29; width
# 2048 (1408): 5.53, 1.25 / 2.37 against 5.31, 1.20 / 2.29; width 1024 (1408): 2.62, 0.86 / 1.30 against 2.42, 0.73 / 1.18.
# The fused tile is 128 gate rows and their 128 up rows wide; its heavier epilogue hides under the products of the next
# tile only where a tile's products take long enough (K = the width).
FUSE_GATE_FROM_WIDTH = 3072


class RoutedFFN(Part):
    role = "ffn"

    def __init__(self, hidden_size: int, experts: int, top: int, expert_size: int, activation: str = "gelu",
                 router_bias: bool = True, shared_size: int = 0, shared_activation: str = None, gated: bool = False,
                 router: str = "softmax_chosen", groups: int = 1, keep_groups: int = 1, limit: float = 0.0, alpha: float = 1.702,
                 prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        if not (0 < top <= experts <= 256):
            raise ValueError(f"routed feed-forward: top {top} of {experts} experts (1 <= top <= experts <= 256)")
        if activation not in ops.ACTIVATIONS and activation != "clamped":
            raise ValueError(f"routed feed-forward: unknown activation '{activation}'")
        self.hidden_size, self.experts, self.top, self.expert_size = hidden_size, experts, top, expert_size
        if router not in ("softmax_chosen", "softmax_all", "sigmoid_groups"):
            raise ValueError(f"routed feed-forward: unknown router '{router}'")
        if gated and activation not in ("silu", "clamped") or (activation == "clamped" and not gated):
            raise ValueError("routed feed-forward: gated experts take the silu activation or the clamped unit, and only they the latter")
        self.clamped, self.limit, self.alpha = activation == "clamped", float(limit), float(alpha)
        if self.clamped and not self.limit > 0:
            raise ValueError("routed feed-forward: the clamped unit needs a positive limit")
        self.sigmoid_groups = None
        if router == "sigmoid_groups":
            if groups <= 0 or experts % groups or not (0 < keep_groups <= groups):
                raise ValueError(f"routed feed-forward: {experts} experts in {groups} groups of which {keep_groups} are kept")
            if top > keep_groups * (experts // groups):
                raise ValueError(f"routed feed-forward: top {top} exceeds the {keep_groups * (experts // groups)} experts of the kept groups")
            self.sigmoid_groups = (int(groups), int(keep_groups))
            router_bias = False
        self.activation, self.router_bias = activation, bool(router_bias)
        self.gated, self.over_all = bool(gated), router == "softmax_all"
        self.shared = (ActMLP(hidden_size, shared_size, shared_activation or activation, prefix=self.name("shared"),
                              dtype=dtype, device=device) if shared_size else None)
        self.w_router = self.b_router = self.w_up = self.w_down = None

    def children(self):
        return [self.shared] if self.shared is not None else []

    def parameters(self):
        p = {self.name("router"): ParamInfo((self.experts, self.hidden_size))}
        if self.router_bias:
            p[self.name("router.b")] = ParamInfo((self.experts,), kind="gain", init="normal")
        if self.sigmoid_groups:
            p[self.name("correction")] = ParamInfo((self.experts,), kind="gain", init="normal")
        for e in range(self.experts):
            if self.gated:
                p[self.name(f"e{e}.gate")] = ParamInfo((self.expert_size, self.hidden_size))
            p[self.name(f"e{e}.up")] = ParamInfo((self.expert_size, self.hidden_size))
            p[self.name(f"e{e}.down")] = ParamInfo((self.hidden_size, self.expert_size))
        return p

    def bind(self, tensors):
        self.w_router = tensors[self.name("router")].contiguous()
        self.b_router = tensors[self.name("router.b")].contiguous() if self.router_bias else None
        if self.sigmoid_groups:
            self.b_router = tensors[self.name("correction")].contiguous()      # enters the choice, not the weights
        if self.gated:      # per expert [gate; up] stacked: one grouped product, then silu(gate) * up over the slots
            self.w_up = torch.stack([torch.cat([tensors[self.name(f"e{e}.gate")], tensors[self.name(f"e{e}.up")]], dim=0)
                                     for e in range(self.experts)]).contiguous()
        else:
            self.w_up = torch.stack([tensors[self.name(f"e{e}.up")] for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([tensors[self.name(f"e{e}.down")] for e in range(self.experts)]).contiguous()

    def _gate(self, act, gate_up, rows: int) -> None:
        """act = silu(gate) * up, or the clamped unit, over the slots' [gate | up] rows."""
        if self.clamped:
            ops.clamped_glu(act, gate_up, None, rows, self.limit, self.alpha)
        else:
            ops.silu_mul(act, gate_up, rows)

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        T, ws, top, E = ctx.n_tokens, ctx.workspace, self.top, self.experts
        # bfloat16 runs the experts on the tensor cores (tiles of 128 slots, rows gathered into slot order
        # first); float32, and shapes the tensor-core kernel refuses, on the CUDA cores (tiles of 64)
        tensor = ops.moe_gemm_tc_available(x, self.w_up) and self.expert_size % 8 == 0
        pairs, tile = T * top, (ops.MOE_TC_TILE if tensor else ops.moe_tile())
        max_tiles = ops.moe_max_tiles(pairs, E, tile)                 # of this step: a function of T alone
        cap_pairs = ws.max_rows * top
        cap_slots = ops.moe_max_tiles(cap_pairs, E, tile) * tile      # of any step: the buffers' sizes
        i32, f32 = torch.int32, torch.float32
        ids, wts = ws.flat("moe_ids", cap_pairs, i32), ws.flat("moe_weights", cap_pairs, f32)
        pair_slot, meta = ws.flat("moe_pair_slot", cap_pairs, i32), ws.flat("moe_meta", 4, i32)
        tile_expert, slot_src = ws.flat("moe_tile_expert", cap_slots // tile, i32), ws.flat("moe_slot_src", cap_slots, i32)
        act = ws.flat("moe_act", cap_slots * self.expert_size, self.dtype).view(cap_slots, self.expert_size)
        y = ws.flat("moe_y", cap_slots * self.hidden_size, f32).view(cap_slots, self.hidden_size)

        logits = ws.get("moe_logits", T, E, f32)
        ops.moe_route(x, self.w_router, self.b_router, logits, ids, wts, T, top, over_all=self.over_all,
                      sigmoid_groups=self.sigmoid_groups)
        ops.moe_group(ids, pairs, E, meta, tile_expert, slot_src, pair_slot, max_tiles, tile)
        if tensor:
            # gated experts: a tile multiplies by its expert's gate rows and up rows and the epilogue makes silu(gate) * up
            rows = ws.flat("moe_rows", cap_slots * self.hidden_size, self.dtype).view(cap_slots, self.hidden_size)
            ops.moe_gather(rows, x, slot_src, meta, top, tile, max_tiles)
            if self.gated and (self.clamped or self.hidden_size < FUSE_GATE_FROM_WIDTH):
                up_out = ws.flat("moe_gate_up", cap_slots * 2 * self.expert_size, self.dtype).view(cap_slots, 2 * self.expert_size)
                ops.moe_gemm_tc(rows, tile_expert, meta, self.w_up, up_out, max_tiles)
                self._gate(act[:max_tiles * tile], up_out[:max_tiles * tile], max_tiles * tile)
            else:
                ops.moe_gemm_tc(rows, tile_expert, meta, self.w_up, act, max_tiles, act="silu_gate" if self.gated else self.activation)
        elif self.gated:
            # on the CUDA cores the up product leaves [gate, up] per slot and a row kernel makes silu(gate) * up of it
            up_out = ws.flat("moe_gate_up", cap_slots * 2 * self.expert_size, self.dtype).view(cap_slots, 2 * self.expert_size)
            ops.moe_gemm(x, top, slot_src, tile_expert, meta, self.w_up, up_out, max_tiles)
            self._gate(act[:max_tiles * tile], up_out[:max_tiles * tile], max_tiles * tile)
        else:
            ops.moe_gemm(x, top, slot_src, tile_expert, meta, self.w_up, act, max_tiles, act=self.activation)
        if tensor:
            ops.moe_gemm_tc(act, tile_expert, meta, self.w_down, y, max_tiles)
        else:
            ops.moe_gemm(act, 0, slot_src, tile_expert, meta, self.w_down, y, max_tiles)
        shared = self.shared.forward(x, ctx, tag="ffn_shared") if self.shared is not None else None
        out = ws.get("ffn_out", T, self.hidden_size, self.dtype)
        ops.moe_combine(out, y, pair_slot, wts, shared, T, top)
        return out


register_part("ffn", "routed", RoutedFFN)
