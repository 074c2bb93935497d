"""Differential attention: every head runs two causal softmax attentions ("maps"), each with queries and keys of its own,
over one set of values, and the output is their difference.

  q = Wq h   [H, 2, D]        k = Wk h   [G, 2, D]        v = Wv h   [G, V]        head h reads key/value head h // (H/G)
  q, k <- RMS norm per head and map over D, one weight vector for all of them (`q.norm`, `k.norm`)
  a_m = softmax(q_m . k_m * scale, causal) v                                       m = 1, 2
  lambda = exp(sum(lq1 * lk1)) - exp(sum(lq2 * lk2)) + diff                        one number for the layer
  o = rms_unit(a_1 - lambda a_2) * (1 - diff)      per head, over V, no weight
  out = Wo (o * sigmoid(Wg h))

On the device the two maps are 2H query heads over 2G key heads: the query rows are stacked group by group as
[kv group][map][head within the group], so that the grouped-query rule (query head i reads key head i // (H/G)) sends map m
of every head in group g to key head 2g + m, the order in which Wk already gives them; the values are cached once per kv head
and key head j reads value head j // 2.  Positions do not enter the scores.  Scores, softmax, the combination and its norm
are float32.  Sizes, scale, diff, eps and tensor names are parameters.
"""
from __future__ import annotations

import math

import torch

from ..csrc import ops
from .base import CacheNeed, ParamInfo, Part, register_part
from .linear import FUSE_PARTIALS, linear

_NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "q_norm": "q.norm", "k_norm": "k.norm",
          "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2"}


class DifferentialAttention(Part):
    role = "mixer"

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, scale: float,
                 diff: float, eps: float, gated: bool = True, names=None, prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        if min(hidden_size, num_heads, num_kv_heads, head_dim, value_dim) <= 0 or num_heads % num_kv_heads:
            raise ValueError(f"differential attention: sizes must be positive and {num_heads} heads divide into {num_kv_heads} kv heads")
        if max(head_dim, value_dim) > 1024:
            raise ValueError("differential attention: head sizes up to 1024")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.value_dim = int(head_dim), int(value_dim)
        self.scale, self.diff, self.eps, self.gated = float(scale), float(diff), float(eps), bool(gated)
        self.names = dict(_NAMES, **(names or {}))
        self.per_group = self.num_heads // self.num_kv_heads
        self.q_size, self.k_size = 2 * self.num_heads * self.head_dim, 2 * self.num_kv_heads * self.head_dim
        self.v_size, self.o_size = self.num_kv_heads * self.value_dim, self.num_heads * self.value_dim
        self.w_in = self.w_o = self.q_gain = self.k_gain = None
        self.lam = 0.0

    def parameters(self):
        n = lambda k: self.name(self.names[k])
        W, D = self.hidden_size, self.head_dim
        p = {n("q"): ParamInfo((self.q_size, W)), n("k"): ParamInfo((self.k_size, W)), n("v"): ParamInfo((self.v_size, W)),
             n("out"): ParamInfo((W, self.o_size)),
             n("q_norm"): ParamInfo((D,), kind="gain", init="ones_normal"), n("k_norm"): ParamInfo((D,), kind="gain", init="ones_normal")}
        for m in ("lq1", "lk1", "lq2", "lk2"):
            p[n(m)] = ParamInfo((D,), kind="gain", init="normal")
        if self.gated:
            p[n("gate")] = ParamInfo((self.o_size, W))
        return p

    def bind(self, tensors):
        n = lambda k: tensors[self.name(self.names[k])]
        H, G, R, D = self.num_heads, self.num_kv_heads, self.per_group, self.head_dim
        # query rows [head][map][D] -> [kv group][map][head within the group][D]
        wq = n("q").view(G, R, 2, D, self.hidden_size).permute(0, 2, 1, 3, 4).reshape(self.q_size, self.hidden_size)
        parts = [wq, n("k"), n("v")] + ([n("gate")] if self.gated else [])
        self.w_in = torch.cat(parts, dim=0).contiguous()
        self.w_o = n("out").contiguous()
        self.q_gain, self.k_gain = n("q_norm").contiguous(), n("k_norm").contiguous()
        f = lambda k: n(k).to(torch.float32)
        self.lam = math.exp(float((f("lq1") * f("lk1")).sum())) - math.exp(float((f("lq2") * f("lk2")).sum())) + self.diff

    def cache_need(self):
        return CacheNeed("full", 2 * self.num_kv_heads, self.head_dim, value_dim=self.value_dim, value_heads=self.num_kv_heads)

    def state_need(self):
        return None

    def forward(self, x: torch.Tensor, ctx, view) -> torch.Tensor:
        T, ws = ctx.n_tokens, ctx.workspace
        H, G, D, V = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        width = self.q_size + self.k_size + self.v_size + (self.o_size if self.gated else 0)
        # the gate is read after the attention, so the product is summed here (partial results live until the next product)
        proj = linear(x, self.w_in, ws.get("diff_in", T, width, self.dtype), T)
        q = ops.head_norm_kv_write(proj, self.q_gain, self.k_gain, self.eps, view.group.slot_map, view.k_pages, view.v_pages,
                                   T, 2 * H, 2 * G, G, D, V)
        maps = ws.get("diff_maps", T, 2 * H * V, self.dtype)
        ops.paged_attention(maps, q, view.k_pages, view.v_pages, view.group, ctx, 2 * H, 2 * G, D, 0, self.scale,
                            value_dim=V, v_share=2)
        gate = proj[:, self.q_size + self.k_size + self.v_size:] if self.gated else None
        out = ws.get("attn_out", T, self.o_size, self.dtype)
        ops.diff_combine(out, maps, gate, T, H, self.per_group, self.lam, 1.0 - self.diff, self.eps)
        return linear(out, self.w_o, ws.get("mixer_out", T, self.hidden_size, self.dtype), T, allow_partial=FUSE_PARTIALS)


register_part("mixer", "diff_attention", DifferentialAttention)
