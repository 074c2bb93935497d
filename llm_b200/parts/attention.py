"""Grouped-query attention over the paged cache.

One product gives q, k and v (the reference fuses the three weights the same way,
model/modules/QKVLinear.h:20-33); q and k are rotated by the position part's table
and k, v are stored in the layer's pages (kernel/Gemm/QKVGemm.h:27-63); every query
head attends to the keys of kv head h // (NH/NKV) that are at or before its own
position and inside the window, if there is one
(kernel/attention/attention_NH_32_NKV_4_HS_64.h:169-172,228-232); then the output
projection (model/modules/Attention.h:19).  Sizes, window and scale are parameters.

Further options, each a parameter and off by default: values of another size than the keys
(value_dim); a soft cap on the scaled scores, s <- cap * tanh(s / cap); a sink, one more term of
score 0 in the softmax's denominator that carries no value, so that a query may attend to
nothing; first tokens of a request that stay visible after the window has passed them
(keep_first; their pages are then never given back); a position part that turns neighbouring
pairs of channels (kind "rope_pairs"); other tensor names.  Further: an RMS norm over the token's whole q projection and
whole k projection, before they are split into heads and before rotation (qk_norm="whole", weights `q.norm`, `k.norm`);
a mask by chunks (a query sees the keys at or before it whose position has the same floor(position / chunk), chunks
counted from the request's first token); and sigmoid weights, sigmoid(score + b_h) with a learned number per head and
no normalisation over the keys (weights="sigmoid").  Further still: a sink whose score is a learned number per head
(sink="learned", tensor `sink`); a bias that grows with the distance, r1_h ln(1 + r2_h (i - j)) taken off the capped score
(dist_bias, tensors `r1`, `r2`); a short causal convolution over time on every channel of the projected (and biased) q, k, v
(qkv_conv = taps, tensors `<projection>.conv` [channels, taps]; the last taps - 1 projected rows are the request's state); and
biases on q, k, v without one on the output (out_bias=False).
"""
from __future__ import annotations

import math

import torch

from ..csrc import ops
from .base import CacheNeed, ParamInfo, Part, StateNeed, build_part, register_part
from .linear import FUSE_PARTIALS, linear


_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
          "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias", "o_bias": "o_proj.bias",
          "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "sink": "sink", "r1": "r1", "r2": "r2"}


class PagedAttention(Part):
    role = "mixer"

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, position=None,
                 window=None, scale=None, shares_cache: bool = False, bias: bool = False, value_dim=None, softcap=None,
                 sink: bool = False, keep_first: int = 0, names=None, chunk=None, weights: str = "softmax", qk_norm=None,
                 norm_eps: float = 1e-6, out_bias=None, qkv_conv: int = 0, dist_bias: bool = False, prefix: str = "",
                 dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        if num_heads % num_kv_heads:
            raise ValueError(f"attention: {num_heads} heads do not divide into {num_kv_heads} kv heads")
        if head_dim <= 0 or head_dim > 256:
            raise ValueError(f"attention: head_dim {head_dim} must be 1 to 256")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.window = int(window) if window else None
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.shares_cache = shares_cache          # reads another layer's pages: no k, v of its own
        self.position = build_part("position", position, dtype, device) if position is not None else None
        self.value_dim = int(value_dim) if value_dim else head_dim
        self.softcap = float(softcap) if softcap else 0.0
        self.sink, self.keep_first = bool(sink), int(keep_first or 0)
        self.learned_sink = sink == "learned"
        self.dist_bias, self.qkv_conv = bool(dist_bias), int(qkv_conv or 0)
        if not (0 <= self.qkv_conv <= 16):
            raise ValueError(f"attention: a convolution of {qkv_conv} taps (0 to 16)")
        if (self.qkv_conv or self.dist_bias or self.learned_sink) and (shares_cache or position is not None):
            raise ValueError("attention: the convolution, the distance bias and the learned sink go with a cache of the "
                             "layer's own and no position part")
        if self.keep_first and not self.window:
            self.keep_first = 0                   # without a window every token is seen anyway
        self.names = dict(_NAMES, **(names or {}))
        self.chunk = int(chunk) if chunk else 0
        if weights not in ("softmax", "sigmoid") or qk_norm not in (None, "whole"):
            raise ValueError(f"attention: weights '{weights}' or qk_norm '{qk_norm}' is not known")
        self.sigmoid, self.qk_norm, self.norm_eps = weights == "sigmoid", qk_norm, float(norm_eps)
        if self.chunk and (self.window or self.keep_first):
            raise ValueError("attention: a chunked mask takes no window and no kept tokens")
        if self.sigmoid and (self.sink or self.softcap):
            raise ValueError("attention: sigmoid weights take no sink and no soft cap")
        # the options above, and pair rotation, run on the path that rotates and stores with one kernel and
        # attends with a kernel that takes them (see forward)
        self.extended = bool(self.value_dim != head_dim or self.softcap or self.sink or self.keep_first or self.qkv_conv
                             or self.dist_bias or self.chunk or self.sigmoid or self.qk_norm
                             or (self.position is not None and hasattr(self.position, "frequencies")))
        self.out_bias = bool(bias) if out_bias is None else bool(out_bias)
        if self.extended and ((bias and self.out_bias) or (self.position is not None and not hasattr(self.position, "frequencies"))):
            raise ValueError("attention: value_dim, softcap, sink and keep_first go with pair rotation or no positions, "
                             "without a bias on the output")
        self.q_size = num_heads * head_dim
        self.kv_size = 0 if shares_cache else num_kv_heads * head_dim
        self.v_size = 0 if shares_cache else num_kv_heads * self.value_dim
        self.bias = bool(bias)        # q/k/v and o projections carry bias vectors (model/modules/Attention.h:16-19)
        self.w_qkv = None
        self.w_o = None
        self.b_qkv = None
        self.b_o = None
        self.score_bias = self.q_gain = self.k_gain = None
        self.sink_values = self.r1 = self.r2 = self.w_conv = None
        self.conv_cols = (max(self.qkv_conv - 1, 0) * (self.q_size + self.kv_size + self.v_size) + 3) // 4 * 4

    def parameters(self):
        n = lambda k: self.name(self.names[k])
        p = {n("q"): ParamInfo((self.q_size, self.hidden_size))}
        if not self.shares_cache:
            p[n("k")] = ParamInfo((self.kv_size, self.hidden_size))
            p[n("v")] = ParamInfo((self.v_size, self.hidden_size))
        p[n("o")] = ParamInfo((self.hidden_size, self.num_heads * self.value_dim))
        if self.sigmoid:
            p[self.name(self.names.get("score_bias", "pb"))] = ParamInfo((self.num_heads,), kind="gain", init="normal")
        if self.qk_norm:
            p[self.name(self.names.get("q_norm", "q.norm"))] = ParamInfo((self.q_size,), kind="gain", init="ones_normal")
            if not self.shares_cache:
                p[self.name(self.names.get("k_norm", "k.norm"))] = ParamInfo((self.kv_size,), kind="gain", init="ones_normal")
        if self.bias:
            p[n("q_bias")] = ParamInfo((self.q_size,), kind="gain", init="normal")
            if not self.shares_cache:
                p[n("k_bias")] = ParamInfo((self.kv_size,), kind="gain", init="normal")
                p[n("v_bias")] = ParamInfo((self.v_size,), kind="gain", init="normal")
            if self.out_bias:
                p[n("o_bias")] = ParamInfo((self.hidden_size,), kind="gain", init="normal")
        if self.learned_sink:
            p[n("sink")] = ParamInfo((self.num_heads,), kind="gain", init="normal")
        if self.dist_bias:
            p[n("r1")] = ParamInfo((self.num_heads,), kind="gain", init="normal")
            p[n("r2")] = ParamInfo((self.num_heads,), kind="gain", init="ones_normal")
        if self.qkv_conv:
            for m, c in (("q_conv", self.q_size), ("k_conv", self.kv_size), ("v_conv", self.v_size)):
                p[n(m)] = ParamInfo((c, self.qkv_conv), kind="gain", init="normal")
        return p

    def bind(self, tensors):
        n = lambda k: tensors[self.name(self.names[k])]
        parts = [n("q")]
        if not self.shares_cache:
            parts += [n("k"), n("v")]
        self.w_qkv = torch.cat(parts, dim=0).contiguous() if len(parts) > 1 else parts[0].contiguous()
        self.w_o = n("o").contiguous()
        if self.sigmoid:
            self.score_bias = tensors[self.name(self.names.get("score_bias", "pb"))].contiguous()
        if self.qk_norm:
            self.q_gain = tensors[self.name(self.names.get("q_norm", "q.norm"))].contiguous()
            if not self.shares_cache:
                self.k_gain = tensors[self.name(self.names.get("k_norm", "k.norm"))].contiguous()
        if self.bias:
            names = ["q_bias"] + ([] if self.shares_cache else ["k_bias", "v_bias"])
            self.b_qkv = torch.cat([n(m) for m in names]).contiguous()
            self.b_o = n("o_bias").contiguous() if self.out_bias else None
        if self.learned_sink:
            self.sink_values = n("sink").contiguous()
        if self.dist_bias:
            self.r1, self.r2 = n("r1").contiguous(), n("r2").contiguous()
        if self.qkv_conv:
            self.w_conv = torch.cat([n("q_conv"), n("k_conv"), n("v_conv")], dim=0).t().contiguous()      # [taps, channels]

    def cache_need(self):
        if self.shares_cache:
            return None
        if self.chunk:      # the keys of a query's chunk lie among the last `chunk` tokens: pages behind them go back
            return CacheNeed("window", self.num_kv_heads, self.head_dim, self.chunk, value_dim=self.value_dim)
        return CacheNeed("window" if self.window else "full", self.num_kv_heads, self.head_dim, self.window,
                         value_dim=self.value_dim, keep_first=self.keep_first)

    def state_need(self):
        # the convolution over the projected rows keeps the request's last taps - 1 of them
        return StateNeed((max(self.conv_cols, 4),), torch.float32) if self.qkv_conv else None

    def children(self):
        return [self.position] if self.position is not None else []

    def _qkv_cta_limit(self, ctx, k_pages) -> int:
        """A decode step whose attention has to read several times the bytes of the QKV weights
        (many requests, long contexts) is bound by that reading, and the attention kernel asks for
        its keys and values before it waits for the product: a product on fewer CTAs leaves it SMs
        to start on.  Measured: 64 requests of 640 keys at TinyLlama sizes, 2 instead of 8 splits
        of K: 5 % off the step; about 30 requests of 1,200 keys at Llama-2-7B sizes: 2 % off; with
        8 requests (of 8,000 keys, Llama-3-8B sizes) or with a cache of under four times the
        weights' bytes the full grid is faster."""
        if not ctx.decode_only or self.w_qkv.dtype != torch.bfloat16 or ctx.n_entries < 24:
            return 0
        keys = min(ctx.kv_bucket or 0, self.window or (1 << 30))
        cache_bytes = 2 * ctx.n_entries * keys * k_pages.shape[1] * self.head_dim * k_pages.element_size()
        weight_bytes = self.w_qkv.numel() * self.w_qkv.element_size()
        if cache_bytes <= 4 * weight_bytes:
            return 0
        # from 32 rows on the product runs one CTA per SM (see ops.NORMAL_MODE_FROM_ROWS): half the SMs
        # then measured best (64 requests: 1.29 ms a step with a third, 1.20 ms with half or all)
        return ops.sm_count() // (2 if ctx.n_tokens >= ops.NORMAL_MODE_FROM_ROWS else 3)

    def forward(self, x: torch.Tensor, ctx, view) -> torch.Tensor:
        T = ctx.n_tokens
        ws = ctx.workspace
        if self.extended:
            return self._forward_extended(x, ctx, view)
        width = self.q_size + 2 * self.kv_size
        cos = sin = None
        own_transform = None
        if self.position is not None:
            if hasattr(self.position, "tables"):
                cos, sin = self.position.tables()
            elif hasattr(self.position, "apply"):
                own_transform = self.position.apply
        k_pages, v_pages = view.k_pages, view.v_pages
        attn = ws.get("attn_out", T, self.q_size, self.dtype)
        if own_transform is not None:
            # a position part with a transform of its own: it runs on the summed projection, between
            # the product and the cache store; the kernels after it neither rotate nor sum
            qkv = linear(x, self.w_qkv, ws.get("qkv", T, width, self.dtype), T, bias=self.b_qkv)
            q_view = qkv[:, :self.q_size].view(T, self.num_heads, self.head_dim)
            k_view = (qkv[:, self.q_size:self.q_size + self.kv_size].view(T, -1, self.head_dim)
                      if self.kv_size else None)
            own_transform(q_view, k_view, ctx)
        elif self.bias:
            # biased projections: the product is summed and the bias added before rotation and store
            qkv = linear(x, self.w_qkv, ws.get("qkv", T, width, self.dtype), T, bias=self.b_qkv)
        else:
            # many rows: one kernel projects, rotates and stores; then the attention over the pages
            q = ops.qkv_rope_store(x, self.w_qkv, lambda: ws.get("q_rot", T, self.q_size, self.dtype), T, cos, sin,
                                   ctx.positions, view.group.slot_map, k_pages, v_pages, self.num_heads,
                                   0 if self.shares_cache else k_pages.shape[1], self.head_dim)
            if q is not None:
                ops.paged_attention(attn, q, k_pages, v_pages, view.group, ctx, self.num_heads, k_pages.shape[1],
                                    self.head_dim, self.window or 0, self.scale)
                return linear(attn, self.w_o, ws.get("mixer_out", T, self.hidden_size, self.dtype), T, allow_partial=FUSE_PARTIALS)
            qkv = linear(x, self.w_qkv, ws.get("qkv", T, width, self.dtype), T, allow_partial=FUSE_PARTIALS,
                         cta_limit=self._qkv_cta_limit(ctx, k_pages))
        ops.rope_store_attend(attn, qkv, cos, sin, k_pages, v_pages, view.group, ctx, self.num_heads,
                              k_pages.shape[1], self.head_dim, self.window or 0, self.scale,
                              write_kv=not self.shares_cache,
                              q_rot=lambda: ws.get("q_rot", T, self.q_size, self.dtype))
        return linear(attn, self.w_o, ws.get("mixer_out", T, self.hidden_size, self.dtype), T, allow_partial=FUSE_PARTIALS,
                      bias=self.b_o)


    def _forward_extended(self, x: torch.Tensor, ctx, view) -> torch.Tensor:
        """One product for q, k, v (its split-K partial results go unsummed to the next kernel); one kernel that
        sums them, turns the pairs of q and k and stores k and v in the pages; the attention kernel that takes
        the options; the output projection."""
        T, ws = ctx.n_tokens, ctx.workspace
        H, D, V = self.num_heads, self.head_dim, self.value_dim
        k_pages, v_pages = view.k_pages, view.v_pages
        n_kv = k_pages.shape[1]
        qkv = linear(x, self.w_qkv, ws.get("qkv", T, self.q_size + self.kv_size + self.v_size, self.dtype), T,
                     allow_partial=FUSE_PARTIALS, bias=self.b_qkv)
        if self.qkv_conv:      # directly behind the (biased) projection; the request's last rows come from its state
            conv = ws.get("qkv_conv", T, qkv.shape[1], self.dtype)
            ops.short_conv(conv, qkv, self.w_conv, None, view.state, ctx)
            qkv = conv
        freqs = self.position.frequencies() if self.position is not None else None
        halves = getattr(self.position, "layout", "pairs") == "halves"
        q_out = ws.get("q_rot", T, self.q_size, self.dtype) if isinstance(qkv, ops.PartialSum) else None
        if self.qk_norm or halves:
            q = ops.norm_rope_kv_write(qkv, self.q_gain, self.k_gain, self.norm_eps, freqs, halves, ctx.positions,
                                       view.group.slot_map, k_pages, v_pages, T, H, 0 if self.shares_cache else n_kv, D, V,
                                       q_out=q_out)
        else:
            q = ops.rope_pairs_kv_write(qkv, freqs, ctx.positions, view.group.slot_map, k_pages, v_pages, T, H,
                                        0 if self.shares_cache else n_kv, D, V, q_out=q_out)
        attn = ws.get("attn_out", T, H * V, self.dtype)
        ops.paged_attention(attn, q, k_pages, v_pages, view.group, ctx, H, n_kv, D, self.window or 0, self.scale,
                            value_dim=V, softcap=self.softcap, sink=self.sink, keep_first=self.keep_first,
                            chunk=self.chunk, sigmoid_bias=self.score_bias, sink_values=self.sink_values,
                            dist_bias=(self.r1, self.r2) if self.dist_bias else None)
        return linear(attn, self.w_o, ws.get("mixer_out", T, self.hidden_size, self.dtype), T, allow_partial=FUSE_PARTIALS)


register_part("mixer", "attention", PagedAttention)
