"""Latent attention: keys and values of every head are linear maps of one small vector per
token, and only that vector is cached.

  c_t   = rms(Wdkv h_t) * gain          [rank]      (kept in the layer's pages; a layer may
                                                      instead read the latents that another
                                                      layer stored, with maps of its own)
  k_t,h = Wuk_h c_t,  v_t,h = Wuv_h c_t
  o_i,h = sigmoid(Wg h_i)_h * sum_{j<=i} softmax_j(scale * q_i,h . k_j,h) v_j,h
  out_i = Wo concat_h(o_i,h)

No position enters: the mask alone orders the tokens.  Because k and v are linear in c, the
engine never forms them.  It carries the query through the key map, q'_i,h = Wuk_h^T q_i,h, so that
q . k = q' . c; runs a multi-query attention whose single key/value head of size `rank` is c
itself (the paged attention kernels the other mixers use, with the key pages given as value
pages too); and carries the result, a mix of latents, through the value map.  The cache holds
rank numbers per token and layer instead of heads x (dim + vdim), and prompts, portions and
decoded tokens all run the same arithmetic.  Sizes, the score scale, the norm's eps and the
tensor names are parameters.

Options, each a parameter and off by default:
  q_rank    the queries pass a latent of their own: c_q = rms(Wdq h) * gain_q, q = Wuq c_q;
  rot_dim   every query head carries rot_dim more channels and the down-projection rot_dim more rows: one key part
            shared by all heads (not normed), both turned by the position part (pairs of neighbours); the score is
            q_plain . k_plain + q_turned . k_turned.  The cached row is then [turned key part | c], the query that meets
            it [turned query part | Wuk_h^T q_plain], and the value map skips the row's first rot_dim numbers;
  window    a query sees itself and the window - 1 tokens before it (pages behind the window go back to the pool);
  sink      the softmax's denominator holds one more term exp(sink_h), a learned number per head without key or value.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import CacheNeed, ParamInfo, Part, build_part, register_part
from .linear import FUSE_PARTIALS, linear

_NAMES = {"q": "q", "down": "dkv", "down_norm": "dkv.norm", "up_k": "uk", "up_v": "uv", "gate": "g", "out": "o",
          "q_down": "dq", "q_down_norm": "dq.norm", "q_up": "uq", "sink": "sink"}


class LatentAttention(Part):
    role = "mixer"

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, rank: int, scale: float,
                 eps: float, gated: bool = True, shares_cache: bool = False, names=None, q_rank: int = 0, rot_dim: int = 0,
                 position=None, window=None, sink: bool = False, prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        if min(hidden_size, num_heads, head_dim, value_dim, rank) <= 0:
            raise ValueError("latent attention: sizes must be positive")
        if rank > 1024:
            raise ValueError(f"latent attention: rank {rank} exceeds 1024, the widest head the attention kernels take")
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim, self.rank = hidden_size, num_heads, head_dim, value_dim, rank
        self.scale, self.eps = float(scale), float(eps)
        self.gated = bool(gated)
        self.shares_cache = bool(shares_cache)      # reads another layer's latents: no down-projection of its own
        self.names = dict(_NAMES, **(names or {}))
        self.q_rank, self.rot_dim = int(q_rank or 0), int(rot_dim or 0)
        self.window, self.sink = (int(window) if window else None), bool(sink)
        self.position = build_part("position", position, dtype, device) if position is not None else None
        # with any of these the mixer runs the path of _forward_rotary (its own layout of the projections)
        self.rotary = bool(self.q_rank or self.rot_dim or self.window or self.sink)
        if self.rotary and (self.gated or self.shares_cache):
            raise ValueError("latent attention: a query latent, a turned key part, a window or a sink go without gate and with latents of the layer's own")
        if self.rot_dim % 2 or (self.position is not None and not hasattr(self.position, "frequencies")):
            raise ValueError("latent attention: the turned part is even and its position part gives frequencies")
        if self.position is not None and self.position.dims > self.rot_dim:
            raise ValueError(f"latent attention: {self.position.dims} turning channels do not fit a part of {self.rot_dim}")
        self.q_size = num_heads * (head_dim + self.rot_dim)
        rank = rank + self.rot_dim          # what a cached row holds: the turned key part, then the latent
        # The width of a cached row.  The tensor-core attention kernels (bfloat16) take heads of 64 or 128: a
        # smaller rank is padded up to the next of the two with zeros (in the cache rows and in the two per-head
        # maps), which changes no score and no output and costs cache, not correctness.  Other ranks, and
        # float32, keep their width and run on the general kernels.
        self.row_width = rank
        if dtype == torch.bfloat16 and rank < 128 and rank != 64:
            self.row_width = 64 if rank < 64 else 128
        self.w_in = None          # [q; down; gate] stacked: one product per step
        self.w_uk_t = None        # [heads, rank, dim]: the key map, transposed per head
        self.w_uv = None          # [heads, vdim, rank]
        self.w_o = None
        self.gain = None
        self.q_gain = self.w_uq = self.sink_values = None

    def children(self):
        return [self.position] if self.position is not None else []

    def parameters(self):
        n = lambda k: self.name(self.names[k])
        if self.rotary:
            W, H, C = self.hidden_size, self.num_heads, self.rank
            p = {n("down"): ParamInfo((C + self.rot_dim, W)), n("down_norm"): ParamInfo((C,), kind="gain", init="ones_normal"),
                 n("up_k"): ParamInfo((H * self.head_dim, C)), n("up_v"): ParamInfo((H * self.value_dim, C)),
                 n("out"): ParamInfo((W, H * self.value_dim))}
            if self.q_rank:
                p[n("q_down")] = ParamInfo((self.q_rank, W))
                p[n("q_down_norm")] = ParamInfo((self.q_rank,), kind="gain", init="ones_normal")
                p[n("q_up")] = ParamInfo((self.q_size, self.q_rank))
            else:
                p[n("q")] = ParamInfo((self.q_size, W))
            if self.sink:
                p[n("sink")] = ParamInfo((H,), kind="gain", init="normal")
            return p
        p = {n("q"): ParamInfo((self.q_size, self.hidden_size))}
        if not self.shares_cache:
            p[n("down")] = ParamInfo((self.rank, self.hidden_size))
            p[n("down_norm")] = ParamInfo((self.rank,), kind="gain", init="ones_normal")
        p[n("up_k")] = ParamInfo((self.q_size, self.rank))
        p[n("up_v")] = ParamInfo((self.num_heads * self.value_dim, self.rank))
        if self.gated:
            p[n("gate")] = ParamInfo((self.num_heads, self.hidden_size))
        p[n("out")] = ParamInfo((self.hidden_size, self.num_heads * self.value_dim))
        return p

    def bind(self, tensors):
        n = lambda k: tensors[self.name(self.names[k])]
        if self.rotary:
            return self._bind_rotary(n)
        parts = [n("q")]
        if not self.shares_cache:
            parts.append(n("down"))
            self.gain = n("down_norm").contiguous()
        if self.gated:
            parts.append(n("gate"))
        self.w_in = torch.cat(parts, dim=0).contiguous() if len(parts) > 1 else parts[0].contiguous()
        H, D, V, R = self.num_heads, self.head_dim, self.value_dim, self.rank
        self.w_uk_t = n("up_k").view(H, D, R).transpose(1, 2).contiguous()
        self.w_uv = n("up_v").view(H, V, R).contiguous()
        if self.row_width != R:
            pad = self.row_width - R
            self.w_uk_t = torch.nn.functional.pad(self.w_uk_t, (0, 0, 0, pad)).contiguous()      # [H, width, D]: zero rows
            self.w_uv = torch.nn.functional.pad(self.w_uv, (0, pad)).contiguous()                # [H, V, width]: zero columns
        self.w_o = n("out").contiguous()

    def _bind_rotary(self, n):
        H, D, V, C, R, RW = self.num_heads, self.head_dim, self.value_dim, self.rank, self.rot_dim, self.row_width
        self.gain = n("down_norm").contiguous()
        # the head's query rows reordered so that the turned part comes first: [turned R | plain D]
        order = torch.cat([torch.cat([torch.arange(D, D + R), torch.arange(D)]) + h * (D + R) for h in range(H)]).to(self.device)
        if self.q_rank:
            self.w_in = torch.cat([n("q_down"), n("down")], dim=0).contiguous()          # [q_rank + C + R, W]
            self.q_gain = n("q_down_norm").contiguous()
            self.w_uq = n("q_up")[order].contiguous()
        else:
            self.w_in = n("down").contiguous()
            self.w_uq = n("q")[order].contiguous()
        # a query [turned R | plain D] -> what meets a cached row [turned R | latent C | zeros]: the turned part passes
        # through an identity, the plain part through the key map
        w_map = torch.zeros((H, RW, R + D), dtype=self.dtype, device=self.device)
        w_map[:, :R, :R] = torch.eye(R, dtype=self.dtype, device=self.device)
        w_map[:, R:R + C, R:] = n("up_k").view(H, D, C).transpose(1, 2)
        self.w_uk_t = w_map.contiguous()
        w_uv = torch.zeros((H, V, RW), dtype=self.dtype, device=self.device)
        w_uv[:, :, R:R + C] = n("up_v").view(H, V, C)
        self.w_uv = w_uv.contiguous()
        self.w_o = n("out").contiguous()
        if self.sink:
            self.sink_values = n("sink").contiguous()

    def cache_need(self):
        if self.shares_cache:
            return None
        if self.window:
            return CacheNeed("window", 1, self.row_width, self.window, values=False)
        return CacheNeed("full", 1, self.row_width, None, values=False)

    def state_need(self):
        return None

    def _forward_rotary(self, x: torch.Tensor, ctx, view) -> torch.Tensor:
        """One product for the two down-projections (float32 out: both are normed next); one kernel for the two norms, the
        turning of the key part and the cache row; the query's up-projection; the turning of the queries' leading
        channels; the per-head map to the cached row's layout; the paged attention with one key/value head (window, sink);
        the per-head value map; the output projection."""
        T, ws = ctx.n_tokens, ctx.workspace
        H, C, R, RW, Q = self.num_heads, self.rank, self.rot_dim, self.row_width, self.q_rank
        pages = view.k_pages
        freqs = self.position.frequencies() if self.position is not None else None
        proj = linear(x, self.w_in, ws.get("latent_down", T, self.w_in.shape[0], torch.float32), T)
        cq = ws.get("latent_cq", T, Q, self.dtype) if Q else None
        ops.latent_rope_norm_store(proj, self.q_gain, Q, cq, self.gain, R, freqs, ctx.positions, self.eps,
                                   view.group.slot_map, pages, T)
        q = linear(cq if Q else x, self.w_uq, ws.get("latent_in", T, self.q_size, self.dtype), T, allow_partial=FUSE_PARTIALS)
        if R or isinstance(q, ops.PartialSum):
            q = ops.rope_pairs_kv_write(q, freqs, ctx.positions, None, None, None, T, H, 0, self.head_dim + R, 0,
                                        q_out=ws.get("latent_in", T, self.q_size, self.dtype) if isinstance(q, ops.PartialSum) else None)
        q_lat = ws.get("latent_q", T, H * RW, self.dtype)
        ops.gemm_heads(q, self.w_uk_t, q_lat, T, H)
        o_lat = ws.get("latent_o", T, H * RW, self.dtype)
        ops.paged_attention(o_lat, q_lat, pages, pages, view.group, ctx, H, 1, RW, self.window or 0, self.scale,
                            sink_values=self.sink_values)
        attn = ws.get("attn_out", T, H * self.value_dim, self.dtype)
        ops.gemm_heads(o_lat, self.w_uv, attn, T, H)
        return linear(attn, self.w_o, ws.get("mixer_out", T, self.hidden_size, self.dtype), T, allow_partial=FUSE_PARTIALS)

    def forward(self, x: torch.Tensor, ctx, view) -> torch.Tensor:
        if self.rotary:
            return self._forward_rotary(x, ctx, view)
        T, ws = ctx.n_tokens, ctx.workspace
        H, R, RW = self.num_heads, self.rank, self.row_width
        proj = linear(x, self.w_in, ws.get("latent_in", T, self.w_in.shape[0], self.dtype), T)
        col = self.q_size
        pages = view.k_pages                        # [pages, 1, page_size, rank]; also the value pages
        if not self.shares_cache:
            ops.latent_norm_store(proj[:, col:col + R], self.gain, self.eps, view.group.slot_map, pages, T)
            col += R
        gate = proj[:, col:col + H] if self.gated else None
        q_lat = ws.get("latent_q", T, H * RW, self.dtype)
        ops.gemm_heads(proj[:, :self.q_size], self.w_uk_t, q_lat, T, H)
        o_lat = ws.get("latent_o", T, H * RW, self.dtype)
        ops.paged_attention(o_lat, q_lat, pages, pages, view.group, ctx, H, 1, RW, 0, self.scale)
        attn = ws.get("attn_out", T, H * self.value_dim, self.dtype)
        ops.gemm_heads(o_lat, self.w_uv, attn, T, H, gate=gate)
        return linear(attn, self.w_o, ws.get("mixer_out", T, self.hidden_size, self.dtype), T, allow_partial=FUSE_PARTIALS)


register_part("mixer", "latent_attention", LatentAttention)
