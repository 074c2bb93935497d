"""Recurrent mixers with a matrix state per head and a diagonal decay, and two mixers that are built from other mixers.

  wkv            RWKV-style time mixing: every projection reads its own blend of the token's row and the previous
                 token's; o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t, S_t = diag(w_t) S_{t-1} + k_t v_t^T
  ssd            state-space duality (Mamba-2): a short convolution on x, B, C; S_t = a_t S_{t-1} + dt_t B_t x_t^T,
                 y_t = S_t^T C_t + D x_t with one decay per head and token
  hgrn2          a forget gate with a lower bound that also decides what is written: S_t = diag(f_t) S_{t-1} + (1 - f_t) v_t^T,
                 o_t = S_t^T silu(q_t); no key
  gated_delta    the gated delta rule: S <- g_t S; u = beta_t (v_t - S^T k_t); S <- S + k_t u^T; o_t = S^T q_t with unit q, k
                 behind a short convolution and silu, one decay and one beta per head
  conv_input     a wrapper: the inner mixer (or feed-forward) reads h + conv(h), a short causal convolution per channel
  parallel       a wrapper: two mixers read the same rows; the result is the mean of their RMS-normed outputs, or a sum of
                 the two with fixed scales

None of them keeps keys: a request's past is its state slot (float32, zero at admission), read at the start of
the step's tokens and written back at their end, so a whole prompt, a portion and a decoded token run the same
recurrence.  A part's state is one flat float32 row per request; a wrapper's row is its own numbers followed by its
inner parts' (each part gets a column range of the row, starting on a 16-byte boundary).  Decays, their logarithms,
step sizes, states and the norms are float32; projections and convolutions run in the compute dtype.
"""
from __future__ import annotations

import dataclasses

import torch

from ..csrc import ops
from .base import ParamInfo, Part, StateNeed, build_part, register_part
from .linear import FUSE_PARTIALS, linear


def _pad4(n: int) -> int:
    return (n + 3) // 4 * 4


def _state_numel(need) -> int:
    if need is None:
        return 0
    if need.dtype != torch.float32:
        raise ValueError("a mixer inside another keeps its state in float32")
    n = 1
    for s in need.shape:
        n *= int(s)
    return n


SEGMENT = 64       # tokens per segment of a prompt step (csrc/scan.cu)
CHUNKED_DELTA = True      # False: the delta rule walks every step token by token (csrc/delta.cu)


def _segments(ctx, tag: str, state_numel: int, decay_numel: int):
    """(seg_len, seg_state, seg_decay): a step with prompt portions runs them as segments side by side in two passes;
    single tokens and short steps take one pass."""
    if ctx.decode_only or ctx.n_tokens < 4 * SEGMENT:
        return 0, None, None
    ws = ctx.workspace
    cap = ws.max_rows // SEGMENT + ctx.cu_tokens.numel()
    return (SEGMENT, ws.flat(tag + "_seg_state", cap * state_numel, torch.float32),
            ws.flat(tag + "_seg_decay", cap * decay_numel, torch.float32))


def _sub_view(view, state):
    """The layer's view as an inner part sees it: the same cache, its own columns of the state row."""
    return dataclasses.replace(view, state=state)


class TimeMixWKV(Part):
    """Tensors (local names): mu.r|k|v|g|w [W] (blend weights), r, k, v, g [H*D, W], w1 [rank, W], w2 [H*D, rank],
    w0 [H*D] (decay through a low rank: w = exp(-exp(w2 tanh(w1 x_w) + w0))), u [H, D] (the current token's bonus),
    norm [H*D], o [W, H*D].  The output of every head is divided by its root mean square, scaled by norm and by
    silu(g x_g).  State row: [the previous token's input: W | S: H * D * D]."""

    role = "mixer"

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, eps: float, decay_rank: int = 16, prefix: str = "",
                 dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        if min(hidden_size, num_heads, head_dim, decay_rank) <= 0:
            raise ValueError("wkv: sizes must be positive")
        if head_dim > 256:
            raise ValueError(f"wkv: head size {head_dim} exceeds 256, the most the recurrence kernel takes")
        self.hidden_size, self.num_heads, self.head_dim = int(hidden_size), int(num_heads), int(head_dim)
        self.eps, self.decay_rank = float(eps), int(decay_rank)
        self.inner = self.num_heads * self.head_dim
        self.shift_cols = _pad4(self.hidden_size)
        self.mu = self.w_rkvg = self.w1 = self.w2 = self.w0 = self.bonus = self.gain = self.w_o = None

    def parameters(self):
        n, W, I, R = self.name, self.hidden_size, self.inner, self.decay_rank
        p = {n("mu." + m): ParamInfo((W,), kind="gain", init="normal") for m in "rkvgw"}
        p.update({n(m): ParamInfo((I, W)) for m in "rkvg"})
        p.update({n("w1"): ParamInfo((R, W), free_dims=(0,)), n("w2"): ParamInfo((I, R), free_dims=(1,)),
                  n("w0"): ParamInfo((I,), kind="gain", init="normal"),
                  n("u"): ParamInfo((self.num_heads, self.head_dim), kind="gain", init="normal"),
                  n("norm"): ParamInfo((I,), kind="gain", init="ones_normal"), n("o"): ParamInfo((W, I))})
        return p

    def bind(self, tensors):
        t = lambda local: tensors[self.name(local)]
        if t("w1").shape[0] != t("w2").shape[1]:
            raise ValueError(f"{self.prefix}: the decay's factors disagree on their rank ({t('w1').shape[0]} and {t('w2').shape[1]})")
        self.decay_rank = int(t("w1").shape[0])
        self.mu = torch.stack([t("mu." + m) for m in "rkvgw"]).contiguous()                  # [5, W] float32
        self.w_rkvg = torch.stack([t(m) for m in "rkvg"]).contiguous()                        # [4, H*D, W]
        self.w1, self.w2 = t("w1").contiguous(), t("w2").contiguous()
        self.w0, self.bonus, self.gain = t("w0").contiguous(), t("u").contiguous(), t("norm").contiguous()
        self.w_o = t("o").contiguous()

    def cache_need(self):
        return None

    def state_need(self):
        return StateNeed((self.shift_cols + self.inner * self.head_dim,), torch.float32)

    def forward(self, x: torch.Tensor, ctx, view) -> torch.Tensor:
        T, ws = ctx.n_tokens, ctx.workspace
        W, I, R = self.hidden_size, self.inner, self.decay_rank
        shift, S = view.state[:, :self.shift_cols], view.state[:, self.shift_cols:]
        mixes = ws.get("wkv_mixes", T, 5 * W, self.dtype)
        ops.token_shift(mixes, x, self.mu, shift, ctx)
        if (self.dtype == torch.bfloat16 and T < ops.NORMAL_MODE_FROM_ROWS
                and all(ops.gemm_fast_available(mixes[:, m * W:], self.w_rkvg[m], None, T) for m in range(4))):
            # few rows: the products are bound by the weights' bytes, which the tensor-core kernel of few rows streams with all
            # SMs; one product per input, each into rows of its own (measured at width 2048, 64 requests: the per-head
            # CUDA-core launch took 156 us, the four products take about 30)
            r_, k_, v_, g_ = (linear(mixes[:, m * W:(m + 1) * W], self.w_rkvg[m], ws.get("wkv_" + "rkvg"[m], T, I, self.dtype), T)
                              for m in range(4))
        else:
            rkvg = ws.get("wkv_rkvg", T, 4 * I, self.dtype)
            ops.gemm_heads(mixes[:, :4 * W], self.w_rkvg, rkvg, T, 4)          # four products of four inputs in one launch
            r_, k_, v_, g_ = (rkvg[:, m * I:(m + 1) * I] for m in range(4))
        low = linear(mixes[:, 4 * W:], self.w1, ws.get("wkv_low", T, R, self.dtype), T)
        low_t = ws.get("wkv_low_t", T, R, self.dtype)
        ops.act_rows(low_t, low, T, "tanh")
        # the decay's pre-activation in float32; bias and the two exponentials are the recurrence kernel's
        z = linear(low_t, self.w2, ws.get("wkv_z", T, I, torch.float32), T)
        o = ws.get("wkv_o", T, I, torch.float32)
        seg, seg_state, seg_decay = _segments(ctx, "wkv", I * self.head_dim, I)
        ops.wkv_scan(o, r_, k_, v_, z, self.w0, self.bonus, S, ctx,
                     shift_src=x, shift_state=shift, seg_len=seg, seg_state=seg_state, seg_decay=seg_decay)
        normed = ws.get("attn_out", T, I, self.dtype)
        ops.group_rmsnorm_gate(normed, o, self.gain, g_, T, self.num_heads, self.eps)
        return linear(normed, self.w_o, ws.get("mixer_out", T, W, self.dtype), T, allow_partial=FUSE_PARTIALS)


register_part("mixer", "wkv", TimeMixWKV)


class StateSpaceDuality(Part):
    """Tensors (local names): in [2 I + 2 G N + H, W] laid out [z: I | x: I | B: G N | C: G N | dt: H] with I = H * V;
    conv [I + 2 G N, taps] and conv.b (x, B and C pass the convolution and silu); dt_bias, A_log, D [H];
    norm [I]; o [W, I].  y * silu(z) is RMS-normed in norm_groups equal parts (the gate comes before the norm).
    State row: [the convolution's last taps - 1 inputs | S: H * N * V]."""

    role = "mixer"

    def __init__(self, hidden_size: int, num_heads: int, value_dim: int, state_size: int, groups: int, norm_groups: int,
                 taps: int, eps: float, prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        if min(hidden_size, num_heads, value_dim, state_size, groups, norm_groups, taps) <= 0:
            raise ValueError("ssd: sizes must be positive")
        if num_heads % groups or (num_heads * value_dim) % norm_groups:
            raise ValueError(f"ssd: {num_heads} heads of {value_dim} do not divide into {groups} groups or {norm_groups} norm groups")
        if state_size > 256:
            raise ValueError(f"ssd: state size {state_size} exceeds 256, the most the recurrence kernel takes")
        self.hidden_size, self.num_heads, self.value_dim, self.state_size = hidden_size, num_heads, value_dim, state_size
        self.groups, self.norm_groups, self.taps, self.eps = groups, norm_groups, taps, float(eps)
        self.inner = num_heads * value_dim
        self.conv_channels = self.inner + 2 * groups * state_size
        self.conv_cols = _pad4((taps - 1) * self.conv_channels)
        self.w_in = self.w_conv = self.b_conv = self.dt_bias = self.a_log = self.skip = self.gain = self.w_o = None

    def parameters(self):
        n, W, I, H, C = self.name, self.hidden_size, self.inner, self.num_heads, self.conv_channels
        return {n("in"): ParamInfo((I + C + H, W)), n("conv"): ParamInfo((C, self.taps), kind="gain", init="normal"),
                n("conv.b"): ParamInfo((C,), kind="gain", init="normal"), n("dt_bias"): ParamInfo((H,), kind="gain", init="normal"),
                n("A_log"): ParamInfo((H,), kind="gain", init="normal"), n("D"): ParamInfo((H,), kind="gain", init="ones_normal"),
                n("norm"): ParamInfo((I,), kind="gain", init="ones_normal"), n("o"): ParamInfo((W, I))}

    def bind(self, tensors):
        t = lambda local: tensors[self.name(local)].contiguous()
        self.w_in, self.w_conv, self.b_conv = t("in"), t("conv").t().contiguous(), t("conv.b")      # [taps, channels]: a row per tap
        self.dt_bias, self.a_log, self.skip, self.gain, self.w_o = t("dt_bias"), t("A_log"), t("D"), t("norm"), t("o")

    def cache_need(self):
        return None

    def state_need(self):
        return StateNeed((self.conv_cols + self.num_heads * self.state_size * self.value_dim,), torch.float32)

    def forward(self, x: torch.Tensor, ctx, view) -> torch.Tensor:
        T, ws = ctx.n_tokens, ctx.workspace
        I, C, H, GN = self.inner, self.conv_channels, self.num_heads, self.groups * self.state_size
        conv_state, S = view.state[:, :self.conv_cols], view.state[:, self.conv_cols:]
        proj = linear(x, self.w_in, ws.get("ssd_in", T, I + C + H, self.dtype), T)
        xbc = ws.get("ssd_xbc", T, C, self.dtype)
        ops.short_conv(xbc, proj[:, I:I + C], self.w_conv, self.b_conv, conv_state, ctx, silu=True)
        y = ws.get("ssd_y", T, I, torch.float32)
        seg, seg_state, seg_decay = _segments(ctx, "ssd", H * self.state_size * self.value_dim, H * self.state_size)
        ops.ssd_scan(y, xbc[:, :I], xbc[:, I:I + GN], xbc[:, I + GN:], proj[:, I + C:], self.dt_bias, self.a_log, self.skip,
                     S, ctx, H, self.groups, self.state_size, self.value_dim, seg_len=seg, seg_state=seg_state, seg_decay=seg_decay)
        normed = ws.get("ssd_normed", T, I, self.dtype)
        ops.group_rmsnorm_gate(normed, y, self.gain, proj[:, :I], T, self.norm_groups, self.eps, gate_first=True)
        return linear(normed, self.w_o, ws.get("ssd_out", T, self.hidden_size, self.dtype), T, allow_partial=FUSE_PARTIALS)


register_part("mixer", "ssd", StateSpaceDuality)


class HGRN2(Part):
    """Tensors (local names): q, f [H*D, W], f.b and lower [H*D], v [H*V, W], norm [V] (shared by the heads), o [W, H*V].
    f = lower + (1 - lower) sigmoid(f h + f.b) per head and key channel is the decay, and 1 - f stands where a key would;
    q passes silu.  Every head's output is RMS-normed over its V values with the plain weight `norm`.  The forget gate's
    pre-activation is a float32 product; the gate, its complement and the state are float32.  State row: S: H * D * V."""

    role = "mixer"

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, eps: float, prefix: str = "",
                 dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        if min(hidden_size, num_heads, head_dim, value_dim) <= 0:
            raise ValueError("hgrn2: sizes must be positive")
        if head_dim > 256:
            raise ValueError(f"hgrn2: key size {head_dim} exceeds 256, the most the recurrence kernel takes")
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim = int(hidden_size), int(num_heads), int(head_dim), int(value_dim)
        self.eps = float(eps)
        self.qk_size, self.v_size = self.num_heads * self.head_dim, self.num_heads * self.value_dim
        self.w_qv = self.w_f = self.b_f = self.lower = self.gain = self.w_o = None

    def parameters(self):
        n, W = self.name, self.hidden_size
        return {n("q"): ParamInfo((self.qk_size, W)), n("f"): ParamInfo((self.qk_size, W)),
                n("f.b"): ParamInfo((self.qk_size,), kind="gain", init="normal"),
                n("lower"): ParamInfo((self.qk_size,), kind="gain", init="normal"),
                n("v"): ParamInfo((self.v_size, W)), n("norm"): ParamInfo((self.value_dim,), kind="gain", init="ones_normal"),
                n("o"): ParamInfo((W, self.v_size))}

    def bind(self, tensors):
        t = lambda local: tensors[self.name(local)]
        self.w_qv = torch.cat([t("q"), t("v")], dim=0).contiguous()
        self.w_f, self.b_f, self.lower = t("f").contiguous(), t("f.b").contiguous(), t("lower").contiguous()
        self.gain, self.w_o = t("norm").contiguous(), t("o").contiguous()

    def cache_need(self):
        return None

    def state_need(self):
        return StateNeed((self.qk_size * self.value_dim,), torch.float32)

    def forward(self, x: torch.Tensor, ctx, view) -> torch.Tensor:
        T, ws = ctx.n_tokens, ctx.workspace
        QK, VS = self.qk_size, self.v_size
        qv = linear(x, self.w_qv, ws.get("hgrn_qv", T, QK + VS, self.dtype), T)
        z = linear(x, self.w_f, ws.get("hgrn_f", T, QK, torch.float32), T)      # float32: bias, sigmoid and the bound are the kernel's
        o = ws.get("hgrn_o", T, VS, torch.float32)
        seg, seg_state, seg_decay = _segments(ctx, "hgrn", QK * self.value_dim, QK)
        ops.gate_scan(o, qv[:, :QK], qv[:, QK:], z, self.b_f, self.lower, view.state, ctx, self.num_heads, self.head_dim,
                      self.value_dim, seg_len=seg, seg_state=seg_state, seg_decay=seg_decay)
        normed = ws.get("attn_out", T, VS, self.dtype)
        ops.head_rmsnorm_gate(normed, o, self.gain, None, T, self.num_heads, self.eps)
        return linear(normed, self.w_o, ws.get("mixer_out", T, self.hidden_size, self.dtype), T, allow_partial=FUSE_PARTIALS)


register_part("mixer", "hgrn2", HGRN2)


class GatedDeltaRule(Part):
    """Tensors (local names): q, k [G*D, W], v [H*V, W], each with `<name>.conv` [channels, taps] (a short causal
    convolution, then silu); b, a [H, W] (beta = sigmoid(b h), decay = exp(-exp(A_log) softplus(a h + dt_bias))); A_log,
    dt_bias [H]; g [H*V, W] (the output gate, silu); norm [V] (shared by the heads); o [W, H*V].  q and k become unit vectors
    per head and q is scaled by D^(-1/2).  Head h reads q/k head h // (H / G).  State row: [the convolution's last
    taps - 1 inputs | S: H * D * V]."""

    role = "mixer"

    def __init__(self, hidden_size: int, num_heads: int, num_qk_heads: int, head_dim: int, value_dim: int, taps: int, eps: float,
                 unit_eps: float = 1e-6, prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        if min(hidden_size, num_heads, num_qk_heads, head_dim, value_dim) <= 0 or not (1 <= taps <= 16):
            raise ValueError("gated delta rule: sizes must be positive and taps 1 to 16")
        if num_heads % num_qk_heads:
            raise ValueError(f"gated delta rule: {num_heads} heads do not divide into {num_qk_heads} key heads")
        if head_dim > 256:
            raise ValueError(f"gated delta rule: key size {head_dim} exceeds 256, the most the recurrence kernel takes")
        self.hidden_size, self.num_heads, self.num_qk_heads = int(hidden_size), int(num_heads), int(num_qk_heads)
        self.head_dim, self.value_dim, self.taps = int(head_dim), int(value_dim), int(taps)
        self.eps, self.unit_eps = float(eps), float(unit_eps)
        self.qk_size, self.v_size = self.num_qk_heads * self.head_dim, self.num_heads * self.value_dim
        self.conv_channels = 2 * self.qk_size + self.v_size
        self.conv_cols = _pad4((self.taps - 1) * self.conv_channels)
        self.w_in = self.w_conv = self.a_log = self.dt_bias = self.gain = self.w_o = None

    def parameters(self):
        n, W, H = self.name, self.hidden_size, self.num_heads
        p = {n("q"): ParamInfo((self.qk_size, W)), n("k"): ParamInfo((self.qk_size, W)), n("v"): ParamInfo((self.v_size, W)),
             n("b"): ParamInfo((H, W)), n("a"): ParamInfo((H, W)), n("g"): ParamInfo((self.v_size, W)),
             n("A_log"): ParamInfo((H,), kind="gain", init="normal"), n("dt_bias"): ParamInfo((H,), kind="gain", init="normal"),
             n("norm"): ParamInfo((self.value_dim,), kind="gain", init="ones_normal"), n("o"): ParamInfo((W, self.v_size))}
        for m, c in (("q", self.qk_size), ("k", self.qk_size), ("v", self.v_size)):
            p[n(m + ".conv")] = ParamInfo((c, self.taps), kind="gain", init="normal")
        return p

    def bind(self, tensors):
        t = lambda local: tensors[self.name(local)]
        # one product for everything the mixer reads from h: [q | k | v | gate | b | a]
        self.w_in = torch.cat([t("q"), t("k"), t("v"), t("g"), t("b"), t("a")], dim=0).contiguous()
        self.w_conv = torch.cat([t("q.conv"), t("k.conv"), t("v.conv")], dim=0).t().contiguous()      # [taps, channels]
        self.a_log, self.dt_bias = t("A_log").contiguous(), t("dt_bias").contiguous()
        self.gain, self.w_o = t("norm").contiguous(), t("o").contiguous()

    def cache_need(self):
        return None

    def state_need(self):
        return StateNeed((self.conv_cols + self.num_heads * self.head_dim * self.value_dim,), torch.float32)

    def forward(self, x: torch.Tensor, ctx, view) -> torch.Tensor:
        T, ws = ctx.n_tokens, ctx.workspace
        QK, VS, C, H = self.qk_size, self.v_size, self.conv_channels, self.num_heads
        conv_state, S = view.state[:, :self.conv_cols], view.state[:, self.conv_cols:]
        proj = linear(x, self.w_in, ws.get("delta_in", T, C + VS + 2 * H, self.dtype), T)
        qkv = ws.get("delta_qkv", T, C, self.dtype)
        ops.short_conv(qkv, proj[:, :C], self.w_conv, None, conv_state, ctx, silu=True)
        o = ws.get("delta_o", T, VS, torch.float32)
        operands = (o, qkv[:, :QK], qkv[:, QK:2 * QK], qkv[:, 2 * QK:], proj[:, C + VS:C + VS + H], proj[:, C + VS + H:],
                    self.a_log, self.dt_bias, S, ctx, H, self.num_qk_heads, self.head_dim, self.value_dim, self.head_dim ** -0.5,
                    self.unit_eps)
        if CHUNKED_DELTA and not ctx.decode_only and T >= 4 * SEGMENT:
            # a step with prompt portions: chunks of 32 tokens solved together, chained through the state
            cap = ws.max_rows // ops.DELTA_CHUNK + ctx.cu_tokens.numel()          # chunks of any step: the buffers' sizes
            scratch = [ws.flat("delta_chunk_" + tag, numel, torch.float32)
                       for tag, numel in zip(("yq", "k", "w", "b", "g"), ops.delta_chunk_scratch(cap, H, self.head_dim, self.value_dim))]
            ops.delta_chunk_scan(*operands, scratch)
        else:
            ops.delta_scan(*operands)
        normed = ws.get("delta_normed", T, VS, self.dtype)
        ops.head_rmsnorm_gate(normed, o, self.gain, proj[:, C:C + VS], T, H, self.eps)
        return linear(normed, self.w_o, ws.get("delta_out", T, self.hidden_size, self.dtype), T, allow_partial=FUSE_PARTIALS)


register_part("mixer", "gated_delta", GatedDeltaRule)


class ConvInput(Part):
    """The inner mixer reads h + conv(h): conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j) per channel, zeros before the
    request's first token, no bias.  Tensor `<prefix>.<weight_name>` [W, taps].  State row: [the last taps - 1
    inputs | the inner mixer's]; the inner mixer's cache is the layer's."""

    role = "mixer"

    def __init__(self, hidden_size: int, taps: int, inner, weight_name: str = "conv", prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        if hidden_size <= 0 or not (1 <= taps <= 16):
            raise ValueError(f"input convolution: width {hidden_size} must be positive and taps {taps} 1 to 16")
        self.hidden_size, self.taps, self.weight_name = int(hidden_size), int(taps), weight_name
        self.inner = build_part("mixer", inner, dtype, device)
        self.own_cols = _pad4((self.taps - 1) * self.hidden_size)
        self.inner_cols = _state_numel(self.inner.state_need())
        self.w = None

    def children(self):
        return [self.inner]

    def parameters(self):
        return {self.name(self.weight_name): ParamInfo((self.hidden_size, self.taps), kind="gain", init="normal")}

    def bind(self, tensors):
        self.w = tensors[self.name(self.weight_name)].t().contiguous()            # [taps, width]: a row per tap

    def cache_need(self):
        return self.inner.cache_need()

    def state_need(self):
        return StateNeed((max(self.own_cols + self.inner_cols, 4),), torch.float32)

    def forward(self, x: torch.Tensor, ctx, view) -> torch.Tensor:
        out = ctx.workspace.get("conv_input", ctx.n_tokens, self.hidden_size, self.dtype)
        ops.short_conv(out, x, self.w, None, view.state[:, :self.own_cols], ctx, residual=True)
        inner_state = view.state[:, self.own_cols:] if self.inner_cols else None
        return self.inner.forward(out, ctx, _sub_view(view, inner_state))


register_part("mixer", "conv_input", ConvInput)


class ConvInputFFN(Part):
    """The same for a feed-forward: the inner feed-forward reads h + conv(h).  Tensor `<prefix>.<weight_name>` [W, taps].
    Unlike other feed-forwards this one keeps something per request, the last taps - 1 inputs, and says so with
    state_need(); the block hands it its columns of the layer's state row."""

    role = "ffn"

    def __init__(self, hidden_size: int, taps: int, inner, weight_name: str = "conv", prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        if hidden_size <= 0 or not (1 <= taps <= 16):
            raise ValueError(f"input convolution: width {hidden_size} must be positive and taps {taps} 1 to 16")
        self.hidden_size, self.taps, self.weight_name = int(hidden_size), int(taps), weight_name
        self.inner = build_part("ffn", inner, dtype, device)
        if hasattr(self.inner, "state_need"):
            raise ValueError("input convolution: the feed-forward inside keeps no state of its own")
        self.w = None

    def children(self):
        return [self.inner]

    def parameters(self):
        return {self.name(self.weight_name): ParamInfo((self.hidden_size, self.taps), kind="gain", init="normal")}

    def bind(self, tensors):
        self.w = tensors[self.name(self.weight_name)].t().contiguous()            # [taps, width]: a row per tap

    def state_need(self):
        return StateNeed((max(_pad4((self.taps - 1) * self.hidden_size), 4),), torch.float32)

    def forward(self, x: torch.Tensor, ctx, state) -> torch.Tensor:
        out = ctx.workspace.get("conv_input_ffn", ctx.n_tokens, self.hidden_size, self.dtype)
        ops.short_conv(out, x, self.w, None, state, ctx, residual=True)
        return self.inner.forward(out, ctx)


register_part("ffn", "conv_input", ConvInputFFN)


class ParallelMixers(Part):
    """out = (rms(left(h)) * g_l + rms(right(h)) * g_r) / 2, each RMS norm over the model width with a plain weight
    (`<prefix>.<left_name>`, `<prefix>.<right_name>`); or, with combine="scaled_sum", out = left_scale * left(h) +
    right_scale * right(h) with two constants and no tensors of its own.  At most one side keeps keys (the layer has one
    cache); the state row is the left side's followed by the right side's."""

    role = "mixer"

    def __init__(self, hidden_size: int, left, right, eps: float = 0.0, left_name: str = "left.out", right_name: str = "right.out",
                 combine: str = "norm_mean", left_scale: float = 1.0, right_scale: float = 1.0, prefix: str = "", dtype=None,
                 device=None):
        super().__init__(prefix, dtype, device)
        if combine not in ("norm_mean", "scaled_sum"):
            raise ValueError(f"parallel mixers: unknown way to combine '{combine}'")
        self.combine, self.left_scale, self.right_scale = combine, float(left_scale), float(right_scale)
        self.hidden_size, self.eps = int(hidden_size), float(eps)
        self.left_name, self.right_name = left_name, right_name
        self.left, self.right = build_part("mixer", left, dtype, device), build_part("mixer", right, dtype, device)
        if self.left.cache_need() is not None and self.right.cache_need() is not None:
            raise ValueError("parallel mixers: only one side may keep keys and values")
        self.left_cols = _pad4(_state_numel(self.left.state_need()))
        self.right_cols = _state_numel(self.right.state_need())
        self.g_left = self.g_right = None

    def children(self):
        return [self.left, self.right]

    def parameters(self):
        W = self.hidden_size
        if self.combine == "scaled_sum":
            return {}
        return {self.name(self.left_name): ParamInfo((W,), kind="gain", init="ones_normal"),
                self.name(self.right_name): ParamInfo((W,), kind="gain", init="ones_normal")}

    def bind(self, tensors):
        if self.combine == "scaled_sum":
            return
        self.g_left = tensors[self.name(self.left_name)].contiguous()
        self.g_right = tensors[self.name(self.right_name)].contiguous()

    def cache_need(self):
        return self.left.cache_need() or self.right.cache_need()

    def state_need(self):
        n = self.left_cols + self.right_cols
        return StateNeed((n,), torch.float32) if n else None

    def forward(self, x: torch.Tensor, ctx, view) -> torch.Tensor:
        T, ws = ctx.n_tokens, ctx.workspace
        ls = view.state[:, :self.left_cols] if self.left_cols else None
        rs = view.state[:, self.left_cols:] if self.right_cols else None
        a = self.left.forward(x, ctx, _sub_view(view, ls))
        # unsummed partial results live until the next product: the left side's are summed before the right side runs
        a = ops.settle(a, ws.get("parallel_left", T, self.hidden_size, self.dtype), T)
        b = self.right.forward(x, ctx, _sub_view(view, rs))
        out = ws.get("parallel_out", T, self.hidden_size, self.dtype)
        if self.combine == "scaled_sum":
            ops.scaled_sum(out, a, b, self.left_scale, self.right_scale, T)
        else:
            ops.pair_norm_mean(out, a, b, self.g_left, self.g_right, T, self.eps)
        return out


register_part("mixer", "parallel", ParallelMixers)
