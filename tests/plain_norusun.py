"""A plain, slow implementation of the Norusun design, one function per mechanism, whole sequences only.

Everything is written from the design's equations in torch on the CPU, in the dtype of the weights it is
given (the tests use float64), token by token where the design has a recurrence.  It shares no code with
the package: no kernels, no parts, no cache.  `forward(config, weights, tokens)` returns the logits at
every position of one sequence and, on request, the summed streams after every layer.

Notation: T tokens, W the model width, h the rows a mixer reads, S streams.
"""
from __future__ import annotations

import math

import torch


# ---- small pieces ------------------------------------------------------------------------------------------
def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose gain is one number for all coordinates."""
    return rms_unit(x, eps) * g


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def causal_conv(x, w, bias=None):
    """y_t = sum_j w[:, j] x_(t - taps + 1 + j) per channel, zeros before the start.  x [T, C], w [C, taps]."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([x.new_zeros(taps - 1, C), x], dim=0)
    y = x.new_zeros(T, C)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    return y if bias is None else y + bias


def input_conv(h, w):
    """What a mixer reads: h + conv(h)."""
    return h + causal_conv(h, w)


def rotate_neighbours(x, positions, dims, base):
    """Pairs (2i, 2i+1), i < dims/2, of the last dimension turn by position * base^(-2i/dims); the rest passes."""
    out = x.clone()
    for i in range(dims // 2):
        a = positions.to(x.dtype) * (float(base) ** (-2.0 * i / dims))
        c, s = torch.cos(a), torch.sin(a)
        while c.dim() < x.dim() - 1:
            c, s = c.unsqueeze(-1), s.unsqueeze(-1)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def rotate_halves(x, positions, dims, base):
    """Pairs (i, i + dims/2), i < dims/2, of the last dimension turn by position * base^(-2i/dims); the rest passes."""
    out = x.clone()
    half = dims // 2
    for i in range(half):
        a = positions.to(x.dtype) * (float(base) ** (-2.0 * i / dims))
        c, s = torch.cos(a), torch.sin(a)
        while c.dim() < x.dim() - 1:
            c, s = c.unsqueeze(-1), s.unsqueeze(-1)
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


# ---- hyper-connections -------------------------------------------------------------------------------------
def streams_read(xs, w_in):
    """u = sum_s w_in[s] x_s.  xs [S, T, W]."""
    return torch.einsum("s,stw->tw", w_in, xs)


def streams_write(xs, mix, w_out, y):
    """x_t <- sum_s mix[s, t] x_s + w_out[t] y, all streams at once from the old ones."""
    return torch.einsum("sr,stw->rtw", mix, xs) + w_out[:, None, None] * y[None]


# ---- mixer: wkv --------------------------------------------------------------------------------------------
def wkv_recurrence(r, k, v, decay, bonus, state=None):
    """o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t, then S_t = diag(w_t) S_(t-1) + k_t v_t^T.  r, k, v, decay [T, H, D];
    bonus [H, D]; state [H, D, D] (key channel, value channel) or None for zeros.  Returns (o [T, H, D], last state)."""
    T, H, D = r.shape
    state = r.new_zeros(H, D, D) if state is None else state.clone()
    o = r.new_zeros(T, H, D)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hi,hij->hj", r[t], state + bonus[:, :, None] * kv)
        state = decay[t][:, :, None] * state + kv
    return o, state


def wkv_mixer(h, p, m, eps):
    """RWKV-style time mixing.  p: the mixer's tensors by their local names; m: its sizes."""
    T, W = h.shape
    H, D = m["heads"], m["dim"]
    prev = torch.cat([h.new_zeros(1, W), h[:-1]], dim=0)
    lerp = lambda name: h + (prev - h) * p["mu." + name]
    r = (lerp("r") @ p["r"].T).view(T, H, D)
    k = (lerp("k") @ p["k"].T).view(T, H, D)
    v = (lerp("v") @ p["v"].T).view(T, H, D)
    gate = silu(lerp("g") @ p["g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(lerp("w") @ p["w1"].T) @ p["w2"].T + p["w0"])).view(T, H, D)
    o, _ = wkv_recurrence(r, k, v, decay, p["u"])
    o = rms_unit(o, eps).reshape(T, H * D) * p["norm"] * gate
    return o @ p["o"].T


# ---- mixer: latent attention -------------------------------------------------------------------------------
def window_sink_softmax(score, size, sink, v, positions=None, key_positions=None):
    """Softmax over the keys j with 0 <= i - j < size, whose denominator also holds exp(sink_h).  score [H, Tq, Tk]
    (already scaled), sink [H], v [Tk, H, V]; positions of queries and keys default to 0, 1, ...  Returns [Tq, H, V]."""
    i = (torch.arange(score.shape[1]) if positions is None else positions)[:, None]
    j = (torch.arange(score.shape[2]) if key_positions is None else key_positions)[None, :]
    seen = (i - j >= 0) & (i - j < size)
    score = score.masked_fill(~seen, -math.inf)
    top = torch.maximum(score.max(dim=-1).values, sink[:, None])                           # [H, Tq]
    e = torch.exp(score - top[..., None])
    weights = e / (e.sum(dim=-1) + torch.exp(sink[:, None] - top))[..., None]
    return torch.einsum("hij,jhv->ihv", weights, v)


def latent_attention_mixer(h, p, m, eps):
    T, W = h.shape
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms_unit(h @ p["dq"].T, eps) * p["dq.norm"]
    q = (cq @ p["uq"].T).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_neighbours(q[..., D:], pos, m["rot"]["dims"], m["rot"]["base"])
    down = h @ p["dkv"].T
    c = rms_unit(down[:, :C], eps) * p["dkv.norm"]
    k_rot = rotate_neighbours(down[:, C:], pos, m["rot"]["dims"], m["rot"]["base"])        # one part for all heads
    k_plain = (c @ p["uk"].T).view(T, H, D)
    v = (c @ p["uv"].T).view(T, H, V)
    score = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihr,jr->hij", q_rot, k_rot)) * m["scale"]
    o = window_sink_softmax(score, m["mask"]["size"], p["sink"], v).reshape(T, H * V)
    return o @ p["o"].T


# ---- mixer: parallel (chunked sigmoid attention beside a state-space layer) ------------------------------------
def chunk_sigmoid_weights(score, size, bias, v):
    """Weights sigmoid(score + bias_h) on the keys j <= i of the query's chunk (floor(i / size) = floor(j / size)), not
    normalised.  score [H, T, T] (already scaled), bias [H], v [T, H, V] (per query head).  Returns [T, H, V]."""
    pos = torch.arange(score.shape[1])
    i, j = pos[:, None], pos[None, :]
    seen = (j <= i) & (i // size == j // size)
    weights = torch.sigmoid(score + bias[:, None, None]) * seen
    return torch.einsum("hij,jhv->ihv", weights, v)


def chunked_sigmoid_attention(h, p, m, eps):
    T, W = h.shape
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (rms_unit(h @ p["q"].T, eps) * p["q.norm"]).view(T, H, D)
    k = (rms_unit(h @ p["k"].T, eps) * p["k.norm"]).view(T, G, D)
    v = (h @ p["v"].T).view(T, G, V)
    q = rotate_halves(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_halves(k, pos, m["rot"]["dims"], m["rot"]["base"])
    group = torch.arange(H) // (H // G)
    score = torch.einsum("ihd,jhd->hij", q, k[:, group]) * m["scale"]
    o = chunk_sigmoid_weights(score, m["mask"]["size"], p["pb"], v[:, group]).reshape(T, H * V)
    return o @ p["o"].T


def ssd_recurrence(x, B, C, dt, decay, skip, state=None):
    """S_t = a_t S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t.  x [T, H, V]; B, C [T, G, N] (head h uses group
    h // (H / G)); dt, decay [T, H]; skip [H]; state [H, N, V] or None for zeros.  Returns (y [T, H, V], last state)."""
    T, H, V = x.shape
    G, N = B.shape[1], B.shape[2]
    group = torch.arange(H) // (H // G)
    state = x.new_zeros(H, N, V) if state is None else state.clone()
    y = x.new_zeros(T, H, V)
    for t in range(T):
        state = decay[t][:, None, None] * state + dt[t][:, None, None] * B[t][group][:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnv,hn->hv", state, C[t][group]) + skip[:, None] * x[t]
    return y, state


def state_space_mixer(h, p, m, eps):
    T, W = h.shape
    H, V, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * V
    proj = h @ p["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, p["conv"], p["conv.b"]))
    x = xbc[:, :inner].view(T, H, V)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + p["dt_bias"])                                # [T, H]
    decay = torch.exp(-torch.exp(p["A_log"]) * dt)
    y, _ = ssd_recurrence(x, B, C, dt, decay, p["D"])
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_unit(y.view(T, parts, inner // parts), eps).reshape(T, inner) * p["norm"]
    return y @ p["o"].T


def parallel_mixer(h, p, m, eps):
    sub = lambda side: {k[len(side) + 1:]: v for k, v in p.items() if k.startswith(side + ".") and k != side + ".out"}
    left = chunked_sigmoid_attention(h, sub("left"), m["left"], eps)
    right = state_space_mixer(h, sub("right"), m["right"], eps)
    return 0.5 * (rms_unit(left, eps) * p["left.out"] + rms_unit(right, eps) * p["right.out"])


# ---- feed-forward ------------------------------------------------------------------------------------------
def clamped_ff(h, p, limit):
    g = torch.clamp(h @ p["gate"].T + p["gate.b"], max=limit)
    u = torch.clamp(h @ p["up"].T + p["up.b"], min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ p["down"].T + p["down.b"]


# ---- the model ---------------------------------------------------------------------------------------------
MIXERS = {"wkv": wkv_mixer, "latent_attention": latent_attention_mixer, "parallel": parallel_mixer}


def forward(config, weights, tokens, with_layers=False):
    """Logits [T, vocab] of one sequence; with_layers also the summed streams after every layer [L, T, W]."""
    eps = config["norm"]["eps"]
    S = config["streams"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    xs = weights["embed"][tokens][None].repeat(S, 1, 1)
    after = []
    for i, layer in enumerate(config["layers"]):
        L = f"l{i}."
        local = lambda prefix: {k[len(L + prefix):]: v for k, v in weights.items() if k.startswith(L + prefix)}
        h = scalar_norm(streams_read(xs, weights[L + "hc1.in"]), weights[L + "norm1"], eps)
        h = input_conv(h, weights[L + "canon1"])
        y = MIXERS[layer["type"]](h, local("mix."), layer["mixer"], eps)
        xs = streams_write(xs, weights[L + "hc1.mix"], weights[L + "hc1.out"], y)
        if layer["mlp"] is not None:
            h = scalar_norm(streams_read(xs, weights[L + "hc2.in"]), weights[L + "norm2"], eps)
            y = clamped_ff(h, local("mlp."), layer["mlp"]["limit"])
            xs = streams_write(xs, weights[L + "hc2.mix"], weights[L + "hc2.out"], y)
        after.append(xs.sum(dim=0))
    x = scalar_norm(xs.sum(dim=0), weights["final.norm"], eps)
    logits = x @ weights["head"].T
    return (logits, torch.stack(after)) if with_layers else logits
