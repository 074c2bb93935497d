"""A plain, slow implementation of the Potipel design, one function per mechanism, whole sequences only.

Everything is written from the design's equations in torch on the CPU, in the dtype of the weights it is
given (the tests use float64), token by token where the design has a recurrence.  It shares no code with
the package: no kernels, no parts, no cache.  `forward(config, weights, tokens)` returns the logits at
every position of one sequence and, on request, the residual stream after every layer run.

Notation: T tokens, W the model width, h the rows a sublayer reads, H query heads, G key/value heads,
D the key size, V the value size.
"""
from __future__ import annotations

import math

import torch


# ---- small pieces ------------------------------------------------------------------------------------------
def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def causal_conv(x, w):
    """y_t = sum_j w[:, j] x_(t - taps + 1 + j) per channel, zeros before the start.  x [T, C], w [C, taps]."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([x.new_zeros(taps - 1, C), x], dim=0)
    y = x.new_zeros(T, C)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    return y


def input_conv(h, w):
    """What a sublayer reads: h + conv(h)."""
    return h + causal_conv(h, w)


def kv_head_of(h, heads, kv_heads):
    return h // (heads // kv_heads)


# ---- differential attention -------------------------------------------------------------------------------
def diff_lambda(lq1, lk1, lq2, lk2, diff):
    return math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + diff


def diff_attention(h, p, m, eps):
    """Two causal softmax maps per head over the same values, a1 - lambda a2, a weightless RMS norm per head times
    (1 - diff), a sigmoid gate from the same input, then the output projection.  p: tensors by local name."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ p["q"].T).view(T, H, 2, D)
    k = (h @ p["k"].T).view(T, G, 2, D)
    v = (h @ p["v"].T).view(T, G, V)
    q = rms_norm(q, p["q.norm"], eps)
    k = rms_norm(k, p["k.norm"], eps)
    lam = diff_lambda(p["lq1"], p["lk1"], p["lq2"], p["lk2"], m["diff"])
    visible = torch.tril(torch.ones(T, T, dtype=torch.bool))
    heads = []
    for hh in range(H):
        g = kv_head_of(hh, H, G)
        maps = []
        for c in range(2):
            s = (q[:, hh, c] @ k[:, g, c].T) * m["scale"]
            s = s.masked_fill(~visible, float("-inf"))
            maps.append(torch.softmax(s, dim=-1) @ v[:, g])
        o = maps[0] - lam * maps[1]
        heads.append(rms_unit(o, eps) * (1.0 - m["diff"]))
    o = torch.cat(heads, dim=-1) * torch.sigmoid(h @ p["g"].T)
    return o @ p["o"].T


# ---- hgrn2 ------------------------------------------------------------------------------------------------
def hgrn2(h, p, m, eps):
    """S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t per head, f bounded below by `lower`."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ p["q"].T).view(T, H, D)
    v = (h @ p["v"].T).view(T, H, V)
    low = p["lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ p["f"].T + p["f.b"])).view(T, H, D)
    S = h.new_zeros(H, D, V)
    out = h.new_zeros(T, H, V)
    for t in range(T):
        S = f[t].unsqueeze(-1) * S + (1.0 - f[t]).unsqueeze(-1) * v[t].unsqueeze(1)
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    out = rms_norm(out, p["norm"], eps)
    return out.reshape(T, H * V) @ p["o"].T


# ---- sliding-window attention with a sink, a capped score and a distance bias -------------------------------
def window_attention(h, p, m):
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv(h @ p["q"].T + p["q.b"], p["q.conv"]).view(T, H, D)
    k = causal_conv(h @ p["k"].T + p["k.b"], p["k.conv"]).view(T, G, D)
    v = causal_conv(h @ p["v"].T + p["v.b"], p["v.conv"]).view(T, G, V)
    i = torch.arange(T).unsqueeze(1)
    j = torch.arange(T).unsqueeze(0)
    dist = (i - j)
    visible = (dist >= 0) & (dist < m["mask"]["size"])
    cap = m["softcap"]
    heads = []
    for hh in range(H):
        g = kv_head_of(hh, H, G)
        s = (q[:, hh] @ k[:, g].T) * m["scale"]
        s = cap * torch.tanh(s / cap)
        s = s - p["r1"][hh] * torch.log1p(p["r2"][hh] * dist.clamp(min=0).to(h.dtype))
        s = s.masked_fill(~visible, float("-inf"))
        sink = p["sink"][hh]
        top = torch.maximum(s.max(dim=-1, keepdim=True).values, sink)
        e = torch.exp(s - top)
        heads.append((e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink - top))) @ v[:, g])
    return torch.cat(heads, dim=-1) @ p["o"].T


# ---- gated delta rule -------------------------------------------------------------------------------------
def gated_delta(h, p, m, eps):
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ p["q"].T, p["q.conv"])).view(T, G, D)
    k = silu(causal_conv(h @ p["k"].T, p["k.conv"])).view(T, G, D)
    v = silu(causal_conv(h @ p["v"].T, p["v.conv"])).view(T, H, V)
    unit = lambda x: x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)
    q = unit(q) * D ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ p["b"].T)                                           # [T, H]
    decay = torch.exp(-torch.exp(p["A_log"]) * softplus(h @ p["a"].T + p["dt_bias"]))   # [T, H]
    S = h.new_zeros(H, D, V)
    out = h.new_zeros(T, H, V)
    for t in range(T):
        for hh in range(H):
            g = kv_head_of(hh, H, G)
            Sh = decay[t, hh] * S[hh]
            u = beta[t, hh] * (v[t, hh] - Sh.T @ k[t, g])
            Sh = Sh + torch.outer(k[t, g], u)
            S[hh] = Sh
            out[t, hh] = Sh.T @ q[t, g]
    out = rms_norm(out, p["norm"], eps) * silu(h @ p["g"].T).view(T, H, V)
    return out.reshape(T, H * V) @ p["o"].T


def sub(p, prefix):
    return {k[len(prefix) + 1:]: v for k, v in p.items() if k.startswith(prefix + ".")}


def parallel(h, p, m, eps):
    return (m["left_scale"] * window_attention(h, sub(p, "left"), m["left"])
            + m["right_scale"] * gated_delta(h, sub(p, "right"), m["right"], eps))


# ---- feed-forward -----------------------------------------------------------------------------------------
def dense_ff(h, p):
    return (torch.relu(h @ p["gate"].T) * (h @ p["up"].T)) @ p["down"].T


def expert_ff(h, p, limit):
    g = torch.clamp(h @ p["gate"].T, max=limit)
    u = torch.clamp(h @ p["up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ p["down"].T


def route(h, p, r):
    """(chosen experts [T, top], their weights [T, top], margin [T]): sigmoid scores, a correction for the choice only,
    experts outside the best groups shut out, weights not renormalised.  margin: the last chosen choice score minus the
    best one left out among the allowed (inf where none is left)."""
    E, top, count, keep = r["experts"], r["top"], r["groups"]["count"], r["groups"]["keep"]
    s = torch.sigmoid(h @ p["router"].T)
    choice = s + p["correction"]
    T = h.shape[0]
    per = E // count
    grouped = choice.view(T, count, per)
    gscore = grouped.topk(min(2, per), dim=-1).values.sum(dim=-1)               # [T, count]
    best = gscore.topk(keep, dim=-1).indices
    allowed = torch.zeros(T, count, dtype=torch.bool)
    allowed.scatter_(1, best, True)
    masked = torch.where(allowed.unsqueeze(-1).expand(T, count, per).reshape(T, E), choice, torch.full_like(choice, float("-inf")))
    order = masked.sort(dim=-1, descending=True)
    ids = order.indices[:, :top]
    margin = (order.values[:, top - 1] - order.values[:, top]) if top < E else torch.full((T,), float("inf"), dtype=h.dtype)
    gmargin = torch.full((T,), float("inf"), dtype=h.dtype)
    if keep < count:
        gs = gscore.sort(dim=-1, descending=True).values
        gmargin = gs[:, keep - 1] - gs[:, keep]
    return ids, s.gather(1, ids), torch.minimum(margin, gmargin)


def moe_ff(h, p, mlp):
    ids, wts, _ = route(h, p, mlp["router"])
    out = h.new_zeros(h.shape[0], p["e0.down"].shape[0])
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            out[t] = out[t] + wts[t, j] * expert_ff(h[t:t + 1], sub(p, f"e{e}"), mlp["expert"]["limit"])[0]
    return out


# ---- the model --------------------------------------------------------------------------------------------
def layer_tensors(weights, i):
    return sub(weights, f"l{i}")


def forward(config, weights, tokens, want_layers=False, margins=None):
    """Logits [T, vocab] of one sequence (and the residual stream after every layer run).  margins: a list that
    receives every routed layer's routing margins [T]."""
    eps = config["norm"]["eps"]
    x = weights["embed"][torch.as_tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]
    after = []
    for i, layer in enumerate(config["layers"]):
        p = layer_tensors(weights, layer.get("weights_of", i) if layer.get("weights_of") is not None else i)
        h = input_conv(rms_norm(x, p["norm1"], eps), p["canon1"])
        kind, m = layer["type"], layer["mixer"]
        if kind == "attention":
            y = diff_attention(h, sub(p, "mix"), m, eps)
        elif kind == "hgrn2":
            y = hgrn2(h, sub(p, "mix"), m, eps)
        elif kind == "parallel":
            y = parallel(h, sub(p, "mix"), m, eps)
        else:
            raise ValueError(kind)
        x = x + y
        mlp = layer.get("mlp")
        if mlp is not None:
            h = input_conv(rms_norm(x, p["norm2"], eps), p["canon2"])
            if mlp["kind"] == "dense":
                x = x + dense_ff(h, sub(p, "mlp"))
            else:
                if margins is not None:
                    margins.append(route(h, sub(p, "mlp"), mlp["router"])[2])
                x = x + moe_ff(h, sub(p, "mlp"), mlp)
        after.append(x)
    logits = rms_norm(x, weights["final.norm"], eps) @ weights["head"].T
    return (logits, torch.stack(after)) if want_layers else logits
