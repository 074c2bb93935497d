"""GPU tests of the Potipel design against the plain implementation (tests/plain_potipel.py): each mechanism alone,
then whole models under every way of cutting the work."""
import copy
import json
import math
import os
from types import SimpleNamespace

import pytest
import torch

import plain_potipel as P
import replay
from potipel_tiny import (CONFIGS, attention, config, dense, hgrn2, layer, make_engine, make_weights, moe, parallel, random_config)
from tiny import max_err, random_tokens

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-5, "bfloat16": 5e-2}       # whole models, relative to the largest logit
KTOL = {"float32": 4e-6, "bfloat16": 6e-3}      # kernels alone: one rounding of the output


def dev(t, dtype="float32"):
    return t.to(device="cuda", dtype=DT[dtype]).contiguous()


def bf(t):
    return t.to(torch.bfloat16).float()


def i32(xs):
    return torch.tensor(xs, dtype=torch.int32, device="cuda")


def step_ctx(lens, slots):
    """What the kernels read of a step: entries of lens tokens laid end to end, each with its state slot."""
    cu, entry = [0], []
    for e, n in enumerate(lens):
        cu.append(cu[-1] + n)
        entry += [e] * n
    return SimpleNamespace(n_tokens=cu[-1], n_entries=len(lens), cu_tokens=i32(cu), token_entry=i32(entry), state_slots=i32(slots))


def split_steps(total, cuts):
    out, at, k = [], 0, 0
    while at < total:
        n = min(cuts[k % len(cuts)], total - at)
        out.append((at, at + n))
        at, k = at + n, k + 1
    return out


# ---- each mechanism alone ---------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_is_scaled_in_float32(dtype):
    from llm_b200.csrc import ops
    g = torch.Generator().manual_seed(3)
    table = bf(torch.randn(19, 100, generator=g))
    resid = torch.zeros(5, 100, device="cuda")
    ops.embedding(resid, dev(table, dtype), i32([3, 18, 0, 3, 7]), 5, torch.zeros(4, dtype=torch.int32, device="cuda"), 0.37)
    assert max_err(resid, table[[3, 18, 0, 3, 7]] * 0.37) < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("ff,rows", [(8, 3), (100, 7), (328, 33)])
def test_relu_gated_unit(dtype, ff, rows):
    from llm_b200.csrc import ops
    g = torch.Generator().manual_seed(ff)
    gu = bf(torch.randn(rows, 2 * ff, generator=g))
    out = torch.empty(rows, ff, device="cuda", dtype=DT[dtype])
    ops.silu_mul(out, dev(gu, dtype), rows, "relu")
    assert max_err(out, torch.relu(gu[:, :ff]) * gu[:, ff:]) < KTOL[dtype]


@pytest.mark.parametrize("rows,ff,width", [(129, 64, 64), (300, 328, 128), (2048, 1024, 512)])
def test_relu_gate_in_the_products_epilogue(rows, ff, width):
    """Many rows in bfloat16: relu(gate) * up is made in the epilogue of the gate/up product."""
    from llm_b200.parts.linear import linear_swiglu
    g = torch.Generator().manual_seed(rows)
    x, w = bf(torch.randn(rows, width, generator=g)), bf(torch.randn(2 * ff, width, generator=g) / math.sqrt(width))
    out = torch.empty(rows, ff, device="cuda", dtype=torch.bfloat16)
    assert linear_swiglu(dev(x, "bfloat16"), dev(w, "bfloat16"), out, rows, "relu")
    gu = x.double() @ w.double().T
    assert max_err(out, torch.relu(gu[:, :ff]) * gu[:, ff:]) < KTOL["bfloat16"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,R,V", [(4, 1, 8), (6, 3, 14), (2, 2, 72), (8, 4, 64), (3, 3, 130)])
def test_two_maps_combined_per_head(dtype, H, R, V):
    """a1 - lambda a2, the weightless norm, (1 - diff), the sigmoid gate; the maps arrive ordered [group][map][head in group]."""
    from llm_b200.csrc import ops
    g = torch.Generator().manual_seed(H * 100 + V)
    T, G, lam, diff, eps = 7, H // R, 0.83, 0.35, 1e-5
    maps = bf(torch.randn(T, H, 2, V, generator=g))                 # by head and map
    gate = bf(torch.randn(T, H * V, generator=g))
    o = maps[:, :, 0] - lam * maps[:, :, 1]
    ref = (P.rms_unit(o.double(), eps) * (1 - diff)).reshape(T, H * V) * torch.sigmoid(gate.double())
    arranged = maps.view(T, G, R, 2, V).permute(0, 1, 3, 2, 4).reshape(T, 2 * H * V)
    out = torch.empty(T, H * V, device="cuda", dtype=DT[dtype])
    ops.diff_combine(out, dev(arranged, dtype), dev(gate, dtype), T, H, R, lam, 1 - diff, eps)
    assert max_err(out, ref) < KTOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_scaled_sum_of_two_rows(dtype):
    from llm_b200.csrc import ops
    g = torch.Generator().manual_seed(1)
    a, b = bf(torch.randn(9, 100, generator=g)), bf(torch.randn(9, 100, generator=g))
    out = torch.empty(9, 100, device="cuda", dtype=DT[dtype])
    ops.scaled_sum(out, dev(a, dtype), dev(b, dtype), 0.7, 1.3, 9)
    assert max_err(out, 0.7 * a + 1.3 * b) < KTOL[dtype]


@pytest.mark.parametrize("E,top,count,keep", [(8, 2, 2, 1), (6, 2, 3, 2), (5, 1, 5, 2), (3, 3, 1, 1), (12, 4, 4, 3), (37, 5, 1, 1), (16, 16, 4, 4)])
def test_router_chooses_among_the_best_groups(E, top, count, keep):
    from llm_b200.csrc import ops
    g = torch.Generator().manual_seed(E * 10 + top)
    T, W = 50, 24
    h = bf(torch.randn(T, W, generator=g))
    p = {"router": bf(torch.randn(E, W, generator=g) * 0.5), "correction": bf(torch.randn(E, generator=g) * 0.5 - 0.6)}
    r = {"experts": E, "top": top, "groups": {"count": count, "keep": keep}}
    ids_ref, w_ref, margin = P.route(h.double(), {k: v.double() for k, v in p.items()}, r)
    logits = torch.empty(T, E, device="cuda")
    ids = torch.empty(T * top, dtype=torch.int32, device="cuda")
    wts = torch.empty(T * top, device="cuda")
    ops.moe_route(dev(h), dev(p["router"]), dev(p["correction"]), logits, ids, wts, T, top, sigmoid_groups=(count, keep))
    ids, wts = ids.view(T, top).cpu().long(), wts.view(T, top).cpu()
    clear = margin > 1e-4
    assert int(clear.sum()) > T // 2
    assert torch.equal(ids[clear], ids_ref[clear])
    assert max_err(wts[clear], w_ref[clear]) < 1e-5
    assert bool((P.route(h.double(), {k: v.double() for k, v in p.items()}, r)[0] >= 0).all())


def _gate_scan_inputs(T, H, D, V, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    q, v = bf(torch.randn(T, H * D, generator=g)), bf(torch.randn(T, H * V, generator=g))
    z = torch.randn(T, H * D, generator=g) * 2
    zb, low = torch.randn(H * D, generator=g), torch.rand(H * D, generator=g) * 0.9
    return q, v, z, zb, low


def _plain_gate_scan(q, v, z, zb, low, H, D, V, S=None):
    T = q.shape[0]
    q, v, z = P.silu(q.double()).view(T, H, D), v.double().view(T, H, V), z.double()
    f = (low.double() + (1 - low.double()) * torch.sigmoid(z + zb.double())).view(T, H, D)
    S = torch.zeros(H, D, V, dtype=torch.float64) if S is None else S.clone()
    out = torch.zeros(T, H, V, dtype=torch.float64)
    for t in range(T):
        S = f[t].unsqueeze(-1) * S + (1 - f[t]).unsqueeze(-1) * v[t].unsqueeze(1)
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out.reshape(T, H * V), S


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,V", [(1, 4, 4), (2, 16, 24), (3, 10, 6), (2, 48, 64), (5, 64, 32), (1, 100, 130), (2, 256, 8)])
def test_forget_gate_recurrence_in_steps_equals_the_plain_loop(dtype, H, D, V):
    """Whole, in portions through other slots, beside single tokens of another request, and as segments of a long step."""
    from llm_b200.csrc import ops
    T = 300
    q, v, z, zb, low = _gate_scan_inputs(T, H, D, V, H * 1000 + D, dtype)
    ref, _ = _plain_gate_scan(q, v, z, zb, low, H, D, V)
    qd, vd, zd, zbd, lowd = dev(q, dtype), dev(v, dtype), dev(z), dev(zb), dev(low)
    state = torch.zeros(4, H * D * V, device="cuda")
    out = torch.empty(T, H * V, device="cuda")
    other = torch.empty(1, H * V, device="cuda")
    for a, b in split_steps(T, (40, 1, 2, 17, 1, 64, 5)):
        # the request in slot 2, a single token of another request (slot 0) in front of it
        ctx = step_ctx([1, b - a], [0, 2])
        cat = lambda t: torch.cat([t[:1], t[a:b]]).contiguous()
        o = torch.empty(1 + b - a, H * V, device="cuda")
        ops.gate_scan(o, cat(qd), cat(vd), cat(zd), zbd, lowd, state, ctx, H, D, V)
        out[a:b] = o[1:]
    assert max_err(out, ref) < 2e-5
    assert float(state[1].abs().max()) == 0 and float(state[3].abs().max()) == 0
    # one long step: segments side by side in two passes
    state.zero_()
    ctx = step_ctx([T], [1])
    seg_state = torch.zeros((T // 64 + 1) * H * D * V, device="cuda")
    seg_decay = torch.zeros((T // 64 + 1) * H * D, device="cuda")
    ops.gate_scan(out, qd, vd, zd.clone(), zbd, lowd, state, ctx, H, D, V, seg_len=64, seg_state=seg_state, seg_decay=seg_decay)
    assert max_err(out, ref) < 2e-5


def _plain_delta(q, k, v, b, a, a_log, dt_bias, H, G, D, V):
    T = q.shape[0]
    unit = lambda x: x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)
    q, k, v = unit(q.double().view(T, G, D)) * D ** -0.5, unit(k.double().view(T, G, D)), v.double().view(T, H, V)
    beta = torch.sigmoid(b.double())
    decay = torch.exp(-torch.exp(a_log.double()) * P.softplus(a.double() + dt_bias.double()))
    S = torch.zeros(H, D, V, dtype=torch.float64)
    out = torch.zeros(T, H, V, dtype=torch.float64)
    for t in range(T):
        for h in range(H):
            g = h // (H // G)
            Sh = decay[t, h] * S[h]
            u = beta[t, h] * (v[t, h] - Sh.T @ k[t, g])
            S[h] = Sh + torch.outer(k[t, g], u)
            out[t, h] = S[h].T @ q[t, g]
    return out.reshape(T, H * V)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,V", [(1, 1, 4, 4), (4, 2, 16, 8), (3, 3, 12, 10), (4, 1, 64, 32), (2, 2, 100, 36), (2, 1, 128, 64), (1, 1, 256, 5),
                                     (6, 2, 8, 130)])
def test_delta_rule_in_steps_equals_the_plain_loop(dtype, H, G, D, V):
    from llm_b200.csrc import ops
    T = 150
    g = torch.Generator().manual_seed(H * 1000 + D)
    q, k = bf(torch.randn(T, G * D, generator=g)), bf(torch.randn(T, G * D, generator=g))
    v = bf(torch.randn(T, H * V, generator=g))
    b, a = bf(torch.randn(T, H, generator=g)), bf(torch.randn(T, H, generator=g))
    a_log, dt_bias = torch.randn(H, generator=g) * 0.7 - 1.0, torch.randn(H, generator=g) - 1.0
    ref = _plain_delta(q, k, v, b, a, a_log, dt_bias, H, G, D, V)
    qk, ba = dev(torch.cat([q, k], dim=1), dtype), dev(torch.cat([b, a], dim=1), dtype)
    vd = dev(v, dtype)
    state = torch.zeros(4, H * D * V, device="cuda")
    out = torch.empty(T, H * V, device="cuda")
    for s, e in split_steps(T, (40, 1, 2, 17, 1, 33)):
        ctx = step_ctx([1, e - s], [3, 1])
        cat = lambda t: torch.cat([t[:1], t[s:e]]).contiguous()
        qk_s, ba_s = cat(qk), cat(ba)
        o = torch.empty(1 + e - s, H * V, device="cuda")
        ops.delta_scan(o, qk_s[:, :G * D], qk_s[:, G * D:], cat(vd), ba_s[:, :H], ba_s[:, H:], dev(a_log), dev(dt_bias), state, ctx,
                       H, G, D, V, D ** -0.5)
        out[s:e] = o[1:]
    assert max_err(out, ref) < 3e-5
    assert float(state[0].abs().max()) == 0 and float(state[2].abs().max()) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,V", [(1, 1, 4, 4), (4, 2, 16, 8), (3, 3, 12, 10), (4, 1, 64, 32), (2, 2, 100, 36), (2, 1, 128, 64), (1, 1, 256, 5),
                                     (6, 2, 8, 130)])
def test_delta_rule_chunk_by_chunk_equals_the_plain_loop(dtype, H, G, D, V):
    """A step of three entries (one token, a portion off every chunk border, a long portion) from non-zero states."""
    from llm_b200.csrc import ops
    lens, T0 = [1, 77, 300], 40
    g = torch.Generator().manual_seed(H * 1000 + D + 7)
    a_log, dt_bias = torch.randn(H, generator=g) * 0.7 - 1.0, torch.randn(H, generator=g) - 1.0
    state = torch.zeros(4, H * D * V, device="cuda")
    seqs, refs = [], []
    for e, n in enumerate(lens):       # every entry: T0 earlier tokens token by token (the state it starts from), then the step
        T = T0 + n
        q, k = bf(torch.randn(T, G * D, generator=g)), bf(torch.randn(T, G * D, generator=g))
        v = bf(torch.randn(T, H * V, generator=g))
        b, a = bf(torch.randn(T, H, generator=g)), bf(torch.randn(T, H, generator=g))
        refs.append(_plain_delta(q, k, v, b, a, a_log, dt_bias, H, G, D, V)[T0:])
        seqs.append((q, k, v, b, a))
        ctx = step_ctx([T0], [e + 1])
        ops.delta_scan(torch.empty(T0, H * V, device="cuda"), dev(q[:T0], dtype), dev(k[:T0], dtype), dev(v[:T0], dtype), dev(b[:T0], dtype),
                       dev(a[:T0], dtype), dev(a_log), dev(dt_bias), state, ctx, H, G, D, V, D ** -0.5)
    cat = lambda i: dev(torch.cat([sq[i][T0:] for sq in seqs]), dtype)
    T = sum(lens)
    ctx = step_ctx(lens, [1, 2, 3])
    out = torch.empty(T, H * V, device="cuda")
    scratch = [torch.full((numel,), float("nan"), device="cuda") for numel in ops.delta_chunk_scratch(T // 32 + len(lens), H, D, V)]
    walked = state.clone()
    ops.delta_chunk_scan(out, cat(0), cat(1), cat(2), cat(3), cat(4), dev(a_log), dev(dt_bias), state, ctx, H, G, D, V, D ** -0.5, 1e-6, scratch)
    assert max_err(out, torch.cat(refs)) < 3e-5
    out2 = torch.empty(T, H * V, device="cuda")
    ops.delta_scan(out2, cat(0), cat(1), cat(2), cat(3), cat(4), dev(a_log), dev(dt_bias), walked, ctx, H, G, D, V, D ** -0.5)
    assert max_err(state, walked) < 3e-5 and float(state[0].abs().max()) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,V,share,page,window", [(4, 4, 16, 8, 2, 16, 0), (8, 4, 40, 80, 2, 16, 0), (6, 2, 10, 14, 1, 8, 19),
                                                       (8, 2, 64, 64, 1, 16, 80), (2, 2, 24, 16, 1, 32, 50), (12, 6, 64, 64, 2, 16, 0)])
def test_attention_with_distance_bias_shared_values_and_a_learned_sink(dtype, H, G, D, V, share, page, window):
    """The general kernel over shuffled pages against the formula: capped scores, r1 ln(1 + r2 distance) taken off, a sink
    with a learned score, a window; with share 2, neighbouring key heads read one value head and there is no bias."""
    from llm_b200.csrc import ops
    g = torch.Generator().manual_seed(H * 100 + D)
    T, cap, scale = 150, 20.0, 0.3
    q, k = bf(torch.randn(T, H, D, generator=g)), bf(torch.randn(T, G, D, generator=g))
    GV = G // share
    v = bf(torch.randn(T, GV, V, generator=g))
    r1, r2, sink = torch.rand(H, generator=g) + 0.2, torch.rand(H, generator=g) * 2, torch.randn(H, generator=g)
    n_pages = -(-T // page)
    perm = torch.randperm(n_pages + 3, generator=g)[:n_pages]
    k_pages = torch.full((n_pages + 3, G, page, D), 1e30).to(DT[dtype])
    v_pages = torch.full((n_pages + 3, GV, page, V), 1e30).to(DT[dtype])
    for t in range(T):
        k_pages[perm[t // page], :, t % page] = k[t].to(DT[dtype])
        v_pages[perm[t // page], :, t % page] = v[t].to(DT[dtype])
    biased = share == 1
    out = torch.empty(T, H * V, device="cuda", dtype=DT[dtype])
    ops.paged_attention_generic(out, dev(q.reshape(T, H * D), dtype), k_pages.cuda(), v_pages.cuda(), i32(perm.tolist()).view(1, -1),
                                i32([0] * T), i32(list(range(T))), T, H, G, D, window, scale, value_dim=V,
                                softcap=cap if biased else 0.0, sink=biased, sink_values=dev(sink) if biased else None,
                                dist_bias=(dev(r1), dev(r2)) if biased else None, v_share=share)
    dist = (torch.arange(T).unsqueeze(1) - torch.arange(T).unsqueeze(0)).double()
    seen = (dist >= 0) & ((dist < window) if window else torch.ones_like(dist, dtype=torch.bool))
    ref = torch.zeros(T, H, V, dtype=torch.float64)
    for h in range(H):
        kh = h // (H // G)
        s = (q[:, h].double() @ k[:, kh].double().T) * scale
        if biased:
            s = cap * torch.tanh(s / cap) - r1[h].double() * torch.log1p(r2[h].double() * dist.clamp(min=0))
        s = s.masked_fill(~seen, float("-inf"))
        if biased:
            s = torch.cat([s, sink[h].double().expand(T, 1)], dim=1)
        w = torch.softmax(s, dim=1)[:, :T]
        ref[:, h] = w @ v[:, kh // share].double()
    assert max_err(out, ref.reshape(T, H * V)) < KTOL[dtype]


@pytest.mark.parametrize("H,G,D,share,page,window", [(8, 2, 64, 1, 16, 80), (4, 2, 128, 1, 16, 0), (16, 4, 128, 1, 32, 300), (8, 8, 64, 2, 16, 0),
                                                     (8, 4, 128, 2, 16, 0), (2, 2, 64, 1, 64, 33)])
def test_fast_attention_kernels_take_the_distance_bias_and_shared_values(H, G, D, share, page, window):
    """The tcgen05 kernel on a prompt portion behind cached tokens, and the split-key kernel on single tokens of several
    requests, against the formula (bfloat16; values as wide as keys)."""
    from llm_b200.csrc import ops
    g = torch.Generator().manual_seed(H * 100 + D + share)
    T, cached, cap, scale = 400, 137, 20.0, 0.2
    q, k = bf(torch.randn(T, H, D, generator=g)), bf(torch.randn(T, G, D, generator=g))
    GV = G // share
    v = bf(torch.randn(T, GV, D, generator=g))
    r1, r2, sink = torch.rand(H, generator=g) + 0.2, torch.rand(H, generator=g) * 2, torch.randn(H, generator=g)
    n_pages = -(-T // page)
    perm = torch.randperm(n_pages + 3, generator=g)[:n_pages]
    k_pages = torch.zeros(n_pages + 3, G, page, D, dtype=torch.bfloat16)
    v_pages = torch.zeros(n_pages + 3, GV, page, D, dtype=torch.bfloat16)
    for t in range(T):
        k_pages[perm[t // page], :, t % page] = k[t].to(torch.bfloat16)
        v_pages[perm[t // page], :, t % page] = v[t].to(torch.bfloat16)
    biased = share == 1
    dist = (torch.arange(T).unsqueeze(1) - torch.arange(T).unsqueeze(0)).double()
    seen = (dist >= 0) & ((dist < window) if window else torch.ones_like(dist, dtype=torch.bool))
    ref = torch.zeros(T, H, D, dtype=torch.float64)
    for h in range(H):
        kh = h // (H // G)
        s = (q[:, h].double() @ k[:, kh].double().T) * scale
        if biased:
            s = cap * torch.tanh(s / cap) - r1[h].double() * torch.log1p(r2[h].double() * dist.clamp(min=0))
        s = s.masked_fill(~seen, float("-inf"))
        if biased:
            s = torch.cat([s, sink[h].double().expand(T, 1)], dim=1)
        ref[:, h] = torch.softmax(s, dim=1)[:, :T] @ v[:, kh // share].double()
    ref = ref.reshape(T, H * D)
    opts = dict(softcap=cap, sink=True, sink_values=dev(sink), dist_bias=(dev(r1), dev(r2))) if biased else dict(v_share=share)
    kd, vd, table = k_pages.cuda(), v_pages.cuda(), i32(perm.tolist()).view(1, -1)
    # a prompt portion of T - cached tokens behind `cached` tokens that the pages already hold
    out = torch.zeros(T - cached, H * D, device="cuda", dtype=torch.bfloat16)
    ops.attention_tc(out, dev(q.reshape(T, H * D)[cached:], "bfloat16"), kd, vd, table, i32([0, T - cached]), i32([T]), T - cached, 1,
                     H, G, D, window, scale, **opts)
    assert ops.attention_tc_take_error() == 0
    assert max_err(out, ref[cached:]) < 1.2e-2          # P is rounded to bfloat16 before the second product
    # single tokens: four requests over the same pages, at different lengths
    lens = [T, T - 19, 100, 3]
    rows = [n - 1 for n in lens]
    out = torch.zeros(4, H * D, device="cuda", dtype=torch.bfloat16)
    for splits in (1, 3, 8):
        ops.paged_attention_decode(out, dev(q.reshape(T, H * D)[rows], "bfloat16"), kd, vd, table.expand(4, -1).contiguous(), i32(lens), 4,
                                   H, G, D, window, scale, splits=splits, **opts)
        assert max_err(out, ref[rows]) < KTOL["bfloat16"]


# ---- whole models ---------------------------------------------------------------------
LENGTHS = {"A": [1, 5, 33, 70, 129], "B": [2, 47, 64, 150, 260], "C": [3, 40, 17, 90], "D": [1, 16, 31, 100], "E": [1, 130, 31, 257],
           "F": [2, 33, 140, 95], "G": [1, 2, 60, 75]}
MARGIN = 0.05      # bfloat16: a choice of experts (or of groups) that hangs on less than this may fall otherwise


def plain(cfg, w, toks, margins=None):
    return P.forward(cfg, {k: v.double() for k, v in w.items()}, toks, margins=margins)


def clear_rows(cfg, w, toks):
    """Rows before the first token whose routing is a close call: after it a bfloat16 engine may have chosen other experts,
    and every later token inherits the difference through attention or state."""
    margins = []
    plain(cfg, w, toks, margins=margins)
    if not margins:
        return len(toks)
    close = torch.nonzero(torch.stack(margins).min(dim=0).values < MARGIN).flatten()
    return int(close[0]) if close.numel() else len(toks)


@pytest.fixture(scope="module")
def models():
    cache = {}

    def get(name):
        if name not in cache:
            cfg, page = CONFIGS[name]
            w = make_weights(cfg, seed=ord(name), slow=3.0 if name == "F" else 0.0)
            reqs = {f"r{i}": random_tokens(n, cfg["vocab"], 300 + i) for i, n in enumerate(LENGTHS[name])}
            ref = {rid: plain(cfg, w, toks) for rid, toks in reqs.items()}
            upto = {rid: clear_rows(cfg, w, toks) for rid, toks in reqs.items()}
            cache[name] = (cfg, page, w, reqs, ref, upto)
        return cache[name]
    return get


def compare(got, ref, dtype, what, upto=None, tol=None, strict=None):
    """Every row's largest difference, relative to the request's largest logit, against the bound of the dtype.  float32:
    every row.  bfloat16: the rows before a request's first close routing call (upto), of which one in fifty (at least one) may
    pass the bound, up to half the largest logit; the rows named in `strict` may not."""
    tol = tol or TOL[dtype]
    for rid, r in ref.items():
        assert got[rid].shape == r.shape, f"{what}: {rid} shape {got[rid].shape} vs {r.shape}"
        err_rows = (got[rid].double() - r).abs().max(dim=1).values / r.abs().max()
        assert bool(torch.isfinite(err_rows).all()), f"{what}: request {rid} has rows that are not finite"
        if dtype == "bfloat16" and upto is not None:
            err_rows = err_rows[:upto[rid]]
            if not err_rows.numel():
                continue
        bad = torch.nonzero(~(err_rows <= tol)).flatten()
        first = f"{what}: request {rid} first differs at position {int(bad[0]) if bad.numel() else -1} " \
                f"(err {float(err_rows.max()):.3e} at most, limit {tol:.1e})"
        if strict:
            assert float(err_rows[strict].max()) <= tol, first
        if dtype == "float32":
            assert bad.numel() == 0, first
        else:
            assert bad.numel() <= max(1, len(err_rows) // 50) and float(err_rows.max()) <= 0.5, first


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_every_cut_matches_plain(models, name, dtype):
    cfg, page, w, reqs, ref, upto = models(name)
    longest = max(len(t) for t in reqs.values())
    eng = make_engine(cfg, w, dtype, page, -(-longest // page) + 1)       # a pool barely larger than the longest request
    compare(replay.run_steps(eng, replay.steps_whole(reqs)), ref, dtype, "whole", upto)
    compare(replay.run_steps(eng, replay.steps_tail_decode(reqs)), ref, dtype, "tail decode", upto)
    compare(replay.run_steps(eng, replay.steps_portions(reqs)), ref, dtype, "portions", upto)
    compare(replay.run_steps(eng, replay.steps_portions(reqs, sizes=(2, 2, 3, 2, 16, 2, 17, 64))), ref, dtype, "small portions", upto)
    eng.check_status()
    eng.cache.check()
    assert all(eng.cache.num_free_pages(g) == eng.cache.group_spec(g).num_pages for g in range(eng.cache.num_groups))
    lens = sorted((len(t) for t in reqs.values()), reverse=True)
    eng = make_engine(cfg, w, dtype, page, sum(-(-n // page) for n in lens[:4]) + 1)
    compare(replay.run_steps(eng, replay.steps_mixed(reqs)), ref, dtype, "mixed", upto)     # freed pages and slots are used again
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_batch_of_unequal_requests_equals_each_alone(models, name, dtype):
    from llm_b200.engine.engine import StepEntry
    cfg, page, w, reqs, ref, upto = models(name)
    eng = make_engine(cfg, w, dtype, page, 60)
    alone = replay.run_steps(eng, replay.steps_whole(reqs))
    entries = [StepEntry(rid, toks, list(range(len(toks)))) for rid, toks in reqs.items()][:4]
    rows = eng.step(entries).float().cpu()
    at = 0
    for e in entries:
        n = len(e.tokens)
        m = n if dtype == "float32" else upto[e.request_id]
        if m:
            assert max_err(rows[at:at + m], alone[e.request_id][:m]) < (1e-5 if dtype == "float32" else 2e-2)
        at += n
        eng.release(e.request_id)


def test_window_pages_go_back():
    """A request far longer than its window holds only the window's pages; the logits say they were the right ones."""
    cfg, page = CONFIGS["E"]
    w = make_weights(cfg, seed=5)
    toks = random_tokens(400, cfg["vocab"], 8)
    ref = {"x": plain(cfg, w, toks)}
    n_pages = 4
    eng = make_engine(cfg, w, "float32", page, n_pages + 3, max_tokens=48, max_seq_len=512)     # 400 tokens would need many more
    compare(replay.run_steps(eng, replay.steps_portions({"x": toks}, sizes=(40, 2, 31, 1, 16, 48))), ref, "float32", "portions")
    eng = make_engine(cfg, w, "float32", page, n_pages, max_tokens=48, max_seq_len=512)
    got = replay.run_steps(eng, replay.steps_tail_decode({"x": toks[:300]}, tail=299))      # token by token
    compare(got, {"x": ref["x"][:300]}, "float32", "decode")
    eng.cache.check()


# ---- keys at the edges: what a row would be if the mask were one token off, on the plain side --------------------------
def _window_model(size, page_hint=16, peak=6.0):
    """The windowed attention alone (the delta rule beside it is scaled by zero, there is no feed-forward), peaked."""
    cfg = config(64, 90, 2, 2.0, [layer(parallel(2, 1, 16, 16, size=size, scale=0.25, softcap=40.0, conv=2, r_heads=1, r_kv=1, r_dim=8,
                                                 r_vdim=8, r_conv=2, left_scale=1.0, right_scale=0.0), None)])
    w = make_weights(cfg, seed=size, peak=peak)
    w["l0.mix.left.r1"] = w["l0.mix.left.r1"] * 0.1      # a weak distance bias: the oldest visible key can still win a row
    return cfg, w


def _resize(cfg, size):
    c = copy.deepcopy(cfg)
    c["layers"][0]["mixer"]["left"]["mask"]["size"] = size
    return c


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size,page", [(16, 16), (17, 16), (15, 16), (33, 8), (80, 16), (50, 32), (2, 16)])
def test_the_oldest_key_of_the_window_is_seen_and_the_one_before_it_is_not(dtype, size, page):
    cfg, w = _window_model(size)
    T = 260 + 4 * size          # the wider the window, the fewer rows its oldest key wins
    toks = random_tokens(T, cfg["vocab"], size)
    ref = plain(cfg, w, toks)
    smaller, larger = plain(_resize(cfg, size - 1), w, toks), plain(_resize(cfg, size + 1), w, toks)
    top = ref.abs().max()
    inside = torch.nonzero(((ref - smaller).abs().max(dim=1).values / top > 0.12)).flatten()      # rows that the edge key carries
    outside = torch.nonzero(((ref - larger).abs().max(dim=1).values / top > 0.12)).flatten()      # rows one more key would change
    assert inside.numel() >= 2 and outside.numel() >= 2, "premise: some rows hang on the key at the edge"
    strict = sorted(set(inside.tolist() + outside.tolist()))
    eng = make_engine(cfg, w, dtype, page, -(-T // page) + 2, max_tokens=T)
    reqs, want = {"x": toks}, {"x": ref}
    compare(replay.run_steps(eng, replay.steps_whole(reqs)), want, dtype, "whole", strict=strict)
    compare(replay.run_steps(eng, replay.steps_tail_decode(reqs, tail=150)), want, dtype, "decode", strict=strict)
    compare(replay.run_steps(eng, replay.steps_portions(reqs, sizes=(7, 2, 13, 3, 2, 29)), ), want, dtype, "portions", strict=strict)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sink_weighs_in_the_denominator_once(dtype):
    cfg, w = _window_model(40, peak=1.0)
    w["l0.mix.left.sink"] = torch.tensor([3.0, 2.0])          # far above the scores: most of the weight goes nowhere
    toks = random_tokens(120, cfg["vocab"], 4)
    ref = plain(cfg, w, toks)
    w0 = dict(w)
    w0["l0.mix.left.sink"] = torch.tensor([-1e4, -1e4])
    assert float((ref - plain(cfg, w0, toks)).abs().max() / ref.abs().max()) > 0.2, "premise: the sink matters"
    eng = make_engine(cfg, w, dtype, 16, 10)
    compare(replay.run_steps(eng, replay.steps_whole({"x": toks})), {"x": ref}, dtype, "whole")
    compare(replay.run_steps(eng, replay.steps_tail_decode({"x": toks}, tail=60)), {"x": ref}, dtype, "decode")


NEEDLE, QUERY = 7, 11


def _far_key_model(kv_heads):
    """A differential attention alone whose first map of head 0 sends the token QUERY to the token NEEDLE: the keys of that
    map are made by the query's own rows, and the needle's embedding is the query token's plus a direction that those rows do
    not see, so the pair scores what a vector scores against itself, several deviations above every other pair, while the
    needle's value is its own.  The embedding is small beside what the mixer writes."""
    cfg = config(64, 80, 2, 2.0, [layer(attention(2, kv_heads, 32, 16, 0.25, 0.3), None)])
    w = make_weights(cfg, seed=11 + kv_heads, peak=5.0)
    w["embed"] = w["embed"] * 0.125
    w["l0.mix.k"][:32] = w["l0.mix.q"][:32]
    w["l0.canon1"] = w["l0.canon1"] * 0.25          # the neighbour's share of a row stays small
    w["l0.norm1"] = torch.ones(64)
    _, _, vh = torch.linalg.svd(w["l0.mix.q"][:32].double())
    hidden = (vh[32:].T @ torch.randn(32, dtype=torch.float64, generator=torch.Generator().manual_seed(1))).float()
    w["embed"][NEEDLE] = (w["embed"][QUERY] + 1.5 * hidden * w["embed"][QUERY].norm() / hidden.norm()).to(torch.bfloat16).float()
    return cfg, w


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kv_heads", [1, 2])
def test_differential_attention_finds_a_key_hundreds_of_tokens_back(dtype, kv_heads):
    """One NEEDLE near the start, QUERY tokens hundreds of tokens later; the rows of the queries change when the needle is
    exchanged (plain side), and those are the strict ones."""
    cfg, w = _far_key_model(kv_heads)
    T, p, asks = 700, 5, [400, 699]
    toks = [t if t not in (NEEDLE, QUERY) else t + 20 for t in random_tokens(T, cfg["vocab"], 3)]
    toks[p] = NEEDLE
    for i in asks:
        toks[i] = QUERY
    other = list(toks)
    other[p] = 33
    ref, ref_other = plain(cfg, w, toks), plain(cfg, w, other)
    moved = (ref - ref_other).abs().max(dim=1).values / ref.abs().max()
    assert float(moved[asks].min()) > 0.06, "premise: the far rows hang on the exchanged token"
    tol = None if dtype == "float32" else 3e-2
    eng = make_engine(cfg, w, dtype, 16, -(-T // 16) + 1, max_tokens=704)
    compare(replay.run_steps(eng, replay.steps_whole({"x": toks})), {"x": ref}, dtype, "whole", strict=asks, tol=tol)
    compare(replay.run_steps(eng, replay.steps_tail_decode({"x": toks}, tail=380)), {"x": ref}, dtype, "decode", strict=asks, tol=tol)
    compare(replay.run_steps(eng, replay.steps_portions({"x": toks}, sizes=(100, 2, 37, 128, 3)), ), {"x": ref}, dtype, "portions", strict=asks, tol=tol)
    compare(replay.run_steps(eng, replay.steps_whole({"y": other})), {"y": ref_other}, dtype, "exchanged", strict=asks, tol=tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["hgrn2", "delta"])
def test_state_remembers_a_token_from_hundreds_back(dtype, kind):
    """Slow decays; the request's state slot was another request's before; portions cut the sequence everywhere."""
    if kind == "hgrn2":
        cfg = config(48, 70, 2, 1.0, [layer(hgrn2(2, 16, 24), None)])
    else:
        cfg = config(48, 70, 2, 1.0, [layer(parallel(1, 1, 8, 8, size=4, scale=0.3, softcap=10.0, conv=2, r_heads=2, r_kv=1, r_dim=16,
                                                     r_vdim=24, r_conv=3, left_scale=0.0, right_scale=1.0), None)])
    w = make_weights(cfg, seed=9, slow=5.0)
    if kind == "delta":
        w["l0.mix.right.b"] = w["l0.mix.right.b"] * 0.0 - 0.0      # beta = 1/2 everywhere: every token writes
        w["l0.mix.right.dt_bias"] = torch.full((2,), -6.0)
        w["l0.mix.right.A_log"] = torch.full((2,), -3.0)
    T, p = 700, 20
    toks = random_tokens(T, cfg["vocab"], 5)
    other = list(toks)
    other[p] = (toks[p] + 9) % cfg["vocab"]
    ref, ref_other = plain(cfg, w, toks), plain(cfg, w, other)
    moved = (ref - ref_other).abs().max(dim=1).values / ref.abs().max()
    assert float(moved[650:].max()) > 1e-3, "premise: the state still holds the exchanged token"      # float32 sees 3e-5
    eng = make_engine(cfg, w, dtype, 16, 50, max_tokens=128, max_seqs=2)
    first = replay.run_steps(eng, replay.steps_whole({"warm": random_tokens(90, cfg["vocab"], 1)}))      # uses and frees a slot
    got = replay.run_steps(eng, replay.steps_portions({"x": toks}, sizes=(100, 2, 64, 1, 128, 31)))
    tol = None if dtype == "float32" else 8e-2
    compare(got, {"x": ref}, dtype, "portions", tol=tol)
    got = replay.run_steps(eng, replay.steps_portions({"y": other}, sizes=(128,)))
    compare(got, {"y": ref_other}, dtype, "exchanged", tol=tol)
    assert first["warm"].shape[0] == 90


def test_a_slot_that_is_used_again_starts_from_zero(models):
    cfg, page, w, reqs, ref, upto = models("A")
    eng = make_engine(cfg, w, "float32", page, 40, max_seqs=1)           # one slot: every request takes the same one
    for _ in range(2):
        compare(replay.run_steps(eng, replay.steps_whole(reqs)), ref, "float32", "whole, one slot")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_long_decode_with_graphs_and_first_tokens(models, name, dtype):
    """One prompt token, then 210 decoded one by one under CUDA graphs, beside a second request that joins late."""
    cfg, page = CONFIGS[name]
    w = make_weights(cfg, seed=77)
    toks, late = random_tokens(211, cfg["vocab"], 21), random_tokens(40, cfg["vocab"], 22)
    ref = {"x": plain(cfg, w, toks), "late": plain(cfg, w, late)}
    upto = {"x": clear_rows(cfg, w, toks), "late": clear_rows(cfg, w, late)}
    eng = make_engine(cfg, w, dtype, page, 40, graphs=True)
    steps = []
    for i in range(len(toks)):
        entries = [{"id": "x", "tokens": toks[i:i + 1], "want": [0]}]
        j = i - 100
        if 0 <= j < len(late):
            entries.append({"id": "late", "tokens": late[j:j + 1], "want": [0]})
        steps.append({"entries": entries, "end": []})
    steps[-1]["end"] = ["x", "late"]
    compare(replay.run_steps(eng, steps), ref, dtype, "decode from the first token", upto)
    eng.check_status()


def test_prefill_equals_token_by_token_from_the_first_token(models):
    for name in ("A", "E", "G"):
        cfg, page = CONFIGS[name]
        w = make_weights(cfg, seed=31)
        toks = random_tokens(70, cfg["vocab"], 6)
        eng = make_engine(cfg, w, "float32", page, 20)
        whole = replay.run_steps(eng, replay.steps_whole({"x": toks}))["x"]
        single = replay.run_steps(eng, replay.steps_tail_decode({"x": toks}, tail=69))["x"]
        assert max_err(single, whole) < 2e-5


def _plain_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(plain(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]


def test_greedy_generation_through_the_scheduler():
    """LLM.generate: the scheduler admits, batches, pages and samples; greedy tokens equal the plain implementation's."""
    from llm_b200 import LLM
    cfg, page = CONFIGS["A"]
    w = make_weights(cfg, seed=41)
    prompts = [random_tokens(n, cfg["vocab"], 500 + n) for n in (1, 9, 30, 47, 18)]
    llm = LLM(None, dtype="float32", max_num_seqs=3, max_num_batched_tokens=16, kv_block_size=page, num_kv_blocks=14,
              eos_token_id=-1, random_config=cfg, tensors={k: v.clone() for k, v in w.items()}, max_seq_len=128)
    got = llm.generate(prompts, max_new_tokens=16)
    for p, g in zip(prompts, got):
        assert g == _plain_greedy(cfg, w, p, 16)
    llm.engine.cache.check()


def test_trace_replay_of_a_folder(models, tmp_path):
    """The trace runner on a folder written to disk in bfloat16: steps in, logit files out."""
    import io
    import numpy as np
    from llm_b200.engine import trace
    from llm_b200.weights.safetensors_io import write_safetensors
    cfg, page = CONFIGS["B"]
    w = make_weights(cfg, seed=51)
    d = tmp_path / "model"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(d / "model.safetensors"), {k: v.to(torch.bfloat16) for k, v in w.items()})
    reqs = {"a": random_tokens(70, cfg["vocab"], 1), "b": random_tokens(45, cfg["vocab"], 2)}
    steps = replay.steps_mixed(reqs, max_live=2)
    lines = "\n".join(json.dumps({"step": i, "entries": s["entries"], "end": s["end"]}) for i, s in enumerate(steps))
    out, said = tmp_path / "out", io.StringIO()
    assert trace.main(["--model", str(d), "--dtype", "float32", "--out", str(out), "--max-tokens", "128"], stdin=io.StringIO(lines),
                      stdout=said) == 0
    assert said.getvalue().split() == [x for i in range(len(steps)) for x in ("done", str(i))]
    rows = {}
    for i, s in enumerate(steps):
        got = torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"]).copy())
        at = 0
        for e in s["entries"]:
            rows.setdefault(e["id"], []).append(got[at:at + len(e["want"])])
            at += len(e["want"])
    got = {rid: torch.cat(parts) for rid, parts in rows.items()}
    compare(got, {rid: plain(cfg, w, toks) for rid, toks in reqs.items()}, "float32", "trace replay")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(10))
def test_seeded_random_configurations(seed, dtype):
    cfg = random_config(seed)
    page = [8, 16, 32][seed % 3]
    w = make_weights(cfg, seed=1000 + seed)
    reqs = {f"r{i}": random_tokens(n, cfg["vocab"], seed * 10 + i) for i, n in enumerate([1, 37, 120, 64])}
    ref = {rid: plain(cfg, w, toks) for rid, toks in reqs.items()}
    upto = {rid: clear_rows(cfg, w, toks) for rid, toks in reqs.items()}
    tol = 1e-4 if dtype == "float32" else 8e-2          # corner sizes and harsh constants among the drawn ones
    eng = make_engine(cfg, w, dtype, page, -(-120 // page) + 1)
    compare(replay.run_steps(eng, replay.steps_whole(reqs)), ref, dtype, f"seed {seed} whole", upto, tol=tol)
    compare(replay.run_steps(eng, replay.steps_tail_decode(reqs, tail=20)), ref, dtype, f"seed {seed} tail decode", upto, tol=tol)
    eng = make_engine(cfg, w, dtype, page, sum(-(-n // page) for n in (37, 120, 64)) + 2)
    compare(replay.run_steps(eng, replay.steps_mixed(reqs)), ref, dtype, f"seed {seed} mixed", upto, tol=tol)
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(4))
def test_seeded_configurations_of_layer_like_sizes(seed, dtype):
    cfg = random_config(100 + seed, large=True)
    w = make_weights(cfg, seed=2000 + seed)
    reqs = {f"r{i}": random_tokens(n, cfg["vocab"], seed * 10 + i) for i, n in enumerate([150, 40, 300])}
    ref = {rid: plain(cfg, w, toks) for rid, toks in reqs.items()}
    upto = {rid: clear_rows(cfg, w, toks) for rid, toks in reqs.items()}
    tol = 1e-4 if dtype == "float32" else 8e-2
    eng = make_engine(cfg, w, dtype, 16, 40)
    compare(replay.run_steps(eng, replay.steps_whole(reqs)), ref, dtype, f"seed {seed} whole", upto, tol=tol)
    compare(replay.run_steps(eng, replay.steps_mixed(reqs, prefill_sizes=(64, 2, 130, 17))), ref, dtype, f"seed {seed} mixed", upto, tol=tol)
    eng.check_status()
