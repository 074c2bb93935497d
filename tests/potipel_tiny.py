"""Tiny Potipel configurations and weights for the tests.

The configurations differ from each other in every size and constant and include the corner values: convolutions of one
tap (none at all) and of many, one head, as many kv heads as query heads and fewer, key and value sizes that differ,
windows smaller than a page, larger, off every page border and larger than any request, one expert chosen and all of
them, one group and as many groups as experts, layers that use an earlier layer's tensors, layers without a feed-forward,
sizes off every grid of 8.  The weights are drawn here (not by the package), with queries scaled so that attention is
peaked, decays spread between fast and slow, every value representable in bfloat16.
"""
from __future__ import annotations

import math

import torch


def attention(heads, kv_heads, dim, vdim, scale, diff):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}}


def hgrn2(heads, dim, vdim):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}}


def parallel(heads, kv_heads, dim, vdim, size, scale, softcap, conv, r_heads, r_kv, r_dim, r_vdim, r_conv, left_scale=0.7, right_scale=0.9):
    return {"type": "parallel", "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap, "conv": conv,
                 "mask": {"size": size}},
        "right": {"heads": r_heads, "kv_heads": r_kv, "dim": r_dim, "vdim": r_vdim, "conv": r_conv},
        "left_scale": left_scale, "right_scale": right_scale}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, limit, experts, top, count, keep):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}


def layer(mixer, mlp, weights_of=None):
    out = dict(mixer, mlp=mlp)
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def config(width, vocab, taps, scale, layers, eps=1e-5):
    return {"architecture": "Potipel", "width": width, "vocab": vocab, "norm": {"eps": eps}, "embedding": {"scale": scale},
            "canon": {"taps": taps}, "layers": layers}


_A0 = layer(attention(4, 2, 16, 8, 0.3, 0.4), dense(40))
_A2 = layer(parallel(4, 2, 16, 8, size=12, scale=0.25, softcap=20.0, conv=3, r_heads=4, r_kv=2, r_dim=16, r_vdim=8, r_conv=2),
            moe(24, 1.0, 6, 2, 3, 2))
# A: every mixer and both feed-forwards; a window inside one page; two layers that run an earlier layer's tensors again
CONFIG_A = config(64, 200, 3, 4.0, [
    _A0,
    layer(hgrn2(2, 16, 24), moe(16, 2.0, 4, 1, 2, 1)),
    _A2,
    layer(_A0, _A0["mlp"], weights_of=0),
    layer(_A2, _A2["mlp"], weights_of=2),
], eps=1e-5)
# B: sizes the tensor-core kernels take; a window across pages; fewer kv heads than heads everywhere
CONFIG_B = config(128, 333, 4, 8.0, [
    layer(parallel(8, 2, 64, 64, size=33, scale=0.125, softcap=30.0, conv=4, r_heads=4, r_kv=1, r_dim=64, r_vdim=32, r_conv=3,
                   left_scale=1.2, right_scale=0.5), dense(64)),
    layer(attention(4, 1, 64, 64, 0.125, 0.7), moe(64, 1.5, 8, 2, 4, 2)),
    layer(hgrn2(4, 32, 64), dense(128)),
    layer(attention(2, 2, 128, 128, 0.09, 0.2), None),
], eps=1e-6)
# C: nothing on a grid of 8; convolutions of one tap (they change nothing or scale); one expert chosen; groups of one
CONFIG_C = config(100, 97, 1, 1.0, [
    layer(attention(3, 3, 10, 14, 0.35, 0.5), moe(14, 0.8, 5, 1, 5, 2)),
    layer(hgrn2(3, 10, 6), dense(22)),
    layer(parallel(5, 5, 6, 14, size=19, scale=0.4, softcap=8.0, conv=1, r_heads=3, r_kv=3, r_dim=12, r_vdim=10, r_conv=1), dense(10)),
], eps=3e-6)
# D: a differential attention alone, without a feed-forward: what the attention does shows in the logits undiluted
CONFIG_D = config(64, 120, 2, 2.0, [layer(attention(2, 1, 32, 16, 0.25, 0.3), None)])
# E: the windowed attention beside the delta rule, alone; a window of several pages that ends off their borders
CONFIG_E = config(48, 150, 4, 3.0, [
    layer(parallel(2, 1, 24, 16, size=50, scale=0.2, softcap=15.0, conv=5, r_heads=2, r_kv=1, r_dim=20, r_vdim=12, r_conv=4), None)])
# F: recurrences only, long memories; every expert chosen; one group; a long input convolution
CONFIG_F = config(56, 130, 7, 0.5, [layer(hgrn2(2, 24, 8), moe(16, 4.0, 3, 3, 1, 1)), layer(hgrn2(7, 8, 8), None),
                                     layer(hgrn2(2, 24, 8), moe(16, 4.0, 3, 3, 1, 1), weights_of=0)])
# G: a window of one token and a window no request reaches
CONFIG_G = config(72, 90, 2, 5.0, [
    layer(parallel(3, 1, 8, 8, size=1, scale=0.5, softcap=5.0, conv=2, r_heads=1, r_kv=1, r_dim=40, r_vdim=36, r_conv=2), dense(24)),
    layer(parallel(2, 2, 16, 4, size=5000, scale=0.3, softcap=50.0, conv=3, r_heads=6, r_kv=2, r_dim=8, r_vdim=4, r_conv=6), None)])

CONFIGS = {"A": (CONFIG_A, 16), "B": (CONFIG_B, 16), "C": (CONFIG_C, 8), "D": (CONFIG_D, 16), "E": (CONFIG_E, 32),
           "F": (CONFIG_F, 16), "G": (CONFIG_G, 16)}   # name -> (config, page size)


def make_weights(cfg: dict, seed: int, peak: float = 1.5, slow: float = 0.0) -> dict:
    """Seeded weights by tensor name.  peak: the standard deviation the attention scores are scaled to; slow: shifts the
    recurrences' decays toward one (larger: longer memory)."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    rnd = lambda *shape, std=1.0, mean=0.0: (mean + torch.randn(tuple(shape), generator=g) * std).to(torch.bfloat16).float()
    gain = lambda *shape: rnd(*shape, std=0.1, mean=1.0)
    w = {"embed": rnd(cfg["vocab"], W, std=1.0 / cfg["embedding"]["scale"]), "head": rnd(cfg["vocab"], W, std=2.0 / math.sqrt(W)),
         "final.norm": gain(W)}
    for i, lay in enumerate(cfg["layers"]):
        if lay.get("weights_of") is not None:
            continue
        p, m, kind = f"l{i}", lay["mixer"], lay["type"]
        for q in (1, 2) if lay["mlp"] is not None else (1,):
            w[f"{p}.norm{q}"] = gain(W)
            w[f"{p}.canon{q}"] = rnd(W, cfg["canon"]["taps"], std=0.3)
        x = p + ".mix."
        if kind == "attention":
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[x + "q"] = rnd(2 * H * D, W, std=1.0 / math.sqrt(W))
            w[x + "k"] = rnd(2 * G * D, W, std=1.0 / math.sqrt(W))
            w[x + "v"] = rnd(G * V, W, std=1.0 / math.sqrt(W))
            w[x + "q.norm"] = rnd(D, std=0.1, mean=peak / (m["scale"] * math.sqrt(D)))
            w[x + "k.norm"] = gain(D)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                w[x + n] = rnd(D, std=0.6 / math.sqrt(D))
            w[x + "g"] = rnd(H * V, W, std=1.5 / math.sqrt(W))
            w[x + "o"] = rnd(W, H * V, std=1.0 / math.sqrt(H * V))
        elif kind == "hgrn2":
            H, D, V = m["heads"], m["dim"], m["vdim"]
            w[x + "q"] = rnd(H * D, W, std=1.5 / math.sqrt(W))
            w[x + "f"] = rnd(H * D, W, std=1.5 / math.sqrt(W))
            w[x + "f.b"] = rnd(H * D, std=1.0, mean=1.0 + slow)
            w[x + "lower"] = (torch.rand(H * D, generator=g) * 0.9).to(torch.bfloat16).float()
            w[x + "v"] = rnd(H * V, W, std=1.0 / math.sqrt(W))
            w[x + "norm"] = gain(V)
            w[x + "o"] = rnd(W, H * V, std=1.0 / math.sqrt(H * V))
        else:
            a, b = m["left"], m["right"]
            H, G, D, V, taps = a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["conv"]
            y = x + "left."
            w[y + "q"] = rnd(H * D, W, std=peak / (a["scale"] * math.sqrt(D)) / math.sqrt(W))
            w[y + "k"] = rnd(G * D, W, std=1.0 / math.sqrt(W))
            w[y + "v"] = rnd(G * V, W, std=1.0 / math.sqrt(W))
            for n, c in (("q", H * D), ("k", G * D), ("v", G * V)):
                w[y + n + ".b"] = rnd(c, std=0.2)
                conv = rnd(c, taps, std=0.3)
                conv[:, -1] += 1.0          # the current token's tap carries most of the weight
                w[y + n + ".conv"] = conv.to(torch.bfloat16).float()
            w[y + "r1"] = rnd(H, std=0.3, mean=0.5)
            w[y + "r2"] = (torch.rand(H, generator=g) * 2.0 + 0.05).to(torch.bfloat16).float()
            w[y + "sink"] = rnd(H, std=1.0, mean=0.5)
            w[y + "o"] = rnd(W, H * V, std=1.0 / math.sqrt(H * V))
            H, G, D, V, taps = b["heads"], b["kv_heads"], b["dim"], b["vdim"], b["conv"]
            y = x + "right."
            w[y + "q"] = rnd(G * D, W, std=1.5 / math.sqrt(W))
            w[y + "k"] = rnd(G * D, W, std=1.5 / math.sqrt(W))
            w[y + "v"] = rnd(H * V, W, std=1.5 / math.sqrt(W))
            for n, c in (("q", G * D), ("k", G * D), ("v", H * V)):
                conv = rnd(c, taps, std=0.3)
                conv[:, -1] += 1.0
                w[y + n + ".conv"] = conv.to(torch.bfloat16).float()
            w[y + "b"] = rnd(H, W, std=1.5 / math.sqrt(W))
            w[y + "a"] = rnd(H, W, std=1.0 / math.sqrt(W))
            w[y + "A_log"] = rnd(H, std=0.7, mean=-slow)
            w[y + "dt_bias"] = rnd(H, std=1.0, mean=-1.0 - slow)
            w[y + "g"] = rnd(H * V, W, std=1.5 / math.sqrt(W))
            w[y + "norm"] = gain(V)
            w[y + "o"] = rnd(W, H * V, std=1.0 / math.sqrt(H * V))
        ff = lay["mlp"]
        if ff is None:
            continue
        y = p + ".mlp."
        if ff["kind"] == "dense":
            F = ff["ff"]
            w[y + "gate"] = rnd(F, W, std=1.5 / math.sqrt(W))
            w[y + "up"] = rnd(F, W, std=1.5 / math.sqrt(W))
            w[y + "down"] = rnd(W, F, std=1.0 / math.sqrt(F))
            continue
        F, L, E = ff["expert"]["ff"], ff["expert"]["limit"], ff["router"]["experts"]
        for e in range(E):      # pre-activations of about the limit's size, so that all three clamps cut
            w[f"{y}e{e}.gate"] = rnd(F, W, std=1.2 * L / math.sqrt(W))
            w[f"{y}e{e}.up"] = rnd(F, W, std=1.2 * L / math.sqrt(W))
            w[f"{y}e{e}.down"] = rnd(W, F, std=1.0 / math.sqrt(F))
        w[y + "router"] = rnd(E, W, std=2.0 / math.sqrt(W))
        w[y + "correction"] = rnd(E, std=0.4)          # large enough to change choices and to make choice scores negative
    return w


def random_config(seed: int, large: bool = False) -> dict:
    """Sizes, constants and layer order drawn from a seed.  large: sizes of some hundreds with heads of 32 to 128."""
    import random
    rng = random.Random(seed)
    pick = rng.choice
    width = pick([192, 256, 320, 384]) if large else pick([40, 56, 72, 88, 100, 128, 136])
    dims = [32, 64, 128] if large else [4, 8, 10, 16, 24, 32, 48, 64]
    vdims = [32, 64, 128] if large else [4, 8, 12, 16, 20, 32, 64]
    layers = []
    for n in range(rng.randint(2, 5)):
        if layers and rng.random() < 0.2:
            src = pick([i for i, l in enumerate(layers) if l.get("weights_of") is None])
            layers.append(dict(layers[src], weights_of=src))
            continue
        kind = rng.random()
        if kind < 0.33:
            kv = pick([1, 2, 3])
            mixer = attention(kv * rng.randint(1, 3), kv, pick(dims), pick(vdims), rng.uniform(0.05, 0.5), rng.uniform(0.1, 0.8))
        elif kind < 0.6:
            mixer = hgrn2(rng.randint(1, 6), pick(dims), pick(vdims))
        else:
            kv, r_kv = pick([1, 2, 4]), pick([1, 2, 3])
            mixer = parallel(kv * rng.randint(1, 3), kv, pick(dims), pick(vdims), size=pick([1, 5, 16, 17, 50, 80, 300]),
                             scale=rng.uniform(0.05, 0.5), softcap=pick([5.0, 30.0, 50.0]), conv=rng.randint(1, 5),
                             r_heads=r_kv * rng.randint(1, 2), r_kv=r_kv, r_dim=pick(dims), r_vdim=pick(vdims), r_conv=rng.randint(1, 5),
                             left_scale=rng.uniform(0.3, 1.5), right_scale=rng.uniform(0.3, 1.5))
        r = rng.random()
        if r < 0.25:
            mlp = None
        elif r < 0.6:
            mlp = dense(pick([256, 344]) if large else pick([8, 12, 24, 40]))
        else:
            count = pick([1, 2, 3, 4])
            per = rng.randint(1, 3)
            keep = rng.randint(1, count)
            top = rng.randint(1, keep * per)
            mlp = moe(pick([64, 80]) if large else pick([8, 12, 20]), pick([0.5, 1.0, 7.0]), count * per, top, count, keep)
        layers.append(layer(mixer, mlp))
    return config(width, pick([61, 128, 200, 333]), rng.randint(1, 6), pick([0.5, 1.0, 4.0, 16.0]), layers, eps=pick([1e-6, 1e-5, 1e-3]))


def make_engine(cfg, weights, dtype, page, num_blocks, max_tokens=512, max_seqs=4, poison=True, graphs=False, max_seq_len=None):
    from llm_b200.config import EngineOptions
    from llm_b200.engine.engine import Engine
    opts = EngineOptions(dtype=dtype, kv_block_size=page, max_num_seqs=max_seqs, max_num_batched_tokens=max_tokens,
                         num_kv_blocks=num_blocks, use_cuda_graphs=graphs, poison_freed_pages=poison,
                         max_seq_len=max_seq_len or min(num_blocks * page, 4096))
    return Engine(None, opts, random_config=cfg, tensors={k: v.clone() for k, v in weights.items()})
