"""Tiny Norusun configurations and weights for the tests.

The configurations differ from each other in every size and constant and include the corner values: one stream and
several, a convolution of one tap (none at all) and of many, one head, as many kv heads as query heads, key and value
sizes that differ, rotation of the whole head and of part of it, windows and chunks smaller than a page, larger, and off
every page border, one group and as many groups as heads, one norm group, sizes off every grid of 8.  The weights are
drawn here (not by the package), with queries scaled so that attention is peaked and decays spread between fast and
slow, every value representable in bfloat16.
"""
from __future__ import annotations

import math

import torch


def wkv(heads, dim):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, size, scale, base=10000.0, rot_dims=None):
    return {"type": "latent_attention", "mixer": {
        "heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
        "mask": {"size": size}, "rot": {"dims": rot_dim if rot_dims is None else rot_dims, "base": base}}}


def parallel(heads, kv_heads, dim, vdim, chunk, rot_dims, scale, s_heads, s_vdim, state, groups, norm_groups, conv, base=10000.0):
    return {"type": "parallel", "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": chunk},
                 "rot": {"dims": rot_dims, "base": base}},
        "right": {"heads": s_heads, "vdim": s_vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}}}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def config(width, vocab, streams, taps, layers, eps=1e-5):
    return {"architecture": "Norusun", "width": width, "vocab": vocab, "norm": {"eps": eps}, "streams": streams,
            "canon": {"taps": taps}, "layers": layers}


# A: every mixer; a window and a chunk inside one page
CONFIG_A = config(64, 200, 2, 3, [
    layer(wkv(2, 16), None),
    layer(latent(4, 16, 8, 8, 24, 12, size=12, scale=0.3), dense(40, 2.0)),
    layer(parallel(4, 2, 16, 8, chunk=10, rot_dims=8, scale=0.25, s_heads=4, s_vdim=8, state=16, groups=2, norm_groups=2, conv=3),
          dense(24, 1.0)),
    layer(wkv(1, 40), dense(32, 0.7)),
], eps=1e-5)
# B: sizes the tensor-core kernels take; windows and chunks across pages; four streams
CONFIG_B = config(128, 333, 4, 4, [
    layer(latent(4, 32, 32, 32, 32, 48, size=33, scale=0.12, base=500000.0), dense(64, 1.5)),
    layer(parallel(8, 2, 64, 64, chunk=32, rot_dims=64, scale=0.125, s_heads=4, s_vdim=32, state=64, groups=1, norm_groups=1, conv=2),
          None),
    layer(wkv(4, 32), dense(128, 3.0)),
    layer(latent(2, 64, 64, 128, 64, 16, size=100, scale=0.09, rot_dims=32), None),
], eps=1e-6)
# C: nothing on a grid of 8; one stream and a convolution of one tap (both mechanisms then change nothing)
CONFIG_C = config(100, 97, 1, 1, [
    layer(latent(3, 10, 6, 14, 18, 7, size=7, scale=0.35, base=100.0), dense(14, 1.2)),
    layer(wkv(3, 10), dense(22, 2.5)),
    layer(parallel(5, 5, 6, 14, chunk=19, rot_dims=2, scale=0.4, s_heads=3, s_vdim=10, state=12, groups=3, norm_groups=5, conv=5),
          dense(10, 0.5)),
], eps=3e-6)
# D: a latent attention alone, without a feed-forward: what the attention does shows in the logits undiluted
CONFIG_D = config(64, 120, 3, 2, [layer(latent(2, 32, 8, 16, 40, 20, size=24, scale=0.25), None)])
# E: the chunked attention beside the state-space layer, alone
CONFIG_E = config(48, 150, 2, 4, [
    layer(parallel(2, 1, 24, 16, chunk=50, rot_dims=12, scale=0.2, s_heads=2, s_vdim=12, state=20, groups=1, norm_groups=3, conv=4), None)])
# F: recurrences only, long memories; eight streams and a long convolution
CONFIG_F = config(56, 130, 8, 7, [layer(wkv(2, 24), dense(16, 4.0)), layer(wkv(7, 8), None)])

CONFIGS = {"A": (CONFIG_A, 16), "B": (CONFIG_B, 16), "C": (CONFIG_C, 8), "D": (CONFIG_D, 16), "E": (CONFIG_E, 32),
           "F": (CONFIG_F, 16)}   # name -> (config, page size)


def make_weights(cfg: dict, seed: int, peak: float = 1.5, decay_rank: int = 6, slow: float = 0.0) -> dict:
    """Seeded weights by tensor name.  peak: the standard deviation the attention scores are scaled to; slow: taken off
    the decay's bias of the wkv layers and off the step's bias of the state-space layers (larger: longer memory)."""
    g = torch.Generator().manual_seed(seed)
    W, S = cfg["width"], cfg["streams"]
    rnd = lambda *shape, std=1.0, mean=0.0: (mean + torch.randn(tuple(shape), generator=g) * std).to(torch.bfloat16).float()
    gain = lambda *shape: rnd(*shape, std=0.1, mean=1.0)
    w = {"embed": rnd(cfg["vocab"], W), "head": rnd(cfg["vocab"], W, std=2.0 / math.sqrt(W)), "final.norm": gain()}
    for i, lay in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}", lay["mixer"], lay["type"]
        for q in (1, 2) if lay["mlp"] is not None else (1,):
            w[f"{p}.norm{q}"] = gain()
            w[f"{p}.hc{q}.in"] = rnd(S, std=0.3, mean=0.7)
            w[f"{p}.hc{q}.out"] = rnd(S, std=0.3, mean=0.8)
            w[f"{p}.hc{q}.mix"] = (0.8 * torch.eye(S) + 0.15 * torch.randn(S, S, generator=g)).to(torch.bfloat16).float()
        w[p + ".canon1"] = rnd(W, cfg["canon"]["taps"], std=0.3)
        x = p + ".mix."
        if kind == "wkv":
            H, D = m["heads"], m["dim"]
            for n in "rkvgw":
                w[x + "mu." + n] = rnd(W, std=0.25, mean=0.5)
            for n in "rkv":
                w[x + n] = rnd(H * D, W, std=1.0 / math.sqrt(W))
            w[x + "g"] = rnd(H * D, W, std=1.5 / math.sqrt(W))
            w[x + "w1"] = rnd(decay_rank, W, std=1.0 / math.sqrt(W))
            w[x + "w2"] = rnd(H * D, decay_rank, std=1.0 / math.sqrt(decay_rank))
            w[x + "w0"] = rnd(H * D, std=1.2, mean=-1.0 - slow)
            w[x + "u"] = rnd(H, D, std=0.5)
            w[x + "norm"] = gain(H * D)
            w[x + "o"] = rnd(W, H * D, std=1.0 / math.sqrt(H * D))
        elif kind == "latent_attention":
            H, D, R, V, C, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            w[x + "dq"] = rnd(Q, W, std=1.0 / math.sqrt(W))
            w[x + "dq.norm"] = gain(Q)
            w[x + "uq"] = rnd(H * (D + R), Q, std=peak / (m["scale"] * math.sqrt(D + R)) / math.sqrt(Q))
            w[x + "dkv"] = rnd(C + R, W, std=1.0 / math.sqrt(W))
            w[x + "dkv.norm"] = gain(C)
            w[x + "uk"] = rnd(H * D, C, std=1.0 / math.sqrt(C))
            w[x + "uv"] = rnd(H * V, C, std=1.0 / math.sqrt(C))
            w[x + "sink"] = rnd(H, std=1.0, mean=0.5)
            w[x + "o"] = rnd(W, H * V, std=1.0 / math.sqrt(H * V))
        else:
            a, b = m["left"], m["right"]
            H, G, D, V = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            w[x + "left.q"] = rnd(H * D, W, std=1.0 / math.sqrt(W))
            w[x + "left.k"] = rnd(G * D, W, std=1.0 / math.sqrt(W))
            w[x + "left.v"] = rnd(G * V, W, std=1.0 / math.sqrt(W))
            w[x + "left.q.norm"] = rnd(H * D, std=0.1, mean=peak / (a["scale"] * math.sqrt(D)))
            w[x + "left.k.norm"] = gain(G * D)
            w[x + "left.pb"] = rnd(H, std=1.0, mean=-2.0)
            w[x + "left.o"] = rnd(W, H * V, std=1.0 / math.sqrt(H * V))
            sH, sV, N, sG, taps = b["heads"], b["vdim"], b["state"], b["groups"], b["conv"]
            inner, chans = sH * sV, sH * sV + 2 * sG * N
            w[x + "right.in"] = rnd(2 * inner + 2 * sG * N + sH, W, std=1.0 / math.sqrt(W))
            w[x + "right.conv"] = rnd(chans, taps, std=0.5)
            w[x + "right.conv.b"] = rnd(chans, std=0.2)
            w[x + "right.dt_bias"] = rnd(sH, std=1.0, mean=-1.0 - slow)
            w[x + "right.A_log"] = rnd(sH, std=0.7)
            w[x + "right.D"] = rnd(sH, std=0.5, mean=1.0)
            w[x + "right.norm"] = gain(inner)
            w[x + "right.o"] = rnd(W, inner, std=1.0 / math.sqrt(inner))
            w[x + "left.out"] = gain(W)
            w[x + "right.out"] = gain(W)
        ff = lay["mlp"]
        if ff is None:
            continue
        F = ff["ff"]
        # pre-activations of about the limit's size, so that all three clamps cut
        w[p + ".mlp.gate"] = rnd(F, W, std=1.2 * ff["limit"] / math.sqrt(W))
        w[p + ".mlp.up"] = rnd(F, W, std=1.2 * ff["limit"] / math.sqrt(W))
        w[p + ".mlp.down"] = rnd(W, F, std=1.0 / math.sqrt(F))
        w[p + ".mlp.gate.b"] = rnd(F, std=0.3)
        w[p + ".mlp.up.b"] = rnd(F, std=0.3)
        w[p + ".mlp.down.b"] = rnd(W, std=0.2)
    return w


def random_layerlike_config(rng) -> dict:
    """Sizes of some hundreds, heads of 32 to 128: what the tensor-core kernels take, with the odd size between."""
    width = rng.choice([192, 256, 320, 384, 512])
    layers = []
    for n in range(rng.randint(3, 6)):
        pick = (n + rng.randint(0, 2)) % 3
        if pick == 0:
            mixer = wkv(rng.randint(2, 8), rng.choice([32, 48, 64, 96]))
        elif pick == 1:
            rot = rng.choice([16, 32, 64])
            mixer = latent(rng.choice([2, 4, 6, 8, 12]), rng.choice([32, 64, 96, 128]), rot, rng.choice([32, 64, 128]),
                           rng.choice([64, 96, 128, 192]), rng.choice([48, 80, 128]), size=rng.choice([48, 100, 129, 256, 1000]),
                           scale=rng.uniform(0.05, 0.2), base=rng.choice([10000.0, 50000.0, 1e6]))
        else:
            kv, dim, groups = rng.choice([1, 2, 4]), rng.choice([32, 64, 128]), rng.choice([1, 2, 4])
            s_heads, s_vdim = groups * rng.choice([1, 2, 4]), rng.choice([32, 48, 64])
            ng = rng.choice([d for d in (1, 2, 4, 8) if (s_heads * s_vdim) % d == 0])
            mixer = parallel(kv * rng.choice([1, 2, 4]), kv, dim, rng.choice([32, 64, 128]), chunk=rng.choice([32, 64, 96, 100, 128, 512]),
                             rot_dims=rng.choice([dim, dim, dim // 2, 0]), scale=rng.uniform(0.05, 0.2), s_heads=s_heads, s_vdim=s_vdim,
                             state=rng.choice([32, 48, 64, 128]), groups=groups, norm_groups=ng, conv=rng.randint(2, 4),
                             base=rng.choice([10000.0, 1e6]))
        mlp = dense(rng.choice([256, 344, 512]), rng.choice([1.0, 2.5, 7.0])) if rng.random() < 0.7 else None
        layers.append(layer(mixer, mlp))
    return config(width, rng.choice([384, 500, 1000]), rng.randint(2, 4), rng.randint(2, 4), layers, eps=rng.choice([1e-6, 1e-5]))


def random_config(seed: int, large: bool = False) -> dict:
    """Sizes, constants and layer order drawn from a seed."""
    import random
    rng = random.Random(seed)
    if large:
        return random_layerlike_config(rng)
    width = rng.choice([40, 56, 72, 88, 100, 128, 136])
    layers = []
    for _ in range(rng.randint(2, 5)):
        pick = rng.random()
        if pick < 0.33:
            mixer = wkv(rng.randint(1, 4), rng.choice([4, 10, 16, 24, 48, 72]))
        elif pick < 0.66:
            rot = rng.choice([2, 4, 8, 16, 32])
            mixer = latent(rng.randint(1, 5), rng.choice([4, 10, 16, 32, 64]), rot, rng.choice([4, 8, 12, 32, 64]),
                           rng.choice([6, 16, 24, 56, 100]), rng.choice([5, 8, 24, 40]), size=rng.choice([1, 5, 16, 17, 50, 300]),
                           scale=rng.uniform(0.1, 0.5), base=rng.choice([100.0, 10000.0, 1e6]), rot_dims=rng.choice([rot, rot, rot // 2 // 2 * 2]))
        else:
            kv = rng.choice([1, 2, 3])
            dim = rng.choice([4, 8, 10, 16, 24, 32, 64])
            groups = rng.choice([1, 2, 3])
            s_heads, s_vdim = groups * rng.randint(1, 2), rng.choice([4, 6, 8, 20, 32])
            ng = rng.choice([d for d in (1, 2, 3, 4, 6) if (s_heads * s_vdim) % d == 0])
            mixer = parallel(kv * rng.randint(1, 3), kv, dim, rng.choice([4, 8, 12, 16, 32, 64]), chunk=rng.choice([1, 5, 16, 17, 50, 300]),
                             rot_dims=rng.choice([0, 2, dim // 2 // 2 * 2, dim // 2 * 2]), scale=rng.uniform(0.1, 0.5),
                             s_heads=s_heads, s_vdim=s_vdim, state=rng.choice([4, 12, 16, 40, 64]), groups=groups, norm_groups=ng,
                             conv=rng.randint(1, 5), base=rng.choice([100.0, 10000.0, 1e6]))
        mlp = dense(rng.choice([8, 12, 24, 40]), rng.choice([0.5, 1.5, 7.0])) if rng.random() < 0.7 else None
        layers.append(layer(mixer, mlp))
    return config(width, rng.choice([61, 128, 200, 333]), rng.randint(1, 5), rng.randint(1, 6), layers,
                  eps=rng.choice([1e-6, 1e-5, 1e-3]))


def make_engine(cfg, weights, dtype, page, num_blocks, max_tokens=512, max_seqs=4, poison=True, graphs=False, max_seq_len=None):
    from llm_b200.config import EngineOptions
    from llm_b200.engine.engine import Engine
    opts = EngineOptions(dtype=dtype, kv_block_size=page, max_num_seqs=max_seqs, max_num_batched_tokens=max_tokens,
                         num_kv_blocks=num_blocks, use_cuda_graphs=graphs, poison_freed_pages=poison,
                         max_seq_len=max_seq_len or min(num_blocks * page, 4096))
    return Engine(None, opts, random_config=cfg, tensors={k: v.clone() for k, v in weights.items()})
