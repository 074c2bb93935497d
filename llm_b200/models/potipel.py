"""Potipel laid out as a ModelSpec: a pre-norm decoder whose config lists its layers one by one.

The embedding is scaled by a constant.  Every sublayer is pre-normed by an RMS norm with a weight and reads its input
through a short causal convolution added to it (h + conv(h)); the convolution's last inputs are part of a request's state,
for the mixer and for the feed-forward.  The mixer is
  attention  differential attention: two causal softmax maps per head with queries and keys of their own (RMS-normed per
             head and map) over one set of values, a1 - lambda a2, a weightless RMS norm per head, a sigmoid gate;
  hgrn2      a recurrence whose forget gate, bounded below, also decides what is written;
  parallel   a sliding-window attention (biased projections behind a short convolution, capped scores, a bias that grows
             with the logarithm of the distance, a learned sink) beside a gated delta rule, summed with two constants.
The feed-forward is a gated unit with relu, or a mixture of clamped gated experts chosen by sigmoid scores with a correction
among the best groups of experts, or absent.  A layer may use an earlier layer's tensors with a cache and state of its own:
the spec's order then names that layer again.  Tensors: `embed`, `l<i>.norm1|norm2`, `l<i>.canon1|canon2`, `l<i>.mix.*`,
`l<i>.mlp.*`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config.model_config import PotipelConfig, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec

GATE_SLOPE = 1.702          # an expert's gate is g * sigmoid(1.702 g)
UNIT_EPS = 1e-6             # added to the sums of squares under the delta rule's unit norms


def _mixer(cfg: PotipelConfig, kind: str, m: dict, prefix: str) -> PartSpec:
    W, eps = cfg.width, cfg.norm_eps
    if kind == "attention":
        return PartSpec("diff_attention", {"hidden_size": W, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"],
                                           "head_dim": m["dim"], "value_dim": m["vdim"], "scale": m["scale"], "diff": m["diff"],
                                           "eps": eps}, prefix)
    if kind == "hgrn2":
        return PartSpec("hgrn2", {"hidden_size": W, "num_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
                                  "eps": eps}, prefix)
    a, b = m["left"], m["right"]
    names = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b"}
    left = PartSpec("attention", {
        "hidden_size": W, "num_heads": a["heads"], "num_kv_heads": a["kv_heads"], "head_dim": a["dim"], "value_dim": a["vdim"],
        "scale": a["scale"], "window": a["window"], "softcap": a["softcap"], "sink": "learned", "dist_bias": True,
        "qkv_conv": a["conv"], "bias": True, "out_bias": False, "names": names}, prefix + ".left")
    right = PartSpec("gated_delta", {"hidden_size": W, "num_heads": b["heads"], "num_qk_heads": b["kv_heads"], "head_dim": b["dim"],
                                     "value_dim": b["vdim"], "taps": b["conv"], "eps": eps, "unit_eps": UNIT_EPS}, prefix + ".right")
    return PartSpec("parallel", {"hidden_size": W, "left": left, "right": right, "combine": "scaled_sum",
                                 "left_scale": m["left_scale"], "right_scale": m["right_scale"]}, prefix)


def _ffn(cfg: PotipelConfig, ff: dict, prefix: str) -> PartSpec:
    W = cfg.width
    if ff["kind"] == "dense":
        return PartSpec("swiglu", {"hidden_size": W, "intermediate_size": ff["ff"], "activation": "relu",
                                   "names": {"gate": "gate", "up": "up", "down": "down"}}, prefix)
    return PartSpec("routed", {"hidden_size": W, "experts": ff["experts"], "top": ff["top"], "expert_size": ff["ff"],
                               "activation": "clamped", "gated": True, "limit": ff["limit"], "alpha": GATE_SLOPE,
                               "router": "sigmoid_groups", "groups": ff["groups"], "keep_groups": ff["keep"],
                               "router_bias": False}, prefix)


def build_potipel_spec(cfg: PotipelConfig) -> ModelSpec:
    W = cfg.width
    norm = lambda p, q: PartSpec("rmsnorm", {"size": W, "eps": cfg.norm_eps, "weight_name": f"norm{q}"}, p)
    own = [i for i, layer in enumerate(cfg.layers) if layer["weights_of"] is None]
    place = {i: n for n, i in enumerate(own)}       # layer index -> its place among the layers that have tensors
    # a layer without tensors runs another layer's parts again, with a cache and state of its own place in the order
    order = [place[i if layer["weights_of"] is None else layer["weights_of"]] for i, layer in enumerate(cfg.layers)]
    layers = []
    for i in own:
        layer = cfg.layers[i]
        p, ff = f"l{i}", layer["mlp"]
        mixer = PartSpec("conv_input", {"hidden_size": W, "taps": cfg.canon_taps, "weight_name": "canon1",
                                        "inner": _mixer(cfg, layer["type"], layer["mixer"], p + ".mix")}, p)
        parts = {"norm1": norm(p, 1), "mixer": mixer, "norm2": None, "ffn": None}
        if ff is not None:
            parts["norm2"] = norm(p, 2)
            parts["ffn"] = PartSpec("conv_input", {"hidden_size": W, "taps": cfg.canon_taps, "weight_name": "canon2",
                                                   "inner": _ffn(cfg, ff, p + ".mlp")}, p)
        layers.append(LayerSpec("prenorm", parts))
    spec = ModelSpec(
        hidden_size=W, vocab_size=cfg.vocab, max_position=cfg.max_position,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "weight_name": "",
                                               "scale": cfg.embedding_scale}, "embed"),
        layers=tuple(layers), order=tuple(order),
        final_norm=PartSpec("rmsnorm", {"size": W, "eps": cfg.norm_eps, "weight_name": ""}, "final.norm"),
        head=PartSpec("lm_head", {"hidden_size": W, "vocab_size": cfg.vocab, "weight_name": ""}, "head"),
        eos_token_id=cfg.eos_token_id,
    )
    spec.validate()
    return spec


register_architecture("Potipel", PotipelConfig, build_potipel_spec)
