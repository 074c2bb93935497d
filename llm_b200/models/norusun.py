"""Norusun laid out as a ModelSpec: a decoder whose config lists its layers one by one, on a residual stream kept
as several copies.

The stream is `streams` copies per token (hyper-connections: every sublayer reads one mix of them and writes back
into all of them; the output is their sum).  Every sublayer is pre-normed by an RMS norm whose gain is one number.
Every mixer reads its input through a short causal convolution added to it (h + conv(h)).  The mixer is
  wkv               RWKV-style time mixing with a matrix state per head and a bonus for the current token,
  latent_attention  queries through a latent of their own, keys and values from one cached latent per token plus one
                    rotated key part shared by the heads (neighbouring pairs), a sliding window and a learned sink,
  parallel          a grouped-query attention (RMS norm over the whole q and k projections, rotate-half, a chunked mask,
                    sigmoid weights with a bias per head) beside a Mamba-2 state-space layer, their RMS-normed outputs
                    averaged.
The feed-forward is a gated unit with clamped branches and biases, or absent.  Tensors: `embed`,
`l<i>.norm1|norm2`, `l<i>.hc1|hc2.in|out|mix`, `l<i>.canon1`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config.model_config import NorusunConfig, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec

GATE_SLOPE = 1.702          # the feed-forward's gate is g * sigmoid(1.702 g)


def _mixer(cfg: NorusunConfig, kind: str, m: dict, prefix: str) -> PartSpec:
    W, eps = cfg.width, cfg.norm_eps
    if kind == "wkv":
        return PartSpec("wkv", {"hidden_size": W, "num_heads": m["heads"], "head_dim": m["dim"], "eps": eps}, prefix)
    if kind == "latent_attention":
        position = PartSpec("rope_pairs", {"dims": m["rot_dims"], "base": m["rot_base"]}) if m["rot_dims"] else None
        return PartSpec("latent_attention", {
            "hidden_size": W, "num_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"], "rank": m["kv_rank"],
            "scale": m["scale"], "eps": eps, "gated": False, "q_rank": m["q_rank"], "rot_dim": m["rot_dim"],
            "position": position, "window": m["window"], "sink": True}, prefix)
    a, b = m["left"], m["right"]
    position = PartSpec("rope_pairs", {"dims": a["rot_dims"], "base": a["rot_base"], "layout": "halves"}) if a["rot_dims"] else None
    left = PartSpec("attention", {
        "hidden_size": W, "num_heads": a["heads"], "num_kv_heads": a["kv_heads"], "head_dim": a["dim"], "value_dim": a["vdim"],
        "scale": a["scale"], "position": position, "chunk": a["chunk"], "weights": "sigmoid", "qk_norm": "whole",
        "norm_eps": eps, "names": {"q": "q", "k": "k", "v": "v", "o": "o"}}, prefix + ".left")
    right = PartSpec("ssd", {"hidden_size": W, "num_heads": b["heads"], "value_dim": b["vdim"], "state_size": b["state"],
                             "groups": b["groups"], "norm_groups": b["norm_groups"], "taps": b["conv"], "eps": eps},
                     prefix + ".right")
    return PartSpec("parallel", {"hidden_size": W, "left": left, "right": right, "eps": eps}, prefix)


def build_norusun_spec(cfg: NorusunConfig) -> ModelSpec:
    W, S = cfg.width, cfg.streams
    norm = lambda p, q: PartSpec("hyper_rmsnorm", {"size": W, "streams": S, "eps": cfg.norm_eps, "gain_name": f"norm{q}",
                                                   "hc_name": f"hc{q}"}, p)
    layers = []
    for i, layer in enumerate(cfg.layers):
        p, ff = f"l{i}", layer["mlp"]
        mixer = PartSpec("conv_input", {"hidden_size": W, "taps": cfg.canon_taps, "weight_name": "canon1",
                                        "inner": _mixer(cfg, layer["type"], layer["mixer"], p + ".mix")}, p)
        parts = {"norm1": norm(p, 1), "mixer": mixer, "norm2": None, "ffn": None}
        if ff is not None:
            parts["norm2"] = norm(p, 2)
            parts["ffn"] = PartSpec("clamped_glu", {"hidden_size": W, "intermediate_size": ff["ff"], "limit": ff["limit"],
                                                    "alpha": GATE_SLOPE, "bias": True}, p + ".mlp")
        layers.append(LayerSpec("hyper", parts))
    spec = ModelSpec(
        hidden_size=W, vocab_size=cfg.vocab, max_position=cfg.max_position,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "weight_name": "", "copies": S}, "embed"),
        layers=tuple(layers), order=tuple(range(len(layers))),
        final_norm=PartSpec("scalar_rmsnorm", {"size": W, "eps": cfg.norm_eps}, "final.norm"),
        head=PartSpec("lm_head", {"hidden_size": W, "vocab_size": cfg.vocab, "weight_name": ""}, "head"),
        eos_token_id=cfg.eos_token_id, stream_copies=S,
    )
    spec.validate()
    return spec


register_architecture("Norusun", NorusunConfig, build_norusun_spec)
