"""CPU tests of the Norusun design: configuration, layout, tensor names, state layout, and the plain implementation's
own consistency (tests/plain_norusun.py is the oracle of the GPU tests)."""
import copy
import math

import pytest
import torch

import plain_norusun as P
from norusun_tiny import CONFIGS, make_weights, random_config
from tiny import random_tokens

from llm_b200.config.model_config import ConfigError, parse_config
from llm_b200.engine.model import Model, collect_parameters


def test_config_reads_every_size_and_constant():
    cfg, _ = CONFIGS["A"]
    arch, c = parse_config(cfg)
    assert arch.name == "Norusun" and c.width == 64 and c.vocab == 200 and c.streams == 2 and c.canon_taps == 3
    assert c.norm_eps == 1e-5 and [l["type"] for l in c.layers] == ["wkv", "latent_attention", "parallel", "wkv"]
    lat = c.layers[1]["mixer"]
    assert (lat["heads"], lat["dim"], lat["rot_dim"], lat["vdim"], lat["kv_rank"], lat["q_rank"], lat["window"]) == (4, 16, 8, 8, 24, 12, 12)
    assert lat["scale"] == 0.3 and lat["rot_dims"] == 8 and lat["rot_base"] == 10000.0
    par = c.layers[2]["mixer"]
    assert par["left"]["chunk"] == 10 and par["left"]["kv_heads"] == 2 and par["right"]["norm_groups"] == 2 and par["right"]["conv"] == 3
    assert c.layers[0]["mlp"] is None and c.layers[3]["mlp"] == {"kind": "dense", "ff": 32, "limit": 0.7}


@pytest.mark.parametrize("path,value", [
    (("streams",), 0), (("streams",), 9), (("canon", "taps"), 0), (("layers", 0, "type"), "conv"), (("layers", 0, "mixer", "dim"), 0),
    (("layers", 1, "mixer", "rot_dim"), 7), (("layers", 1, "mixer", "rot", "dims"), 10), (("layers", 1, "mixer", "mask", "size"), 0),
    (("layers", 2, "mixer", "left", "kv_heads"), 3), (("layers", 2, "mixer", "right", "groups"), 3),
    (("layers", 2, "mixer", "right", "norm_groups"), 5), (("layers", 1, "mlp", "kind"), "moe"), (("layers", 1, "mlp", "limit"), 0.0),
    (("width",), -1), (("norm", "eps"), "x")])
def test_config_errors_name_the_key(path, value):
    cfg = copy.deepcopy(CONFIGS["A"][0])
    at = cfg
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError):
        parse_config(cfg)


@pytest.mark.parametrize("missing", ["streams", "canon", "norm", "layers", "width", "vocab"])
def test_config_requires_its_keys(missing):
    cfg = copy.deepcopy(CONFIGS["B"][0])
    del cfg[missing]
    with pytest.raises(ConfigError):
        parse_config(cfg)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_names_and_shapes_are_those_of_the_weights(name):
    cfg, _ = CONFIGS[name]
    w = make_weights(cfg, seed=1)
    want = collect_parameters(cfg)
    assert sorted(want) == sorted(w)
    for n, info in want.items():
        assert info.fits(w[n].shape), (n, info.shape, tuple(w[n].shape))


def test_layout_streams_and_state_rows():
    cfg, _ = CONFIGS["A"]
    arch, c = parse_config(cfg)
    spec = arch.build_spec(c)
    assert spec.stream_copies == 2 and [l.block for l in spec.layers] == ["hyper"] * 4
    model = Model(spec, torch.float32, torch.device("cpu"))
    W, taps = 64, 3
    conv = (taps - 1) * W
    # wkv: convolution inputs, previous row, a matrix per head
    assert model.state_needs[0].shape == (conv + W + 2 * 16 * 16,)
    # latent attention: convolution inputs only; its latents are a window cache of one head of rot_dim + kv_rank numbers
    assert model.state_needs[1].shape == (conv,)
    need = model.blocks[1].mixer.cache_need()
    assert (need.kind, need.window, need.num_kv_heads, need.values) == ("window", 12, 1, False) and need.head_dim >= 8 + 24
    # parallel: the left side keeps keys of its chunk, the right side the convolution's inputs and its matrices
    need = model.blocks[2].mixer.cache_need()
    assert (need.kind, need.window, need.num_kv_heads, need.head_dim, need.value_dim) == ("window", 10, 2, 16, 8)
    chans = 4 * 8 + 2 * 2 * 16
    assert model.state_needs[2].shape == (conv + (3 - 1) * chans + 4 * 16 * 8,)
    assert len(model.cache_instances) == 2 and len(model.group_keys) == 2


def test_one_tap_and_one_stream_change_nothing():
    """With one stream whose weights are 1 and a convolution of one tap whose weight is 0 the design is a plain pre-norm
    decoder: the plain implementation agrees with itself written that way."""
    cfg, _ = CONFIGS["C"]
    w = {k: v.double() for k, v in make_weights(cfg, seed=3).items()}
    for k in w:
        if ".hc" in k:
            w[k] = torch.ones_like(w[k])
        if k.endswith("canon1"):
            w[k] = torch.zeros_like(w[k])
    toks = random_tokens(23, cfg["vocab"], 5)
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(toks)]
    for i, lay in enumerate(cfg["layers"]):
        L = f"l{i}."
        local = lambda prefix: {k[len(L + prefix):]: v for k, v in w.items() if k.startswith(L + prefix)}
        x = x + P.MIXERS[lay["type"]](P.scalar_norm(x, w[L + "norm1"], eps), local("mix."), lay["mixer"], eps)
        if lay["mlp"] is not None:
            x = x + P.clamped_ff(P.scalar_norm(x, w[L + "norm2"], eps), local("mlp."), lay["mlp"]["limit"])
    ref = P.scalar_norm(x, w["final.norm"], eps) @ w["head"].T
    assert torch.allclose(P.forward(cfg, w, toks), ref, rtol=1e-10, atol=1e-10)


def test_plain_recurrences_agree_with_their_closed_forms():
    """The token-by-token loops of the plain implementation against sums written out over all earlier tokens."""
    torch.manual_seed(0)
    T, H, D = 9, 2, 5
    m = {"heads": H, "dim": D}
    W = 12
    p = {"mu." + n: torch.rand(W, dtype=torch.float64) for n in "rkvgw"}
    p.update({n: torch.randn(H * D, W, dtype=torch.float64) / math.sqrt(W) for n in "rkvg"})
    p.update({"w1": torch.randn(3, W, dtype=torch.float64), "w2": torch.randn(H * D, 3, dtype=torch.float64), "w0": torch.randn(H * D, dtype=torch.float64),
              "u": torch.randn(H, D, dtype=torch.float64), "norm": torch.ones(H * D, dtype=torch.float64), "o": torch.eye(H * D, dtype=torch.float64)})
    h = torch.randn(T, W, dtype=torch.float64)
    got = P.wkv_mixer(h, p, m, 1e-6)
    prev = torch.cat([torch.zeros(1, W, dtype=torch.float64), h[:-1]])
    mix = lambda n: h + (prev - h) * p["mu." + n]
    r, k, v = ((mix(n) @ p[n].T).view(T, H, D) for n in "rkv")
    dec = torch.exp(-torch.exp(torch.tanh(mix("w") @ p["w1"].T) @ p["w2"].T + p["w0"])).view(T, H, D)
    o = torch.zeros(T, H, D, dtype=torch.float64)
    for t in range(T):
        for j in range(t + 1):
            wgt = p["u"] if j == t else dec[j + 1:t].prod(dim=0)           # the decays strictly between j and t
            o[t] += (r[t] * wgt * k[j]).sum(-1, keepdim=True) * v[j]
    ref = (P.rms_unit(o, 1e-6).reshape(T, H * D) * P.silu(mix("g") @ p["g"].T))
    assert torch.allclose(got, ref, rtol=1e-9, atol=1e-9)


@pytest.mark.parametrize("seed", range(6))
def test_random_configurations_parse_and_name_their_tensors(seed):
    cfg = random_config(3000 + seed)
    w = make_weights(cfg, seed=seed)
    assert sorted(collect_parameters(cfg)) == sorted(w)
    logits = P.forward(cfg, {k: v.double() for k, v in w.items()}, random_tokens(17, cfg["vocab"], seed))
    assert logits.shape == (17, cfg["vocab"]) and bool(torch.isfinite(logits).all())
