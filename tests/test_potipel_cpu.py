"""CPU tests of the Potipel design: configuration, layout, tensor names, the state row, and the plain implementation's
own consistency (tests/plain_potipel.py is the oracle of the GPU tests)."""
import copy
import math

import pytest
import torch

import plain_potipel as P
from potipel_tiny import CONFIGS, make_weights, random_config
from tiny import random_tokens

from llm_b200.config.model_config import ConfigError, parse_config
from llm_b200.engine.model import Model, collect_parameters


def test_config_reads_every_size_and_constant():
    cfg, _ = CONFIGS["A"]
    arch, c = parse_config(cfg)
    assert arch.name == "Potipel" and c.width == 64 and c.vocab == 200 and c.canon_taps == 3 and c.embedding_scale == 4.0
    assert c.norm_eps == 1e-5 and [l["type"] for l in c.layers] == ["attention", "hgrn2", "parallel", "attention", "parallel"]
    assert [l["weights_of"] for l in c.layers] == [None, None, None, 0, 2]
    att = c.layers[0]["mixer"]
    assert (att["heads"], att["kv_heads"], att["dim"], att["vdim"], att["scale"], att["diff"]) == (4, 2, 16, 8, 0.3, 0.4)
    par = c.layers[2]["mixer"]
    assert par["left"]["window"] == 12 and par["left"]["softcap"] == 20.0 and par["left"]["conv"] == 3 and par["right"]["conv"] == 2
    assert (par["left_scale"], par["right_scale"]) == (0.7, 0.9)
    assert c.layers[0]["mlp"] == {"kind": "dense", "ff": 40}
    assert c.layers[1]["mlp"] == {"kind": "moe", "ff": 16, "limit": 2.0, "experts": 4, "top": 1, "groups": 2, "keep": 1}


@pytest.mark.parametrize("path,value", [
    (("canon", "taps"), 0), (("canon", "taps"), 17), (("layers", 0, "type"), "conv"), (("layers", 0, "mixer", "dim"), 0),
    (("layers", 0, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "diff"), "x"), (("layers", 1, "mixer", "vdim"), -1),
    (("layers", 2, "mixer", "left", "mask", "size"), 0), (("layers", 2, "mixer", "left", "kv_heads"), 3),
    (("layers", 2, "mixer", "right", "kv_heads"), 3), (("layers", 2, "mixer", "left", "softcap"), 0.0),
    (("layers", 1, "mlp", "kind"), "sparse"), (("layers", 1, "mlp", "expert", "limit"), 0.0), (("layers", 1, "mlp", "router", "top"), 5),
    (("layers", 1, "mlp", "router", "groups", "count"), 3), (("layers", 1, "mlp", "router", "groups", "keep"), 3),
    (("layers", 2, "mlp", "router", "top"), 5), (("layers", 3, "weights_of"), 3), (("layers", 3, "weights_of"), 1),
    (("layers", 4, "weights_of"), 3), (("width",), -1), (("norm", "eps"), "x"), (("embedding", "scale"), "x")])
def test_config_errors_name_the_key(path, value):
    cfg = copy.deepcopy(CONFIGS["A"][0])
    at = cfg
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError):
        parse_config(cfg)


@pytest.mark.parametrize("missing", ["embedding", "canon", "norm", "layers", "width", "vocab"])
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


def test_layout_order_caches_and_state_rows():
    cfg, _ = CONFIGS["A"]
    arch, c = parse_config(cfg)
    spec = arch.build_spec(c)
    # three layers have tensors; the order runs two of them a second time
    assert len(spec.layers) == 3 and spec.order == (0, 1, 2, 0, 2) and [l.block for l in spec.layers] == ["prenorm"] * 3
    model = Model(spec, torch.float32, torch.device("cpu"))
    W, taps = 64, 3
    conv = (taps - 1) * W
    # every run has a state of its own: the mixer's input convolution, the mixer's own numbers, the feed-forward's convolution
    assert len(model.state_needs) == 5 and len(model.cache_instances) == 4
    assert model.state_needs[0].shape == (conv + conv,) == model.state_needs[3].shape
    assert model.state_needs[1].shape == (conv + 2 * 16 * 24 + conv,)
    left = (3 - 1) * (4 * 16 + 2 * 16 + 2 * 8)
    right = (2 - 1) * (2 * 2 * 16 + 4 * 8) + 4 * 16 * 8
    assert model.state_needs[2].shape == (conv + left + right + conv,) == model.state_needs[4].shape
    # two maps per head: twice the key heads, the values once
    need = model.blocks[0].mixer.cache_need()
    assert (need.kind, need.num_kv_heads, need.head_dim, need.value_dim, need.value_heads) == ("full", 4, 16, 8, 2)
    need = model.blocks[2].mixer.cache_need()
    assert (need.kind, need.window, need.num_kv_heads, need.head_dim, need.value_dim) == ("window", 12, 2, 16, 8)
    assert len(model.group_keys) == 2
    occ = model.occurrences
    assert occ[0].cache_instance != occ[3].cache_instance and occ[2].cache_instance != occ[4].cache_instance


def test_a_layer_may_name_one_that_names_another_or_one_that_comes_later():
    cfg = copy.deepcopy(CONFIGS["A"][0])
    cfg["layers"].append(dict(cfg["layers"][3], weights_of=3))           # 5 -> 3 -> 0
    arch, c = parse_config(cfg)
    assert [l["weights_of"] for l in c.layers] == [None, None, None, 0, 2, 0] and arch.build_spec(c).order == (0, 1, 2, 0, 2, 0)
    cfg = copy.deepcopy(CONFIGS["A"][0])
    L = cfg["layers"]
    L[0], L[3] = L[3], L[0]                                               # the layer with the tensors now comes after its user
    L[0]["weights_of"] = 3
    arch, c = parse_config(cfg)
    spec = arch.build_spec(c)
    assert spec.order == (2, 0, 1, 2, 1) and sorted(n for n in Model(spec, torch.float32, torch.device("cpu")).parameters() if n.endswith(".norm1")) \
        == ["l1.norm1", "l2.norm1", "l3.norm1"]
    cfg["layers"][3]["weights_of"] = 0                                    # a circle
    with pytest.raises(ConfigError):
        parse_config(cfg)


def test_a_layer_without_feed_forward_keeps_only_its_mixers_state():
    cfg, _ = CONFIGS["D"]
    arch, c = parse_config(cfg)
    model = Model(arch.build_spec(c), torch.float32, torch.device("cpu"))
    assert model.state_needs[0].shape == ((2 - 1) * 64,)


def test_one_tap_with_weight_zero_changes_nothing():
    """With input convolutions of one tap whose weight is 0 the design is a plain pre-norm decoder: the plain implementation
    agrees with itself written that way."""
    cfg, _ = CONFIGS["C"]
    w = {k: v.double() for k, v in make_weights(cfg, seed=3).items()}
    for k in w:
        if ".canon" in k:
            w[k] = torch.zeros_like(w[k])
    toks = random_tokens(23, cfg["vocab"], 5)
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(toks)] * cfg["embedding"]["scale"]
    for i, lay in enumerate(cfg["layers"]):
        p = P.layer_tensors(w, i)
        h = P.rms_norm(x, p["norm1"], eps)
        mix = {"attention": P.diff_attention, "hgrn2": P.hgrn2, "parallel": P.parallel}[lay["type"]]
        x = x + mix(h, P.sub(p, "mix"), lay["mixer"], eps)
        h = P.rms_norm(x, p["norm2"], eps)
        x = x + (P.dense_ff(h, P.sub(p, "mlp")) if lay["mlp"]["kind"] == "dense" else P.moe_ff(h, P.sub(p, "mlp"), lay["mlp"]))
    ref = P.rms_norm(x, w["final.norm"], eps) @ w["head"].T
    assert torch.allclose(P.forward(cfg, w, toks), ref, rtol=1e-10, atol=1e-10)


def test_plain_recurrences_agree_with_their_closed_forms():
    """The token-by-token loops of the plain implementation against sums written out over all earlier tokens."""
    torch.manual_seed(0)
    T, H, D, V, W = 9, 2, 5, 3, 12
    f64 = lambda *s: torch.randn(*s, dtype=torch.float64)
    p = {"q": f64(H * D, W) / math.sqrt(W), "f": f64(H * D, W), "f.b": f64(H * D), "lower": torch.rand(H * D, dtype=torch.float64),
         "v": f64(H * V, W), "norm": torch.ones(V, dtype=torch.float64), "o": torch.eye(H * V, dtype=torch.float64)}
    h = f64(T, W)
    got = P.hgrn2(h, p, {"heads": H, "dim": D, "vdim": V}, 1e-6)
    q, v = P.silu(h @ p["q"].T).view(T, H, D), (h @ p["v"].T).view(T, H, V)
    f = (p["lower"] + (1 - p["lower"]) * torch.sigmoid(h @ p["f"].T + p["f.b"])).view(T, H, D)
    o = torch.zeros(T, H, V, dtype=torch.float64)
    for t in range(T):
        for j in range(t + 1):
            wgt = f[j + 1:t + 1].prod(dim=0) * (1 - f[j])                   # the gates after j, and what j wrote
            o[t] += (q[t] * wgt).sum(-1, keepdim=True) * v[j]
    assert torch.allclose(got, P.rms_unit(o, 1e-6).reshape(T, H * V), rtol=1e-9, atol=1e-9)
    # the delta rule with beta = 1, no decay and orthonormal keys stores each value under its key and reads it back
    D = 4
    keys = torch.eye(D, dtype=torch.float64)
    S = torch.zeros(D, V, dtype=torch.float64)
    vals = f64(D, V)
    for t in range(D):
        S = S + torch.outer(keys[t], vals[t] - S.T @ keys[t])
    assert torch.allclose(S.T @ keys[2], vals[2])


def test_router_strikes_out_groups_not_scores():
    """A group that is not kept cannot be chosen from even where its corrected scores are the largest left, and negative
    corrected scores inside kept groups still can."""
    h = torch.eye(4, dtype=torch.float64)[:1]
    p = {"router": torch.zeros(4, 4, dtype=torch.float64), "correction": torch.tensor([-0.9, -0.8, 0.3, -2.0], dtype=torch.float64)}
    r = {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 1}}
    ids, wts, _ = P.route(h, p, r)
    # group scores: (-0.4) + (-0.3) = -0.7 against 0.8 + (-1.5) = -0.7 + ... the second group wins by its best expert
    g0, g1 = (0.5 - 0.9) + (0.5 - 0.8), (0.5 + 0.3) + (0.5 - 2.0)
    want = [2, 3] if g1 > g0 else [1, 0]
    assert ids[0].tolist() == want and torch.allclose(wts, torch.full((1, 2), 0.5, dtype=torch.float64))


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations_parse_and_name_their_tensors(seed):
    cfg = random_config(3000 + seed)
    w = make_weights(cfg, seed=seed)
    assert sorted(collect_parameters(cfg)) == sorted(w)
    logits = P.forward(cfg, {k: v.double() for k, v in w.items()}, random_tokens(17, cfg["vocab"], seed))
    assert logits.shape == (17, cfg["vocab"]) and bool(torch.isfinite(logits).all())
