"""Bilurax without a GPU: the configuration and its checks, the model description (parts, run order of a looped span,
tensor names), and properties of the plain implementation that the GPU
tests lean on."""
import copy
import math

import pytest
import torch

import plain_bilurax as plain
from bilurax_models import CONFIGS, _config, attention, dense, layer, make_weights, moe, tensor_shapes

from sandyrt_b200.config.base import ConfigError, config_from_normalised
from sandyrt_b200.config.bilurax import BiluraxConfig


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_description_names_every_tensor_with_its_shape(name):
    from sandyrt_b200.models.model import build_model

    cfg = config_from_normalised(CONFIGS[name])
    assert isinstance(cfg, BiluraxConfig) and cfg.vocab_size == CONFIGS[name]["vocab"]
    cfg.validate()
    got = {k: list(v.shape) for k, v in build_model(cfg).tensor_requests().items()}
    assert got == tensor_shapes(CONFIGS[name])


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_run_order_of_a_looped_span(name):
    """Every pass of the span is a call of the same layers with cache entries of its own; a pass is entered through a
    remix that adds its row of the table, and from the second pass on the embedding's output."""
    from sandyrt_b200.models.model import describe

    raw = CONFIGS[name]
    spec = describe(config_from_normalised(raw))
    order = plain.run_order(raw)
    assert len(spec.layers) == len(raw["layers"])
    assert [c.layer for c in spec.schedule] == [i for i, _ in order]
    assert [c.cache for c in spec.schedule] == list(range(len(order)))
    entered = [c.remix for c in spec.schedule]
    assert entered == [t for _, t in order]
    times = raw["loop"]["times"] if raw.get("loop") else 0
    assert len(spec.remixes) == times
    for t, r in enumerate(spec.remixes):
        assert r.kind == "add_row" and r.params["row"] == t and r.params["rows"] == times
        assert r.params["add_embedding"] is (t > 0) and r.tensors == {"table": "loop.step"}
    for l, src in zip(spec.layers, raw["layers"]):
        assert l.block == "pre_norm" and l.mixer.kind == "normed_attention"
        assert l.feed_forward.kind == {None: "none", "dense": "dense_mlp", "moe": "routed_experts"}[src["mlp"] and src["mlp"]["kind"]]
    assert spec.position.kind == "none" and spec.head.params["tied"] is True
    assert spec.head.params["logit_softcap"] == raw["logit_softcap"] and spec.embedding.params["scale"] == raw["embedding"]["scale"]


def test_config_round_trip_and_constants_reach_the_parts():
    from sandyrt_b200.models.model import describe

    raw = CONFIGS["A"]
    cfg = BiluraxConfig.from_dict(raw)
    assert BiluraxConfig.from_dict(cfg.to_dict()) == cfg
    assert cfg.to_dict()["layers"] == raw["layers"] and cfg.to_dict()["loop"] == raw["loop"]
    spec = describe(cfg)
    p, m = spec.layers[2].mixer.params, raw["layers"][2]["mixer"]
    assert (p["n_heads"], p["n_kv_heads"], p["qk_dim"], p["v_dim"], p["chunk"]) == (2, 1, 16, 48, 24)
    assert p["softcap"] == m["softcap"] == 6.0 and p["scale"] == m["scale"] and p["eps"] == raw["norm"]["eps"]
    assert all(p[k] is True for k in ("bias", "qk_norm", "v_norm", "head_temperature", "token_shift"))
    f, r = spec.layers[1].feed_forward.params, raw["layers"][1]["mlp"]
    assert (f["n_experts"], f["top"], f["inner"], f["n_groups"], f["keep_groups"]) == (6, 2, 24, 3, 2)
    assert f["weight_scale"] == r["router"]["scale"] and f["limit"] == r["expert"]["limit"]
    assert (f["scoring"], f["activation"], f["group_rank"], f["glu_alpha"], f["weight_eps"]) == ("sigmoid", "clamped_glu", 2, 1.702, 1e-20)
    d = spec.layers[0].feed_forward.params
    assert (d["activation"], d["inner"], d["bias"]) == ("relu_squared", 96, False)
    no_loop = BiluraxConfig.from_dict(CONFIGS["B"])
    assert no_loop.loop is None and "loop" not in no_loop.to_dict() and not describe(no_loop).remixes


def _broken(path, value):
    raw = copy.deepcopy(CONFIGS["A"])
    node = raw
    for k in path[:-1]:
        node = node[k]
    if value is KeyError:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    return raw


@pytest.mark.parametrize("path,value,message", [
    (("layers", 0, "type"), "rotated", "unknown layer type"),
    (("layers", 0, "mixer", "kv_heads"), 3, "do not divide"),
    (("layers", 0, "mixer", "dim"), 648, "at most 640"),
    (("layers", 0, "mixer", "softcap"), 0.0, "softcap"),
    (("layers", 0, "mixer", "mask"), KeyError, "mask"),
    (("layers", 0, "mixer", "mask", "size"), 0, "size"),
    (("layers", 0, "mixer", "vdim"), "8", "int"),
    (("layers", 1, "mlp", "kind"), "routed", "dense"),
    (("layers", 1, "mlp", "router", "top"), 5, "top"),
    (("layers", 1, "mlp", "router", "groups", "count"), 4, "divide"),
    (("layers", 1, "mlp", "router", "groups", "keep"), 4, "keep"),
    (("layers", 1, "mlp", "expert", "limit"), -1.0, "limit"),
    (("loop", "stop"), 5, "start < stop"),
    (("loop", "times"), 0, "times"),
    (("logit_softcap",), KeyError, "logit_softcap"),
    (("embedding",), KeyError, "embedding"),
    (("norm",), KeyError, "norm"),
])
def test_configurations_that_are_refused(path, value, message):
    with pytest.raises(ConfigError, match=message):
        BiluraxConfig.from_dict(_broken(path, value)).validate()


# ---- the plain implementation --------------------------------------------------------------------------------
def test_plain_chunks_count_from_position_zero():
    see = plain.visible(10, 4)
    assert see[3].tolist() == [True] * 4 + [False] * 6          # the chunk's last position sees all of it
    assert see[4].tolist() == [False] * 4 + [True] + [False] * 5      # the next chunk's first sees itself alone
    assert see[9].tolist() == [False] * 8 + [True, True]
    assert torch.equal(plain.visible(6, 1), torch.eye(6, dtype=torch.bool))
    assert torch.equal(plain.visible(6, 100), torch.ones(6, 6).tril().bool())


def test_plain_token_shift_reads_the_row_before():
    h = torch.randn(5, 3, dtype=torch.float64)
    mix = torch.tensor([0.0, 1.0, 0.25], dtype=torch.float64)
    u = plain.token_shift(h, mix)
    assert torch.equal(u[:, 0], h[:, 0])
    assert torch.allclose(u[1:, 1], h[:-1, 1]) and abs(float(u[0, 1])) < 1e-12
    assert torch.allclose(u[2, 2], 0.75 * h[2, 2] + 0.25 * h[1, 2]) and torch.allclose(u[0, 2], 0.75 * h[0, 2])


def test_plain_routing_stays_inside_the_best_groups():
    """Six experts in three pairs, two pairs kept.  The best single expert sits in the pair with the smallest sum: it
    is not chosen.  Corrections move the choice but not the weights."""
    r = {"experts": 6, "top": 2, "scale": 1.5, "groups": {"count": 3, "keep": 2}}
    width = 4
    w = {"r.router": torch.zeros(6, width, dtype=torch.float64), "r.correction": torch.zeros(6, dtype=torch.float64)}
    z = torch.tensor([2.0, -8.0, 1.0, 0.9, 0.5, 0.4], dtype=torch.float64)      # sigmoid: .88 .0003 | .73 .71 | .62 .60
    w["r.router"][:, 0] = z
    n = torch.zeros(3, width, dtype=torch.float64)
    n[:, 0] = 1.0
    chosen, weights, margin = plain.route(r, w, "r.", n, plain.Products(False))
    assert chosen[0].tolist() == [2, 3]                     # groups 1 and 2 stay (1.44, 1.22 against 0.88)
    s = torch.sigmoid(z)
    assert torch.allclose(weights[0], s[[2, 3]] / s[[2, 3]].sum() * 1.5) and float(margin[0]) > 0.05
    w["r.correction"] = torch.tensor([0.0, 1.0, 0.0, 0.0, 0.0, 0.0], dtype=torch.float64)     # now group 0 sums to 1.88
    chosen, weights, _ = plain.route(r, w, "r.", n, plain.Products(False))
    assert chosen[0].tolist() == [1, 0]                     # 1.0003 with the correction, 0.88
    assert torch.allclose(weights[0], s[[1, 0]] / s[[1, 0]].sum() * 1.5)       # the weights are the scores without it
    w["r.correction"] = torch.tensor([-5.0, -5.0, -3.0, -3.1, -9.0, -9.0], dtype=torch.float64)   # all negative
    chosen, _, _ = plain.route(r, w, "r.", n, plain.Products(False))
    assert chosen[0].tolist() == [2, 3]                     # experts outside the kept groups are out, not zero


def test_plain_expert_clamps_before_the_gate():
    w = {"e.gate": torch.eye(3, dtype=torch.float64), "e.up": torch.eye(3, dtype=torch.float64), "e.down": torch.eye(3, dtype=torch.float64)}
    n = torch.tensor([[5.0, -5.0, 0.5]], dtype=torch.float64)
    y = plain.expert(2.0, w, "e.", n, plain.Products(False))
    sig = lambda g: 1.0 / (1.0 + math.exp(-1.702 * g))
    want = [2.0 * sig(2.0) * (2.0 + 1.0), -5.0 * sig(-5.0) * (-2.0 + 1.0), 0.5 * sig(0.5) * 1.5]     # the gate has no lower limit
    assert torch.allclose(y[0], torch.tensor(want, dtype=torch.float64))


def test_plain_model_is_causal_and_every_mechanism_matters():
    cfg = CONFIGS["A"]
    w = make_weights(cfg, 1)
    ids = list(range(3, 60))
    full = plain.forward(cfg, w, ids)
    assert torch.allclose(plain.forward(cfg, w, ids[:30]), full[:30])
    for name in ("l0.shift", "l1.mix.temp", "l1.mix.q.norm", "l2.mix.k.norm", "l1.mlp.correction", "loop.step", "l3.mix.v.b", "l0.mix.o.b"):
        w2 = dict(w)
        w2[name] = w[name] + torch.linspace(0.5, 3.0, w[name].numel()).view_as(w[name])
        assert (plain.forward(cfg, w2, ids) - full).abs().max() > 1e-3, name
    for path, value in ((("layers", 0, "mixer", "mask", "size"), 25), (("layers", 2, "mixer", "softcap"), 60.0),
                        (("loop", "times"), 1), (("layers", 1, "mlp", "router", "groups", "keep"), 3),
                        (("layers", 3, "mlp", "expert", "limit"), 5.0), (("embedding", "scale"), 2.0)):
        assert (plain.forward(_broken(path, value), w, ids) - full).abs().max() > 1e-3, path
    # chunks: a token at a chunk's start sees nothing of the chunk before, in a model of attention alone without a shift
    one = _config(50, 32, [layer(attention(2, 1, 8, 8, 5), None)])
    w1 = make_weights(one, 2)
    w1["l0.shift"] = torch.zeros(32)
    a, b = list(range(10, 22)), list(range(30, 35)) + list(range(15, 22))
    assert torch.allclose(plain.forward(one, w1, a)[5:], plain.forward(one, w1, b)[5:])
    assert not torch.allclose(plain.forward(one, w1, a)[4], plain.forward(one, w1, b)[4])
