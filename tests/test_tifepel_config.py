"""Tifepel without a GPU: the configuration and its checks, the model description (parts, run order of a looped span,
tensor names, cache entries with the block's and the embedding's states), and properties of the plain implementation
that the GPU tests lean on."""
import copy
import math

import pytest
import torch

import plain_tifepel as plain
from tifepel_models import CONFIGS, _config, attention, layer, make_weights, mamba2, moe, tensor_shapes

from sandyrt_b200.config.base import ConfigError, config_from_normalised
from sandyrt_b200.config.tifepel import TifepelConfig


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_description_names_every_tensor_with_its_shape(name):
    from sandyrt_b200.models.model import build_model

    cfg = config_from_normalised(CONFIGS[name])
    assert isinstance(cfg, TifepelConfig) and cfg.vocab_size == CONFIGS[name]["vocab"]
    cfg.validate()
    got = {k: list(v.shape) for k, v in build_model(cfg).tensor_requests().items()}
    assert got == tensor_shapes(CONFIGS[name])


def test_a_bias_table_takes_its_length_from_the_file():
    """Without `bias_rows` the description asks for a table of any length with one column a head."""
    from sandyrt_b200.models.model import build_model

    raw = copy.deepcopy(CONFIGS["A"])
    for l in raw["layers"]:
        l["mixer"].pop("bias_rows", None)
    got = {k: list(v.shape) for k, v in build_model(config_from_normalised(raw)).tensor_requests().items()}
    assert got["l0.mix.rel"] == [-1, 4] and got["l2.mix.rel"] == [-1, 2]
    want = tensor_shapes(CONFIGS["A"])
    assert {k: v for k, v in got.items() if not k.endswith(".rel")} == {k: v for k, v in want.items() if not k.endswith(".rel")}


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_run_order_and_cache_entries(name):
    """Every pass of a looped span is a call of the same layers with a cache entry of its own, nothing runs between the
    passes, and the embedding's state has the entry behind the layers'."""
    from sandyrt_b200.models.model import describe

    raw = CONFIGS[name]
    spec = describe(config_from_normalised(raw))
    order = plain.run_order(raw)
    assert [c.layer for c in spec.schedule] == order
    assert [c.cache for c in spec.schedule] == list(range(len(order)))
    assert all(c.remix is None for c in spec.schedule) and len(spec.remixes) == 0
    assert spec.embedding_cache == len(order) and spec.n_caches() == len(order) + 1
    assert spec.streams == raw["streams"] and spec.max_positions == raw["max_positions"]
    for l, src in zip(spec.layers, raw["layers"]):
        assert l.block == "wrapped_sublayers" and not l.norms
        assert l.mixer.kind == {"attention": "biased_attention", "mamba2": "state_space"}[src["type"]]
        assert l.feed_forward.kind == ("routed_experts" if src["mlp"] else "none")
        assert sorted(l.wraps) == (["feed_forward", "mixer"] if src["mlp"] else ["mixer"])
        for wrap in l.wraps.values():
            assert wrap.kind == "hyper_gated_conv" and wrap.params["streams"] == raw["streams"] and wrap.params["taps"] == raw["canon"]["taps"]
    assert spec.embedding.kind == "bigram_embedding" and spec.position.kind == "learned_absolute"
    assert spec.head.params["tied"] is False and spec.final_norm.kind == "layernorm" and spec.final_norm.params["bias"] is False


def test_config_round_trip_and_constants_reach_the_parts():
    from sandyrt_b200.models.model import describe

    raw = CONFIGS["A"]
    cfg = TifepelConfig.from_dict(raw)
    assert TifepelConfig.from_dict(cfg.to_dict()) == cfg
    assert cfg.to_dict()["layers"] == raw["layers"] and cfg.to_dict()["loop"] == raw["loop"]
    assert cfg.to_dict()["embedding"] == raw["embedding"] and cfg.to_dict()["canon"] == raw["canon"]
    spec = describe(cfg)
    m = spec.layers[0].mixer.params
    src = raw["layers"][0]["mixer"]
    assert (m["n_heads"], m["n_kv_heads"], m["qk_dim"], m["v_dim"]) == (src["heads"], src["kv_heads"], src["dim"], src["vdim"])
    assert m["scale"] == src["scale"] and m["q_pos_coef"] == src["q_temp"]["coef"] and m["q_pos_every"] == src["q_temp"]["every"]
    assert m["bias_max"] == src["bias_max"] and m["distance_bias"] is True and m["qk_unit_norm"] is True
    s = spec.layers[1].mixer.params
    src = raw["layers"][1]["mixer"]
    assert (s["n_heads"], s["n_groups"], s["state"], s["v_dim"], s["conv_taps"], s["norm_groups"]) == \
           (src["heads"], src["groups"], src["state"], src["vdim"], src["conv"], src["norm_groups"])
    f = spec.layers[0].feed_forward.params
    r = raw["layers"][0]["mlp"]
    assert (f["n_experts"], f["n_identity"], f["top"], f["inner"], f["shared_inner"]) == \
           (r["router"]["experts"], r["router"]["identity"], r["router"]["top"], r["expert"]["ff"], r["shared"]["ff"])
    assert f["scoring"] == "softmax_all" and f["activation"] == "silu_glu" and f["correction"] is True
    e = spec.embedding.params
    assert (e["buckets"], e["mul_prev"], e["mul_cur"]) == (31, 7, 3)


BAD = {
    "no streams": lambda c: c.pop("streams"),
    "nine streams": lambda c: c.update(streams=9),
    "no taps": lambda c: c["canon"].update(taps=0),
    "an unknown layer type": lambda c: c["layers"][0].update(type="lstm"),
    "heads that do not divide": lambda c: c["layers"][0]["mixer"].update(kv_heads=3),
    "groups that do not divide": lambda c: c["layers"][1]["mixer"].update(groups=3),
    "a state beyond the kernels": lambda c: c["layers"][1]["mixer"].update(state=300),
    "norm groups that do not divide": lambda c: c["layers"][1]["mixer"].update(norm_groups=5),
    "more experts chosen than there are": lambda c: c["layers"][0]["mlp"]["router"].update(top=9),
    "a bias table whose far end lies in its first half": lambda c: c["layers"][0]["mixer"].update(bias_max=3),
    "a loop beyond the layers": lambda c: c["loop"].update(stop=7),
    "a dense feed-forward": lambda c: c["layers"][0]["mlp"].update(kind="dense"),
    "no pair table": lambda c: c["embedding"].pop("bigram"),
    "a step of zero positions": lambda c: c["layers"][0]["mixer"]["q_temp"].update(every=0),
}


@pytest.mark.parametrize("what", sorted(BAD))
def test_refusals_name_the_key(what):
    raw = copy.deepcopy(CONFIGS["A"])
    BAD[what](raw)
    with pytest.raises(ConfigError):
        config_from_normalised(raw).validate()


def test_cache_layout_has_pages_and_states():
    """Attention layers get pages and the block's tails as a state; state-space layers one state that holds the matrix,
    the mixer's tail and the block's tails; the embedding one integer."""
    from sandyrt_b200.models.model import build_model

    raw = CONFIGS["A"]
    specs = build_model(config_from_normalised(raw)).cache_specs()
    w, taps = raw["width"], raw["canon"]["taps"]
    order = plain.run_order(raw)
    assert len(specs) == len(order) + 1
    for spec, i in zip(specs, order):
        l = raw["layers"][i]
        m = l["mixer"]
        tails = (2 if l["mlp"] else 1) * (taps - 1) * w
        if l["type"] == "attention":
            assert spec["kind"] == "paged_state" and spec["n_kv_heads"] == m["kv_heads"] and spec["head_dim"] == 16 * math.ceil(max(m["dim"], m["vdim"]) / 16)
            assert spec["shape"] == [tails] and spec["dtype"] == "float32"
        else:
            own = m["heads"] * m["vdim"] * m["state"] + (m["conv"] - 1) * (m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"])
            assert spec["kind"] == "state" and spec["shape"] == [own + tails]
    assert specs[-1]["kind"] == "state" and specs[-1]["shape"] == [1] and specs[-1]["dtype"] == "int32"


# ---- the plain implementation --------------------------------------------------------------------------------------
def test_plain_buckets():
    rows, far = 24, 150
    b = [plain.distance_bucket(n, rows, far) for n in range(400)]
    assert b[:12] == list(range(12)) and b[12] == 12 and b[far] == rows - 1 and b[399] == rows - 1
    assert all(y >= x for x, y in zip(b, b[1:])) and set(b) == set(range(rows))
    assert plain.distance_bucket(1, 2, 2) == 1 and plain.distance_bucket(0, 2, 2) == 0


def test_plain_is_causal_and_keeps_no_state_between_sequences():
    cfg = CONFIGS["A"]
    w = make_weights(cfg, seed=1)
    ids = list(range(3, 40))
    full = plain.forward(cfg, w, ids)
    assert torch.allclose(plain.forward(cfg, w, ids[:20]), full[:20], atol=1e-9)
    other = list(ids)
    other[30] = 99
    assert torch.allclose(plain.forward(cfg, w, other)[:30], full[:30], atol=1e-9)
    assert not torch.allclose(plain.forward(cfg, w, other)[31], full[31], atol=1e-3)      # the token before enters the pair table


def test_plain_convolution_and_recurrence():
    h = torch.randn(9, 5, dtype=torch.float64)
    taps = torch.randn(5, 3, dtype=torch.float64)
    c = plain.causal_conv(h, taps)
    assert torch.allclose(c[0], h[0] * taps[:, 2]) and torch.allclose(c[4], h[2] * taps[:, 0] + h[3] * taps[:, 1] + h[4] * taps[:, 2])
    # a state-space layer whose decay is zero forgets everything but the token itself
    cfg = _config(31, 16, [layer(mamba2(2, 1, 4, 8, conv=1, norm_groups=1), None)], streams=1, taps=1)
    w = make_weights(cfg, seed=2)
    w["l0.mix.A_log"] = torch.full((2,), 5.0)
    w["l0.mix.dt_bias"] = torch.full((2,), 3.0)
    a = plain.forward(cfg, w, [1, 2, 3, 4])
    b = plain.forward(cfg, w, [9, 8, 3, 4])
    assert torch.allclose(a[3], b[3], atol=1e-6)


def test_plain_routing_weights_are_the_scores_themselves():
    cfg = _config(31, 16, [layer(attention(1, 1, 8, 8, rows=4, far=8), moe(3, 2, 2, 8))])
    w = {k: v.to(torch.float64) for k, v in make_weights(cfg, seed=3).items()}
    h = torch.randn(7, 16, dtype=torch.float64)
    chosen, weights, margin = plain.route(cfg["layers"][0]["mlp"]["router"], w, "l0.mlp.", h, plain.Products(False))
    s = torch.softmax(h @ w["l0.mlp.router"].t(), -1)
    assert torch.allclose(weights, s.gather(1, chosen)) and (weights.sum(-1) < 1.0).all() and (margin > 0).all()
