"""Bilurax through the engine against the plain implementation (tests/plain_bilurax.py, float64).

Three small models that differ in every size and option (tests/bilurax_models.py) are run whole, as a prompt
followed by single tokens, in portions down to two tokens, and as mixed batches in a pool whose pages and slots
are used again; single mechanisms are isolated by one-layer configurations; weights are bent where random ones
would hide a fault (a far key among hundreds, a key at a chunk's edge, the token before, one group among many).

Bounds.  The measure is the RMS over the vocabulary of the logits' difference (mean taken off) over the RMS of
the wanted logits, the largest over the rows.  float32: the engine computes what the plain implementation
computes in another order of float additions: 2e-4.  bfloat16: what rounding alone does depends on the model, so it
is measured: the plain implementation is run once more with the operands and results of its products rounded to
bfloat16 values, and the engine may be three times as far from the exact logits as that run is (at least 2e-2).
The bfloat16 runs use routers whose choices no rounding can turn (bilurax_models.make_weights says why); routers
that choose token by token run in float32.  A lost key, chunk edge, shift or expert moves the logits by their own
size, and where a test rests on that it checks it with the plain implementation first.
"""
import copy

import numpy as np
import pytest
import torch

import plain_bilurax as plain
from bilurax_models import CONFIGS, _config, attention, dense, layer, make_weights, moe, rel_error, write_model

pytestmark = pytest.mark.gpu

BOUND_F32 = 2e-4
_cache = {}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """(name, dtype) -> (config, weights, model folder); the bfloat16 models have decisive routers."""
    base = tmp_path_factory.mktemp("bilurax")
    out = {}
    for i, (name, cfg) in enumerate(sorted(CONFIGS.items())):
        for dtype in ("float32", "bfloat16"):
            w = make_weights(cfg, seed=300 + i, decisive_router=dtype == "bfloat16")
            out[name, dtype] = (cfg, w, write_model(cfg, w, str(base / f"{name}_{dtype}")))
    return out


def _engine(model_dir, dtype, max_tokens=512, page_size=16, max_requests=4):
    from sandyrt_b200.engine.step import Engine
    from sandyrt_b200.models.model import load_model

    model = load_model(model_dir, device="cuda:0", dtype=getattr(torch, dtype))
    eng = Engine(model, max_tokens=max_tokens, page_size=page_size, max_requests=max_requests)
    eng.cache.device_caches.poison()
    return eng


def _tokens(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).tolist()


def _want(cfg, w, ids):
    key = (id(w), tuple(ids))
    if key not in _cache:
        _cache[key] = [plain.forward(cfg, w, ids).numpy(), None]
    return _cache[key][0]


def _bound(cfg, w, ids, dtype):
    if dtype == "float32":
        return BOUND_F32
    want = _want(cfg, w, ids)
    entry = _cache[(id(w), tuple(ids))]
    if entry[1] is None:
        entry[1] = rel_error(plain.forward_rounded(cfg, w, ids).numpy(), want)
    return max(2e-2, 3 * entry[1])


def _run_cuts(eng, rid, ids, cuts, release=True):
    from sandyrt_b200.engine.step import StepEntry

    rows, pos = [], 0
    for n in cuts:
        rows.append(eng.step([StepEntry(rid, ids[pos:pos + n], list(range(n)))]).cpu().numpy().copy())
        pos += n
    assert pos == len(ids)
    eng.check_status()
    if release:
        eng.release(rid)
    return np.concatenate(rows, axis=0)


def _check(got, model, ids, dtype, what):
    cfg, w = model
    e, bound = rel_error(got, _want(cfg, w, ids)), _bound(cfg, w, ids, dtype)
    assert e < bound, f"{what}: relative error {e:.3e} (bound {bound:.1e})"


# ---- whole models under every way of cutting the work -------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompts_and_first_tokens(models, name, dtype):
    cfg, w, path = models[name, dtype]
    eng = _engine(path, dtype)
    for i, n in enumerate([1, 2, 5, 33, 150]):
        ids = _tokens(cfg, n, seed=i)
        _check(_run_cuts(eng, f"r{i}", ids, [n]), (cfg, w), ids, dtype, f"{name}: whole prompt of {n}")
    eng.cache.alloc.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_prompt_then_single_tokens(models, name, dtype):
    """Most of the request in one step, the last 60 tokens one by one (the later ones replay a recorded graph); the
    single tokens cross the edges of every model's chunks."""
    cfg, w, path = models[name, dtype]
    eng = _engine(path, dtype)
    ids = _tokens(cfg, 131, seed=7)
    got = _run_cuts(eng, "r", ids, [71] + [1] * 60)
    _check(got, (cfg, w), ids, dtype, f"{name}: prompt + 60 single tokens")
    assert eng.graph_replays > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_portions_of_changing_size(models, name, dtype):
    """Portions that end before, at and behind the chunks' edges (24, 40, 48, 64, 7, 33), down to two tokens."""
    cfg, w, path = models[name, dtype]
    eng = _engine(path, dtype)
    ids = _tokens(cfg, 101, seed=11)
    for cuts in ([24, 24, 24, 24, 5], [2, 3, 17, 16, 15, 31, 2, 13, 2], [1, 2, 1, 3, 94], [64, 37], [16, 16, 32, 1, 1, 35],
                 [23, 2, 14, 2, 7, 1, 23, 29], [47, 1, 2, 14, 1, 36]):
        assert sum(cuts) == len(ids)
        _check(_run_cuts(eng, "r", ids, cuts), (cfg, w), ids, dtype, f"{name}: portions {cuts}")
    eng.cache.alloc.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens_in_every_division(models, name, dtype):
    """The first few tokens of a request: the token before the first is zeros, a lone token's softmax holds itself."""
    cfg, w, path = models[name, dtype]
    eng = _engine(path, dtype)
    ids = _tokens(cfg, 6, seed=13)
    for cuts in ([1] * 6, [2, 2, 2], [1, 5], [5, 1], [3, 1, 2], [6]):
        _check(_run_cuts(eng, "r", ids, cuts), (cfg, w), ids, dtype, f"first tokens as {cuts}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_mixed_batches_with_pages_and_slots_used_again(models, name, dtype):
    """Up to four live requests, portions of some beside single tokens of others; the pool holds 12 pages of 16
    tokens for requests that need 24 in all, pages poisoned.  Each request's rows must equal what it gives alone
    (its token-shift state sits in a slot that other requests held before)."""
    from sandyrt_b200.engine.step import StepEntry

    cfg, w, path = models[name, dtype]
    eng = _engine(path, dtype, max_tokens=192, page_size=16, max_requests=4)
    lengths = [37, 50, 21, 64, 45, 30, 58, 17]
    prompts = [_tokens(cfg, n, seed=20 + i) for i, n in enumerate(lengths)]
    rng = np.random.default_rng(1)
    fed = [0] * len(prompts)
    got = [[] for _ in prompts]
    live, nxt, slots_seen = [], 0, []
    while nxt < len(prompts) or live:
        while nxt < len(prompts) and len(live) < 4:
            if sum(-(-lengths[r] // 16) for r in live) + -(-lengths[nxt] // 16) > 12:
                break
            live.append(nxt)
            nxt += 1
        entries = []
        for r in live:
            left = lengths[r] - fed[r]
            n = int(rng.integers(2, min(left, 19) + 1)) if left > 8 and rng.random() < 0.6 else 1
            entries.append(StepEntry(r, prompts[r][fed[r]:fed[r] + n], list(range(n))))
        if rng.random() < 0.3 and len(entries) > 1:
            entries.pop(int(rng.integers(0, len(entries))))
        out = eng.step(entries).cpu().numpy()
        row = 0
        for e in entries:
            n = len(e.tokens)
            got[e.rid].append(out[row:row + n].copy())
            row += n
            fed[e.rid] += n
            slots_seen.append((e.rid, eng.cache.alloc.slot(e.rid)))
        for r in list(live):
            if fed[r] == lengths[r]:
                eng.release(r)
                live.remove(r)
        eng.cache.alloc.check()
    eng.check_status()
    assert len({s for _, s in slots_seen}) <= 4 and len({r for r, _ in slots_seen}) == 8      # slots were used again
    for r, ids in enumerate(prompts):
        _check(np.concatenate(got[r], axis=0), (cfg, w), ids, dtype, f"{name}: mixed request {r}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_a_batch_gives_each_request_what_it_gives_alone(models, name, dtype):
    """Unequal requests in one step against each alone: same rows, beyond rounding.  The experts see other
    neighbours in their groups, the attention other tiles, the token shift other rows before a request's first."""
    from sandyrt_b200.engine.step import StepEntry

    cfg, w, path = models[name, dtype]
    eng = _engine(path, dtype)
    prompts = [_tokens(cfg, n, seed=40 + n) for n in (70, 3, 29, 1)]
    alone = [_run_cuts(eng, f"a{i}", p, [len(p)]) for i, p in enumerate(prompts)]
    out = eng.step([StepEntry(f"b{i}", p, list(range(len(p)))) for i, p in enumerate(prompts)]).cpu().numpy()
    row = 0
    for i, p in enumerate(prompts):
        e = rel_error(out[row:row + len(p)], alone[i])
        assert e < (1e-5 if dtype == "float32" else 2e-2), f"request {i} in a batch differs from itself alone by {e:.2e}"
        row += len(p)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_across_page_borders_and_chunk_edges(models, dtype):
    """300 single tokens behind a short prompt, pages of 8: every page border and a dozen chunk edges (24 and 40
    positions) are crossed by a decoded token."""
    cfg, w, path = models["A", dtype]
    eng = _engine(path, dtype, max_tokens=512, page_size=8)
    ids = _tokens(cfg, 310, seed=3)
    got = _run_cuts(eng, "r", ids, [10] + [1] * 300)
    _check(got, (cfg, w), ids, dtype, "A: 300 decoded tokens")


# ---- single mechanisms --------------------------------------------------------------------------------
def _one_model(tmp_path, cfg, seed, bend=None, decisive=False):
    w = make_weights(cfg, seed, decisive_router=decisive)
    if bend:
        bend(w)
        w = {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}
    return w, write_model(cfg, w, str(tmp_path / f"m{seed}"))


ONE_LAYER = {
    "attention alone, values wider than keys": lambda: [layer(attention(3, 1, 24, 40, 30), None)],
    "attention alone, keys wider than values": lambda: [layer(attention(4, 2, 48, 16, 17, softcap=4.0), None)],
    "attention alone, a chunk beyond the sequence": lambda: [layer(attention(2, 2, 32, 32, 4096), None)],
    "dense feed-forward": lambda: [layer(attention(1, 1, 8, 8, 16), dense(72))],
    "routed feed-forward, one group": lambda: [layer(attention(1, 1, 8, 8, 16), moe(6, 3, 24, scale=1.7, limit=0.8))],
    "routed feed-forward, groups": lambda: [layer(attention(1, 1, 8, 8, 16), moe(12, 3, 16, groups=4, keep=2, scale=0.6))],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(ONE_LAYER))
def test_each_mechanism_alone(tmp_path, which, dtype):
    cfg = _config(61, 48, ONE_LAYER[which](), eps=1e-5, logit_softcap=9.0, embedding_scale=2.0)
    w, path = _one_model(tmp_path, cfg, seed=5, decisive=dtype == "bfloat16")
    eng = _engine(path, dtype)
    ids = _tokens(cfg, 90, seed=1)
    _check(_run_cuts(eng, "r", ids, [90]), (cfg, w), ids, dtype, f"{which}, whole")
    _check(_run_cuts(eng, "r", ids, [40, 2, 30] + [1] * 18), (cfg, w), ids, dtype, f"{which}, in portions")


def _without(cfg, w, ids, change_cfg=None, change_w=None):
    """Logits of the plain implementation with one thing changed, to show that the thing matters."""
    cfg2, w2 = copy.deepcopy(cfg), dict(w)
    if change_cfg:
        change_cfg(cfg2)
    if change_w:
        change_w(w2)
    return plain.forward(cfg2, w2, ids).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds(tmp_path, dtype):
    """Attention alone, 400 tokens in one chunk.  Queries and keys are normed, so a larger projection sharpens
    nothing; the temperatures do, up to the cap of 12: every query then looks at one or two keys, mostly far back,
    and a key that is lost or off by one moves the logits by far more than the bound."""
    cfg = _config(53, 64, [layer(attention(4, 2, 16, 16, 512, softcap=12.0, scale=1.0), None)], eps=1e-5, logit_softcap=30.0)

    def sharp(w):
        w["l0.mix.temp"] = torch.full((4,), 3.0)
        w["l0.shift"] *= 0.2

    w, path = _one_model(tmp_path, cfg, seed=9, bend=sharp)
    ids = _tokens(cfg, 400, seed=2)
    want = _want(cfg, w, ids)
    # the cap matters too: without it the sharpest scores are sharper still
    assert rel_error(_without(cfg, w, ids, change_cfg=lambda c: c["layers"][0]["mixer"].update(softcap=1e6)), want) > 0.05
    eng = _engine(path, dtype, max_tokens=512, page_size=16)
    _check(_run_cuts(eng, "r", ids, [400]), (cfg, w), ids, dtype, "sharp scores, whole")
    _check(_run_cuts(eng, "r", ids, [250, 100, 18] + [1] * 32), (cfg, w), ids, dtype, "sharp scores, portions and single tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("chunk", [24, 37])
def test_keys_just_inside_and_just_outside_a_chunk(tmp_path, chunk, dtype):
    """Sharp scores and chunks of 24 (a page and a half) or 37 positions.  A chunk that is one position longer, shorter
    or counted from elsewhere lets another key win for some query; the plain implementation shows first that each
    of these moves the logits by their own size.  Whole, in portions that end one token before, at and behind
    an edge, and with the tokens around the edges decoded one by one."""
    cfg = _config(53, 64, [layer(attention(2, 1, 16, 16, chunk, softcap=14.0, scale=1.0), None)], eps=1e-5, logit_softcap=30.0)

    def sharp(w):
        w["l0.mix.temp"] = torch.full((2,), 4.0)
        w["l0.shift"] *= 0.1

    w, path = _one_model(tmp_path, cfg, seed=12, bend=sharp)
    n = 4 * chunk + 9
    ids = _tokens(cfg, n, seed=6)
    want = _want(cfg, w, ids)
    for other in (chunk - 1, chunk + 1):
        assert rel_error(_without(cfg, w, ids, change_cfg=lambda c: c["layers"][0]["mixer"]["mask"].update(size=other)), want) > 0.2
    eng = _engine(path, dtype, max_tokens=512, page_size=16)
    _check(_run_cuts(eng, "r", ids, [n]), (cfg, w), ids, dtype, "chunk edges, whole")
    _check(_run_cuts(eng, "r", ids, [chunk - 1, 1, 1, chunk - 1, chunk + 1, 2, n - 3 * chunk - 3]), (cfg, w), ids, dtype,
           "chunk edges, portions around the edges")
    _check(_run_cuts(eng, "r", ids, [2 * chunk - 3] + [1] * (n - 2 * chunk + 3)), (cfg, w), ids, dtype, "chunk edges, decoded over two edges")
    # a portion that starts in the middle of a chunk still counts chunks from position 0
    _check(_run_cuts(eng, "r", ids, [chunk // 2, chunk, chunk, n - 2 * chunk - chunk // 2]), (cfg, w), ids, dtype, "chunk edges, portions out of step")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_token_before_is_all_the_mixer_reads(tmp_path, dtype):
    """A shift of one everywhere: the mixer reads the token before and nothing of its own, the first token reads
    zeros.  Losing the state between steps (or taking another request's) then changes everything, which the plain
    implementation shows with the shift switched off.  Portions down to one token, two layers, a looped span: every
    run of a layer keeps a token of its own."""
    cfg = _config(47, 48, [layer(attention(2, 2, 8, 24, 16), dense(40)), layer(attention(3, 1, 16, 8, 64), None)],
                  eps=1e-5, logit_softcap=20.0, embedding_scale=1.5, loop=(0, 2, 2))

    def bend(w):
        w["l0.shift"] = torch.ones(48)
        w["l1.shift"] = torch.ones(48)

    w, path = _one_model(tmp_path, cfg, seed=14, bend=bend)
    ids = _tokens(cfg, 60, seed=5)
    want = _want(cfg, w, ids)

    def off(w2):
        w2["l0.shift"] = torch.zeros(48)
        w2["l1.shift"] = torch.zeros(48)

    assert rel_error(_without(cfg, w, ids, change_w=off), want) > 0.2
    eng = _engine(path, dtype)
    for cuts in ([60], [1] * 60, [2] * 30, [17, 1, 2, 1, 39], [59, 1]):
        _check(_run_cuts(eng, "r", ids, cuts), (cfg, w), ids, dtype, f"shift of one, {cuts[:5]}")


def test_groups_are_judged_by_their_two_best_and_scores_may_be_negative(tmp_path):
    """float32.  Corrections push every choice score below zero, and one expert of each group far above its
    neighbours: the group with the single best expert is then often not the group with the best pair, and an expert
    outside the kept groups would win if it counted as zero instead of being out of the race (both checked on the
    plain routing first).  The token-by-token choice is then the engine's own."""
    cfg = _config(59, 48, [layer(attention(2, 1, 8, 8, 32), moe(12, 3, 16, groups=4, keep=2, scale=1.3, limit=1.5))],
                  eps=1e-5, logit_softcap=25.0)

    def bend(w):
        c = -2.0 + 0.3 * torch.randn(12, generator=torch.Generator().manual_seed(3))
        c[0::3] += 0.5                                            # one strong expert a group
        w["l0.mlp.correction"] = c
        w["l0.mlp.router"] *= 2.0

    w, path = _one_model(tmp_path, cfg, seed=16, bend=bend)
    ids = _tokens(cfg, 200, seed=7)
    assert plain.router_margin(cfg, w, ids) > 1e-5
    w64 = {k: v.to(torch.float64) for k, v in w.items()}
    x = w64["embed"][torch.tensor(ids)]
    u = plain.token_shift(plain.rms_norm(x, w64["l0.norm1"], 1e-5), w64["l0.shift"])
    x = x + plain.attention(cfg["layers"][0]["mixer"], 1e-5, w64, "l0.mix.", u, plain.Products(False))
    n = plain.rms_norm(x, w64["l0.norm2"], 1e-5)
    c = torch.sigmoid(n @ w64["l0.mlp.router"].t()) + w64["l0.mlp.correction"]
    chosen, _, _ = plain.route(cfg["layers"][0]["mlp"]["router"], w64, "l0.mlp.", n, plain.Products(False))
    assert float(c.max()) < 0.0                                                    # all negative
    assert ((c.argmax(-1) // 3)[:, None] != chosen // 3).all(-1).float().mean() > 0.05  # the single best expert's group is often out
    assert len({tuple(sorted(r)) for r in chosen.tolist()}) > 6                   # and the choice changes from token to token
    eng = _engine(path, "float32")
    _check(_run_cuts(eng, "r", ids, [200]), (cfg, w), ids, "float32", "groups, whole")
    _check(_run_cuts(eng, "r", ids, [33, 2, 140, 5] + [1] * 20), (cfg, w), ids, "float32", "groups, portions and single tokens")


def test_routers_that_choose_token_by_token(tmp_path):
    """float32, ordinary routers in a looped span: the choices change from token to token and from pass to pass, a
    step of many tokens groups them by expert while single tokens go one by one."""
    cfg = _config(89, 56, [layer(attention(2, 1, 8, 16, 20), moe(8, 2, 16, groups=2, keep=1, scale=2.0, limit=2.0)),
                           layer(attention(2, 2, 8, 8, 50), moe(9, 3, 24, groups=3, keep=3, scale=0.7))],
                  eps=1e-5, logit_softcap=15.0, embedding_scale=2.0, loop=(0, 1, 3))
    w, path = _one_model(tmp_path, cfg, seed=31)
    ids = _tokens(cfg, 260, seed=8)
    assert plain.router_margin(cfg, w, ids) > 1e-5
    eng = _engine(path, "float32")
    _check(_run_cuts(eng, "r", ids, [260]), (cfg, w), ids, "float32", "token-by-token routing, whole")
    _check(_run_cuts(eng, "r", ids, [33, 2, 190, 5] + [1] * 30), (cfg, w), ids, "float32", "token-by-token routing, portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_experts_clamp(tmp_path, dtype):
    """A limit of 0.25 cuts most of what gate and up give (the plain implementation without a limit lands elsewhere);
    the gate is cut from above only, the other factor on both sides."""
    cfg = _config(53, 48, [layer(attention(1, 1, 8, 8, 16), moe(4, 2, 24, scale=3.0, limit=0.25))], eps=1e-5, logit_softcap=30.0)
    w, path = _one_model(tmp_path, cfg, seed=18, decisive=True)
    ids = _tokens(cfg, 80, seed=9)
    want = _want(cfg, w, ids)
    assert rel_error(_without(cfg, w, ids, change_cfg=lambda c: c["layers"][0]["mlp"]["expert"].update(limit=1e9)), want) > 0.2
    eng = _engine(path, dtype)
    _check(_run_cuts(eng, "r", ids, [80]), (cfg, w), ids, dtype, "clamped experts, whole")
    _check(_run_cuts(eng, "r", ids, [50, 2] + [1] * 28), (cfg, w), ids, dtype, "clamped experts, portions and single tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_heads_of_64_in_long_prompts(tmp_path, dtype):
    """Heads of 64 take the tcgen05 prompt kernel in bfloat16: chunks of 210 and 96 positions cut through its tiles of 128
    queries and 128 keys, portions start inside chunks and tiles, then single tokens pass a chunk's edge."""
    cfg = _config(97, 128, [layer(attention(4, 2, 64, 64, 210, softcap=10.0), dense(64)),
                            layer(attention(2, 1, 64, 64, 96, softcap=25.0), None)], eps=1e-5, logit_softcap=20.0)
    w, path = _one_model(tmp_path, cfg, seed=21)
    eng = _engine(path, dtype, max_tokens=1024)
    ids = _tokens(cfg, 420, seed=2)
    _check(_run_cuts(eng, "r", ids, [420]), (cfg, w), ids, dtype, "heads of 64, whole")
    _check(_run_cuts(eng, "r", ids, [130, 2, 209, 60] + [1] * 19), (cfg, w), ids, dtype, "heads of 64, portions and single tokens")


def test_options_at_their_edges(tmp_path):
    """float32.  A span that runs once, a span of the last layer alone, every expert of the kept groups chosen, as
    many key/value heads as query heads, a chunk of one position, a layer without a feed-forward whose file still
    holds its second norm (it is read past), an embedding scale and temperatures of one."""
    a = _config(67, 40, [layer(attention(3, 3, 8, 8, 1), moe(8, 4, 8, groups=4, keep=2)), layer(attention(2, 1, 8, 16, 9), None)],
                eps=1e-5, logit_softcap=50.0, embedding_scale=1.0, loop=(0, 2, 1))
    b = _config(67, 40, [layer(attention(1, 1, 16, 8, 13), dense(24)), layer(attention(2, 2, 8, 8, 5), moe(3, 1, 8))],
                eps=1e-5, logit_softcap=5.0, embedding_scale=1.0, loop=(1, 2, 4))
    for k, cfg in enumerate((a, b)):
        w = make_weights(cfg, seed=41 + k)
        for name in w:
            if name.endswith("temp"):
                w[name] = torch.ones_like(w[name])
        on_disk = dict(w)
        if k == 0:
            on_disk["l1.norm2"] = torch.ones(40)
        path = write_model(cfg, on_disk, str(tmp_path / f"edges{k}"))
        ids = _tokens(cfg, 70, seed=9 + k)
        assert plain.router_margin(cfg, w, ids) > 1e-5
        eng = _engine(path, "float32")
        _check(_run_cuts(eng, "r", ids, [70]), (cfg, w), ids, "float32", f"edges {k}, whole")
        _check(_run_cuts(eng, "r", ids, [31, 2, 30] + [1] * 7), (cfg, w), ids, "float32", f"edges {k}, in portions")


# ---- the entry point --------------------------------------------------------------------------------------
def test_greedy_generation_through_the_entry_point(models):
    """LLM.generate (scheduler, prompt portions, decode bursts) on three requests at once, float32: the same tokens
    as greedy decoding with the plain implementation, wherever its top two logits are clearly apart."""
    from sandyrt_b200.engine.llm import LLM

    cfg, w, path = models["A", "float32"]
    llm = LLM(path, dtype="float32", cache_tokens=1024, max_live=4, prefill_chunk_tokens=24, max_step_tokens=64)
    prompts = [_tokens(cfg, n, seed=60 + n) for n in (5, 40, 71)]
    outs = llm.generate(prompts, max_tokens=20)
    for p, r in zip(prompts, outs):
        assert r.finish_reason == "length" and len(r.output_ids) == 20
        ids = list(p)
        for tok in r.output_ids:
            l = _want(cfg, w, ids)[-1]
            top2 = np.sort(l)[-2:]
            if top2[1] - top2[0] > 1e-3:
                assert tok == int(np.argmax(l)), f"token {len(ids) - len(p)} of the request with {len(p)} prompt tokens"
            ids.append(tok)
