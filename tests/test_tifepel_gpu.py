"""Tifepel through the engine against the plain implementation (tests/plain_tifepel.py, float64).

Three small models that differ in every size and option (tests/tifepel_models.py) are run whole, as a prompt
followed by single tokens, in portions down to two tokens, and as mixed batches in a pool whose pages and slots
are used again; single mechanisms are isolated by one-layer configurations; weights are bent where random ones
would hide a fault (a far key among hundreds, the edges of the bias table's buckets, a state that must still hold
its first token, the token before).

Bounds.  The measure is the RMS over the vocabulary of the logits' difference (mean taken off) over the RMS of
the wanted logits, the largest over the rows.  float32: the engine computes what the plain implementation
computes in another order of float additions: 2e-4.  bfloat16: what rounding alone does depends on the model, so it
is measured: the plain implementation is run once more with the operands and results of its products rounded to
bfloat16 values, and the engine may be three times as far from the exact logits as that run is (at least 2e-2).
The bfloat16 runs use routers whose choices no rounding can turn (tifepel_models.make_weights says why); routers
that choose token by token run in float32.  Where a test rests on a mechanism mattering, it checks that with the
plain implementation first.
"""
import copy

import numpy as np
import pytest
import torch

import plain_tifepel as plain
from tifepel_models import CONFIGS, _config, attention, layer, make_weights, mamba2, moe, rel_error, write_model

pytestmark = pytest.mark.gpu

BOUND_F32 = 2e-4
_cache = {}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """(name, dtype) -> (config, weights, model folder); the bfloat16 models have decisive routers."""
    base = tmp_path_factory.mktemp("tifepel")
    out = {}
    for i, (name, cfg) in enumerate(sorted(CONFIGS.items())):
        for dtype in ("float32", "bfloat16"):
            w = make_weights(cfg, seed=500 + i, decisive_router=dtype == "bfloat16")
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
    """Most of the request in one step, the last 60 tokens one by one (the later ones replay a recorded graph): every
    single token reads the token before, the convolutions' tails and the recurrent states that the steps before left."""
    cfg, w, path = models[name, dtype]
    eng = _engine(path, dtype)
    ids = _tokens(cfg, 131, seed=7)
    got = _run_cuts(eng, "r", ids, [71] + [1] * 60)
    _check(got, (cfg, w), ids, dtype, f"{name}: prompt + 60 single tokens")
    assert eng.graph_replays > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_portions_of_changing_size(models, name, dtype):
    """Portions shorter and longer than the convolutions' taps and the recurrence's staging of eight tokens, down to
    two tokens, ending before, at and behind page borders."""
    cfg, w, path = models[name, dtype]
    eng = _engine(path, dtype)
    ids = _tokens(cfg, 101, seed=11)
    for cuts in ([24, 24, 24, 24, 5], [2, 3, 17, 16, 15, 31, 2, 13, 2], [1, 2, 1, 3, 94], [64, 37], [16, 16, 32, 1, 1, 35],
                 [23, 2, 14, 2, 7, 1, 23, 29], [47, 1, 2, 14, 1, 36], [8, 8, 9, 7, 69]):
        assert sum(cuts) == len(ids)
        _check(_run_cuts(eng, "r", ids, cuts), (cfg, w), ids, dtype, f"{name}: portions {cuts}")
    eng.cache.alloc.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_first_tokens_in_every_division(models, name, dtype):
    """The first few tokens of a request: the first reads the pair table's last row and zeros before the convolutions,
    the second is the first whose pair is hashed, a lone token's softmax holds itself."""
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
    (its states sit in a slot that other requests held before)."""
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
    """Unequal requests in one step against each alone: same rows, beyond rounding."""
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
def test_long_decoding_across_page_borders(models, dtype):
    """300 single tokens behind a short prompt, pages of 8: every page border is crossed by a decoded token, the
    distances pass the last bucket of both bias tables, the factor on the query steps up every 5 positions."""
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
    "attention alone, values wider than keys": lambda: dict(layers=[layer(attention(3, 1, 24, 40, rows=10, far=30, every=7), None)]),
    "attention alone, keys wider than values": lambda: dict(layers=[layer(attention(4, 2, 48, 16, rows=16, far=64, every=3, coef=1.5), None)]),
    "attention alone, one stream and one tap": lambda: dict(layers=[layer(attention(2, 2, 32, 32, rows=2, far=3), None)], streams=1, taps=1),
    "state space alone": lambda: dict(layers=[layer(mamba2(3, 1, 20, 24, conv=4, norm_groups=2), None)]),
    "state space alone, a state of 200 and five streams": lambda: dict(layers=[layer(mamba2(2, 2, 200, 40, conv=2, norm_groups=1), None)], streams=5, taps=5),
    "routed feed-forward, identities chosen": lambda: dict(layers=[layer(attention(1, 1, 8, 8, rows=4, far=8), moe(3, 5, 4, 24, shared=8))]),
    "routed feed-forward, no identities, no shared": lambda: dict(layers=[layer(mamba2(1, 1, 8, 8, conv=2, norm_groups=1), moe(6, 0, 2, 16))]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(ONE_LAYER))
def test_each_mechanism_alone(tmp_path, which, dtype):
    cfg = _config(61, 48, **ONE_LAYER[which]())
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
    """Attention alone over 400 tokens.  Queries and keys have unit root mean square, so a larger projection sharpens
    nothing; the scale does: with a scale of 3 on heads of 16 every query looks at one or two keys, mostly far back,
    and a key that is lost or off by one moves the logits by far more than the bound.  The bias table is flat here."""
    cfg = _config(53, 64, [layer(attention(4, 2, 16, 16, rows=8, far=300, every=100, coef=0.3, scale=3.0), None)], max_positions=512)

    def flat(w):
        w["l0.mix.rel"] = torch.zeros_like(w["l0.mix.rel"])

    w, path = _one_model(tmp_path, cfg, seed=9, bend=flat)
    ids = _tokens(cfg, 400, seed=2)
    want = _want(cfg, w, ids)
    assert rel_error(_without(cfg, w, ids, change_cfg=lambda c: c["layers"][0]["mixer"].update(scale=0.25)), want) > 0.05
    eng = _engine(path, dtype, max_tokens=512, page_size=16)
    _check(_run_cuts(eng, "r", ids, [400]), (cfg, w), ids, dtype, "sharp scores, whole")
    _check(_run_cuts(eng, "r", ids, [250, 100, 18] + [1] * 32), (cfg, w), ids, dtype, "sharp scores, portions and single tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows,far", [(8, 40), (6, 17), (32, 200)])
def test_the_edges_of_the_bias_table(tmp_path, rows, far, dtype):
    """The bias alone decides: a tiny scale, and a table whose rows differ by several units, so that a distance put into
    the bucket next door, a table read with another head's column, or a last bucket that starts one position early
    moves the logits by their own size (the plain implementation shows it with the table's rows moved on by one, and
    with buckets that are twice as long).  Whole, in portions,
    and decoded one by one across every bucket's first distance up to beyond bias_max."""
    cfg = _config(53, 64, [layer(attention(3, 1, 16, 16, rows=rows, far=far, every=1000, coef=0.0, scale=0.01), None)], max_positions=512)

    def steep(w):
        g = torch.Generator().manual_seed(rows)
        w["l0.mix.rel"] = 4.0 * torch.randn(rows, 3, generator=g)

    w, path = _one_model(tmp_path, cfg, seed=12, bend=steep)
    n = min(far + 40, 300)
    ids = _tokens(cfg, n, seed=6)
    want = _want(cfg, w, ids)
    def next_door(w2):
        w2["l0.mix.rel"] = torch.roll(w2["l0.mix.rel"], 1, 0)

    assert rel_error(_without(cfg, w, ids, change_w=next_door), want) > 0.05
    assert rel_error(_without(cfg, w, ids, change_cfg=lambda c: c["layers"][0]["mixer"].update(bias_max=far * far)), want) > 0.05
    eng = _engine(path, dtype, max_tokens=512, page_size=16)
    _check(_run_cuts(eng, "r", ids, [n]), (cfg, w), ids, dtype, "bias buckets, whole")
    _check(_run_cuts(eng, "r", ids, [rows // 2, 1, 2, rows, n - rows - rows // 2 - 3]), (cfg, w), ids, dtype, "bias buckets, portions")
    _check(_run_cuts(eng, "r", ids, [3] + [1] * (n - 3)), (cfg, w), ids, dtype, "bias buckets, decoded")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_factor_on_the_query_steps_with_the_position(tmp_path, dtype):
    """A large coefficient and steps every 7 positions: the scores' sharpness changes at positions 6, 13, 20, ... (the
    position plus one is what is divided), which the plain implementation shows with steps every 8."""
    cfg = _config(53, 64, [layer(attention(2, 2, 16, 16, rows=4, far=20, every=7, coef=3.0, scale=0.5), None)])
    w, path = _one_model(tmp_path, cfg, seed=13)
    ids = _tokens(cfg, 75, seed=4)
    want = _want(cfg, w, ids)
    assert rel_error(_without(cfg, w, ids, change_cfg=lambda c: c["layers"][0]["mixer"]["q_temp"].update(every=8)), want) > 0.05
    eng = _engine(path, dtype)
    _check(_run_cuts(eng, "r", ids, [75]), (cfg, w), ids, dtype, "query factor, whole")
    _check(_run_cuts(eng, "r", ids, [5, 1, 1, 6, 2] + [1] * 60), (cfg, w), ids, dtype, "query factor, decoded over its steps")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_state_that_still_holds_its_first_tokens(tmp_path, dtype):
    """State space alone with decays close to one (a small step size): what the first tokens wrote is still most of the
    state after 200, so a state that is lost between steps, starts from another request's numbers or is cleared late
    shows.  Run beside another request, then again in the slot the other one left."""
    from sandyrt_b200.engine.step import StepEntry

    cfg = _config(53, 48, [layer(mamba2(4, 2, 32, 16, conv=3, norm_groups=2), None)], streams=2, taps=2)

    def slow(w):
        w["l0.mix.A_log"] = torch.full((4,), -4.0)
        w["l0.mix.dt_bias"] = torch.full((4,), -1.0)

    w, path = _one_model(tmp_path, cfg, seed=15, bend=slow)
    ids = _tokens(cfg, 220, seed=5)
    want = _want(cfg, w, ids)
    cut = plain.forward(cfg, w, ids[20:]).numpy()
    assert rel_error(cut[-10:], want[-10:]) > 0.05          # the first 20 tokens still matter 200 tokens later
    eng = _engine(path, dtype, max_tokens=768, max_requests=2)
    other = _tokens(cfg, 90, seed=6)
    got, pos = [], 0
    eng.step([StepEntry("other", other[:50], [])])
    for n in [30, 2, 1, 80, 7] + [1] * 100:
        entries = [StepEntry("r", ids[pos:pos + n], list(range(n)))]
        if pos < 40:
            entries.append(StepEntry("other", other[50 + pos:50 + pos + 1], []))
        got.append(eng.step(entries).cpu().numpy()[:n].copy())
        pos += n
    assert pos == 220
    eng.check_status()
    _check(np.concatenate(got), (cfg, w), ids, dtype, "long memory beside another request")
    eng.release("other")
    eng.release("r")
    _check(_run_cuts(eng, "again", ids, [219, 1]), (cfg, w), ids, dtype, "long memory in a slot used before")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_token_before_and_the_rows_before_decide(tmp_path, dtype):
    """A pair table much larger than the token table, and convolutions whose weight lies on the rows before: losing the
    token before or a convolution's tail between steps (or taking another request's) then changes everything, which the
    plain implementation shows with both switched off.  Portions down to one token, two layers, a looped span: every
    run of a layer keeps tails of its own."""
    cfg = _config(47, 48, [layer(attention(2, 2, 8, 24, rows=4, far=9), moe(2, 1, 2, 16, shared=8)),
                           layer(mamba2(2, 1, 8, 12, conv=3, norm_groups=1), None)], streams=2, taps=4, bigram=(97, 13, 5), loop=(0, 2, 2))

    def bend(w):
        w["bigram"] = 4.0 * w["bigram"]
        for name in ("l0.canon1", "l0.canon2", "l1.canon1"):
            t = 0.05 * w[name]
            t[:, :3] += 1.0
            w[name] = t

    w, path = _one_model(tmp_path, cfg, seed=14, bend=bend, decisive=dtype == "bfloat16")
    ids = _tokens(cfg, 60, seed=5)
    want = _want(cfg, w, ids)

    def no_pairs(w2):
        w2["bigram"] = torch.zeros_like(w2["bigram"])

    def no_tails(w2):
        for name in ("l0.canon1", "l0.canon2", "l1.canon1"):
            t = w2[name].clone()
            t[:, :3] = 0.0
            w2[name] = t

    assert rel_error(_without(cfg, w, ids, change_w=no_pairs), want) > 0.2
    assert rel_error(_without(cfg, w, ids, change_w=no_tails), want) > 0.2
    eng = _engine(path, dtype)
    for cuts in ([60], [1] * 60, [2] * 30, [17, 1, 2, 1, 39], [59, 1], [3, 3, 3, 51]):
        _check(_run_cuts(eng, "r", ids, cuts), (cfg, w), ids, dtype, f"token and rows before, {cuts[:5]}")


def test_routers_that_choose_token_by_token(tmp_path):
    """float32, ordinary routers in a looped span: the choices change from token to token and from pass to pass, identity
    experts are chosen for some tokens and not for others, a step of many tokens groups them by expert while single
    tokens go one by one.  The correction moves the choice and not the weights (the plain implementation shows it)."""
    cfg = _config(89, 56, [layer(attention(2, 1, 8, 16, rows=6, far=20), moe(5, 3, 2, 16, shared=24)),
                           layer(mamba2(2, 2, 12, 8, conv=2, norm_groups=2), moe(9, 1, 3, 24))], loop=(0, 1, 3))

    def bend(w):
        w["l0.mlp.correction"] = 0.3 * torch.randn(8, generator=torch.Generator().manual_seed(2))

    w, path = _one_model(tmp_path, cfg, seed=31, bend=bend)
    ids = _tokens(cfg, 260, seed=8)
    assert plain.router_margin(cfg, w, ids) > 1e-6
    want = _want(cfg, w, ids)

    def no_correction(w2):
        w2["l0.mlp.correction"] = torch.zeros(8)

    assert rel_error(_without(cfg, w, ids, change_w=no_correction), want) > 0.02
    eng = _engine(path, "float32")
    _check(_run_cuts(eng, "r", ids, [260]), (cfg, w), ids, "float32", "token-by-token routing, whole")
    _check(_run_cuts(eng, "r", ids, [33, 2, 190, 5] + [1] * 30), (cfg, w), ids, "float32", "token-by-token routing, portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompts_with_heads_of_64_and_a_wide_state(tmp_path, dtype):
    """Prompts of several hundred tokens through heads of 64 and a state of 128 x 64: portions start inside pages and
    inside the recurrence's groups of eight tokens, then single tokens."""
    cfg = _config(97, 128, [layer(attention(4, 2, 64, 64, rows=16, far=128, every=50), moe(4, 2, 2, 32, shared=32)),
                            layer(mamba2(2, 1, 128, 64, conv=4, norm_groups=1), None)], max_positions=512)
    w, path = _one_model(tmp_path, cfg, seed=21, decisive=dtype == "bfloat16")
    eng = _engine(path, dtype, max_tokens=1024)
    ids = _tokens(cfg, 420, seed=2)
    _check(_run_cuts(eng, "r", ids, [420]), (cfg, w), ids, dtype, "long prompt, whole")
    _check(_run_cuts(eng, "r", ids, [130, 2, 209, 60] + [1] * 19), (cfg, w), ids, dtype, "long prompt, portions and single tokens")


def test_options_at_their_edges(tmp_path):
    """float32.  A span that runs once, a span of the last layer alone, every routed output chosen, one expert and many
    identities, a bias table of two rows, a mixer's convolution of one tap, a layer without a feed-forward whose file
    still holds what would surround one (it is read past), a bias table whose length the configuration states."""
    a = _config(67, 40, [layer(attention(3, 3, 8, 8, rows=2, far=2), moe(1, 6, 7, 8)), layer(mamba2(1, 1, 4, 40, conv=1, norm_groups=8), None)],
                streams=2, taps=1, loop=(0, 2, 1))
    b = _config(67, 40, [layer(mamba2(4, 4, 16, 4, conv=8, norm_groups=1), moe(2, 0, 1, 8, shared=4)),
                         layer(attention(2, 2, 8, 8, rows=5, far=6, every=2), moe(3, 1, 1, 8))], streams=8, taps=8, loop=(1, 2, 4))
    for k, cfg in enumerate((a, b)):
        w = make_weights(cfg, seed=41 + k)
        on_disk = dict(w)
        if k == 0:
            on_disk.update({"l1.norm2": torch.ones(40), "l1.canon2": torch.zeros(40, 1), "l1.hc2.in": torch.ones(2)})
        path = write_model(cfg, on_disk, str(tmp_path / f"edges{k}"), drop_bias_rows=k == 0)
        ids = _tokens(cfg, 70, seed=9 + k)
        assert plain.router_margin(cfg, w, ids) > 1e-6
        eng = _engine(path, "float32")
        _check(_run_cuts(eng, "r", ids, [70]), (cfg, w), ids, "float32", f"edges {k}, whole")
        _check(_run_cuts(eng, "r", ids, [31, 2, 30] + [1] * 7), (cfg, w), ids, "float32", f"edges {k}, in portions")


# ---- the entry point --------------------------------------------------------------------------------------
def test_greedy_generation_through_the_entry_point(models):
    """LLM.generate (scheduler, prompt portions, decode bursts) on three requests at once, float32: the same tokens
    as greedy decoding with the plain implementation, wherever its top two logits are clearly apart.  In a burst the
    sampler hands its token to the next step on the device, which is also where the pair table's token before comes from."""
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
