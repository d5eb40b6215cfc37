"""Tifepel configurations drawn at random, each through the engine whole, as a prompt with single tokens behind it and
in portions, in both compute types, against the plain implementation (tests/plain_tifepel.py).

The sizes divide by nothing in particular: widths of 44 to 136 (some no multiple of 8), 1 to 5 copies of the stream, 1 to
5 taps, head sizes of 5 to 72 with query and value sizes apart, states of 3 to 150 rows with values of 3 to 72, bias
tables of 2 to 40 rows, 1 to 10 experts with 0 to 5 identities, loops over any span.  Bounds as in test_tifepel_gpu.py."""
import numpy as np
import pytest
import torch

import plain_tifepel as plain
from tifepel_models import _config, attention, layer, make_weights, mamba2, moe, rel_error, write_model

pytestmark = pytest.mark.gpu


def draw(seed: int) -> dict:
    r = np.random.default_rng(seed)
    pick = lambda *xs: xs[int(r.integers(0, len(xs)))]
    width = int(pick(44, 48, 66, 72, 90, 100, 128, 136))
    layers = []
    for _ in range(int(r.integers(1, 5))):
        if r.random() < 0.5:
            kv = int(pick(1, 2, 3))
            rows = 2 * int(r.integers(1, 21))
            mixer = attention(kv * int(pick(1, 2, 4)), kv, int(pick(5, 8, 16, 24, 40, 64, 72)), int(pick(6, 8, 16, 20, 48, 64)), rows=rows,
                              far=rows // 2 + int(r.integers(1, 60)), every=int(pick(1, 3, 16, 50)), coef=float(pick(0.0, 0.4, 1.2)),
                              scale=float(pick(0.1, 0.3, 0.5)))
        else:
            groups = int(pick(1, 2, 3))
            heads = groups * int(pick(1, 2, 3))
            vdim = int(pick(3, 8, 12, 30, 64, 72))
            inner = heads * vdim
            mixer = mamba2(heads, groups, int(pick(3, 7, 16, 24, 40, 64, 100, 150)), vdim, conv=int(r.integers(1, 6)),
                           norm_groups=int(pick(*[d for d in (1, 2, 3, 4, 6) if inner % d == 0])))
        if r.random() < 0.8:
            experts, identity = int(r.integers(1, 11)), int(r.integers(0, 6))
            mlp = moe(experts, identity, int(r.integers(1, experts + identity + 1)), int(pick(4, 8, 12, 24, 40)),
                      shared=int(pick(8, 20, 36)) if r.random() < 0.6 else None)
        else:
            mlp = None
        layers.append(layer(mixer, mlp))
    loop = None
    if r.random() < 0.6:
        start = int(r.integers(0, len(layers)))
        loop = (start, int(r.integers(start + 1, len(layers) + 1)), int(r.integers(1, 4)))
    return _config(int(r.integers(50, 200)), width, layers, streams=int(r.integers(1, 6)), taps=int(r.integers(1, 6)),
                   eps=float(pick(1e-5, 1e-6)), max_positions=128,
                   bigram=(int(r.integers(1, 300)), int(r.integers(0, 1000)), int(r.integers(0, 1000))), loop=loop)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(20))
def test_a_configuration_drawn_at_random(tmp_path, seed, dtype):
    from sandyrt_b200.engine.step import Engine, StepEntry
    from sandyrt_b200.models.model import load_model

    cfg = draw(seed)
    ids = np.random.default_rng(1000 + seed).integers(0, cfg["vocab"], size=70).tolist()
    w = make_weights(cfg, seed=seed, decisive_router=dtype == "bfloat16")
    if dtype == "float32" and plain.router_margin(cfg, w, ids) < 1e-5:
        w = make_weights(cfg, seed=seed, decisive_router=True)
    path = write_model(cfg, w, str(tmp_path / "m"))
    want = plain.forward(cfg, w, ids).numpy()
    bound = 2e-4 if dtype == "float32" else max(2e-2, 3 * rel_error(plain.forward_rounded(cfg, w, ids).numpy(), want))
    eng = Engine(load_model(path, device="cuda:0", dtype=getattr(torch, dtype)), max_tokens=256, page_size=16, max_requests=2)
    eng.cache.device_caches.poison()
    for cuts in ([70], [41] + [1] * 29, [2, 9, 1, 30, 3, 25]):
        rows, pos = [], 0
        for n in cuts:
            rows.append(eng.step([StepEntry("r", ids[pos:pos + n], list(range(n)))]).cpu().numpy().copy())
            pos += n
        eng.check_status()
        eng.release("r")
        e = rel_error(np.concatenate(rows), want)
        assert e < bound, f"seed {seed}, cuts {cuts[:4]}: relative error {e:.3e} (bound {bound:.1e}); {cfg}"
