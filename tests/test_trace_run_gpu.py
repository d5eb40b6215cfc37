"""bin/trace_run as a user runs it: a subprocess fed JSON lines, logits in files."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT, TINY

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,store,tol", [("float32", "f32", 2e-5), ("bfloat16", "bf16", 6e-3)])
def test_trace_run_protocol(model_dirs, plain_models, tmp_path, dtype, store, tol):
    name = "B"
    rng = np.random.default_rng(5)
    seqs = {k: rng.integers(0, TINY[name]["vocab_size"], size=n).tolist() for k, n in (("a", 70), ("b", 40), ("c", 90))}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": seqs["a"][:38], "want": [0, 37]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": seqs["a"][38:40], "want": []},
                                {"id": "b", "tokens": seqs["b"][:40], "want": [39]}], "end": ["b"]},
        {"step": 2, "entries": [], "end": []},
        {"step": 3, "entries": [{"id": "c", "tokens": seqs["c"][:64], "want": [63]},
                                {"id": "a", "tokens": seqs["a"][40:41], "want": [0]}], "end": []},
        {"step": 4, "entries": [{"id": "a", "tokens": seqs["a"][41:70], "want": list(range(29))},
                                {"id": "c", "tokens": seqs["c"][64:90], "want": [25]}], "end": ["a", "c"]},
    ]
    out_dir = tmp_path / "out"
    # the pool holds 192 tokens: a (70 -> 128) + c (90 -> 128) would not fit beside b, so b's pages are reused
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dirs[name],
                           "--dtype", dtype, "--out", str(out_dir), "--max-tokens", "256"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=280)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(5)]
    plain = plain_models(name, store)
    full = {k: plain.logits(v) for k, v in seqs.items()}
    V = TINY[name]["vocab_size"]
    read = lambda i: np.fromfile(out_dir / f"{i}.f32", dtype="<f4").reshape(-1, V)
    close = lambda got, want: np.testing.assert_allclose(got, want, atol=tol, rtol=10 * tol)
    close(read(0), full["a"][[0, 37]])
    close(read(1), full["b"][[39]])
    assert not (out_dir / "2.f32").exists()
    close(read(3), np.stack([full["c"][63], full["a"][40]]))
    close(read(4), np.concatenate([full["a"][41:70], full["c"][[89]]]))


@pytest.mark.parametrize("dtype,bound", [("float32", 2e-4), ("bfloat16", 0.2)])
def test_trace_run_serves_the_hybrid_design(tmp_path, dtype, bound):
    """The same runner on a Panupel folder (config.json chooses the model): six requests through four state slots
    and a pool of 160 tokens, portions beside single tokens, a request that sits steps out, slots and pages used
    again.  bfloat16's bound is loose here (these small models move by a tenth under rounding alone); the float32
    run is the sharp one."""
    import plain_panupel as plain
    from panupel_models import CONFIGS, make_weights, rel_error, write_model

    cfg = CONFIGS["A"]
    w = make_weights(cfg, seed=31)
    model_dir = write_model(cfg, w, str(tmp_path / "model"))
    rng = np.random.default_rng(8)
    lengths = {"a": 40, "b": 9, "c": 33, "d": 21, "e": 30, "f": 12}
    seqs = {k: rng.integers(0, cfg["vocab"], size=n).tolist() for k, n in lengths.items()}
    cut = lambda k, lo, hi, want: {"id": k, "tokens": seqs[k][lo:hi], "want": want}
    steps = [
        {"step": 0, "entries": [cut("a", 0, 17, [16]), cut("b", 0, 2, [0, 1]), cut("c", 0, 30, [])], "end": []},
        {"step": 1, "entries": [cut("a", 17, 18, [0]), cut("b", 2, 9, [6]), cut("d", 0, 21, [20])], "end": ["b", "d"]},
        {"step": 2, "entries": [cut("a", 18, 40, [0, 21]), cut("e", 0, 29, [28]), cut("f", 0, 3, [2])], "end": ["a"]},
        {"step": 3, "entries": [cut("c", 30, 31, [0]), cut("e", 29, 30, [0]), cut("f", 3, 12, [8])], "end": ["e", "f"]},
        {"step": 4, "entries": [cut("c", 31, 33, [0, 1])], "end": ["c"]},
    ]
    out_dir = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", "160"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=560)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(5)]
    full = {k: plain.forward(cfg, w, v)[0].numpy() for k, v in seqs.items()}
    read = lambda i: np.fromfile(out_dir / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
    want = [np.stack([full["a"][16], full["b"][0], full["b"][1]]),
            np.stack([full["a"][17], full["b"][8], full["d"][20]]),
            np.stack([full["a"][18], full["a"][39], full["e"][28], full["f"][2]]),
            np.stack([full["c"][30], full["e"][29], full["f"][11]]),
            np.stack([full["c"][31], full["c"][32]])]
    for i, wanted in enumerate(want):
        assert rel_error(read(i), wanted) < bound, f"step {i}"


@pytest.mark.parametrize("dtype,bound", [("float32", 2e-4), ("bfloat16", 6e-2)])
def test_trace_run_serves_the_latent_attention_design(tmp_path, dtype, bound):
    """The same runner on a Sovezen folder: six requests through four slots and a pool of 160 tokens, portions beside
    single tokens, a request that sits steps out, pages used again."""
    import plain_sovezen as plain
    from sovezen_models import CONFIGS, make_weights, rel_error, write_model

    cfg = CONFIGS["A"]
    w = make_weights(cfg, seed=31, decisive_router=dtype == "bfloat16")
    model_dir = write_model(cfg, w, str(tmp_path / "model"))
    rng = np.random.default_rng(8)
    lengths = {"a": 40, "b": 9, "c": 33, "d": 21, "e": 30, "f": 12}
    seqs = {k: rng.integers(0, cfg["vocab"], size=n).tolist() for k, n in lengths.items()}
    cut = lambda k, lo, hi, want: {"id": k, "tokens": seqs[k][lo:hi], "want": want}
    steps = [
        {"step": 0, "entries": [cut("a", 0, 17, [16]), cut("b", 0, 2, [0, 1]), cut("c", 0, 30, [])], "end": []},
        {"step": 1, "entries": [cut("a", 17, 18, [0]), cut("b", 2, 9, [6]), cut("d", 0, 21, [20])], "end": ["b", "d"]},
        {"step": 2, "entries": [cut("a", 18, 40, [0, 21]), cut("e", 0, 29, [28]), cut("f", 0, 3, [2])], "end": ["a"]},
        {"step": 3, "entries": [cut("c", 30, 31, [0]), cut("e", 29, 30, [0]), cut("f", 3, 12, [8])], "end": ["e", "f"]},
        {"step": 4, "entries": [cut("c", 31, 33, [0, 1])], "end": ["c"]},
    ]
    out_dir = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", "160"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=560)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(5)]
    full = {k: plain.forward(cfg, w, v).numpy() for k, v in seqs.items()}
    read = lambda i: np.fromfile(out_dir / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
    want = [np.stack([full["a"][16], full["b"][0], full["b"][1]]),
            np.stack([full["a"][17], full["b"][8], full["d"][20]]),
            np.stack([full["a"][18], full["a"][39], full["e"][28], full["f"][2]]),
            np.stack([full["c"][30], full["e"][29], full["f"][11]]),
            np.stack([full["c"][31], full["c"][32]])]
    for i, wanted in enumerate(want):
        assert rel_error(read(i), wanted) < bound, f"step {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_serves_the_design_with_several_streams(tmp_path, dtype):
    """The same runner on a Tifepel folder whose configuration leaves the bias tables' lengths to the weight file: six
    requests through four slots and a pool of 160 tokens, portions beside single tokens, a request that sits steps out;
    the slots hold recurrent states, convolution tails and the token before, and are used again.  float32 within 2e-4;
    bfloat16 within three times what rounding alone does to these requests (the plain implementation with its products'
    operands and results rounded), at least 2e-2."""
    import plain_tifepel as plain
    from tifepel_models import CONFIGS, make_weights, rel_error, write_model

    cfg = CONFIGS["A"]
    w = make_weights(cfg, seed=31, decisive_router=dtype == "bfloat16")
    model_dir = write_model(cfg, w, str(tmp_path / "model"), drop_bias_rows=True)
    rng = np.random.default_rng(8)
    lengths = {"a": 40, "b": 9, "c": 33, "d": 21, "e": 30, "f": 12}
    seqs = {k: rng.integers(0, cfg["vocab"], size=n).tolist() for k, n in lengths.items()}
    cut = lambda k, lo, hi, want: {"id": k, "tokens": seqs[k][lo:hi], "want": want}
    steps = [
        {"step": 0, "entries": [cut("a", 0, 17, [16]), cut("b", 0, 2, [0, 1]), cut("c", 0, 30, [])], "end": []},
        {"step": 1, "entries": [cut("a", 17, 18, [0]), cut("b", 2, 9, [6]), cut("d", 0, 21, [20])], "end": ["b", "d"]},
        {"step": 2, "entries": [cut("a", 18, 40, [0, 21]), cut("e", 0, 29, [28]), cut("f", 0, 3, [2])], "end": ["a"]},
        {"step": 3, "entries": [cut("c", 30, 31, [0]), cut("e", 29, 30, [0]), cut("f", 3, 12, [8])], "end": ["e", "f"]},
        {"step": 4, "entries": [cut("c", 31, 33, [0, 1])], "end": ["c"]},
    ]
    out_dir = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", "160"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=560)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(5)]
    full = {k: plain.forward(cfg, w, v).numpy() for k, v in seqs.items()}
    bound = 2e-4
    if dtype == "bfloat16":
        bound = max(2e-2, 3 * max(rel_error(plain.forward_rounded(cfg, w, v).numpy(), full[k]) for k, v in seqs.items()))
    read = lambda i: np.fromfile(out_dir / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
    want = [np.stack([full["a"][16], full["b"][0], full["b"][1]]),
            np.stack([full["a"][17], full["b"][8], full["d"][20]]),
            np.stack([full["a"][18], full["a"][39], full["e"][28], full["f"][2]]),
            np.stack([full["c"][30], full["e"][29], full["f"][11]]),
            np.stack([full["c"][31], full["c"][32]])]
    for i, wanted in enumerate(want):
        assert rel_error(read(i), wanted) < bound, f"step {i}"


def test_the_command_line_writes_and_runs_a_random_model_of_the_design(tmp_path):
    """`python -m sandyrt_b200 random-model` from a configuration file that states the bias tables' lengths, then `generate`."""
    from tifepel_models import CONFIGS

    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(CONFIGS["A"]))
    run = lambda *args: subprocess.run([sys.executable, "-m", "sandyrt_b200", *args], capture_output=True, text=True, timeout=560,
                                       cwd=ROOT)
    made = run("random-model", "--config", str(cfg_path), "--out", str(tmp_path / "m"), "--seed", "3")
    assert made.returncode == 0, made.stderr[-2000:]
    out = run("generate", "--model", str(tmp_path / "m"), "--dtype", "float32", "--prompt-ids", "5,17,3,9", "--max-tokens", "6")
    assert out.returncode == 0, out.stderr[-2000:]
