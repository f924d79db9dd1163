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
