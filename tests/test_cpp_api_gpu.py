"""The C++ API on its own: examples/generate.cpp, built with make against the host library, generates
from a model folder in a process that holds no Python interpreter.  Its tokens must equal those of the
Python entry point (which is a face of the same library) and of the plain implementation."""
import os
import subprocess

import numpy as np
import pytest

from conftest import TINY

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_example_generates_the_same_tokens(model_dirs, plain_models):
    from plain_gpt2 import generate_greedy
    from sandyrt_b200.csrc import build
    from sandyrt_b200.engine.llm import LLM

    build.build_all(verbose=False)                       # the kernel libraries and the host library, where make looks for them
    env = dict(os.environ, CUDA_HOME=os.path.dirname(os.path.dirname(os.path.realpath(build._find_nvcc()))))
    made = subprocess.run(["make", "-C", os.path.join(ROOT, "examples"), "generate"], capture_output=True, text=True, env=env)
    assert made.returncode == 0, made.stdout + made.stderr
    exe = os.path.join(ROOT, "examples", "generate")
    prompt = np.random.default_rng(5).integers(0, TINY["A"]["vocab_size"], size=21).tolist()
    want, reason = generate_greedy(plain_models("A", "f32"), prompt, 14)
    run = subprocess.run([exe, model_dirs["A"], "--dtype", "float32", "--max-tokens", "14"] + [str(t) for t in prompt],
                         capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    lines = run.stdout.strip().splitlines()
    got = [int(t) for t in lines[0].split()]
    assert got == want
    assert f"finish_reason={reason}" in lines[1] and "completion_tokens=14" in lines[1]
    assert LLM(model_dirs["A"], dtype="float32", cache_tokens=512, max_live=2).generate(prompt, max_tokens=14)[0].output_ids == got
    # a folder that is not a model: the error comes out as text, not as a crash
    bad = subprocess.run([exe, os.path.join(ROOT, "examples"), "1", "2"], capture_output=True, text=True, timeout=60)
    assert bad.returncode == 1 and "ConfigError" in bad.stderr and "config.json" in bad.stderr
