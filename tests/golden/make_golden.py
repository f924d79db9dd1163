#!/usr/bin/env python3
"""Makes tests/golden/*.json: top-5 logits per position computed by the REFERENCE's own CPU
code (sunho/SandyRT, `cpu_runner`: test/engine/CpuRunner.cpp -> Engine -> CpuDevice ->
src/core/TensorCalc.cpp) on tiny random GPT-2 models.  tests/test_plain.py compares the plain
implementation (tests/plain_gpt2.py) with these numbers; that anchors the plain
implementation, which every engine test is then compared with, on the reference.

What it does, offline:
  1. builds the reference's `cpu_runner` out of tree (cmake + ninja, tests off);
  2. for each case writes a model program in the reference's own language with the case's
     sizes (the structure of src/models/gpt2_small.sandy.go, whose sizes are literals),
     seeded random weights in the reference's converted naming (q/k/v split out of c_attn and
     every matrix transposed to [out, in], as scripts/run_gpt2.py:151-192 does), and the inputs;
  3. runs cpu_runner and parses its `top5[row]: id(logit) ...` lines
     (test/engine/CpuRunner.cpp:337-343, printed with %.6g).

Cases: tiny A as it is; tiny B with gelu_new in place of the exact gelu, because the
reference has no erf (its `gelu` is the tanh form, src/ir/BuiltinLowering.cpp:116-140): the
exact-gelu option of B rests on the formula alone.  B's other options (eps 1e-6, n_inner
that is not 4x, 3 heads of 32, attention scaled by 1/(layer+1) through the `scale=`
attribute of `__attention`) are all exercised.

Weights are NOT stored: `golden_weights(case)` below regenerates them from the seed with
numpy's PCG64, and the test calls the same function.

    python tests/golden/make_golden.py --reference <checkout of sunho/SandyRT> [--build-dir DIR]
"""
import argparse
import json
import math
import os
import re
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = {
    "tiny_a": dict(n_layer=2, n_embd=64, n_head=4, n_inner=256, vocab_size=512, n_positions=128,
                   layer_norm_epsilon=1e-5, activation_function="gelu_new",
                   scale_attn_by_inverse_layer_idx=False, seed=101, n_tokens=12),
    "tiny_b_tanh": dict(n_layer=3, n_embd=96, n_head=3, n_inner=320, vocab_size=1000, n_positions=256,
                        layer_norm_epsilon=1e-6, activation_function="gelu_new",
                        scale_attn_by_inverse_layer_idx=True, seed=202, n_tokens=9),
}


def golden_weights(case: dict) -> dict:
    """HF-named float32 tensors of a case, from its seed (N(0,0.02) weights, N(0,0.01) biases,
    gains 1+N(0,0.02), offsets N(0,0.02)), and its token ids under the key '__ids__'."""
    rng = np.random.default_rng(case["seed"])
    E, I, V, P = case["n_embd"], case["n_inner"], case["vocab_size"], case["n_positions"]
    w = {}
    nrm = lambda shape, std, mean=0.0: (rng.standard_normal(shape) * std + mean).astype(np.float32)
    w["wte.weight"] = nrm((V, E), 0.02)
    w["wpe.weight"] = nrm((P, E), 0.02)
    for i in range(case["n_layer"]):
        p = f"h.{i}."
        for ln in ("ln_1", "ln_2"):
            w[p + ln + ".weight"] = nrm((E,), 0.02, 1.0)
            w[p + ln + ".bias"] = nrm((E,), 0.02)
        w[p + "attn.c_attn.weight"] = nrm((E, 3 * E), 0.02)
        w[p + "attn.c_attn.bias"] = nrm((3 * E,), 0.01)
        w[p + "attn.c_proj.weight"] = nrm((E, E), 0.02)
        w[p + "attn.c_proj.bias"] = nrm((E,), 0.01)
        w[p + "mlp.c_fc.weight"] = nrm((E, I), 0.02)
        w[p + "mlp.c_fc.bias"] = nrm((I,), 0.01)
        w[p + "mlp.c_proj.weight"] = nrm((I, E), 0.02)
        w[p + "mlp.c_proj.bias"] = nrm((E,), 0.01)
    w["ln_f.weight"] = nrm((E,), 0.02, 1.0)
    w["ln_f.bias"] = nrm((E,), 0.02)
    w["__ids__"] = rng.integers(0, V, size=case["n_tokens"]).astype(np.int64)
    return w


def write_safetensors(path, tensors):
    header, blobs, off = {}, [], 0
    for name in sorted(tensors):
        a = np.ascontiguousarray(tensors[name])
        dt = {"float32": "F32", "int64": "I64"}[str(a.dtype)]
        raw = a.astype("<f4" if dt == "F32" else "<i8").tobytes()
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    head = json.dumps(header, separators=(",", ":")).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)) + head + b"".join(blobs))


def to_reference_names(w, case):
    """scripts/run_gpt2.py:151-192: split c_attn into q/k/v, transpose every matrix to [out, in]."""
    E = case["n_embd"]
    out = {k: w[k] for k in ("wte.weight", "wpe.weight", "ln_f.weight", "ln_f.bias")}
    for i in range(case["n_layer"]):
        p = f"h.{i}."
        for n in ("ln_1.weight", "ln_1.bias", "ln_2.weight", "ln_2.bias", "attn.c_proj.bias", "mlp.c_fc.bias",
                  "mlp.c_proj.bias"):
            out[p + n] = w[p + n]
        for j, proj in enumerate(("q_proj", "k_proj", "v_proj")):
            out[p + f"attn.{proj}.weight"] = w[p + "attn.c_attn.weight"][:, j * E:(j + 1) * E].T.copy()
            out[p + f"attn.{proj}.bias"] = w[p + "attn.c_attn.bias"][j * E:(j + 1) * E].copy()
        for n in ("attn.c_proj.weight", "mlp.c_fc.weight", "mlp.c_proj.weight"):
            out[p + n] = w[p + n].T.copy()
    return out


def program_text(case):
    """A model program in the reference's language with this case's sizes (layers unrolled so
    that each can carry its own attention scale)."""
    E, H, T = case["n_embd"], case["n_head"], case["n_tokens"]
    D = E // H
    eps = f"{case['layer_norm_epsilon']:.10f}".rstrip("0")
    lines = []
    for i in range(case["n_layer"]):
        scale = 1.0 / math.sqrt(D)
        if case["scale_attn_by_inverse_layer_idx"]:
            scale /= (i + 1)
        lines += [
            f"func block_{i}(x Tensor) Tensor {{",
            f"    weight_scope \"h.{i}\" {{",
            f"        h := __layer_norm(x, @ln_1.weight, @ln_1.bias, epsilon={eps})",
            "        weight_scope \"attn\" {",
            "            q := __linear(h, @q_proj.weight, @q_proj.bias)",
            "            k := __linear(h, @k_proj.weight, @k_proj.bias)",
            "            v := __linear(h, @v_proj.weight, @v_proj.bias)",
            f"            q = __reshape(q, shape=[-1, {T}, {H}, {D}])",
            f"            k = __reshape(k, shape=[-1, {T}, {H}, {D}])",
            f"            v = __reshape(v, shape=[-1, {T}, {H}, {D}])",
            "            q = __permute(q, dims=[0, 2, 1, 3])",
            "            k = __permute(k, dims=[0, 2, 1, 3])",
            "            v = __permute(v, dims=[0, 2, 1, 3])",
            f"            ctx := __attention(q, k, v, window=0, scale={scale:.9f})",
            "            ctx = __permute(ctx, dims=[0, 2, 1, 3])",
            f"            ctx = __reshape(ctx, shape=[-1, {T}, {E}])",
            "            h = __linear(ctx, @c_proj.weight, @c_proj.bias)",
            "        }",
            "        x = __add(x, h)",
            f"        h = __layer_norm(x, @ln_2.weight, @ln_2.bias, epsilon={eps})",
            "        weight_scope \"mlp\" {",
            "            h = __linear(h, @c_fc.weight, @c_fc.bias)",
            "            h = __gelu(h)",
            "            h = __linear(h, @c_proj.weight, @c_proj.bias)",
            "        }",
            "        x = __add(x, h)",
            "    }",
            "    return x",
            "}",
            "",
        ]
    lines += ["func main(input_ids Tensor, position_ids Tensor) Tensor {",
              "    x := __embedding(input_ids, @wte.weight)",
              "    pos := __embedding(position_ids, @wpe.weight)",
              "    x = __add(x, pos)"]
    lines += [f"    x = block_{i}(x)" for i in range(case["n_layer"])]
    lines += [f"    x = __layer_norm(x, @ln_f.weight, @ln_f.bias, epsilon={eps})",
              "    logits := __matmul(x, __transpose(@wte.weight))",
              "    return logits",
              "}", ""]
    return "\n".join(lines)


def build_runner(reference, build_dir):
    def find():
        for cand in (os.path.join(build_dir, "cpu_runner"), os.path.join(build_dir, "test", "cpu_runner")):
            if os.path.isfile(cand):
                return cand
        return None

    if find():
        return find()
    subprocess.run(["cmake", "-S", reference, "-B", build_dir, "-G", "Ninja", "-DSANDY_BUILD_TESTS=OFF",
                    "-DCMAKE_BUILD_TYPE=Release"], check=True, stdout=subprocess.DEVNULL)
    subprocess.run(["cmake", "--build", build_dir, "--target", "cpu_runner"], check=True, stdout=subprocess.DEVNULL)
    runner = find()
    if runner is None:
        raise SystemExit("cpu_runner was not produced by the reference's build")
    return runner


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="a checkout of sunho/SandyRT")
    ap.add_argument("--build-dir", default=None, help="where cpu_runner is built (default: a fresh temporary folder)")
    args = ap.parse_args()
    runner = build_runner(args.reference, args.build_dir or tempfile.mkdtemp(prefix="sandy_ref_build_"))
    for name, case in CASES.items():
        w = golden_weights(case)
        ids = w.pop("__ids__")
        with tempfile.TemporaryDirectory() as d:
            prog = os.path.join(d, "model.sandy.go")
            with open(prog, "w") as f:
                f.write(program_text(case))
            write_safetensors(os.path.join(d, "weights.safetensors"), to_reference_names(w, case))
            write_safetensors(os.path.join(d, "inputs.safetensors"),
                              {"input_ids": ids.reshape(1, -1),
                               "position_ids": np.arange(len(ids), dtype=np.int64).reshape(1, -1)})
            res = subprocess.run([runner, prog, os.path.join(d, "weights.safetensors"),
                                  os.path.join(d, "inputs.safetensors")], capture_output=True, text=True)
            if res.returncode != 0:
                sys.stderr.write(res.stdout[-3000:] + res.stderr[-3000:])
                raise SystemExit(f"cpu_runner failed for {name}")
        top5 = {}
        for m in re.finditer(r"^\s+top5\[(\d+)\]:(.*)$", res.stdout, re.MULTILINE):
            top5[int(m.group(1))] = [[int(i), float(v)] for i, v in re.findall(r"\s(\d+)\(([^)]+)\)", m.group(2))]
        assert sorted(top5) == list(range(len(ids))), f"{name}: expected one top5 line per position"
        out = {"case": name, "config": {k: v for k, v in case.items()}, "ids": ids.tolist(),
               "source": "sunho/SandyRT cpu_runner (CpuDevice / TensorCalc), float32",
               "top5": [top5[r] for r in range(len(ids))]}
        with open(os.path.join(HERE, name + ".json"), "w") as f:
            json.dump(out, f, indent=1)
        print(f"{name}: wrote {len(ids)} positions; argmax at last position {top5[len(ids) - 1][0]}")


if __name__ == "__main__":
    main()
