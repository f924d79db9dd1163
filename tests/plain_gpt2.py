"""A plain, slow GPT-2 written from the reference's formulas.  numpy only.

Whole sequences, no cache, one function per part.  It shares no code with the engine: it
has its own safetensors reader, its own config reading, its own sampler.  Every function
cites the reference file and lines it follows (paths inside sunho/SandyRT).

Arithmetic: sums are carried in float64 and the result of each op is rounded to float32
(`store="f32"`), which is at least as exact as the reference's float/double mix.  With
`store="bf16"` the weights and the tensors that the engine keeps in bfloat16 (norm
outputs, q/k/v, attention output, activation output) are rounded to bfloat16
(round-to-nearest-even, src/core/Tensor.h:43-49); the residual stream and the logits stay
float32, as in the engine.
"""
from __future__ import annotations

import json
import math
import struct
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np


# ---- container -----------------------------------------------------------------------
def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """src/core/Tensor.h:36-41: the 16 bits are the high half of a float."""
    return (bits.astype(np.uint32) << 16).view(np.float32)


def round_bf16(x: np.ndarray) -> np.ndarray:
    """src/core/Tensor.h:43-49: bits + 0x7fff + lsb, then drop the low half."""
    f = np.ascontiguousarray(x, dtype=np.float32)
    b = f.view(np.uint32)
    lsb = (b >> 16) & 1
    r = ((b + 0x7FFF + lsb) >> 16).astype(np.uint32) << 16
    out = r.view(np.float32).copy()
    out[np.isnan(f)] = np.nan
    return out.reshape(f.shape)


def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    """scripts/run_gpt2.py:39-59: u64 header length, JSON header, payload; floats -> float32."""
    with open(path, "rb") as f:
        blob = f.read()
    (hlen,) = struct.unpack_from("<Q", blob, 0)
    header = json.loads(blob[8:8 + hlen])
    base = 8 + hlen
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        raw = blob[base + b:base + e]
        dt = meta["dtype"]
        if dt == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float32)
        elif dt == "BF16":
            a = bf16_bits_to_f32(np.frombuffer(raw, dtype="<u2"))
        elif dt == "F16":
            a = np.frombuffer(raw, dtype="<f2").astype(np.float32)
        elif dt == "I64":
            a = np.frombuffer(raw, dtype="<i8").astype(np.int64)
        elif dt == "I32":
            a = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"{name}: dtype {dt}")
        out[name] = a.reshape(meta["shape"])
    return out


def read_config(model_dir: str) -> dict:
    """experiments/gpt2_small/config.json:1-30: the keys; absent ones get GPT-2's defaults."""
    with open(f"{model_dir}/config.json") as f:
        c = json.load(f)
    c.setdefault("n_inner", None)
    if c["n_inner"] is None:
        c["n_inner"] = 4 * c["n_embd"]
    c.setdefault("layer_norm_epsilon", 1e-5)
    c.setdefault("activation_function", "gelu_new")
    c.setdefault("scale_attn_weights", True)
    c.setdefault("scale_attn_by_inverse_layer_idx", False)
    c.setdefault("tie_word_embeddings", True)
    return c


# ---- parts -----------------------------------------------------------------------------
def _store(x: np.ndarray, store: str) -> np.ndarray:
    x = np.asarray(x, dtype=np.float32)
    return round_bf16(x) if store == "bf16" else x


def embedding(ids: Sequence[int], table: np.ndarray) -> np.ndarray:
    """src/core/TensorCalc.cpp:1546-1560: row gather; an id outside the table is an error."""
    ids = np.asarray(ids, dtype=np.int64)
    if ids.min(initial=0) < 0 or ids.max(initial=0) >= table.shape[0]:
        raise ValueError("embedding id out of range")
    return table[ids].astype(np.float32)


def layer_norm(x: np.ndarray, gamma: np.ndarray, beta: np.ndarray, eps: float) -> np.ndarray:
    """src/core/TensorCalc.cpp:2048-2072: mean and biased variance in double (two passes),
    inv = 1/sqrt(float(var) + eps), y = (x - float(mean)) * inv * gamma + beta."""
    x64 = x.astype(np.float64)
    mean = x64.mean(axis=-1, keepdims=True)
    var = ((x64 - mean) ** 2).mean(axis=-1, keepdims=True)
    inv = 1.0 / np.sqrt(var.astype(np.float32).astype(np.float64) + np.float64(np.float32(eps)))
    y = (x64 - mean.astype(np.float32)) * inv * gamma.astype(np.float64) + beta.astype(np.float64)
    return y.astype(np.float32)


def linear_in_out(x: np.ndarray, w_in_out: np.ndarray, bias: Optional[np.ndarray]) -> np.ndarray:
    """src/core/TensorCalc.cpp:759-770: acc = bias; acc += x[i] * w[o][i] over i.  The file
    keeps GPT-2's matrices as [in, out] (scripts/run_gpt2.py:171-189 transposes them for the
    reference); here y = x @ W + b with W as stored."""
    y = x.astype(np.float64) @ w_in_out.astype(np.float64)
    if bias is not None:
        y = y + bias.astype(np.float64)
    return y.astype(np.float32)


def gelu_new(u: np.ndarray) -> np.ndarray:
    """src/ir/BuiltinLowering.cpp:116-140: 0.5*u*(1 + tanh(0.7978845608028654*(u + 0.044715*u^3)))."""
    u = u.astype(np.float64)
    inner = u + 0.044715 * (u * u * u)
    return ((0.5 * u) * (1.0 + np.tanh(0.7978845608028654 * inner))).astype(np.float32)


def gelu_erf(u: np.ndarray) -> np.ndarray:
    """Exact gelu, 0.5*u*(1 + erf(u/sqrt 2)).  The reference has no erf
    (ScalarOp list src/ir/KernelIR.h:317-337); this rests on the formula."""
    u = u.astype(np.float64)
    erf = np.vectorize(math.erf)
    return (0.5 * u * (1.0 + erf(u / math.sqrt(2.0)))).astype(np.float32)


def causal_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float,
                     window: int = 0) -> np.ndarray:
    """src/core/TensorCalc.cpp:1241-1311.  q: [H, T, D]; k, v: [Hkv, T, D].
    score = (q.k)*scale for max(0, i+1-window) <= j <= i, else -inf (:1257-1272);
    p = exp(score - max) / sum (sum in double, :1275-1279); out = sum p*v (:1281-1297);
    query head h reads kv head h / (H/Hkv) (:1246)."""
    H, T, D = q.shape
    Hkv = k.shape[0]
    out = np.zeros((H, T, D), dtype=np.float32)
    for h in range(H):
        kh = h // (H // Hkv)
        for i in range(T):
            lo = max(0, i + 1 - window) if window > 0 else 0
            s = (k[kh, lo:i + 1].astype(np.float64) @ q[h, i].astype(np.float64)) * np.float64(np.float32(scale))
            s = s.astype(np.float32).astype(np.float64)
            p = np.exp(s - s.max())
            p = p / p.sum()
            out[h, i] = (p @ v[kh, lo:i + 1].astype(np.float64)).astype(np.float32)
    return out


def attention_block(h: np.ndarray, w: Dict[str, np.ndarray], prefix: str, n_head: int,
                    scale: float, store: str) -> np.ndarray:
    """src/models/gpt2_small.sandy.go:1-23: q/k/v projections, heads split [T,E]->[H,T,D],
    attention, heads merged, output projection.  q, k, v are column ranges 0/E/2E of the fused
    c_attn (scripts/run_gpt2.py:170-175)."""
    T, E = h.shape
    D = E // n_head
    qkv = _store(linear_in_out(h, w[prefix + "attn.c_attn.weight"], w[prefix + "attn.c_attn.bias"]), store)
    q, k, v = qkv[:, :E], qkv[:, E:2 * E], qkv[:, 2 * E:]
    split = lambda t: t.reshape(T, n_head, D).transpose(1, 0, 2)
    ctx = causal_attention(split(q), split(k), split(v), scale)
    ctx = _store(ctx.transpose(1, 0, 2).reshape(T, E), store)
    return linear_in_out(ctx, w[prefix + "attn.c_proj.weight"], w[prefix + "attn.c_proj.bias"])


def mlp_block(h: np.ndarray, w: Dict[str, np.ndarray], prefix: str, activation: str, store: str) -> np.ndarray:
    """src/models/gpt2_small.sandy.go:25-32: c_fc, gelu, c_proj."""
    u = linear_in_out(h, w[prefix + "mlp.c_fc.weight"], w[prefix + "mlp.c_fc.bias"])
    g = _store(gelu_new(u) if activation == "gelu_new" else gelu_erf(u), store)
    return linear_in_out(g, w[prefix + "mlp.c_proj.weight"], w[prefix + "mlp.c_proj.bias"])


def block(x: np.ndarray, w: Dict[str, np.ndarray], i: int, cfg: dict, store: str) -> np.ndarray:
    """src/models/gpt2_small.sandy.go:34-45: x += attn(ln_1(x)); x += mlp(ln_2(x))."""
    p = f"h.{i}."
    eps = cfg["layer_norm_epsilon"]
    D = cfg["n_embd"] // cfg["n_head"]
    scale = 1.0
    if cfg["scale_attn_weights"]:
        scale /= math.sqrt(D)                 # src/core/TensorCalc.cpp:1236-1237
    if cfg["scale_attn_by_inverse_layer_idx"]:
        scale /= float(i + 1)                 # the `scale` attribute of attention, per layer
    h = _store(layer_norm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"], eps), store)
    x = (x.astype(np.float64) + attention_block(h, w, p, cfg["n_head"], scale, store)).astype(np.float32)
    h = _store(layer_norm(x, w[p + "ln_2.weight"], w[p + "ln_2.bias"], eps), store)
    x = (x.astype(np.float64) + mlp_block(h, w, p, cfg["activation_function"], store)).astype(np.float32)
    return x


class PlainGPT2:
    def __init__(self, model_dir: str, store: str = "f32"):
        assert store in ("f32", "bf16")
        self.cfg = read_config(model_dir)
        w = read_safetensors(f"{model_dir}/model.safetensors")
        w = {(k[len("transformer."):] if k.startswith("transformer.") else k): a for k, a in w.items()}
        if store == "bf16":
            w = {k: round_bf16(a) if a.dtype == np.float32 else a for k, a in w.items()}
        self.w = w
        self.store = store

    def logits(self, ids: Sequence[int], rows: Optional[Sequence[int]] = None) -> np.ndarray:
        """src/models/gpt2_small.sandy.go:47-59: x = wte[ids] + wpe[0..T-1]; blocks; ln_f;
        logits = x @ wte^T for every position.  Returns float32 [T, vocab], or only the given
        rows of it (the final norm and the head work row by row, so leaving rows out changes
        nothing in the others)."""
        cfg, w = self.cfg, self.w
        T = len(ids)
        if T > cfg["n_positions"]:
            raise ValueError("sequence longer than n_positions")
        x = (embedding(ids, w["wte.weight"]).astype(np.float64)
             + embedding(range(T), w["wpe.weight"]).astype(np.float64)).astype(np.float32)
        for i in range(cfg["n_layer"]):
            x = block(x, w, i, cfg, self.store)
        if rows is not None:
            x = x[np.asarray(list(rows), dtype=np.int64)]
        y = _store(layer_norm(x, w["ln_f.weight"], w["ln_f.bias"], cfg["layer_norm_epsilon"]), self.store)
        head = w["wte.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
        return (y.astype(np.float64) @ head.astype(np.float64).T).astype(np.float32)


# ---- sampling and generation ------------------------------------------------------------
def sample_token(logits: np.ndarray, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
                 u: float = 0.0) -> int:
    """src/server/Sampler.cpp:55-107: stable sort high to low (ties: lower id first); keep top_k
    (0 = all here); temperature 0 -> the first; weights exp(l/T - best/T) in double; shortest
    prefix whose cumulative share reaches top_p; draw in proportion.  The draw here is an
    inverse CDF with the given uniform number `u` over the kept ids in id order."""
    l = np.asarray(logits, dtype=np.float32)
    if np.isnan(l).any():
        raise ValueError("sampling logits must not contain NaN")
    order = np.argsort(-l.astype(np.float64), kind="stable")
    if top_k and top_k > 0:
        order = order[:top_k]
    if temperature == 0.0 or not np.isfinite(l[order[0]]):
        return int(order[0])
    scaled = l[order].astype(np.float64) / temperature
    wts = np.exp(scaled - scaled[0])
    total = wts.sum()
    keep, cum = 0, 0.0
    while True:
        cum += wts[keep] / total
        keep += 1
        if not (keep < len(wts) and cum < top_p):
            break
    kept_ids = np.sort(order[:keep])
    kept_w = np.exp(l[kept_ids].astype(np.float64) / temperature - scaled[0])
    cdf = np.cumsum(kept_w)
    target = u * cdf[-1]
    idx = int(np.searchsorted(cdf, target, side="right"))
    return int(kept_ids[min(idx, len(kept_ids) - 1)])


def kept_set_and_cdf(logits: np.ndarray, temperature: float, top_k: int = 0, top_p: float = 1.0):
    """The ids a draw may return (in id order) and their cumulative shares (for tests that
    check a device draw against the distribution rather than bit for bit)."""
    l = np.asarray(logits, dtype=np.float32)
    order = np.argsort(-l.astype(np.float64), kind="stable")
    if top_k and top_k > 0:
        order = order[:top_k]
    scaled = l[order].astype(np.float64) / temperature
    wts = np.exp(scaled - scaled[0])
    total = wts.sum()
    keep, cum = 0, 0.0
    while True:
        cum += wts[keep] / total
        keep += 1
        if not (keep < len(wts) and cum < top_p):
            break
    kept_ids = np.sort(order[:keep])
    kept_w = np.exp(l[kept_ids].astype(np.float64) / temperature - scaled[0])
    cdf = np.cumsum(kept_w) / kept_w.sum()
    return kept_ids, cdf


def generate_greedy(model: PlainGPT2, prompt: Sequence[int], max_tokens: int,
                    stop_ids: Sequence[int] = ()) -> Tuple[List[int], str]:
    """src/server/Session.cpp:477-514: emit the next token, stop on a stop token (which is
    part of the output) or after max_tokens; every step recomputes the whole sequence."""
    ids = list(prompt)
    out: List[int] = []
    if max_tokens == 0:
        return out, "length"
    while True:
        nxt = sample_token(model.logits(ids, rows=[len(ids) - 1])[0])
        out.append(nxt)
        ids.append(nxt)
        if nxt in stop_ids:
            return out, "stop"
        if len(out) >= max_tokens or len(ids) >= model.cfg["n_positions"]:
            return out, "length"
