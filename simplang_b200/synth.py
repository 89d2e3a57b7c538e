"""Seeded synthetic LLaMA weights for the decode workloads (random init, as the reference's own
benchmarks use: examples/llama2/test_stories110M.cpp:120-134, bench_llama_quant.cpp:43-49).

Every tensor is ~N(0, 0.02) (norm weights ~N(1, 0.02)), one numpy Generator per tensor seeded with
``seed + index`` in the .sl argument order.  The W4 variant quantises the seven projection families
symmetrically to int4 per group of ``gs`` weights along K: scale = max|w|/7, q = clip(rint(w/scale), -8, 7),
stored as nibble = q + 8 in the reference's layout (two per byte, low nibble = even flat index), which
the reference form w = nibble*scale + zero reproduces with zero = -8*scale.
"""
from __future__ import annotations

import concurrent.futures as cf

import numpy as np

STORIES_110M = dict(dim=768, hidden_dim=2048, n_layers=12, n_heads=12, n_kv_heads=12, vocab_size=32000, seq_len=1024)
LLAMA_3B_W4 = dict(dim=3200, hidden_dim=8640, n_layers=26, n_heads=32, n_kv_heads=32, vocab_size=32000, seq_len=2048,
                   group_size=64)
FAMILIES = ("wq", "wk", "wv", "wo", "w1", "w2", "w3")


def family_shapes(cfg):
    d, h = cfg["dim"], cfg["hidden_dim"]
    kv = d * cfg["n_kv_heads"] // cfg["n_heads"]
    return {"wq": (d, d), "wk": (kv, d), "wv": (kv, d), "wo": (d, d), "w1": (h, d), "w2": (d, h), "w3": (h, d)}


def _normal(seed, shape, mean=0.0, std=0.02):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal(shape, dtype=np.float32)
    a *= std
    if mean:
        a += mean
    return a


def common_tensors(cfg, seed):
    d, L, V = cfg["dim"], cfg["n_layers"], cfg["vocab_size"]
    return {
        "token_embedding": _normal(seed + 1, (V, d)),
        "rms_att_w": _normal(seed + 2, (L, d), mean=1.0),
        "rms_ffn_w": _normal(seed + 7, (L, d), mean=1.0),
        "rms_final_w": _normal(seed + 11, (d,), mean=1.0),
        "wcls": _normal(seed + 12, (V, d)),
    }


def llama_f32_tensors(cfg, seed=0):
    t = common_tensors(cfg, seed)
    L = cfg["n_layers"]
    for i, (f, (r, c)) in enumerate(family_shapes(cfg).items()):
        t[f] = _normal(seed + 100 + i, (L, r, c))
    return t


def quantize_sym_w4(w, gs):
    """(packed bytes, scales) of a float32 array, symmetric per group of gs consecutive weights."""
    g = w.reshape(-1, gs)
    scale = np.abs(g).max(axis=1) / np.float32(7.0)
    scale[scale < 1e-8] = 1e-8
    q = np.rint(g / scale[:, None])
    np.clip(q, -8, 7, out=q)
    q = (q + 8).astype(np.uint8).reshape(-1)
    return (q[0::2] | (q[1::2] << 4)).astype(np.uint8), scale.astype(np.float32)


def llama_w4_tensors(cfg, seed=0, threads=16):
    """Returns (tensors, offsets): qweights/scales concatenated over families and layers in FAMILIES order."""
    gs, L = cfg["group_size"], cfg["n_layers"]
    shapes = family_shapes(cfg)
    offsets, total = {}, 0
    for f in FAMILIES:
        offsets[f] = total
        total += L * shapes[f][0] * shapes[f][1]
    qweights = np.empty(total // 2, np.uint8)
    scales = np.empty(total // gs, np.float32)

    def work(job):
        fi, f, layer = job
        r, c = shapes[f]
        o = offsets[f] + layer * r * c
        w = _normal(seed + 1000 + fi * 1000 + layer, (r * c,))
        qb, sc = quantize_sym_w4(w, gs)
        qweights[o // 2:(o + r * c) // 2] = qb
        scales[o // gs:(o + r * c) // gs] = sc

    jobs = [(fi, f, layer) for fi, f in enumerate(FAMILIES) for layer in range(L)]
    with cf.ThreadPoolExecutor(max_workers=threads) as ex:
        list(ex.map(work, jobs))
    t = common_tensors(cfg, seed)
    t["qweights"], t["scales"] = qweights, scales
    return t, offsets


def prompt_tokens(n, vocab, seed=1234):
    return np.random.default_rng(seed).integers(0, vocab, n).astype(np.int32)


# --------------------------------------------------------------------------- int8 LLaMA-3.2-1B-style model
# Shapes of examples/llama2/llama32_1b_int8_tensor.sl:5-13; the host bench_llama32_1b_int8.cpp:62-75, 184-195
# fills int8 tensors with uniform integers in [-64, 63] and f32 tensors with uniform [-0.01, 0.01].
LLAMA32_1B_INT8 = dict(dim=2048, hidden_dim=8192, n_layers=16, n_heads=32, n_kv_heads=8, vocab_size=128256,
                       max_seq_len=4096, head_dim=64)


def llama_i8_shapes(cfg):
    d, h, L, V = cfg["dim"], cfg["hidden_dim"], cfg["n_layers"], cfg["vocab_size"]
    kv = cfg["n_kv_heads"] * cfg["head_dim"]
    return dict(rms_att_w=(L, d), rms_ffn_w=(L, d), rms_final_w=(d,), wcls=(V, d),
                wq_t=(L, d, d), wk_t=(L, kv, d), wv_t=(L, kv, d), wo_t=(L, d, d),
                w1_t=(L, h, d), w2_t=(L, d, h), w3_t=(L, h, d))


def llama_i8_tensors(cfg, seed=0, style="bench"):
    """Random-init tensors of the int8 model.  style "bench": the distributions of the reference's host
    (int8 uniform [-64, 63]; f32 uniform [-0.01, 0.01]).  style "unit-norm": norm weights ~ N(1, 0.02),
    which drives the quantised activations into their clamps and wrap-arounds (the harder parity case)."""
    out = {}
    for k, (name, shape) in enumerate(llama_i8_shapes(cfg).items()):
        rng = np.random.default_rng([seed, k])
        if name.endswith("_t"):
            out[name] = rng.integers(-64, 64, size=shape, dtype=np.int8)
        elif style == "unit-norm" and name.startswith("rms_"):
            out[name] = (1.0 + 0.02 * rng.standard_normal(shape)).astype(np.float32)
        else:
            out[name] = rng.uniform(-0.01, 0.01, size=shape).astype(np.float32)
    return out


def llama_i8_input(cfg, seed=1):
    return np.random.default_rng([seed, 99]).integers(-64, 64, size=cfg["dim"], dtype=np.int8)
