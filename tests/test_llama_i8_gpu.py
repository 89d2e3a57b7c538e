"""GPU parity: token forward of the int8 LLaMA-3.2-1B-style model vs the CPU oracle.

All projections accumulate in i32 and are exact; f32 enters through the norms, the attention and the
classifier.  Tolerance (north star, LLaMA logits): max |gpu - ref| / max |ref| <= 1e-3 per step.
The reference holds no known-answer test for this model (parity unpinned): the oracle restates
examples/llama2/llama32_1b_int8_tensor.sl line by line.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SMALL = dict(dim=128, hidden_dim=256, n_layers=2, n_heads=8, n_kv_heads=2, vocab_size=300, max_seq_len=48, head_dim=16)
MID = dict(dim=512, hidden_dim=1376 // 16 * 16, n_layers=3, n_heads=8, n_kv_heads=4, vocab_size=1000, max_seq_len=160, head_dim=64)


def run_positions(gpu, oracle, cfg, seed, style, positions, x_seed=1):
    from simplang_b200 import synth
    t = synth.llama_i8_tensors(cfg, seed, style)
    x = synth.llama_i8_input(cfg, x_seed)
    gm = gpu.LlamaI8(cfg, t)
    om = oracle.LlamaI8(cfg, t)
    worst = 0.0
    for pos in positions:
        a = gm.forward(x, pos)
        b = om.forward(x, pos)
        err = float(np.max(np.abs(a - b)) / (np.max(np.abs(b)) + 1e-30))
        worst = max(worst, err)
        assert err <= 1e-3, (pos, err)
    gm.close()
    return worst


@pytest.mark.parametrize("style", ["bench", "unit-norm"])
def test_small(gpu, oracle, style):
    run_positions(gpu, oracle, SMALL, 3, style, range(0, 40))


@pytest.mark.parametrize("style", ["bench", "unit-norm"])
def test_mid_gqa(gpu, oracle, style):
    """head_dim 64 (the divisor 8.0 is then sqrt(head_dim)), 2 query heads per KV head, hidden_dim not a power
    of two, context long enough for every warp of the attention kernel to hold several timesteps."""
    run_positions(gpu, oracle, MID, 5, style, range(0, 150))


@pytest.mark.parametrize("style", ["bench", "unit-norm"])
def test_long_context_sequence_splits(gpu, oracle, style):
    """max_seq_len 1100 gives the attention kernel 4 sequence splits per head; positions are visited sparsely
    (rows never visited stay zero in both caches), including split boundaries and the last position."""
    cfg = dict(dim=256, hidden_dim=512, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=400, max_seq_len=1100, head_dim=64)
    positions = list(range(0, 9)) + list(range(270, 280)) + list(range(548, 553)) + list(range(1090, 1100))
    run_positions(gpu, oracle, cfg, 11, style, positions)


def test_decode_loop_matches_single_forwards(gpu, oracle):
    from simplang_b200 import synth
    t = synth.llama_i8_tensors(SMALL, 7, "unit-norm")
    x = synth.llama_i8_input(SMALL, 2)
    gm = gpu.LlamaI8(SMALL, t)
    om = oracle.LlamaI8(SMALL, t)
    last, ms = gm.decode_loop(x, 4, 20)          # positions 4 .. 23 on a zeroed cache below position 4
    for pos in range(4, 24):
        ref = om.forward(x, pos)
    assert np.max(np.abs(last - ref)) <= 1e-3 * np.max(np.abs(ref))
    assert ms > 0
    gm.reset_cache()
    a = gm.forward(x, 0)
    om2 = oracle.LlamaI8(SMALL, t)
    assert np.max(np.abs(a - om2.forward(x, 0))) <= 1e-3 * np.max(np.abs(a))
    gm.close()


def test_llama32_1b_full_size(gpu, oracle):
    """The reference's configuration (dim 2048, 16 layers, 32 / 8 heads, hidden 8192, vocab 128256): a few
    positions with the host's own distributions; the CPU oracle needs ~1 s per token."""
    from simplang_b200 import synth
    cfg = dict(synth.LLAMA32_1B_INT8, max_seq_len=256)
    worst = run_positions(gpu, oracle, cfg, 0, "bench", [0, 1, 2, 3])
    print(f"llama-3.2-1B int8: worst logit rel err {worst:.2e}")


def test_errors(gpu):
    from simplang_b200 import synth
    with pytest.raises(gpu.SimpGpuError):
        gpu.LlamaI8(dict(SMALL, dim=120), {})            # n_heads * head_dim != dim
    gm = gpu.LlamaI8(SMALL, {})
    with pytest.raises(gpu.SimpGpuError):
        gm.forward(np.zeros(SMALL["dim"], np.int8), 0)   # tensors not loaded
    gm.close()
    t = synth.llama_i8_tensors(SMALL, 1)
    gm = gpu.LlamaI8(SMALL, t)
    with pytest.raises(gpu.SimpGpuError):
        gm.forward(np.zeros(SMALL["dim"], np.int8), SMALL["max_seq_len"])
    with pytest.raises(gpu.SimpGpuError):
        check = gpu.check
        check(gpu.lib().simp_llama_i8_load(gm.h, b"wq_t", t["wq_t"].ctypes.data, 5))
    gm.close()


# --------------------------------------------------------------------------- prefill (llama32_1b_int8_prefill.sl)
def run_prefill(gpu, oracle, cfg, seed, style, M, x_seed=0):
    from simplang_b200 import synth
    t = synth.llama_i8_tensors(cfg, seed, style)
    x = np.random.default_rng([x_seed, M]).integers(-64, 64, (M, cfg["dim"]), dtype=np.int8)
    gm = gpu.LlamaI8(cfg, t)
    om = oracle.LlamaI8(cfg, t)
    xg, kg, vg, ms = gm.prefill(x, M)
    xo, ko, vo = om.prefill(x, M)
    err = float(np.max(np.abs(xg - xo)) / (np.max(np.abs(xo)) + 1e-30))
    # the caches are integers: count mismatching entries (a flip needs an f32 difference at a truncation boundary)
    bad = int(np.count_nonzero(kg != ko) + np.count_nonzero(vg != vo))
    gm.close()
    return err, bad, ko.size + vo.size, ms, (gm, om, t, x, ko, vo)


@pytest.mark.parametrize("style", ["bench", "unit-norm"])
@pytest.mark.parametrize("M", [1, 8, 13, 48])
def test_prefill_small(gpu, oracle, style, M):
    err, bad, total, _, _ = run_prefill(gpu, oracle, SMALL, 3, style, M)
    assert err <= 1e-3, err
    assert bad <= total // 1000, (bad, total)


@pytest.mark.parametrize("M", [64, 150])
def test_prefill_mid_gqa(gpu, oracle, M):
    err, bad, total, _, _ = run_prefill(gpu, oracle, MID, 5, "bench", M)
    assert err <= 1e-3, err
    assert bad <= total // 1000, (bad, total)


def test_prefill_then_decode_continues(gpu, oracle):
    """The prefill leaves its K/V rows in the device cache; a decode step at position M must see them."""
    from simplang_b200 import synth
    cfg, M = SMALL, 16
    t = synth.llama_i8_tensors(cfg, 9, "bench")
    x = np.random.default_rng(5).integers(-64, 64, (M, cfg["dim"]), dtype=np.int8)
    gm, om = gpu.LlamaI8(cfg, t), oracle.LlamaI8(cfg, t)
    gm.prefill(x, M)
    _, ko, vo = om.prefill(x, M)
    kv = cfg["n_kv_heads"] * cfg["head_dim"]
    om.k_cache.reshape(cfg["n_layers"], cfg["max_seq_len"], kv)[:, :M] = ko
    om.v_cache.reshape(cfg["n_layers"], cfg["max_seq_len"], kv)[:, :M] = vo
    xi = synth.llama_i8_input(cfg, 3)
    a, b = gm.forward(xi, M), om.forward(xi, M)
    assert np.max(np.abs(a - b)) <= 1e-3 * np.max(np.abs(b))
    gm.close()


@pytest.mark.parametrize("M", [8, 64])
def test_prefill_llama32_1b_full_size(gpu, oracle, M):
    """The reference's configuration and its host's distributions (bench_llama32_1b_int8_prefill.cpp)."""
    from simplang_b200 import synth
    cfg = dict(synth.LLAMA32_1B_INT8, max_seq_len=256)
    err, bad, total, ms, _ = run_prefill(gpu, oracle, cfg, 0, "bench", M)
    print(f"llama-3.2-1B int8 prefill M={M}: rel err {err:.2e}, cache mismatches {bad}/{total}, {ms:.2f} ms")
    assert err <= 1e-3, err
    assert bad <= total // 1000, (bad, total)
