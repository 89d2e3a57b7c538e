"""GPU parity: whole-token LLaMA decode (f32 110M-style and W4 3B-style) vs the CPU oracle.

Tolerance (north star): logits within relative error 1e-3 (max |gpu - ref| / max |ref| per step) and an
identical greedy token sequence for the first 64 generated tokens.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def run_pair(gpu, oracle, cfg, tensors, w4, offsets, n_prompt, n_new, seed=1234):
    from simplang_b200 import synth
    prompt = synth.prompt_tokens(n_prompt, cfg["vocab_size"], seed)
    gm = gpu.Llama(cfg, tensors, w4=w4, offsets=offsets)
    toks, trace, ms = gm.generate(prompt, n_new, trace_logits=True)
    ot = dict(tensors)
    off = None
    if w4:
        off = {k + "_off": v for k, v in offsets.items()}
    om = oracle.Llama(cfg, ot, w4=w4, offsets=off, threads=0)
    ref_toks, worst, tok = [], 0.0, int(prompt[0])
    for pos in range(n_prompt + n_new - 1):
        logits = om.forward(tok, pos)
        err = np.max(np.abs(trace[pos] - logits)) / (np.max(np.abs(logits)) + 1e-30)
        worst = max(worst, float(err))
        nxt = oracle.argmax(logits)
        if pos + 1 < n_prompt:
            tok = int(prompt[pos + 1])
        else:
            tok = nxt
            ref_toks.append(nxt)
        if pos + 1 >= n_prompt and toks[pos + 1 - n_prompt] != nxt:
            top2 = np.sort(logits)[-2:]
            raise AssertionError(f"token mismatch at generated index {pos + 1 - n_prompt}: gpu {toks[pos + 1 - n_prompt]} "
                                 f"ref {nxt}; oracle top-2 margin {top2[1] - top2[0]:.3e}, worst logit err so far {worst:.3e}")
    gm.close()
    assert worst <= 1e-3, worst
    assert list(toks) == ref_toks
    return worst, ms


TINY = dict(dim=128, hidden_dim=256, n_layers=3, n_heads=4, n_kv_heads=4, vocab_size=300, seq_len=64)


@pytest.fixture(params=["persistent", "graph"])
def decode_mode(request, monkeypatch):
    """The f32 model has two device forms: one cooperative kernel per token (default), or a graph of per-op kernels
    (SIMP_DECODE_MODE=graph, read when a model builds its token graph).  The W4 model has the graph form only."""
    monkeypatch.setenv("SIMP_DECODE_MODE", request.param)
    return request.param


def test_tiny_f32(gpu, oracle, decode_mode):
    from simplang_b200 import synth
    run_pair(gpu, oracle, TINY, synth.llama_f32_tensors(TINY, 3), False, None, 5, 40)


def test_small_f32_gqa_long(gpu, oracle, decode_mode):
    """Grouped-query heads (kv_mul 2), rows not divisible by the SM count, context long enough for every
    sequence split of the attention phase to hold several timesteps."""
    from simplang_b200 import synth
    cfg = dict(dim=256, hidden_dim=688, n_layers=2, n_heads=8, n_kv_heads=4, vocab_size=515, seq_len=320)
    run_pair(gpu, oracle, cfg, synth.llama_f32_tensors(cfg, 11), False, None, 6, 300)


def test_tiny_f32_gqa_odd_head(gpu, oracle):
    from simplang_b200 import synth
    cfg = dict(dim=200, hidden_dim=320, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=97, seq_len=300)  # hs = 50
    run_pair(gpu, oracle, cfg, synth.llama_f32_tensors(cfg, 5), False, None, 3, 280)


@pytest.mark.parametrize("gs", [32, 64, 128])
def test_tiny_w4(gpu, oracle, gs):
    from simplang_b200 import synth
    cfg = dict(TINY, group_size=gs)
    t, off = synth.llama_w4_tensors(cfg, 7, threads=4)
    run_pair(gpu, oracle, cfg, t, True, off, 4, 30)


def test_tiny_w4_asymmetric(gpu, oracle):
    """Reference-style asymmetric groups (zeros array present), quantised by the host quantiser's formula."""
    from simplang_b200 import synth
    cfg = dict(TINY, group_size=64)
    f32 = synth.llama_f32_tensors(cfg, 9)
    shapes = synth.family_shapes(cfg)
    flat, offsets, total = [], {}, 0
    for f in synth.FAMILIES:
        offsets[f] = total
        flat.append(f32[f].reshape(-1))
        total += f32[f].size
    qw, sc, zr = oracle.quantize_w4(np.concatenate(flat), 64)
    t = {k: v for k, v in f32.items() if k not in synth.FAMILIES}
    t.update(qweights=qw, scales=sc, zeros=zr)
    run_pair(gpu, oracle, cfg, t, True, offsets, 4, 20)


def test_stories110m_f32(gpu, oracle, decode_mode):
    """BASELINE config: dim 768, 12 layers, 12 heads, FFN 2048, vocab 32000, seq 1024; 16-token prompt, 64 greedy tokens."""
    from simplang_b200 import synth
    cfg = synth.STORIES_110M
    worst, ms = run_pair(gpu, oracle, cfg, synth.llama_f32_tensors(cfg, 0), False, None, 16, 64)
    print(f"110M f32 ({decode_mode}): worst logit rel err {worst:.2e}, {79 / ms * 1e3:.0f} tok/s")


def test_llama3b_w4(gpu, oracle):
    """BASELINE config: dim 3200, 26 layers, 32 heads (hs 100), FFN 8640, W4 gs 64; 16-token prompt, 64 greedy tokens."""
    from simplang_b200 import synth
    cfg = synth.LLAMA_3B_W4
    t, off = synth.llama_w4_tensors(cfg, 0, threads=16)
    worst, ms = run_pair(gpu, oracle, cfg, t, True, off, 16, 64)
    print(f"3B W4: worst logit rel err {worst:.2e}, {79 / ms * 1e3:.0f} tok/s")


def test_forward_api_and_errors(gpu, oracle):
    from simplang_b200 import synth
    t = synth.llama_f32_tensors(TINY, 3)
    gm = gpu.Llama(TINY, t)
    om = oracle.Llama(TINY, t, threads=1)
    for pos, tok in enumerate([5, 17, 3]):
        a, b = gm.forward(tok, pos), om.forward(tok, pos)
        assert np.max(np.abs(a - b)) <= 1e-3 * np.max(np.abs(b))
    with pytest.raises(gpu.SimpGpuError):
        gm.forward(TINY["vocab_size"], 0)
    with pytest.raises(gpu.SimpGpuError):
        gm.forward(0, TINY["seq_len"])
    gm.close()
    with pytest.raises(gpu.SimpGpuError):
        gpu.Llama(dict(TINY, dim=130), {})  # dim % n_heads != 0
