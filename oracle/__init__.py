"""ctypes binding of the CPU oracle (``libsimp_oracle.so``) and of the reference's own
compiled int8 kernels (``_ref/*.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the
CPU-baseline / reference legs of ``bench.py`` -- as the checker, never as the thing shipped.
The CUDA library must not import this package.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = {}

i64 = C.c_int64
_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(dtype=np.int8, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")


def reference_dir():
    """Path of the reference checkout: $SIMP_REFERENCE_DIR, else a directory named ``reference`` beside this
    repository; None when neither exists (the prebuilt oracle/_ref objects are then used as they are)."""
    cand = os.environ.get("SIMP_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "simptensor")) else None


def build(with_ref: bool = True) -> None:
    """Compile the oracle (and oracle/_ref when the reference checkout is present)."""
    cmd = ["make", "-C", _HERE, "all" if with_ref else "oracle"]
    ref_dir = reference_dir() if with_ref else None
    if ref_dir:
        cmd.append(f"REF={ref_dir}")
    subprocess.run(cmd, check=True, stdout=subprocess.DEVNULL)


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libsimp_oracle.so")
        if not os.path.exists(path):
            build(with_ref=False)
        _LIB = C.CDLL(path)
        L = _LIB
        L.simp_oracle_max_threads.restype = C.c_int
        L.simp_oracle_set_threads.argtypes = [C.c_int]
        L.simp_oracle_set_threads.restype = C.c_int
        L.simp_oracle_matmul_f32.argtypes = [_f32p, i64, _f32p, i64, _f32p, i64, i64, i64, i64, C.c_int]
        L.simp_oracle_tensor_matmul_f32.argtypes = [_f32p, _f32p, _f32p, i64, i64, i64, C.c_int, C.c_int]
        L.simp_oracle_tensor_matmul_f64.argtypes = [_f64p, _f64p, _f64p, i64, i64, i64, C.c_int, C.c_int]
        L.simp_oracle_tensor_matmul_i8.argtypes = [C.c_void_p, _i8p, _i32p, i64, i64, i64, C.c_int, C.c_int, C.c_int]
        L.simp_oracle_checksum_i32.argtypes = [_i32p, i64]
        L.simp_oracle_checksum_i32.restype = C.c_int32
        L.simp_oracle_dequant_w4.argtypes = [_u8p, _f32p, C.c_void_p, i64, i64, i64, _f32p]
        L.simp_oracle_matmul_quant.argtypes = [_u8p, _f32p, C.c_void_p, _f32p, _f32p, i64, i64, i64, i64, C.c_int, C.c_int]
        L.simp_oracle_quantize_w4.argtypes = [_f32p, i64, i64, _u8p, _f32p, _f32p]
        L.simp_oracle_rmsnorm.argtypes = [_f32p, _f32p, _f32p, i64, C.c_float, i64]
        L.simp_oracle_softmax.argtypes = [_f32p, _f32p, i64, i64, i64]
        L.simp_oracle_silu.argtypes = [_f32p, C.c_void_p, _f32p, i64]
        L.simp_oracle_quantize_i8.argtypes = [_f32p, _i8p, i64, C.c_float, C.c_int]
        L.simp_oracle_dequantize_i32.argtypes = [_i32p, _f32p, i64, C.c_float]
        L.simp_oracle_llama_forward.argtypes = [C.c_void_p, i64, i64]
        L.simp_oracle_llama_forward.restype = C.c_int
        L.simp_oracle_argmax.argtypes = [_f32p, i64]
        L.simp_oracle_argmax.restype = i64
    return _LIB


def use_all_cores() -> int:
    """Sets the OpenMP team size of this process to the cores it may run on (its affinity mask) and returns
    that count.  torch.distributed.run exports OMP_NUM_THREADS=1 to every rank; the CPU baselines call this so
    that they are timed on all host cores whatever launched them."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return int(lib().simp_oracle_set_threads(n))


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


# --------------------------------------------------------------------------- numpy front-ends
def matmul_f32(A, aoff, B, boff, Cbuf, coff, m, k, n, threads=1):
    """In-place C += A.B on flat arrays with element offsets (simp.matmul)."""
    lib().simp_oracle_matmul_f32(A, aoff, B, boff, Cbuf, coff, m, k, n, threads)
    return Cbuf


def tensor_matmul_f32(A, B, b_transposed=False, threads=1):
    M, K = A.shape
    N = B.shape[0] if b_transposed else B.shape[1]
    out = np.empty((M, N), np.float32)
    lib().simp_oracle_tensor_matmul_f32(np.ascontiguousarray(A), np.ascontiguousarray(B), out, M, K, N,
                                        int(b_transposed), threads)
    return out


def tensor_matmul_f64(A, B, b_transposed=False, threads=1):
    M, K = A.shape
    N = B.shape[0] if b_transposed else B.shape[1]
    out = np.empty((M, N), np.float64)
    lib().simp_oracle_tensor_matmul_f64(np.ascontiguousarray(A), np.ascontiguousarray(B), out, M, K, N,
                                        int(b_transposed), threads)
    return out


def tensor_matmul_i8(A, B, b_transposed=False, threads=0):
    """A int8 (signed x signed) or uint8 (vpdpbusd form) [M,K]; B int8 [K,N] or [N,K]."""
    M, K = A.shape
    N = B.shape[0] if b_transposed else B.shape[1]
    A = np.ascontiguousarray(A)
    out = np.empty((M, N), np.int32)
    lib().simp_oracle_tensor_matmul_i8(_ptr(A), np.ascontiguousarray(B), out, M, K, N,
                                       int(A.dtype == np.uint8), int(b_transposed), threads)
    return out


def checksum_i32(Cm):
    return int(lib().simp_oracle_checksum_i32(np.ascontiguousarray(Cm, np.int32).ravel(), Cm.size))


def dequant_w4(qw, sc, zr, idx0, count, gs):
    out = np.empty(count, np.float32)
    lib().simp_oracle_dequant_w4(qw, sc, _ptr(zr), idx0, count, gs, out)
    return out


def matmul_quant(qw, sc, zr, x, rows, cols, gs, offset=0, scale_mode=0, threads=1):
    out = np.empty(rows, np.float32)
    lib().simp_oracle_matmul_quant(qw, sc, _ptr(zr), x, out, rows, cols, gs, offset, scale_mode, threads)
    return out


def quantize_w4(w, gs):
    w = np.ascontiguousarray(w, np.float32).ravel()
    ng = (w.size + gs - 1) // gs
    qw = np.zeros((w.size + 1) // 2, np.uint8)
    sc = np.empty(ng, np.float32)
    zr = np.empty(ng, np.float32)
    lib().simp_oracle_quantize_w4(w, w.size, gs, qw, sc, zr)
    return qw, sc, zr


def rmsnorm(x, w, eps=1e-5, woff=0):
    y = np.empty(x.size, np.float32)
    lib().simp_oracle_rmsnorm(x, w, y, x.size, eps, woff)
    return y


def softmax(x, n=None, xoff=0, yoff=0, out=None):
    n = x.size if n is None else n
    y = np.zeros(yoff + n, np.float32) if out is None else out
    lib().simp_oracle_softmax(x, y, n, xoff, yoff)
    return y


def silu(x, mul=None):
    y = np.empty(x.size, np.float32)
    lib().simp_oracle_silu(x, _ptr(mul), y, x.size)
    return y


def quantize_i8(x, scale=127.0, clamp=True):
    y = np.empty(x.size, np.int8)
    lib().simp_oracle_quantize_i8(x, y, x.size, scale, int(clamp))
    return y


def dequantize_i32(acc, divisor=65536.0):
    y = np.empty(acc.size, np.float32)
    lib().simp_oracle_dequantize_i32(acc, y, acc.size, divisor)
    return y


def pack_i4(values):
    """[rows, cols] integers in [-8, 7] -> [rows, ceil(cols / 2)] bytes, low nibble = even column."""
    v = np.asarray(values)
    rows, cols = v.shape
    n = (v.astype(np.int64) & 15).astype(np.uint8)
    if cols & 1:
        n = np.concatenate([n, np.zeros((rows, 1), np.uint8)], axis=1)
    return np.ascontiguousarray(n[:, 0::2] | (n[:, 1::2] << 4))


def tensor_matmul_i4(A_packed, B_packed, M, K, N, threads=0):
    """Packed signed i4 x i4 -> i16 (wrapping): A [M, ceil(K/2)] bytes, B [K, ceil(N/2)] bytes."""
    A_packed = np.ascontiguousarray(A_packed, np.uint8)
    B_packed = np.ascontiguousarray(B_packed, np.uint8)
    out = np.empty((M, N), np.int16)
    f = lib().simp_oracle_tensor_matmul_i4
    f.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, i64, i64, i64, C.c_int32]
    f.restype = None
    f(_ptr(A_packed), _ptr(B_packed), _ptr(out), M, K, N, threads if threads > 0 else lib().simp_oracle_max_threads())
    return out


def ref_int4_checksums(N):
    """(scalar, packed) checksums of the reference's own i4 runner code, or None when oracle/_ref is absent."""
    L = ref("int4runner")
    if L is None:
        return None
    a, b = C.c_int32(), C.c_int32()
    if L.simp_ref_int4_checksums(N, C.byref(a), C.byref(b)) != 0:
        raise ValueError(f"size {N} not instantiated")
    return int(a.value), int(b.value)


def tensor_gather(source, indices, axis=0):
    """tensor_gather on a numpy array of any rank and dtype; indices are int64."""
    source = np.ascontiguousarray(source)
    indices = np.ascontiguousarray(indices, np.int64)
    axis = axis + source.ndim if axis < 0 else axis
    shape = source.shape
    outer = int(np.prod(shape[:axis], dtype=np.int64))
    inner = int(np.prod(shape[axis + 1:], dtype=np.int64))
    out = np.empty(shape[:axis] + (indices.size,) + shape[axis + 1:], source.dtype)
    f = lib().simp_oracle_tensor_gather
    f.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, i64, i64, i64, i64, i64]
    f.restype = C.c_int
    if f(_ptr(source), _ptr(indices), _ptr(out), outer, shape[axis], inner, indices.size, source.dtype.itemsize) != 0:
        raise IndexError("gather index out of range")
    return out


def conv2d_f32(x, w, bias, stride=(1, 1), pad=(0, 0), threads=0):
    """conv2d: x [N, H, W, IC] f32, w [OC, KH, KW, IC], bias [OC] -> [N, OH, OW, OC]."""
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    bias = np.ascontiguousarray(bias, np.float32)
    n, h, wd, ic = x.shape
    oc, kh, kw, ic2 = w.shape
    assert ic == ic2 and bias.size == oc
    oh, ow = (h + 2 * pad[0] - kh) // stride[0] + 1, (wd + 2 * pad[1] - kw) // stride[1] + 1
    out = np.empty((n, oh, ow, oc), np.float32)
    f = lib().simp_oracle_conv2d_f32
    f.argtypes = [C.c_void_p] * 4 + [i64] * 11 + [C.c_int32]
    f.restype = None
    f(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), n, h, wd, ic, oc, kh, kw, stride[0], stride[1], pad[0], pad[1],
      threads if threads > 0 else lib().simp_oracle_max_threads())
    return out


def argmax(v):
    return int(lib().simp_oracle_argmax(v, v.size))


class LlamaStruct(C.Structure):
    _fields_ = [(n, i64) for n in ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "vocab_size",
                                   "seq_len", "w4", "group_size")] + \
               [(n, C.c_void_p) for n in ("token_embedding", "rms_att_w", "rms_ffn_w", "rms_final_w", "wcls",
                                          "wq", "wk", "wv", "wo", "w1", "w2", "w3",
                                          "qweights", "scales", "zeros")] + \
               [(n, i64) for n in ("wq_off", "wk_off", "wv_off", "wo_off", "w1_off", "w2_off", "w3_off")] + \
               [(n, C.c_void_p) for n in ("key_cache", "value_cache", "logits")] + \
               [("threads", C.c_int32)]


class Llama:
    """Whole-token forward of the f32 (stories110M.sl) or W4 (llama2_quant.sl) model on the CPU.

    ``cfg``: dict with dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len
    (+ group_size for W4).  ``tensors``: dict of numpy arrays named like the struct fields.
    """

    def __init__(self, cfg, tensors, w4=False, offsets=None, threads=0):
        self.cfg = dict(cfg)
        self._keep = dict(tensors)
        kv_dim = cfg["dim"] * cfg["n_kv_heads"] // cfg["n_heads"]
        self.key_cache = np.zeros(cfg["n_layers"] * cfg["seq_len"] * kv_dim, np.float32)
        self.value_cache = np.zeros_like(self.key_cache)
        self.logits = np.zeros(cfg["vocab_size"], np.float32)
        s = LlamaStruct()
        for n in ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "vocab_size", "seq_len"):
            setattr(s, n, cfg[n])
        s.w4 = int(w4)
        s.group_size = cfg.get("group_size", 0)
        for n, a in tensors.items():
            setattr(s, n, _ptr(a))
        for n, v in (offsets or {}).items():
            setattr(s, n, v)
        s.key_cache, s.value_cache, s.logits = _ptr(self.key_cache), _ptr(self.value_cache), _ptr(self.logits)
        s.threads = threads if threads > 0 else lib().simp_oracle_max_threads()
        self._s = s

    def forward(self, token, pos):
        rc = lib().simp_oracle_llama_forward(C.byref(self._s), token, pos)
        if rc != 0:
            raise ValueError("token/pos out of range")
        return self.logits


I8_TENSORS = ("rms_att_w", "rms_ffn_w", "rms_final_w", "wcls", "wq_t", "wk_t", "wv_t", "wo_t", "w1_t", "w2_t", "w3_t")


class LlamaI8Struct(C.Structure):
    _fields_ = [(n, i64) for n in ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "vocab_size",
                                   "max_seq_len", "head_dim")] + \
               [(n, C.c_void_p) for n in I8_TENSORS] + \
               [(n, C.c_void_p) for n in ("k_cache", "v_cache")]


class LlamaI8:
    """Whole-token forward of the int8 LLaMA-3.2-1B-style model (llama32_1b_int8_tensor.sl) on the CPU.

    ``cfg``: dict with dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, max_seq_len, head_dim.
    ``tensors``: dict of numpy arrays named as in ``I8_TENSORS`` (int8 weights pre-transposed [N, K]).
    The int8 KV cache lives in the object; ``forward(x_i8, pos)`` returns the logits.
    """

    def __init__(self, cfg, tensors, threads=0):
        self.cfg = dict(cfg)
        self._keep = {k: np.ascontiguousarray(v) for k, v in tensors.items()}
        kv_dim = cfg["n_kv_heads"] * cfg["head_dim"]
        self.k_cache = np.zeros(cfg["n_layers"] * cfg["max_seq_len"] * kv_dim, np.int8)
        self.v_cache = np.zeros_like(self.k_cache)
        self.logits = np.zeros(cfg["vocab_size"], np.float32)
        s = LlamaI8Struct()
        for n in ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "vocab_size", "max_seq_len", "head_dim"):
            setattr(s, n, cfg[n])
        for n in I8_TENSORS:
            setattr(s, n, _ptr(self._keep[n]))
        s.k_cache, s.v_cache = _ptr(self.k_cache), _ptr(self.v_cache)
        self._s = s
        self.threads = threads if threads > 0 else lib().simp_oracle_max_threads()

    def forward(self, x_i8, pos):
        x_i8 = np.ascontiguousarray(x_i8, np.int8)
        assert x_i8.size == self.cfg["dim"] and 0 <= pos < self.cfg["max_seq_len"]
        f = lib().simp_oracle_llama_i8_forward
        f.argtypes = [C.c_void_p, C.c_void_p, i64, C.c_void_p, C.c_int32]
        f.restype = None
        f(C.byref(self._s), _ptr(x_i8), pos, _ptr(self.logits), self.threads)
        return self.logits


    def prefill(self, x_i8, seq_len):
        """llama32_prefill_<seq_len>: x_i8 [seq_len, dim] -> (x_fp32 [seq_len, dim], k_cache, v_cache
        [n_layers, seq_len, kv_dim]).  Does not touch the object's decode cache."""
        c = self.cfg
        x_i8 = np.ascontiguousarray(x_i8, np.int8)
        assert x_i8.size == seq_len * c["dim"]
        kv_dim = c["n_kv_heads"] * c["head_dim"]
        x = np.zeros((seq_len, c["dim"]), np.float32)
        kc = np.zeros((c["n_layers"], seq_len, kv_dim), np.int8)
        vc = np.zeros_like(kc)
        f = lib().simp_oracle_llama_i8_prefill
        f.argtypes = [C.c_void_p, C.c_void_p, i64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32]
        f.restype = None
        f(C.byref(self._s), _ptr(x_i8), seq_len, _ptr(x), _ptr(kc), _ptr(vc), self.threads)
        return x, kc, vc


# --------------------------------------------------------------------------- reference's own kernels
def cpu_has_vnni() -> bool:
    try:
        with open("/proc/cpuinfo") as f:
            flags = f.read()
    except OSError:
        return False
    return all(x in flags for x in ("avx512_vnni", "avx512bw", "avx512vl", "avx512dq", "avx512cd"))


def ref(unit: str):
    """Load oracle/_ref/libref_<unit>.so, or return None when it is absent or the CPU lacks AVX512-VNNI."""
    if unit not in _REF:
        path = os.path.join(_HERE, "_ref", f"libref_{unit}.so")
        _REF[unit] = C.CDLL(path) if (os.path.exists(path) and cpu_has_vnni()) else None
    return _REF[unit]


def ref_vnni_square(A, B_T, multicore=True):
    """The reference's OpenMP VNNI GEMM (s8 x s8, B pre-transposed, N % 64 == 0)."""
    L = ref("multicore")
    N = A.shape[0]
    out = np.empty((N, N), np.int32)
    L.simp_ref_vnni_square.argtypes = [_i8p, _i8p, _i32p, C.c_int, C.c_int]
    rc = L.simp_ref_vnni_square(np.ascontiguousarray(A), np.ascontiguousarray(B_T), out, N, int(multicore))
    if rc != 0:
        raise ValueError(f"size {N} not instantiated")
    return out


def ref_vnni_mnk(A, B_T, threads=1):
    """The reference's non-square VNNI kernel: A [M,K] s8, B_T [N,K] s8, K % 64 == 0."""
    L = ref("qkv")
    M, K = A.shape
    N = B_T.shape[0]
    out = np.empty((M, N), np.int32)
    L.simp_ref_vnni_mnk.argtypes = [_i8p, _i8p, _i32p, C.c_int, C.c_int, C.c_int, C.c_int]
    rc = L.simp_ref_vnni_mnk(np.ascontiguousarray(A), np.ascontiguousarray(B_T), out, M, N, K, threads)
    if rc != 0:
        raise ValueError("K must be a multiple of 64")
    return out
