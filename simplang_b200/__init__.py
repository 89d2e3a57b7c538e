"""simplang_b200 -- Python binding of ``libsimp_gpu.so``, the B200 (sm_100a) runtime library for
SimpLang's tensor hot path.

The product is the C-ABI library (``include/simp_gpu.h``); this module only loads it with ctypes and
offers numpy conveniences for tests and benchmarks.  There is no CPU fallback: if the shared
library is missing or an op fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("SIMP_GPU_LIB") or os.path.join(_HERE, "libsimp_gpu.so")   # SIMP_GPU_LIB: another build of the library
_LIB = None

i64 = C.c_int64
vp = C.c_void_p


class SimpGpuError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"simp_gpu error {code}: {msg}")
        self.code = code


_SIGNATURES = {
    "simp_gpu_init": [C.c_int],
    "simp_gpu_shutdown": [],
    "simp_gpu_device_count": [C.POINTER(C.c_int)],
    "simp_gpu_alloc": [C.POINTER(vp), C.c_size_t],
    "simp_gpu_free": [vp],
    "simp_gpu_upload": [vp, vp, C.c_size_t],
    "simp_gpu_download": [vp, vp, C.c_size_t],
    "simp_gpu_memset": [vp, C.c_int, C.c_size_t],
    "simp_gpu_sync": [],
    "simp_gpu_check_device_status": [],
    "simp_gpu_matmul_f32": [vp, i64, vp, i64, vp, i64, i64, i64, i64, C.c_int, C.c_int],
    "simp_gpu_matmul_f32_batched": [vp, vp, vp, i64, i64, i64, i64, C.c_int],
    "simp_gpu_matmul_i8": [vp, vp, vp, i64, i64, i64, C.c_int, C.c_int],
    "simp_gpu_matmul_w4": [vp, vp, vp, vp, vp, i64, i64, i64, i64, C.c_int],
    "simp_gpu_dequant_w4": [vp, vp, vp, i64, i64, i64, vp],
    "simp_gpu_matmul_w4_noalloc": [vp, vp, vp, vp, vp, i64, i64, i64, i64, C.c_int],
    "simp_gpu_rmsnorm_f32": [vp, vp, vp, i64, i64, C.c_float, i64, i64, vp],
    "simp_gpu_softmax_f32": [vp, vp, i64, i64, i64, i64, i64],
    "simp_gpu_silu_f32": [vp, vp, vp, i64],
    "simp_gpu_quantize_i8": [vp, vp, i64, C.c_float, C.c_int],
    "simp_gpu_dequantize_i32": [vp, vp, i64, C.c_float],
    "simp_gpu_host_alloc": [C.POINTER(vp), C.c_size_t],
    "simp_gpu_host_free": [vp],
    "simp_gpu_register_host": [vp, C.c_size_t],
    "simp_gpu_unregister_host": [vp],
    "simp_gpu_event_create": [C.POINTER(vp)],
    "simp_gpu_event_record": [vp],
    "simp_gpu_event_elapsed_ms": [vp, vp, C.POINTER(C.c_float)],
    "simp_gpu_event_destroy": [vp],
    "simp_host_tensor_matmul_i8": [vp, vp, vp, i64, i64, i64, C.c_int, C.c_int],
    "simp_host_matmul_f32": [vp, i64, vp, i64, vp, i64, i64, i64, i64, C.c_int, C.c_int],
    "simp_host_matmul_quant": [vp, C.c_size_t, vp, vp, C.c_size_t, vp, vp, i64, i64, i64, i64, C.c_int],
    "simp_host_rmsnorm_f32": [vp, vp, vp, i64, i64, C.c_float, i64],
    "simp_host_softmax_f32": [vp, vp, i64, i64, i64, i64, i64],
    "simp_host_silu_f32": [vp, vp, vp, i64],
    "simp_gpu_matmul_i4": [vp, vp, vp, i64, i64, i64],
    "simp_gpu_tensor_gather": [vp, vp, vp, i64, i64, i64, i64, i64],
    "simp_gpu_conv2d_f32": [vp, vp, vp, vp] + [i64] * 11,
    "simp_gpu_record_begin": [],
    "simp_gpu_record_end": [C.POINTER(vp)],
    "simp_gpu_replay": [vp, i64],
    "simp_gpu_recording_destroy": [vp],
    "simp_llama_create": [vp, C.POINTER(vp)],
    "simp_llama_load": [vp, C.c_char_p, vp, C.c_size_t],
    "simp_llama_set_w4_offsets": [vp, C.POINTER(i64)],
    "simp_llama_forward": [vp, i64, i64, vp],
    "simp_llama_generate": [vp, vp, i64, i64, vp, vp, C.POINTER(C.c_float)],
    "simp_llama_kernels_per_token": [vp, C.POINTER(i64)],
    "simp_llama_destroy": [vp],
    "simp_llama_i8_create": [vp, C.POINTER(vp)],
    "simp_llama_i8_load": [vp, C.c_char_p, vp, C.c_size_t],
    "simp_llama_i8_forward": [vp, vp, i64, vp],
    "simp_llama_i8_decode_loop": [vp, vp, i64, i64, vp, C.POINTER(C.c_float)],
    "simp_llama_i8_prefill": [vp, vp, i64, vp, vp, vp, C.POINTER(C.c_float)],
    "simp_llama_i8_reset_cache": [vp],
    "simp_llama_i8_destroy": [vp],
    "simp_dist_unique_id": [vp, C.c_size_t],
    "simp_dist_init": [C.c_int, C.c_int, vp, C.c_size_t],
    "simp_dist_shutdown": [],
    "simp_dist_rank": [],
    "simp_dist_world": [],
    "simp_dist_allgather": [vp, vp, C.c_size_t],
    "simp_dist_allreduce_f32": [vp, C.c_size_t],
    "simp_dist_matmul_i8_nsharded": [vp, vp, vp, i64, i64, i64, C.c_int, C.c_int],
    "simp_dist_symm_alloc": [C.c_size_t, C.POINTER(vp)],
    "simp_dist_symm_free": [vp],
    "simp_dist_barrier": [],
    "simp_dist_matmul_i8_nsharded_fused": [vp, vp, vp, i64, i64, i64, C.c_int, C.c_int],
}


def lib() -> C.CDLL:
    """The loaded C-ABI library.  Raises if it has not been built (``python -m simplang_b200.build``)."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m simplang_b200.build`; "
                              "there is no CPU fallback")
        L = C.CDLL(LIB_PATH)
        for name, args in _SIGNATURES.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = C.c_int
        L.simp_gpu_last_error.restype = C.c_char_p
        L.simp_gpu_stream.restype = vp
        _LIB = L
    return _LIB


def check(rc: int) -> None:
    if rc != 0:
        raise SimpGpuError(rc, lib().simp_gpu_last_error().decode())


def init(device: int = 0) -> None:
    check(lib().simp_gpu_init(device))


def shutdown() -> None:
    check(lib().simp_gpu_shutdown())


def sync() -> None:
    check(lib().simp_gpu_sync())


def stream_handle() -> int:
    return int(lib().simp_gpu_stream() or 0)


class DeviceBuffer:
    """Device memory owned through the C-ABI (simp_gpu_alloc / simp_gpu_free)."""

    def __init__(self, nbytes: int):
        p = vp()
        check(lib().simp_gpu_alloc(C.byref(p), nbytes))
        self.ptr = p.value
        self.nbytes = nbytes

    @classmethod
    def from_numpy(cls, a: np.ndarray) -> "DeviceBuffer":
        a = np.ascontiguousarray(a)
        b = cls(max(a.nbytes, 16))
        if a.nbytes:
            check(lib().simp_gpu_upload(b.ptr, a.ctypes.data, a.nbytes))
            sync()  # `a` may be a temporary
        return b

    def to_numpy(self, dtype, shape) -> np.ndarray:
        out = np.empty(shape, dtype)
        assert out.nbytes <= self.nbytes
        check(lib().simp_gpu_download(out.ctypes.data, self.ptr, out.nbytes))
        return out

    def upload(self, a: np.ndarray) -> None:
        a = np.ascontiguousarray(a)
        assert a.nbytes <= self.nbytes
        check(lib().simp_gpu_upload(self.ptr, a.ctypes.data, a.nbytes))
        sync()

    def zero(self) -> None:
        check(lib().simp_gpu_memset(self.ptr, 0, self.nbytes))

    def offset(self, nbytes: int) -> int:
        return self.ptr + nbytes

    def free(self) -> None:
        if self.ptr:
            lib().simp_gpu_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _p(b):
    if b is None:
        return None
    return b.ptr if isinstance(b, DeviceBuffer) else int(b)


# ------------------------------------------------------------------------- device-pointer ops
def matmul_f32(A, aoff, B, boff, Cb, coff, m, k, n, accumulate=True, b_transposed=False):
    check(lib().simp_gpu_matmul_f32(_p(A), aoff, _p(B), boff, _p(Cb), coff, m, k, n, int(accumulate),
                                    int(b_transposed)))


def matmul_i8(A, B, Cb, M, K, N, a_unsigned=False, b_transposed=False):
    check(lib().simp_gpu_matmul_i8(_p(A), _p(B), _p(Cb), M, K, N, int(a_unsigned), int(b_transposed)))


def matmul_w4(qw, sc, zr, x, out, rows, cols, gs, offset=0, scale_mode=0):
    check(lib().simp_gpu_matmul_w4(_p(qw), _p(sc), _p(zr), _p(x), _p(out), rows, cols, gs, offset, scale_mode))


def dequant_w4(qw, sc, zr, first, count, gs, out):
    check(lib().simp_gpu_dequant_w4(_p(qw), _p(sc), _p(zr), first, count, gs, _p(out)))


def rmsnorm_f32(x, w, y, rows, n, eps=1e-5, woff=0, row_stride=0, residual=None):
    check(lib().simp_gpu_rmsnorm_f32(_p(x), _p(w), _p(y), rows, n, eps, woff, row_stride, _p(residual)))


def softmax_f32(x, y, rows, n, xoff=0, yoff=0, row_stride=0):
    check(lib().simp_gpu_softmax_f32(_p(x), _p(y), rows, n, xoff, yoff, row_stride))


def silu_f32(x, mul, y, n):
    check(lib().simp_gpu_silu_f32(_p(x), _p(mul), _p(y), n))


def quantize_i8(x, y, n, scale=127.0, clamp=True):
    check(lib().simp_gpu_quantize_i8(_p(x), _p(y), n, scale, int(clamp)))


def dequantize_i32(acc, y, n, divisor=65536.0):
    check(lib().simp_gpu_dequantize_i32(_p(acc), _p(y), n, divisor))


# ------------------------------------------------------------------------- numpy round trips (tests)
def np_matmul_i8(A: np.ndarray, B: np.ndarray, b_transposed=False) -> np.ndarray:
    """Upload, run the int8 GEMM, download.  A int8 or uint8 [M,K]; B int8 [K,N] or [N,K]."""
    M, K = A.shape
    N = B.shape[0] if b_transposed else B.shape[1]
    dA, dB = DeviceBuffer.from_numpy(A), DeviceBuffer.from_numpy(B)
    dC = DeviceBuffer(max(M * N * 4, 16))
    matmul_i8(dA, dB, dC, M, K, N, a_unsigned=(A.dtype == np.uint8), b_transposed=b_transposed)
    out = dC.to_numpy(np.int32, (M, N))
    check(lib().simp_gpu_check_device_status())
    return out


# ------------------------------------------------------------------------- timing, pinned memory
class Event:
    """CUDA event on the library stream (simp_gpu_event_*)."""

    def __init__(self):
        p = vp()
        check(lib().simp_gpu_event_create(C.byref(p)))
        self.ptr = p.value

    def record(self):
        check(lib().simp_gpu_event_record(self.ptr))
        return self

    def elapsed_ms(self, stop: "Event") -> float:
        ms = C.c_float()
        check(lib().simp_gpu_event_elapsed_ms(self.ptr, stop.ptr, C.byref(ms)))
        return float(ms.value)

    def __del__(self):
        try:
            lib().simp_gpu_event_destroy(self.ptr)
        except Exception:
            pass


def pinned_empty(shape, dtype) -> np.ndarray:
    """numpy array backed by pinned host memory from simp_gpu_host_alloc (kept alive by the array)."""
    dtype = np.dtype(dtype)
    n = int(np.prod(shape)) * dtype.itemsize
    p = vp()
    check(lib().simp_gpu_host_alloc(C.byref(p), max(n, 16)))
    buf = (C.c_uint8 * max(n, 16)).from_address(p.value)
    arr = np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape)
    _PINNED.append((p.value, buf))
    return arr


_PINNED = []


# ------------------------------------------------------------------------- host-pointer ops (numpy in, numpy out)
def host_tensor_matmul_i8(A: np.ndarray, B: np.ndarray, out: np.ndarray = None, b_transposed=False) -> np.ndarray:
    M, K = A.shape
    N = B.shape[0] if b_transposed else B.shape[1]
    if out is None:
        out = np.empty((M, N), np.int32)
    check(lib().simp_host_tensor_matmul_i8(A.ctypes.data, B.ctypes.data, out.ctypes.data, M, K, N,
                                           int(A.dtype == np.uint8), int(b_transposed)))
    return out


# ------------------------------------------------------------------------- LLaMA decode driver
def np_matmul_i4(A_packed: np.ndarray, B_packed: np.ndarray, M: int, K: int, N: int) -> np.ndarray:
    """Packed signed i4 x i4 -> i16 (numpy in / out): A [M, ceil(K/2)] bytes, B [K, ceil(N/2)] bytes."""
    dA = DeviceBuffer.from_numpy(np.ascontiguousarray(A_packed, np.uint8))
    dB = DeviceBuffer.from_numpy(np.ascontiguousarray(B_packed, np.uint8))
    dC = DeviceBuffer(max(M * N * 2, 16))
    check(lib().simp_gpu_matmul_i4(dA.ptr, dB.ptr, dC.ptr, M, K, N))
    return dC.to_numpy(np.int16, (M, N))


def np_tensor_gather(source: np.ndarray, indices, axis: int = 0) -> np.ndarray:
    """tensor_gather on a numpy array of any rank and dtype (numpy in / out)."""
    source = np.ascontiguousarray(source)
    indices = np.ascontiguousarray(indices, np.int64)
    axis = axis + source.ndim if axis < 0 else axis
    shape = source.shape
    outer = int(np.prod(shape[:axis], dtype=np.int64))
    inner = int(np.prod(shape[axis + 1:], dtype=np.int64))
    out_shape = shape[:axis] + (indices.size,) + shape[axis + 1:]
    dS, dI = DeviceBuffer.from_numpy(source), DeviceBuffer.from_numpy(indices)
    nbytes = int(np.prod(out_shape, dtype=np.int64)) * source.dtype.itemsize
    dD = DeviceBuffer(max(nbytes, 16))
    check(lib().simp_gpu_tensor_gather(dS.ptr, dI.ptr, dD.ptr, outer, shape[axis], inner, indices.size, source.dtype.itemsize))
    check(lib().simp_gpu_check_device_status())
    return dD.to_numpy(source.dtype, out_shape)


def np_conv2d_f32(x: np.ndarray, w: np.ndarray, bias: np.ndarray, stride=(1, 1), pad=(0, 0)) -> np.ndarray:
    """conv2d (numpy in / out): x [N, H, W, IC], w [OC, KH, KW, IC], bias [OC] -> [N, OH, OW, OC]."""
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    bias = np.ascontiguousarray(bias, np.float32)
    n, h, wd, ic = x.shape
    oc, kh, kw, _ = w.shape
    oh, ow = (h + 2 * pad[0] - kh) // stride[0] + 1, (wd + 2 * pad[1] - kw) // stride[1] + 1
    dX, dW, dB = DeviceBuffer.from_numpy(x), DeviceBuffer.from_numpy(w), DeviceBuffer.from_numpy(bias)
    dY = DeviceBuffer(max(n * oh * ow * oc * 4, 16))
    check(lib().simp_gpu_conv2d_f32(dX.ptr, dW.ptr, dB.ptr, dY.ptr, n, h, wd, ic, oc, kh, kw, stride[0], stride[1], pad[0], pad[1]))
    return dY.to_numpy(np.float32, (n, oh, ow, oc))


class Recording:
    """``with Recording() as r: <device-pointer calls>`` records the calls; ``r.replay(n)`` enqueues them n times."""

    def __init__(self):
        self.h = None

    def __enter__(self):
        check(lib().simp_gpu_record_begin())
        return self

    def __exit__(self, et, ev, tb):
        h = vp()
        rc = lib().simp_gpu_record_end(C.byref(h))
        if et is None:
            check(rc)
            self.h = h
        return False

    def replay(self, times=1):
        check(lib().simp_gpu_replay(self.h, times))

    def close(self):
        if self.h:
            lib().simp_gpu_recording_destroy(self.h)
            self.h = None


class LlamaConfig(C.Structure):
    _fields_ = [(n, i64) for n in ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "vocab_size", "seq_len",
                                   "w4", "group_size", "tp_size")]


W4_FAMILIES = ("wq", "wk", "wv", "wo", "w1", "w2", "w3")


class Llama:
    """Device-resident LLaMA decoder (simp_llama_*).  ``tensors`` maps the .sl argument names to numpy arrays;
    for W4 pass qweights / scales [/ zeros] and ``offsets`` = {family: element offset}."""

    def __init__(self, cfg: dict, tensors: dict, w4=False, offsets=None, tp_size=1):
        c = LlamaConfig(**{k: cfg[k] for k in ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "vocab_size",
                                                "seq_len")}, w4=int(w4), group_size=cfg.get("group_size", 0),
                        tp_size=tp_size)
        h = vp()
        check(lib().simp_llama_create(C.byref(c), C.byref(h)))
        self.h = h
        self.vocab = cfg["vocab_size"]
        if w4:  # offsets first: under tensor parallelism the loader slices the shared arrays with them
            off = (i64 * 7)(*[offsets[f] if isinstance(offsets, dict) else offsets[i] for i, f in enumerate(W4_FAMILIES)])
            check(lib().simp_llama_set_w4_offsets(self.h, off))
        for name, arr in tensors.items():
            arr = np.ascontiguousarray(arr)
            check(lib().simp_llama_load(self.h, name.encode(), arr.ctypes.data, arr.nbytes))

    def forward(self, token: int, pos: int) -> np.ndarray:
        out = np.empty(self.vocab, np.float32)
        check(lib().simp_llama_forward(self.h, token, pos, out.ctypes.data))
        return out

    def generate(self, prompt, n_new: int, trace_logits=False):
        prompt = np.ascontiguousarray(prompt, np.int32)
        toks = np.empty(n_new, np.int32)
        steps = len(prompt) + n_new - 1
        trace = np.empty((steps, self.vocab), np.float32) if trace_logits else None
        ms = C.c_float()
        check(lib().simp_llama_generate(self.h, prompt.ctypes.data, len(prompt), n_new, toks.ctypes.data,
                                        trace.ctypes.data if trace_logits else None, C.byref(ms)))
        return toks, trace, float(ms.value)

    def kernels_per_token(self) -> int:
        n = i64()
        check(lib().simp_llama_kernels_per_token(self.h, C.byref(n)))
        return int(n.value)

    def close(self):
        if self.h:
            lib().simp_llama_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class LlamaI8Config(C.Structure):
    _fields_ = [(n, i64) for n in ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "vocab_size",
                                   "max_seq_len", "head_dim")]


class LlamaI8:
    """Device-resident int8 LLaMA-3.2-1B-style model (simp_llama_i8_*): int8 input vector and position in,
    f32 logits out.  ``tensors`` maps the .sl argument names (rms_att_w, wq_t, ...) to numpy arrays."""

    def __init__(self, cfg: dict, tensors: dict):
        c = LlamaI8Config(**{k: cfg[k] for k in ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "vocab_size",
                                                  "max_seq_len", "head_dim")})
        h = vp()
        check(lib().simp_llama_i8_create(C.byref(c), C.byref(h)))
        self.h = h
        self.dim, self.vocab = cfg["dim"], cfg["vocab_size"]
        self.n_layers, self.kv_dim = cfg["n_layers"], cfg["n_kv_heads"] * cfg["head_dim"]
        for name, arr in tensors.items():
            arr = np.ascontiguousarray(arr)
            check(lib().simp_llama_i8_load(self.h, name.encode(), arr.ctypes.data, arr.nbytes))

    def forward(self, x_i8, pos: int) -> np.ndarray:
        x_i8 = np.ascontiguousarray(x_i8, np.int8)
        assert x_i8.size == self.dim
        out = np.empty(self.vocab, np.float32)
        check(lib().simp_llama_i8_forward(self.h, x_i8.ctypes.data, pos, out.ctypes.data))
        return out

    def decode_loop(self, x_i8, start_pos: int, n_tokens: int):
        """n_tokens forwards at consecutive positions; returns (logits of the last one, device ms of the loop)."""
        x_i8 = np.ascontiguousarray(x_i8, np.int8)
        assert x_i8.size == self.dim
        out = np.empty(self.vocab, np.float32)
        ms = C.c_float()
        check(lib().simp_llama_i8_decode_loop(self.h, x_i8.ctypes.data, start_pos, n_tokens, out.ctypes.data, C.byref(ms)))
        return out, float(ms.value)

    def prefill(self, x_i8, seq_len: int):
        """llama32_prefill_<seq_len>: returns (x_fp32 [seq_len, dim], k_cache, v_cache [n_layers, seq_len, kv_dim], ms)."""
        x_i8 = np.ascontiguousarray(x_i8, np.int8)
        assert x_i8.size == seq_len * self.dim
        x = np.empty((seq_len, self.dim), np.float32)
        kc = np.empty((self.n_layers, seq_len, self.kv_dim), np.int8)
        vc = np.empty_like(kc)
        ms = C.c_float()
        check(lib().simp_llama_i8_prefill(self.h, x_i8.ctypes.data, seq_len, x.ctypes.data, kc.ctypes.data, vc.ctypes.data,
                                          C.byref(ms)))
        return x, kc, vc, float(ms.value)

    def reset_cache(self):
        check(lib().simp_llama_i8_reset_cache(self.h))

    def close(self):
        if self.h:
            lib().simp_llama_i8_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
