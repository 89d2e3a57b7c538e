// host_api.cu -- the reference-facing layer: entry points that take HOST pointers, as the
// reference's compiled kernels do (its hosts pass std::vector::data() on every call,
// examples/llama2/generate_stories110M.cpp:236-251; simptensor/benchmarks/bench_prefill_matmul_runner.cpp:18-23).
//
// Operands are copied to the device, the device op runs, results are copied back; the call
// returns when the results are in host memory.  Long-lived operands (weights) can be registered
// once with simp_gpu_register_host(): later calls that pass a pointer inside a registered range
// use the resident device mirror instead of copying.
// Also here: pinned host memory and CUDA-event timing for the host drivers.
#include <cstdint>
#include <map>
#include <mutex>
#include <vector>

#include <cstdlib>
#include "common.cuh"

namespace simp {

struct Mirror {
  size_t bytes;
  void* dev;
};
static std::map<uintptr_t, Mirror> g_mirrors;  // keyed by host base address
static std::mutex g_reg_mu;

// Device address mirroring host pointer `h`, or nullptr when `h` is not inside a registered range.
static void* lookup_mirror(const void* h, size_t bytes) {
  std::lock_guard<std::mutex> lk(g_reg_mu);
  const uintptr_t a = reinterpret_cast<uintptr_t>(h);
  auto it = g_mirrors.upper_bound(a);
  if (it == g_mirrors.begin()) return nullptr;
  --it;
  if (a >= it->first && a + bytes <= it->first + it->second.bytes)
    return static_cast<uint8_t*>(it->second.dev) + (a - it->first);
  return nullptr;
}

// Device copy of a host input: the registered mirror, or a staged copy in arena `slot`.
static int stage_in(const void* h, size_t bytes, int slot, cudaStream_t st, void** dev) {
  if (void* m = lookup_mirror(h, bytes)) {
    *dev = m;
    return SIMP_OK;
  }
  void* d = scratch(bytes ? bytes : 16, slot);
  SIMP_REQUIRE(d != nullptr, SIMP_ERR_CUDA, "out of device memory staging %zu bytes", bytes);
  if (bytes) SIMP_CUDA(cudaMemcpyAsync(d, h, bytes, cudaMemcpyHostToDevice, st));
  *dev = d;
  return SIMP_OK;
}

}  // namespace simp

using namespace simp;

// ---- pinned memory, registration, events ------------------------------------------------------
SIMP_API int simp_gpu_host_alloc(void** hptr, size_t bytes) {
  SIMP_REQUIRE(hptr != nullptr, SIMP_ERR_ARG, "host_alloc: null pointer");
  if (int rc = ensure_ready()) return rc;
  SIMP_CUDA(cudaMallocHost(hptr, bytes ? bytes : 16));
  return SIMP_OK;
}
SIMP_API int simp_gpu_host_free(void* hptr) {
  if (!hptr) return SIMP_OK;
  SIMP_CUDA(cudaFreeHost(hptr));
  return SIMP_OK;
}
SIMP_API int simp_gpu_register_host(const void* host, size_t bytes) {
  SIMP_REQUIRE(host != nullptr && bytes > 0, SIMP_ERR_ARG, "register_host: null pointer or empty range");
  if (int rc = ensure_ready()) return rc;
  void* d = nullptr;
  SIMP_CUDA(cudaMalloc(&d, bytes));
  SIMP_CUDA(cudaMemcpyAsync(d, host, bytes, cudaMemcpyHostToDevice, ctx().stream));
  SIMP_CUDA(cudaStreamSynchronize(ctx().stream));
  std::lock_guard<std::mutex> lk(g_reg_mu);
  auto old = g_mirrors.find(reinterpret_cast<uintptr_t>(host));
  if (old != g_mirrors.end()) {
    cudaFree(old->second.dev);
    g_mirrors.erase(old);
  }
  g_mirrors[reinterpret_cast<uintptr_t>(host)] = Mirror{bytes, d};
  return SIMP_OK;
}
SIMP_API int simp_gpu_unregister_host(const void* host) {
  std::lock_guard<std::mutex> lk(g_reg_mu);
  auto it = g_mirrors.find(reinterpret_cast<uintptr_t>(host));
  SIMP_REQUIRE(it != g_mirrors.end(), SIMP_ERR_ARG, "unregister_host: pointer was not registered");
  cudaStreamSynchronize(ctx().stream);
  cudaFree(it->second.dev);
  g_mirrors.erase(it);
  return SIMP_OK;
}
SIMP_API int simp_gpu_event_create(void** ev) {
  SIMP_REQUIRE(ev != nullptr, SIMP_ERR_ARG, "event_create: null pointer");
  if (int rc = ensure_ready()) return rc;
  cudaEvent_t e;
  SIMP_CUDA(cudaEventCreate(&e));
  *ev = e;
  return SIMP_OK;
}
SIMP_API int simp_gpu_event_record(void* ev) {
  SIMP_REQUIRE(ev != nullptr, SIMP_ERR_ARG, "event_record: null event");
  SIMP_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(ev), ctx().stream));
  return SIMP_OK;
}
SIMP_API int simp_gpu_event_elapsed_ms(void* start, void* stop, float* ms) {
  SIMP_REQUIRE(start && stop && ms, SIMP_ERR_ARG, "event_elapsed_ms: null pointer");
  SIMP_CUDA(cudaEventSynchronize(static_cast<cudaEvent_t>(stop)));
  SIMP_CUDA(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)));
  return SIMP_OK;
}
SIMP_API int simp_gpu_event_destroy(void* ev) {
  if (ev) SIMP_CUDA(cudaEventDestroy(static_cast<cudaEvent_t>(ev)));
  return SIMP_OK;
}

// ---- replaying a sequence of calls ----------------------------------------------------------
// A host that repeats the same sequence of device-pointer calls (a benchmark loop, a layer applied to resident
// buffers) can record it once and replay it: the replay costs one launch instead of one per call, which is
// what a microsecond-scale kernel needs to be measured (or used) at its device speed.
SIMP_API int simp_gpu_record_begin(void) {
  if (int rc = ensure_ready()) return rc;
  SIMP_CUDA(cudaStreamBeginCapture(ctx().stream, cudaStreamCaptureModeThreadLocal));
  scratch_capture(true);
  return SIMP_OK;
}
SIMP_API int simp_gpu_record_end(void** recording) {
  SIMP_REQUIRE(recording != nullptr, SIMP_ERR_ARG, "record_end: null pointer");
  cudaGraph_t g = nullptr;
  cudaError_t e = cudaStreamEndCapture(ctx().stream, &g);
  scratch_capture(false);
  SIMP_REQUIRE(e == cudaSuccess && g != nullptr, SIMP_ERR_CUDA, "record_end: capture failed: %s", cudaGetErrorString(e));
  cudaGraphExec_t ex = nullptr;
  e = cudaGraphInstantiate(&ex, g, 0);
  cudaGraphDestroy(g);
  SIMP_REQUIRE(e == cudaSuccess, SIMP_ERR_CUDA, "record_end: instantiate failed: %s", cudaGetErrorString(e));
  *recording = ex;
  scratch_recordings(+1);
  return SIMP_OK;
}
SIMP_API int simp_gpu_replay(void* recording, int64_t times) {
  SIMP_REQUIRE(recording != nullptr && times >= 0, SIMP_ERR_ARG, "replay: null recording or negative count");
  for (int64_t i = 0; i < times; ++i) SIMP_CUDA(cudaGraphLaunch(static_cast<cudaGraphExec_t>(recording), ctx().stream));
  return SIMP_OK;
}
SIMP_API int simp_gpu_recording_destroy(void* recording) {
  if (recording) {
    SIMP_CUDA(cudaStreamSynchronize(ctx().stream));
    SIMP_CUDA(cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(recording)));
    scratch_recordings(-1);
  }
  return SIMP_OK;
}

// ---- host-pointer ops -------------------------------------------------------------------------
namespace {
// Large host-to-host tensor_matmul on i8 whose operands are not resident on the device: the time is the PCIe time of
// the 4-byte result (twice the bytes of both operands together at square shapes), so what matters is how soon the
// first piece of C can leave and that the download never waits afterwards.  C is cut into row chunks x column blocks:
// a block needs only its row chunk of A and its column block of B, so the first download starts after ~1/5 of the
// operand bytes have arrived instead of after all of B.  Uploads are ordered so that every upload unlocks blocks
// (B_0, A_0, A_1, B_1, A_2, A_3, B_2, ...); a block's GEMM is enqueued as soon as both of its operands are on the
// way; three streams (upload, compute, download) chained by events.  On the device every column block of B and of C
// is a dense matrix of its own (2-D copies repack them), so the GEMM sees ordinary dense operands.
int host_matmul_i8_blocked(const void* A, const int8_t* B, int32_t* C, int64_t M, int64_t K, int64_t N, int a_unsigned,
                           int b_transposed, int64_t chunk, int64_t nb) {
  Context& c = ctx();
  const int nrow = int(cdiv(M, chunk)), ncol = int(cdiv(N, nb));
  uint8_t* dA = static_cast<uint8_t*>(scratch(size_t(M) * K + 16, 0));
  int8_t* dB = static_cast<int8_t*>(scratch(size_t(K) * N + 16, 1));
  int32_t* dC = static_cast<int32_t*>(scratch(size_t(M) * N * 4, 2));
  SIMP_REQUIRE(dA && dB && dC, SIMP_ERR_CUDA, "host tensor_matmul_i8: out of device memory for the staged operands");
  std::vector<cudaEvent_t> ev_a(nrow, nullptr), ev_b(ncol, nullptr), ev_done(size_t(nrow) * ncol, nullptr);
  std::vector<char> a_up(nrow, 0), b_up(ncol, 0), done(size_t(nrow) * ncol, 0);
  int rc = SIMP_OK;
  cudaError_t ce = cudaSuccess;
  auto note = [&](cudaError_t e) { if (ce == cudaSuccess && e != cudaSuccess) ce = e; };
  auto col_width = [&](int j) { return (int64_t(j) + 1) * nb <= N ? nb : N - int64_t(j) * nb; };
  auto row_count = [&](int i) { return (int64_t(i) + 1) * chunk <= M ? chunk : M - int64_t(i) * chunk; };
  // device layout: column block j of B is dense [K, w_j] (or [w_j, K] when transposed) at dB + K * j * nb; column block
  // j of C is dense [M, w_j] at dC + M * j * nb
  auto upload_a = [&](int i) {
    const int64_t r0 = int64_t(i) * chunk;
    note(cudaMemcpyAsync(dA + r0 * K, static_cast<const uint8_t*>(A) + r0 * K, size_t(row_count(i)) * K, cudaMemcpyHostToDevice,
                         c.copy_in));
    note(cudaEventCreateWithFlags(&ev_a[i], cudaEventDisableTiming));
    note(cudaEventRecord(ev_a[i], c.copy_in));
    a_up[i] = 1;
  };
  auto upload_b = [&](int j) {
    const int64_t c0 = int64_t(j) * nb, w = col_width(j);
    int8_t* dst = dB + K * c0;
    if (b_transposed) note(cudaMemcpyAsync(dst, B + c0 * K, size_t(w) * K, cudaMemcpyHostToDevice, c.copy_in));
    else note(cudaMemcpy2DAsync(dst, size_t(w), B + c0, size_t(N), size_t(w), size_t(K), cudaMemcpyHostToDevice, c.copy_in));
    note(cudaEventCreateWithFlags(&ev_b[j], cudaEventDisableTiming));
    note(cudaEventRecord(ev_b[j], c.copy_in));
    b_up[j] = 1;
  };
  auto run_ready_blocks = [&]() {
    for (int j = 0; j < ncol && rc == SIMP_OK; ++j)
      for (int i = 0; i < nrow && rc == SIMP_OK; ++i) {
        const size_t id = size_t(j) * nrow + i;
        if (done[id] || !a_up[i] || !b_up[j]) continue;
        done[id] = 1;
        const int64_t r0 = int64_t(i) * chunk, c0 = int64_t(j) * nb, w = col_width(j), rows = row_count(i);
        int32_t* cblk = dC + M * c0 + r0 * w;
        note(cudaStreamWaitEvent(c.stream, ev_a[i], 0));
        note(cudaStreamWaitEvent(c.stream, ev_b[j], 0));
        rc = simp_gpu_matmul_i8(dA + r0 * K, dB + K * c0, cblk, rows, K, w, a_unsigned, b_transposed);
        if (rc != SIMP_OK) break;
        note(cudaEventCreateWithFlags(&ev_done[id], cudaEventDisableTiming));
        note(cudaEventRecord(ev_done[id], c.stream));
        note(cudaStreamWaitEvent(c.copy_out, ev_done[id], 0));
        note(cudaMemcpy2DAsync(C + r0 * N + c0, size_t(N) * 4, cblk, size_t(w) * 4, size_t(w) * 4, size_t(rows),
                               cudaMemcpyDeviceToHost, c.copy_out));
      }
  };
  // upload order: B_0, then two row chunks of A per further column block of B, the rest of A (or B) at the end
  int ia = 0, jb = 0;
  upload_b(jb++);
  while ((ia < nrow || jb < ncol) && rc == SIMP_OK) {
    for (int t = 0; t < 2 && ia < nrow; ++t) {
      upload_a(ia++);
      run_ready_blocks();
    }
    if (jb < ncol) {
      upload_b(jb++);
      run_ready_blocks();
    }
  }
  const cudaError_t e1 = cudaStreamSynchronize(c.copy_out), e2 = cudaStreamSynchronize(c.stream),
                    e3 = cudaStreamSynchronize(c.copy_in);
  for (auto e : ev_a) if (e) cudaEventDestroy(e);
  for (auto e : ev_b) if (e) cudaEventDestroy(e);
  for (auto e : ev_done) if (e) cudaEventDestroy(e);
  if (rc != SIMP_OK) return rc;
  note(e1); note(e2); note(e3);
  SIMP_REQUIRE(ce == cudaSuccess, SIMP_ERR_CUDA, "host tensor_matmul_i8: %s", cudaGetErrorString(ce));
  return SIMP_OK;
}
}  // namespace

// tensor_matmul on i8 with host operands.  Rows of A are processed in chunks so that the upload of
// chunk c+1, the GEMM of chunk c and the download of chunk c-1 overlap on three streams; large products whose
// operands are both staged from the host also cut B and C into column blocks (host_matmul_i8_blocked).
SIMP_API int simp_host_tensor_matmul_i8(const void* A, const int8_t* B, int32_t* C, int64_t M, int64_t K,
                                        int64_t N, int a_unsigned, int b_transposed) {
  if (int rc = ensure_ready()) return rc;
  SIMP_REQUIRE(M >= 0 && K >= 0 && N >= 0, SIMP_ERR_ARG, "host tensor_matmul_i8: negative size");
  if (M == 0 || N == 0) return SIMP_OK;
  SIMP_REQUIRE(A && B && C, SIMP_ERR_ARG, "host tensor_matmul_i8: null pointer");
  Context& c = ctx();
  if (K > 0 && M >= 1024 && N >= 2048 && N % 1024 == 0 && size_t(K) * size_t(N) >= (size_t(16) << 20) &&
      lookup_mirror(A, size_t(M) * K) == nullptr && lookup_mirror(B, size_t(K) * N) == nullptr) {
    const int64_t chunk = ((cdiv(M, 8) + 127) / 128) * 128;
    // four column blocks: measured at 8192^3 with pinned buffers, ms per call: one block (row chunks only) 6.34,
    // two 6.14, four 5.83, eight 6.43 (shorter row segments in the strided download cost more than the earlier start gains)
    const int64_t nb = ((cdiv(N, 4) + 255) / 256) * 256;
    return host_matmul_i8_blocked(A, B, C, M, K, N, a_unsigned, b_transposed, chunk, nb);
  }
  void *dA = nullptr, *dB = nullptr;
  const bool a_resident = lookup_mirror(A, size_t(M) * K) != nullptr;
  if (int rc = stage_in(B, size_t(K) * N, 1, c.copy_in, &dB)) return rc;
  int32_t* dC = static_cast<int32_t*>(scratch(size_t(M) * N * 4, 2));
  SIMP_REQUIRE(dC != nullptr, SIMP_ERR_CUDA, "out of device memory for C");
  if (a_resident) dA = lookup_mirror(A, size_t(M) * K);
  else {
    dA = scratch(size_t(M) * K + 16, 0);
    SIMP_REQUIRE(dA != nullptr, SIMP_ERR_CUDA, "out of device memory for A");
  }
  int64_t chunk = ((cdiv(M, 8) + 127) / 128) * 128;
  if (M * N * 4 < (int64_t(8) << 20)) chunk = M;  // small results: one piece
  const int nchunks = int(cdiv(M, chunk));
  std::vector<cudaEvent_t> ev_in(nchunks), ev_done(nchunks);
  cudaEvent_t ev_b;
  SIMP_CUDA(cudaEventCreateWithFlags(&ev_b, cudaEventDisableTiming));
  SIMP_CUDA(cudaEventRecord(ev_b, c.copy_in));
  SIMP_CUDA(cudaStreamWaitEvent(c.stream, ev_b, 0));
  int rc = SIMP_OK;
  for (int i = 0; i < nchunks && rc == SIMP_OK; ++i) {
    const int64_t r0 = i * chunk, rows = (r0 + chunk <= M) ? chunk : M - r0;
    cudaEventCreateWithFlags(&ev_in[i], cudaEventDisableTiming);
    cudaEventCreateWithFlags(&ev_done[i], cudaEventDisableTiming);
    const uint8_t* a_dev = static_cast<const uint8_t*>(dA) + r0 * K;
    if (!a_resident)
      cudaMemcpyAsync(const_cast<uint8_t*>(a_dev), static_cast<const uint8_t*>(A) + r0 * K, size_t(rows) * K,
                      cudaMemcpyHostToDevice, c.copy_in);
    cudaEventRecord(ev_in[i], c.copy_in);
    cudaStreamWaitEvent(c.stream, ev_in[i], 0);
    rc = simp_gpu_matmul_i8(a_dev, static_cast<const int8_t*>(dB), dC + r0 * N, rows, K, N, a_unsigned, b_transposed);
    cudaEventRecord(ev_done[i], c.stream);
    cudaStreamWaitEvent(c.copy_out, ev_done[i], 0);
    cudaMemcpyAsync(C + r0 * N, dC + r0 * N, size_t(rows) * N * 4, cudaMemcpyDeviceToHost, c.copy_out);
  }
  cudaError_t e1 = cudaStreamSynchronize(c.copy_out);
  cudaError_t e2 = cudaStreamSynchronize(c.stream);
  for (int i = 0; i < nchunks; ++i) {
    if (ev_in[i]) cudaEventDestroy(ev_in[i]);
    if (ev_done[i]) cudaEventDestroy(ev_done[i]);
  }
  cudaEventDestroy(ev_b);
  if (rc != SIMP_OK) return rc;
  SIMP_REQUIRE(e1 == cudaSuccess && e2 == cudaSuccess, SIMP_ERR_CUDA, "host tensor_matmul_i8: %s",
               cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
  return SIMP_OK;
}

// simp.matmul with host operands (C is read when accumulating, then written back).
SIMP_API int simp_host_matmul_f32(const float* A, int64_t aoff, const float* B, int64_t boff, float* C, int64_t coff,
                                  int64_t m, int64_t k, int64_t n, int accumulate, int b_transposed) {
  if (int rc = ensure_ready()) return rc;
  SIMP_REQUIRE(m >= 0 && k >= 0 && n >= 0 && aoff >= 0 && boff >= 0 && coff >= 0, SIMP_ERR_ARG,
               "host matmul_f32: negative size or offset");
  if (m == 0 || n == 0) return SIMP_OK;
  SIMP_REQUIRE(A && B && C, SIMP_ERR_ARG, "host matmul_f32: null pointer");
  cudaStream_t st = ctx().stream;
  void *dA, *dB, *dC;
  if (int rc = stage_in(A + aoff, size_t(m) * k * 4, 0, st, &dA)) return rc;
  if (int rc = stage_in(B + boff, size_t(k) * n * 4, 1, st, &dB)) return rc;
  dC = scratch(size_t(m) * n * 4, 2);
  SIMP_REQUIRE(dC != nullptr, SIMP_ERR_CUDA, "out of device memory for C");
  if (accumulate) SIMP_CUDA(cudaMemcpyAsync(dC, C + coff, size_t(m) * n * 4, cudaMemcpyHostToDevice, st));
  if (int rc = simp_gpu_matmul_f32(static_cast<float*>(dA), 0, static_cast<float*>(dB), 0, static_cast<float*>(dC), 0,
                                   m, k, n, accumulate, b_transposed))
    return rc;
  SIMP_CUDA(cudaMemcpyAsync(C + coff, dC, size_t(m) * n * 4, cudaMemcpyDeviceToHost, st));
  SIMP_CUDA(cudaStreamSynchronize(st));
  return SIMP_OK;
}

// matmul_quant with host operands.  qweights/scales/zeros are normally registered (resident).
SIMP_API int simp_host_matmul_quant(const uint8_t* qw, size_t qw_bytes, const float* sc, const float* zr,
                                    size_t n_groups, const float* x, float* out, int64_t rows, int64_t cols,
                                    int64_t gs, int64_t offset, int scale_mode) {
  SIMP_REQUIRE(qw && sc && x && out && rows >= 0 && cols >= 0 && offset >= 0 && gs > 0, SIMP_ERR_ARG,
               "host matmul_quant: bad argument");
  SIMP_REQUIRE(scale_mode == 0 || scale_mode == 1, SIMP_ERR_ARG, "host matmul_quant: scale_mode must be 0 or 1");
  // The kernels index qw[(offset + row*cols + k) >> 1] and scales[(row*cols [+ offset]) / gs + g], g < cols / gs:
  // a wrong offset / rows / cols must come back as an error, not as an out-of-range device read.
  SIMP_REQUIRE(rows <= (INT64_MAX - offset) / (cols > 0 ? cols : 1), SIMP_ERR_SHAPE, "host matmul_quant: size overflow");
  SIMP_REQUIRE(size_t(offset + rows * cols + 1) / 2 <= qw_bytes, SIMP_ERR_SHAPE,
               "host matmul_quant: offset %lld + %lld x %lld weights need %zu bytes of qweights, the array holds %zu",
               (long long)offset, (long long)rows, (long long)cols, size_t(offset + rows * cols + 1) / 2, qw_bytes);
  if (cols >= gs) {
    const int64_t last = ((scale_mode == 1 ? offset : 0) + (rows - 1) * cols) / gs + cols / gs - 1;
    SIMP_REQUIRE(last >= 0 && size_t(last) < n_groups, SIMP_ERR_SHAPE,
                 "host matmul_quant: the last group read is %lld, scales / zeros hold %zu groups", (long long)last, n_groups);
  }
  if (int rc = ensure_ready()) return rc;
  cudaStream_t st = ctx().stream;
  void *dq, *ds, *dz = nullptr, *dx;
  if (int rc = stage_in(qw, qw_bytes, 0, st, &dq)) return rc;
  if (int rc = stage_in(sc, n_groups * 4, 1, st, &ds)) return rc;
  if (zr)
    if (int rc = stage_in(zr, n_groups * 4, 3, st, &dz)) return rc;
  if (int rc = stage_in(x, size_t(cols) * 4, 4, st, &dx)) return rc;
  float* dout = static_cast<float*>(scratch(size_t(rows) * 4 + 16, 2));
  SIMP_REQUIRE(dout != nullptr, SIMP_ERR_CUDA, "out of device memory");
  if (int rc = simp_gpu_matmul_w4(static_cast<uint8_t*>(dq), static_cast<float*>(ds), static_cast<float*>(dz),
                                  static_cast<float*>(dx), dout, rows, cols, gs, offset, scale_mode))
    return rc;
  SIMP_CUDA(cudaMemcpyAsync(out, dout, size_t(rows) * 4, cudaMemcpyDeviceToHost, st));
  SIMP_CUDA(cudaStreamSynchronize(st));
  return SIMP_OK;
}

// rmsnorm / softmax / silu with host operands (single call = `rows` rows).
SIMP_API int simp_host_rmsnorm_f32(const float* x, const float* w, float* y, int64_t rows, int64_t n, float eps,
                                   int64_t woff) {
  if (int rc = ensure_ready()) return rc;
  SIMP_REQUIRE(rows >= 0 && n >= 0 && woff >= 0, SIMP_ERR_ARG, "host rmsnorm: negative size");
  if (rows == 0 || n == 0) return SIMP_OK;
  SIMP_REQUIRE(x && w && y, SIMP_ERR_ARG, "host rmsnorm: null pointer");
  cudaStream_t st = ctx().stream;
  void *dx, *dw;
  if (int rc = stage_in(x, size_t(rows) * n * 4, 0, st, &dx)) return rc;
  if (int rc = stage_in(w + woff, size_t(n) * 4, 1, st, &dw)) return rc;
  float* dy = static_cast<float*>(scratch(size_t(rows) * n * 4, 2));
  SIMP_REQUIRE(dy != nullptr, SIMP_ERR_CUDA, "out of device memory");
  if (int rc = simp_gpu_rmsnorm_f32(static_cast<float*>(dx), static_cast<float*>(dw), dy, rows, n, eps, 0, n, nullptr))
    return rc;
  SIMP_CUDA(cudaMemcpyAsync(y, dy, size_t(rows) * n * 4, cudaMemcpyDeviceToHost, st));
  SIMP_CUDA(cudaStreamSynchronize(st));
  return SIMP_OK;
}
SIMP_API int simp_host_softmax_f32(const float* x, float* y, int64_t rows, int64_t n, int64_t xoff, int64_t yoff,
                                   int64_t row_stride) {
  if (int rc = ensure_ready()) return rc;
  SIMP_REQUIRE(rows >= 0 && n >= 0 && xoff >= 0 && yoff >= 0, SIMP_ERR_ARG, "host softmax: negative size");
  if (rows == 0 || n == 0) return SIMP_OK;
  SIMP_REQUIRE(x && y, SIMP_ERR_ARG, "host softmax: null pointer");
  if (row_stride == 0) row_stride = n;
  const size_t span = size_t((rows - 1) * row_stride + n) * 4;
  cudaStream_t st = ctx().stream;
  void* dx;
  if (int rc = stage_in(x + xoff, span, 0, st, &dx)) return rc;
  float* dy = static_cast<float*>(scratch(span, 2));
  SIMP_REQUIRE(dy != nullptr, SIMP_ERR_CUDA, "out of device memory");
  if (row_stride != n) SIMP_CUDA(cudaMemcpyAsync(dy, y + yoff, span, cudaMemcpyHostToDevice, st));
  if (int rc = simp_gpu_softmax_f32(static_cast<float*>(dx), dy, rows, n, 0, 0, row_stride)) return rc;
  SIMP_CUDA(cudaMemcpyAsync(y + yoff, dy, span, cudaMemcpyDeviceToHost, st));
  SIMP_CUDA(cudaStreamSynchronize(st));
  return SIMP_OK;
}
SIMP_API int simp_host_silu_f32(const float* x, const float* mul, float* y, int64_t n) {
  if (int rc = ensure_ready()) return rc;
  SIMP_REQUIRE(n >= 0, SIMP_ERR_ARG, "host silu: negative size");
  if (n == 0) return SIMP_OK;
  SIMP_REQUIRE(x && y, SIMP_ERR_ARG, "host silu: null pointer");
  cudaStream_t st = ctx().stream;
  void *dx, *dm = nullptr;
  if (int rc = stage_in(x, size_t(n) * 4, 0, st, &dx)) return rc;
  if (mul)
    if (int rc = stage_in(mul, size_t(n) * 4, 1, st, &dm)) return rc;
  float* dy = static_cast<float*>(scratch(size_t(n) * 4, 2));
  SIMP_REQUIRE(dy != nullptr, SIMP_ERR_CUDA, "out of device memory");
  if (int rc = simp_gpu_silu_f32(static_cast<float*>(dx), static_cast<float*>(dm), dy, n)) return rc;
  SIMP_CUDA(cudaMemcpyAsync(y, dy, size_t(n) * 4, cudaMemcpyDeviceToHost, st));
  SIMP_CUDA(cudaStreamSynchronize(st));
  return SIMP_OK;
}
