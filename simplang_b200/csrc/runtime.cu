// runtime.cu -- life cycle, memory and stream of libsimp_gpu.
//
// The reference has no device runtime: its hosts keep every tensor in a std::vector and hand
// host pointers to the compiled kernel (examples/llama2/generate_stories110M.cpp:236-251).
// This module is the part of the GPU back end that owns device memory and the stream all ops
// are enqueued on.
#include <mutex>
#include <vector>

#include "common.cuh"

namespace simp {

static Context g_ctx;
static thread_local char g_err[512] = "";
static std::mutex g_mu;
struct Arena {
  void* p = nullptr;
  size_t cap = 0;
};
static Arena g_arena[16];
static bool g_capturing = false;          // the library stream is being captured into a recording
static int g_recordings = 0;              // live recordings (their graphs hold arena pointers)
static std::vector<void*> g_retired;      // outgrown arena blocks a live recording may still use
static thread_local bool g_scratch_refused = false;

Context& ctx() { return g_ctx; }

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int ensure_ready() {
  if (g_ctx.ready) return SIMP_OK;
  return simp_gpu_init(0);
}

void* scratch(size_t bytes, int slot) {
  std::lock_guard<std::mutex> lk(g_mu);
  Arena& a = g_arena[slot];
  g_scratch_refused = false;
  if (a.cap < bytes) {
    if (g_capturing) {
      g_scratch_refused = true;
      // growing would synchronise and free on the capturing stream, and the capture would keep a stale pointer
      set_error(SIMP_ERR_STATE, "scratch slot %d must grow to %zu bytes while a recording is being captured: run the "
                "same call once before simp_gpu_record_begin", slot, bytes);
      return nullptr;
    }
    if (a.p) {
      if (g_recordings > 0) {
        g_retired.push_back(a.p);   // a recording may replay kernels that use this block
      } else {
        cudaStreamSynchronize(g_ctx.stream);
        cudaFree(a.p);
      }
      a.p = nullptr;
      a.cap = 0;
    }
    size_t cap = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    if (cudaMalloc(&a.p, cap) != cudaSuccess) {
      a.p = nullptr;
      return nullptr;
    }
    a.cap = cap;
  }
  return a.p;
}

int scratch_failed(const char* who) {
  if (g_scratch_refused) return SIMP_ERR_STATE;   // message already set by scratch()
  return set_error(SIMP_ERR_CUDA, "%s: out of device memory for library scratch", who);
}

void scratch_capture(bool on) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_capturing = on;
}

void scratch_recordings(int delta) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_recordings += delta;
  if (g_recordings <= 0) {
    g_recordings = 0;
    if (!g_retired.empty() && g_ctx.ready) {
      cudaStreamSynchronize(g_ctx.stream);
      for (void* p : g_retired) cudaFree(p);
    }
    g_retired.clear();
  }
}

}  // namespace simp

using namespace simp;

SIMP_API int simp_gpu_init(int device) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_ctx.ready && g_ctx.device == device) return SIMP_OK;
  SIMP_REQUIRE(!g_ctx.ready, SIMP_ERR_STATE,
               "simp_gpu_init(%d): already initialised on device %d; call simp_gpu_shutdown first",
               device, g_ctx.device);
  int n = 0;
  SIMP_CUDA(cudaGetDeviceCount(&n));
  SIMP_REQUIRE(device >= 0 && device < n, SIMP_ERR_ARG, "device %d out of range (have %d)", device, n);
  SIMP_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  SIMP_CUDA(cudaGetDeviceProperties(&prop, device));
  SIMP_REQUIRE(prop.major == 10, SIMP_ERR_UNSUPPORTED,
               "device %d is sm_%d%d; this library contains sm_100a code only", device, prop.major,
               prop.minor);
  g_ctx.sm_count = prop.multiProcessorCount;
  SIMP_CUDA(cudaStreamCreateWithFlags(&g_ctx.stream, cudaStreamNonBlocking));
  SIMP_CUDA(cudaStreamCreateWithFlags(&g_ctx.copy_in, cudaStreamNonBlocking));
  SIMP_CUDA(cudaStreamCreateWithFlags(&g_ctx.copy_out, cudaStreamNonBlocking));
  SIMP_CUDA(cudaMalloc(&g_ctx.dev_status, 64));
  SIMP_CUDA(cudaMemset(g_ctx.dev_status, 0, 64));
  SIMP_CUDA(cudaMallocHost(&g_ctx.host_status, 64));
  g_ctx.host_status[0] = 0;
  g_ctx.device = device;
  g_ctx.ready = true;
  return SIMP_OK;
}

SIMP_API int simp_gpu_shutdown(void) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_ctx.ready) return SIMP_OK;
  cudaSetDevice(g_ctx.device);
  cudaStreamSynchronize(g_ctx.stream);
  for (auto& a : g_arena) {
    if (a.p) cudaFree(a.p);
    a = Arena{};
  }
  for (void* p : g_retired) cudaFree(p);
  g_retired.clear();
  g_recordings = 0;
  g_capturing = false;
  cudaFree(g_ctx.dev_status);
  cudaFreeHost(g_ctx.host_status);
  cudaStreamDestroy(g_ctx.stream);
  cudaStreamDestroy(g_ctx.copy_in);
  cudaStreamDestroy(g_ctx.copy_out);
  g_ctx = Context{};
  return SIMP_OK;
}

SIMP_API const char* simp_gpu_last_error(void) { return g_err; }

SIMP_API int simp_gpu_device_count(int* count) {
  SIMP_REQUIRE(count != nullptr, SIMP_ERR_ARG, "count is null");
  SIMP_CUDA(cudaGetDeviceCount(count));
  return SIMP_OK;
}

SIMP_API int simp_gpu_alloc(void** dptr, size_t bytes) {
  SIMP_REQUIRE(dptr != nullptr, SIMP_ERR_ARG, "dptr is null");
  if (int rc = ensure_ready()) return rc;
  *dptr = nullptr;
  if (bytes == 0) bytes = 16;
  SIMP_CUDA(cudaMalloc(dptr, bytes));
  return SIMP_OK;
}

SIMP_API int simp_gpu_free(void* dptr) {
  if (!dptr) return SIMP_OK;
  if (int rc = ensure_ready()) return rc;
  SIMP_CUDA(cudaStreamSynchronize(g_ctx.stream));
  SIMP_CUDA(cudaFree(dptr));
  return SIMP_OK;
}

SIMP_API int simp_gpu_upload(void* dst_dev, const void* src_host, size_t bytes) {
  if (bytes == 0) return SIMP_OK;
  SIMP_REQUIRE(dst_dev && src_host, SIMP_ERR_ARG, "upload: null pointer");
  if (int rc = ensure_ready()) return rc;
  SIMP_CUDA(cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, g_ctx.stream));
  return SIMP_OK;
}

SIMP_API int simp_gpu_download(void* dst_host, const void* src_dev, size_t bytes) {
  if (int rc = ensure_ready()) return rc;
  if (bytes) {
    SIMP_REQUIRE(dst_host && src_dev, SIMP_ERR_ARG, "download: null pointer");
    SIMP_CUDA(cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, g_ctx.stream));
  }
  SIMP_CUDA(cudaStreamSynchronize(g_ctx.stream));
  return SIMP_OK;
}

SIMP_API int simp_gpu_memset(void* dptr, int value, size_t bytes) {
  if (bytes == 0) return SIMP_OK;
  SIMP_REQUIRE(dptr != nullptr, SIMP_ERR_ARG, "memset: null pointer");
  if (int rc = ensure_ready()) return rc;
  SIMP_CUDA(cudaMemsetAsync(dptr, value, bytes, g_ctx.stream));
  return SIMP_OK;
}

SIMP_API int simp_gpu_sync(void) {
  if (int rc = ensure_ready()) return rc;
  SIMP_CUDA(cudaStreamSynchronize(g_ctx.stream));
  return SIMP_OK;
}

SIMP_API void* simp_gpu_stream(void) {
  if (ensure_ready() != SIMP_OK) return nullptr;
  return (void*)g_ctx.stream;
}

SIMP_API int simp_gpu_check_device_status(void) {
  if (int rc = ensure_ready()) return rc;
  SIMP_CUDA(cudaMemcpyAsync(g_ctx.host_status, g_ctx.dev_status, 16, cudaMemcpyDeviceToHost,
                            g_ctx.stream));
  SIMP_CUDA(cudaStreamSynchronize(g_ctx.stream));
  if (g_ctx.host_status[0] != 0) {
    const int code = g_ctx.host_status[0], where = g_ctx.host_status[1];
    cudaMemsetAsync(g_ctx.dev_status, 0, 16, g_ctx.stream);
    if (code == 2)   // raised by tensor_gather: an index outside the gathered axis
      return set_error(SIMP_ERR_ARG, "tensor_gather: index %d is outside the gathered axis (row skipped)", where);
    return set_error(SIMP_ERR_TIMEOUT, "a bounded device-side wait gave up (code %d, site %d)", code,
                     where);
  }
  return SIMP_OK;
}
