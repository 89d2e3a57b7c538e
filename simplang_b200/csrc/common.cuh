// common.cuh -- shared host/device helpers of libsimp_gpu (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "simp_gpu.h"

#define SIMP_API extern "C" __attribute__((visibility("default")))

namespace simp {

// ---- per-process state (runtime.cu) ---------------------------------------------------------
struct Context {
  int device = -1;
  cudaStream_t stream = nullptr;     // all ops
  cudaStream_t copy_in = nullptr;    // host->device staging of the host-pointer entry points
  cudaStream_t copy_out = nullptr;   // device->host staging
  int sm_count = 148;
  int* dev_status = nullptr;   // device word written by bounded waits (0 = ok)
  int* host_status = nullptr;  // pinned mirror for polling
  bool ready = false;
};
Context& ctx();
int set_error(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
int ensure_ready();

// Scratch arena owned by the library (grows, never shrinks until shutdown).  Recordings freeze the arena
// pointers they saw: while one is being captured a slot does not grow (nullptr is returned and the call fails),
// and while recordings are alive a slot that must grow keeps its old block until the last of them is destroyed.
void* scratch(size_t bytes, int slot);
int scratch_failed(const char* who); // status + message for a nullptr from scratch(): refused growth or out of memory
void scratch_capture(bool on);      // a stream capture of the library stream begins / ends
void scratch_recordings(int delta); // a recording was created (+1) / destroyed (-1)

#define SIMP_CUDA(call)                                                                     \
  do {                                                                                      \
    cudaError_t e__ = (call);                                                               \
    if (e__ != cudaSuccess)                                                                 \
      return ::simp::set_error(SIMP_ERR_CUDA, "%s failed: %s (%s:%d)", #call,               \
                               cudaGetErrorString(e__), __FILE__, __LINE__);                \
  } while (0)

#define SIMP_REQUIRE(cond, code, ...)                              \
  do {                                                             \
    if (!(cond)) return ::simp::set_error(code, __VA_ARGS__);      \
  } while (0)

#define SIMP_LAUNCH_CHECK()                                                                  \
  do {                                                                                       \
    cudaError_t e__ = cudaGetLastError();                                                    \
    if (e__ != cudaSuccess)                                                                  \
      return ::simp::set_error(SIMP_ERR_CUDA, "kernel launch failed: %s (%s:%d)",            \
                               cudaGetErrorString(e__), __FILE__, __LINE__);                 \
  } while (0)

inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Kernel launch with optional programmatic dependent launch: the kernel may begin (and run the part of
// its prologue that touches only immutable weights) before the previous kernel on the stream has
// finished; it must execute pdl_wait() before touching anything a predecessor writes or reads.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                                 Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// ---- tensor-parallel exchange fused into the producing / consuming kernels --------------------
// Every rank holds the exchanged activation vectors in a symmetric arena (same layout on every rank, all ranks'
// arenas mapped through CUDA IPC).  In such a vector every element is one 64-bit word { value (low 32 bits), tag
// (high 32 bits) }, written with ONE 64-bit store and read with ONE 64-bit load.  A kernel that produces a slice
// stores its words into EVERY rank's copy (over NVLink for the peers); a kernel that consumes the vector polls the
// words of its own copy until they carry the tag of the launch that produces them.  Data and flag travel together:
// no fence, no atomic, no exchange kernel, no collective call -- an exchange costs one NVLink store latency.
// tag = tokens completed * per_token + id, id = 1 for the embedding, 2 + 4 * layer + k for the four exchanged vectors
// of a layer (attention output, x after wo, hidden, x after down): strictly increasing, never 0.
typedef unsigned long long ll_word;
struct TpLL {
  int n = 0, rank = 0;          // ranks (0 or 1: plain vectors, no exchange), this rank
  uint8_t* arena[8] = {};       // arena base of every rank as seen from this process (arena[rank] = local)
  const int* tokens = nullptr;  // tokens completed so far (device word, advanced once per token)
  uint32_t per_token = 0;       // tags per token
};

// ---- device helpers -------------------------------------------------------------------------
#ifdef __CUDACC__
// Programmatic dependent launch: no-ops when the kernel was launched without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// First tag of the current token (add the id of a vector).  The token counter is written by the previous token's
// last kernel, so a kernel may read it before it waits for its predecessor.
__device__ __forceinline__ uint32_t ll_tag_base(const TpLL& t) { return t.n > 1 ? uint32_t(__ldcg(t.tokens)) * t.per_token : 0u; }
__device__ __forceinline__ void ll_store_sys(ll_word* p, float v, uint32_t tag) {
  const ll_word w = (ll_word(tag) << 32) | ll_word(__float_as_uint(v));
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
// One value to the same word of every rank's copy (byte offset `off` inside the arena).
__device__ __forceinline__ void ll_store_all(const TpLL& t, uint32_t off, float v, uint32_t tag) {
#pragma unroll
  for (int r = 0; r < 8; ++r)   // fixed trip count: the arena table stays in the parameter bank
    if (r < t.n) ll_store_sys(reinterpret_cast<ll_word*>(t.arena[r] + off), v, tag);
}
__device__ __forceinline__ ll_word ll_load_sys(const ll_word* p) {
  ll_word w;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
  return w;
}
// Polls `p` until it carries `tag` (bounded: 1 s, then the library status word is set and 0 is returned).
static __device__ __noinline__ float ll_spin(const ll_word* p, uint32_t tag, int* status, int site) {
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (unsigned spin = 1;; ++spin) {
    const ll_word w = ll_load_sys(p);
    if (uint32_t(w >> 32) == tag) return __uint_as_float(uint32_t(w));
    if ((spin & 63u) == 0) {
      unsigned long long t1;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
      if (t1 - t0 > 1000000000ull || *reinterpret_cast<volatile int*>(status) == 1) {
        if (atomicCAS(status, 0, 1) == 0) status[1] = site;
        return 0.0f;
      }
    }
  }
}
__device__ __forceinline__ float ll_get(const ll_word* p, uint32_t tag, int* status, int site) {
  const ll_word w = ll_load_sys(p);
  if (uint32_t(w >> 32) == tag) return __uint_as_float(uint32_t(w));
  return ll_spin(p, tag, status, site);
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum / max over blockDim.x threads (multiple of 32, <= 1024); `red` holds 33 floats.
// Every thread gets the result.  The same fixed tree each call, so results are run-to-run stable.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
// 128-bit streaming load that does not allocate in L1 (weights are read once per token).
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ float4 ld_stream_f4(const void* p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}
#endif

}  // namespace simp
