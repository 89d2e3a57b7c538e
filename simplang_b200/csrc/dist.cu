// dist.cu -- multi-GPU entry points: one process per GPU, NCCL over NVLink / NVSwitch.
//
// The reference has no distributed code; its only parallel schemes are OpenMP over row tiles
// (src/mlir/mlir_pipeline.cpp:265-364) and host-side row chunking with a shared B
// (simptensor/benchmarks/bench_int8_parallel_runner.cpp:70-91).  Here large GEMMs are N-sharded:
// rank r owns columns [r*N/R, (r+1)*N/R) of B, A is replicated, and the column blocks of C are
// exchanged with one all-gather -- the only collective on the path (integer results, so the
// exchange cannot change a bit).
// NCCL is loaded at run time (dlopen "libnccl.so.2", the copy the process already has when torch is
// imported) so the library has no link-time dependency on it.  The unique id is created on rank 0
// (simp_dist_unique_id) and carried to the other ranks by the host (torch.distributed, MPI, a file).
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace simp {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  ncclResult_t (*GetVersion)(int*) = nullptr;
};
static NcclApi g_nccl;
static ncclComm_t g_comm = nullptr;
static int g_rank = 0, g_world = 1;
static std::mutex g_dist_mu;

static int load_nccl() {
  if (g_nccl.handle) return SIMP_OK;
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  for (const char* n : names) {
    g_nccl.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (g_nccl.handle) break;
  }
  SIMP_REQUIRE(g_nccl.handle != nullptr, SIMP_ERR_COMM, "cannot load libnccl.so.2: %s", dlerror());
#define SIMP_SYM(field, name)                                                          \
  g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(g_nccl.handle, name)); \
  SIMP_REQUIRE(g_nccl.field != nullptr, SIMP_ERR_COMM, "libnccl lacks %s", name)
  SIMP_SYM(GetUniqueId, "ncclGetUniqueId");
  SIMP_SYM(CommInitRank, "ncclCommInitRank");
  SIMP_SYM(CommDestroy, "ncclCommDestroy");
  SIMP_SYM(AllGather, "ncclAllGather");
  SIMP_SYM(AllReduce, "ncclAllReduce");
  SIMP_SYM(GetErrorString, "ncclGetErrorString");
  SIMP_SYM(GetVersion, "ncclGetVersion");
#undef SIMP_SYM
  return SIMP_OK;
}

#define SIMP_NCCL(call)                                                                              \
  do {                                                                                               \
    ncclResult_t r__ = (call);                                                                       \
    if (r__ != ncclSuccess)                                                                          \
      return set_error(SIMP_ERR_COMM, "%s failed: %s", #call, g_nccl.GetErrorString(r__));           \
  } while (0)

// Symmetric buffers: one cudaMalloc per rank, made addressable from every rank of the node through CUDA IPC.
struct SymmBuf {
  void* local = nullptr;
  size_t bytes = 0;
  void* peer[8] = {};  // peer[r] = rank r's buffer as seen from this process (peer[rank] == local)
};
static std::vector<SymmBuf> g_symm;

int gemm_i8_run(const void* A, const int8_t* B, int32_t* C, int64_t M, int64_t K, int64_t N, int a_unsigned,
                int b_transposed, int32_t* const* peer_c, int n_peers, int64_t ldc, int64_t col_offset, int self_rank);
int dist_rendezvous(bool pdl = false);

// ---- peer-store all-gather ---------------------------------------------------------------------
// In-place all-gather of a small vector that lives in a symmetric buffer: every rank stores its slice straight
// into the other ranks' copies (plain stores through the CUDA IPC mappings, i.e. over NVLink), publishes a
// per-source epoch word in each peer's flag array, and waits for the epochs of the other sources.  One block,
// no NCCL call: for the kilobyte-sized slices of batch-1 decode the cost is a launch plus one NVLink round trip.
// The wait is bounded (1 s); on expiry the library status word is set and the kernel returns.
struct LlPeers {
  uint8_t* buf[8];
  unsigned* flags[8];
};
static unsigned* g_ll_flags = nullptr;   // symmetric: [8] epoch words, written by the peers
static unsigned* g_ll_seq = nullptr;     // local: epochs issued so far

__device__ __forceinline__ void st_release_sys_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__global__ void __launch_bounds__(256) ll_allgather_kernel(LlPeers peers, unsigned* seq, int rank, int world, size_t offset,
                                                           size_t slice, int* status) {
  // a consumer launched as a programmatic dependent may start its prologue (weight requests) now; its
  // griddepcontrol.wait still returns only when this exchange has completed
  pdl_launch_dependents();
  pdl_wait();   // launched as a programmatic dependent by the fused GEMM: the predecessor's stores have been performed
  const unsigned epoch = *seq + 1u;
  const uint8_t* mine = peers.buf[rank] + offset + size_t(rank) * slice;
  const bool vec = ((reinterpret_cast<uintptr_t>(mine) | slice) & 15u) == 0;
  for (int r = 0; r < world; ++r) {
    if (r == rank) continue;
    uint8_t* dst = peers.buf[r] + offset + size_t(rank) * slice;
    if (vec) {
      for (size_t i = threadIdx.x; i < (slice >> 4); i += blockDim.x)
        reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(mine)[i];
    } else {
      for (size_t i = threadIdx.x; i < slice; i += blockDim.x) dst[i] = mine[i];
    }
  }
  __threadfence_system();
  __syncthreads();
  const int t = threadIdx.x;
  if (t < world && t != rank) {
    st_release_sys_u32(peers.flags[t] + rank, epoch);   // "rank's slice of this epoch has landed in t's buffer"
    const unsigned long long t0 = ptx::globaltimer_ns();
    for (unsigned spin = 1;; ++spin) {
      if (int(ld_acquire_sys_u32(peers.flags[rank] + t) - epoch) >= 0) break;
      if ((spin & 63u) == 0 && ptx::globaltimer_ns() - t0 > 1000000000ull) {
        if (atomicCAS(status, 0, 1) == 0) status[1] = 90 + t;
        break;
      }
    }
  }
  __syncthreads();
  if (t == 0) *seq = epoch;
}

}  // namespace simp

using namespace simp;

// Collective: every rank allocates `bytes` and learns the addresses of all ranks' buffers (cudaIpc handles
// travel through one NCCL all-gather).  Stores from a kernel to a peer address go over NVLink.
SIMP_API int simp_dist_symm_alloc(size_t bytes, void** local_ptr) {
  SIMP_REQUIRE(local_ptr != nullptr && bytes > 0, SIMP_ERR_ARG, "dist_symm_alloc: null pointer or empty buffer");
  if (int rc = ensure_ready()) return rc;
  SIMP_REQUIRE(g_world <= 8, SIMP_ERR_UNSUPPORTED, "dist_symm_alloc: at most 8 ranks");
  SymmBuf b;
  b.bytes = bytes;
  SIMP_CUDA(cudaMalloc(&b.local, bytes));
  b.peer[g_rank] = b.local;
  if (g_world > 1) {
    SIMP_REQUIRE(g_comm != nullptr, SIMP_ERR_STATE, "dist_symm_alloc: call simp_dist_init first");
    cudaIpcMemHandle_t mine;
    SIMP_CUDA(cudaIpcGetMemHandle(&mine, b.local));
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "unexpected IPC handle size");
    uint8_t* dev = nullptr;
    SIMP_CUDA(cudaMalloc(&dev, 64 * size_t(g_world)));
    cudaStream_t st = ctx().stream;
    SIMP_CUDA(cudaMemcpyAsync(dev + 64 * g_rank, &mine, 64, cudaMemcpyHostToDevice, st));
    SIMP_NCCL(g_nccl.AllGather(dev + 64 * g_rank, dev, 64, ncclInt8, g_comm, st));
    std::vector<cudaIpcMemHandle_t> all(g_world);
    SIMP_CUDA(cudaMemcpyAsync(all.data(), dev, 64 * size_t(g_world), cudaMemcpyDeviceToHost, st));
    SIMP_CUDA(cudaStreamSynchronize(st));
    SIMP_CUDA(cudaFree(dev));
    for (int r = 0; r < g_world; ++r) {
      if (r == g_rank) continue;
      SIMP_CUDA(cudaIpcOpenMemHandle(&b.peer[r], all[r], cudaIpcMemLazyEnablePeerAccess));
    }
  }
  g_symm.push_back(b);
  *local_ptr = b.local;
  return SIMP_OK;
}

SIMP_API int simp_dist_symm_free(void* local_ptr) {
  for (size_t i = 0; i < g_symm.size(); ++i) {
    if (g_symm[i].local != local_ptr) continue;
    cudaStreamSynchronize(ctx().stream);
    for (int r = 0; r < g_world; ++r)
      if (r != g_rank && g_symm[i].peer[r]) cudaIpcCloseMemHandle(g_symm[i].peer[r]);
    cudaFree(g_symm[i].local);
    g_symm.erase(g_symm.begin() + i);
    return SIMP_OK;
  }
  return set_error(SIMP_ERR_ARG, "dist_symm_free: pointer was not returned by simp_dist_symm_alloc");
}

// Rendezvous on the library stream: returns (in stream order) only after every rank's earlier work on its own
// stream has completed -- one 4-byte all-reduce.
SIMP_API int simp_dist_barrier(void) {
  if (int rc = ensure_ready()) return rc;
  if (g_world == 1) return SIMP_OK;
  SIMP_REQUIRE(g_comm != nullptr, SIMP_ERR_STATE, "dist_barrier: call simp_dist_init first");
  float* word = static_cast<float*>(scratch(256, 7));
  SIMP_REQUIRE(word != nullptr, SIMP_ERR_CUDA, "dist_barrier: out of device memory");
  SIMP_NCCL(g_nccl.AllReduce(word, word, 1, ncclFloat, ncclSum, g_comm, ctx().stream));
  return SIMP_OK;
}

// N-sharded tensor_matmul on i8 with the all-gather fused into the GEMM epilogue: each C tile is staged once
// in shared memory and TMA-stored into every rank's copy of the full row-major C[M, N_local*world] -- the
// exchange overlaps the tensor-core main loop tile by tile instead of following it.  C_symm must come from
// simp_dist_symm_alloc (M * N_local * world * 4 bytes).  A trailing simp_dist_barrier orders the peers'
// stores before later work on this stream.
SIMP_API int simp_dist_matmul_i8_nsharded_fused(const void* A_dev, const int8_t* B_local_dev, int32_t* C_symm,
                                                int64_t M, int64_t K, int64_t N_local, int a_unsigned,
                                                int b_transposed) {
  if (int rc = ensure_ready()) return rc;
  const SymmBuf* sb = nullptr;
  for (const auto& b : g_symm)
    if (b.local == C_symm) sb = &b;
  SIMP_REQUIRE(sb != nullptr, SIMP_ERR_ARG, "dist_matmul_i8_nsharded_fused: C must come from simp_dist_symm_alloc");
  const int64_t ldc = N_local * g_world;
  SIMP_REQUIRE(size_t(M) * size_t(ldc) * 4 <= sb->bytes, SIMP_ERR_SHAPE, "dist_matmul_i8_nsharded_fused: C buffer too small");
  int32_t* peers[8];
  for (int r = 0; r < g_world; ++r) peers[r] = static_cast<int32_t*>(sb->peer[r]);
  if (int rc = gemm_i8_run(A_dev, B_local_dev, nullptr, M, K, N_local, a_unsigned, b_transposed, peers, g_world, ldc,
                           int64_t(g_rank) * N_local, g_rank))
    return rc;
  return dist_rendezvous(true);   // resident early; its wait returns when the GEMM's stores have been performed
}

SIMP_API int simp_dist_unique_id(void* id_out, size_t bytes) {
  SIMP_REQUIRE(id_out != nullptr && bytes >= sizeof(ncclUniqueId), SIMP_ERR_ARG,
               "dist_unique_id: need a buffer of at least %zu bytes", sizeof(ncclUniqueId));
  if (int rc = load_nccl()) return rc;
  ncclUniqueId id;
  SIMP_NCCL(g_nccl.GetUniqueId(&id));
  memcpy(id_out, &id, sizeof(id));
  return SIMP_OK;
}

SIMP_API int simp_dist_init(int rank, int world, const void* id, size_t bytes) {
  std::lock_guard<std::mutex> lk(g_dist_mu);
  SIMP_REQUIRE(world >= 1 && rank >= 0 && rank < world, SIMP_ERR_ARG, "dist_init: bad rank %d of %d", rank, world);
  SIMP_REQUIRE(g_comm == nullptr, SIMP_ERR_STATE, "dist_init: already initialised");
  if (int rc = ensure_ready()) return rc;
  g_rank = rank;
  g_world = world;
  if (world == 1) return SIMP_OK;
  SIMP_REQUIRE(id != nullptr && bytes >= sizeof(ncclUniqueId), SIMP_ERR_ARG, "dist_init: unique id missing");
  if (int rc = load_nccl()) return rc;
  ncclUniqueId uid;
  memcpy(&uid, id, sizeof(uid));
  SIMP_NCCL(g_nccl.CommInitRank(&g_comm, world, uid, rank));
  return SIMP_OK;
}

SIMP_API int simp_dist_shutdown(void) {
  if (g_ll_flags) {
    simp_dist_symm_free(g_ll_flags);
    g_ll_flags = nullptr;
  }
  if (g_ll_seq) {
    cudaFree(g_ll_seq);
    g_ll_seq = nullptr;
  }
  std::lock_guard<std::mutex> lk(g_dist_mu);
  if (g_comm) {
    cudaStreamSynchronize(ctx().stream);
    g_nccl.CommDestroy(g_comm);
    g_comm = nullptr;
  }
  g_rank = 0;
  g_world = 1;
  return SIMP_OK;
}

SIMP_API int simp_dist_rank(void) { return g_rank; }
SIMP_API int simp_dist_world(void) { return g_world; }

// recv[r*bytes_per_rank ...] = rank r's send buffer, on the library stream.
SIMP_API int simp_dist_allgather(const void* send_dev, void* recv_dev, size_t bytes_per_rank) {
  if (int rc = ensure_ready()) return rc;
  SIMP_REQUIRE(send_dev && recv_dev, SIMP_ERR_ARG, "dist_allgather: null pointer");
  if (g_world == 1) {
    if (send_dev != recv_dev)
      SIMP_CUDA(cudaMemcpyAsync(recv_dev, send_dev, bytes_per_rank, cudaMemcpyDeviceToDevice, ctx().stream));
    return SIMP_OK;
  }
  SIMP_REQUIRE(g_comm != nullptr, SIMP_ERR_STATE, "dist_allgather: call simp_dist_init first");
  SIMP_NCCL(g_nccl.AllGather(send_dev, recv_dev, bytes_per_rank, ncclInt8, g_comm, ctx().stream));
  return SIMP_OK;
}

// In-place all-gather inside a symmetric buffer without NCCL: on return (in stream order) the bytes
// [offset, offset + world * slice) of `symm_local` hold every rank's slice; this rank's slice must already be at
// offset + rank * slice.  Every rank calls it in the same order.  The first call allocates the flag words
// (a collective): make it outside stream capture.
// The epoch words of the peer exchange (a collective on first use: allocates, so the first call must come
// outside any stream capture).
static int ll_flags_ready(const SymmBuf** fb_out) {
  if (!g_ll_flags) {
    void* f = nullptr;
    if (int rc = simp_dist_symm_alloc(256, &f)) return rc;
    SIMP_CUDA(cudaMemsetAsync(f, 0, 256, ctx().stream));
    SIMP_CUDA(cudaMalloc(&g_ll_seq, 64));
    SIMP_CUDA(cudaMemsetAsync(g_ll_seq, 0, 64, ctx().stream));
    g_ll_flags = static_cast<unsigned*>(f);
    if (int rc = simp_dist_barrier()) return rc;   // every rank's flags are zero before anyone publishes
    SIMP_CUDA(cudaStreamSynchronize(ctx().stream));
  }
  const SymmBuf* fb = nullptr;
  for (const auto& b : g_symm)
    if (b.local == g_ll_flags) fb = &b;
  SIMP_REQUIRE(fb != nullptr, SIMP_ERR_STATE, "peer exchange: flag buffer missing");
  *fb_out = fb;
  return SIMP_OK;
}

namespace simp {
// The addresses of all ranks' copies of a symmetric buffer (peers[rank] = local); false if `local` is unknown.
bool dist_symm_peers(const void* local, uint8_t** peers8) {
  for (const auto& b : g_symm)
    if (b.local == local) {
      for (int r = 0; r < 8; ++r) peers8[r] = static_cast<uint8_t*>(b.peer[r]);
      return true;
    }
  return false;
}
// Rendezvous on the library stream without NCCL: the one-block exchange kernel with empty slices publishes this
// rank's next epoch to every peer and waits (bounded) for theirs.  Work queued before it on this stream has
// completed, with its stores to peer memory performed, before the epoch is published.
int dist_rendezvous(bool pdl) {
  if (g_world == 1) return SIMP_OK;
  const SymmBuf* fb = nullptr;
  if (int rc = ll_flags_ready(&fb)) return rc;
  LlPeers peers{};
  for (int r = 0; r < g_world; ++r) {
    peers.buf[r] = static_cast<uint8_t*>(fb->peer[r]);   // not touched: the slices are empty
    peers.flags[r] = static_cast<unsigned*>(fb->peer[r]);
  }
  SIMP_CUDA(launch_kernel(ll_allgather_kernel, dim3(1), dim3(256), 0, ctx().stream, pdl, peers, g_ll_seq, g_rank, g_world,
                          size_t(0), size_t(0), ctx().dev_status));
  return SIMP_OK;
}
}  // namespace simp

SIMP_API int simp_dist_allgather_peer(void* symm_local, size_t offset, size_t slice) {
  if (int rc = ensure_ready()) return rc;
  if (g_world == 1 || slice == 0) return SIMP_OK;
  const SymmBuf* fb = nullptr;
  if (int rc = ll_flags_ready(&fb)) return rc;
  const SymmBuf* sb = nullptr;
  for (const auto& b : g_symm)
    if (b.local == symm_local) sb = &b;
  SIMP_REQUIRE(sb != nullptr, SIMP_ERR_ARG, "dist_allgather_peer: buffer must come from simp_dist_symm_alloc");
  SIMP_REQUIRE(offset + slice * size_t(g_world) <= sb->bytes, SIMP_ERR_SHAPE, "dist_allgather_peer: range outside the buffer");
  LlPeers peers{};
  for (int r = 0; r < g_world; ++r) {
    peers.buf[r] = static_cast<uint8_t*>(sb->peer[r]);
    peers.flags[r] = static_cast<unsigned*>(fb->peer[r]);
  }
  ll_allgather_kernel<<<1, 256, 0, ctx().stream>>>(peers, g_ll_seq, g_rank, g_world, offset, slice, ctx().dev_status);
  SIMP_LAUNCH_CHECK();
  return SIMP_OK;
}

SIMP_API int simp_dist_allreduce_f32(float* buf_dev, size_t count) {
  if (int rc = ensure_ready()) return rc;
  SIMP_REQUIRE(buf_dev != nullptr, SIMP_ERR_ARG, "dist_allreduce_f32: null pointer");
  if (g_world == 1) return SIMP_OK;
  SIMP_REQUIRE(g_comm != nullptr, SIMP_ERR_STATE, "dist_allreduce_f32: call simp_dist_init first");
  SIMP_NCCL(g_nccl.AllReduce(buf_dev, buf_dev, count, ncclFloat, ncclSum, g_comm, ctx().stream));
  return SIMP_OK;
}

// N-sharded tensor_matmul on i8: this rank multiplies A[M,K] by its column block of B
// (B_local: [K, N/R] or, transposed, [N/R, K]) and the column blocks of C are all-gathered.
// C_blocks_dev receives R blocks of M x (N/R) i32, block r = C[:, r*N/R : (r+1)*N/R].
SIMP_API int simp_dist_matmul_i8_nsharded(const void* A_dev, const int8_t* B_local_dev, int32_t* C_blocks_dev,
                                          int64_t M, int64_t K, int64_t N_local, int a_unsigned, int b_transposed) {
  if (int rc = ensure_ready()) return rc;
  SIMP_REQUIRE(C_blocks_dev != nullptr, SIMP_ERR_ARG, "dist_matmul_i8_nsharded: null pointer");
  int32_t* mine = C_blocks_dev + size_t(g_rank) * size_t(M) * size_t(N_local);
  if (int rc = simp_gpu_matmul_i8(A_dev, B_local_dev, mine, M, K, N_local, a_unsigned, b_transposed)) return rc;
  if (g_world == 1) return SIMP_OK;
  return simp_dist_allgather(mine, C_blocks_dev, size_t(M) * size_t(N_local) * sizeof(int32_t));
}
