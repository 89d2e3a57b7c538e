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
                int b_transposed, int32_t* const* peer_c, int n_peers, int64_t ldc, int64_t col_offset);

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
                           int64_t(g_rank) * N_local))
    return rc;
  return simp_dist_barrier();
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
