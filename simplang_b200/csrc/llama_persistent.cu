// llama_persistent.cu -- one token of the f32 LLaMA model (examples/llama2/stories110M.sl:5-247) as ONE
// persistent cooperative kernel: one block per SM (16 compute warps + 1 producer warp), the phases of the
// forward pass separated by grid-wide barriers instead of kernel launches.
//
// Why: at batch 1 the per-op graph is a chain of ~64 dependent kernels whose launch floor (~1.2 us each)
// and cold first loads dominate, while a layer's weights are only ~190 KB per SM.  Here every block owns a
// fixed, contiguous slice of the rows of each projection, and shared memory holds one buffer per
// projection group (q/k/v + norm weights | wo | gate/up + norm weights | down).  The producer warp refills
// a buffer with the next layer's slice (cp.async.bulk + mbarrier) the moment the compute warps release it,
// so each slice has a whole layer's time to arrive, HBM streams continuously under the dependency chain,
// and a phase costs one grid barrier plus its short compute out of shared memory.
// Per layer: q/k/v (rmsnorm folded in) | attention (RoPE, KV store, split-sequence online softmax) |
// wo + residual (merging the attention partials) | gate/up + silu*mul (rmsnorm folded in) | down + residual;
// then rmsnorm + classifier streamed from HBM + greedy argmax.  Arithmetic and reduction orders are fixed,
// so results are run-to-run identical.
//
// Grid barrier: one global arrival counter, monotonic within a launch (zeroed by a memset node before the
// kernel).  The wait is bounded (1 s): on expiry an error word is set that every waiter polls, all blocks
// leave, and the host reports the timeout; cooperative launch guarantees all blocks are co-resident.
#include "llama_persistent.cuh"
#include "llama_model.hpp"

namespace simp {

constexpr size_t PK_MAX_DYN_SMEM = PK_SMEM_LIMIT - 2560;   // per-block limit less this kernel's static shared memory

struct PersistArgs {
  PkCommon c;
  const float *wq, *wk, *wv, *wo, *w1, *w2, *w3;
  uint32_t koff[5];     // shared-memory byte offset of the weight buffer of each phase kind (kind 1 has none)
  uint32_t xs_off;      // offset of the staged-vector buffer
};

__global__ void __launch_bounds__(PK_BLOCK, 1) llama_f32_token_kernel(const PersistArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ PkStatic S;
  __shared__ __align__(8) uint64_t full[5];   // weights of a phase kind have landed (phase parity = layer parity)
  __shared__ __align__(8) uint64_t freeb[5];  // the compute warps are done with that kind's buffer
  const PkCommon& c = a.c;
  float* xs = reinterpret_cast<float*>(smem + a.xs_off);   // staged input vector
  float* sm_acc = xs;                                      // [PK_WARPS][128] attention scratch (xs is idle then)
  const int G = gridDim.x, b = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int dim = c.dim, hd = c.hd, kv = c.kv, hs = c.hs;
  unsigned epoch = 0;
  // this block's row slices of the three output widths
  const int n_dim = share_rows(dim, G, b), r0_dim = share_row0(dim, G, b);
  const int n_kv = share_rows(kv, G, b), r0_kv = share_row0(kv, G, b);
  const int n_hd = share_rows(hd, G, b), r0_hd = share_row0(hd, G, b);

  if (threadIdx.x == 0) {
#pragma unroll
    for (int k = 0; k < 5; ++k) {
      ptx::mbar_init(ptx::smem_u32(&full[k]), 1);
      ptx::mbar_init(ptx::smem_u32(&freeb[k]), 1);
    }
    S.sh_abort = 0;
    S.prod_done = 0;
    ptx::fence_barrier_init();
  }
  __syncthreads();

  // ================================================================== producer warp
  // Requests this block's slice of every layer for each phase kind (0 q/k/v, 2 wo, 3 gate/up, 4 down) into
  // that kind's own buffer, as soon as the compute warps have released the buffer.  A slice therefore has a
  // whole layer's time to arrive, HBM streams continuously under the dependency chain, and the time the copy
  // engine takes to accept the requests is not on the compute warps' path.
  if (warp == PK_WARPS) {
    if (lane != 0) return;
    int outstanding = 0, parity = 0;   // bit k: kind k has a request in flight / parity of its layer
    auto issue = [&](int l, int kind) {
      const uint32_t bar = ptx::smem_u32(&full[kind]);
      uint8_t* dst = smem + a.koff[kind];
      auto vec = [&](const float* w, uint32_t& off, uint32_t& total, bool count_only) {   // norm weights of layer l
        const uint32_t bytes = uint32_t(dim) * 4u;
        if (count_only) { total += bytes; return; }
        ptx::bulk_load(ptx::smem_u32(dst + off), w + size_t(l) * dim, bytes, bar);
        off += bytes;
      };
      auto one = [&](const float* W, int R, int K, uint32_t& off, uint32_t& total, bool count_only) {
        const int n = R == dim ? n_dim : (R == hd ? n_hd : n_kv);
        const int first = R == dim ? r0_dim : (R == hd ? r0_hd : r0_kv);
        const uint32_t bytes = uint32_t(n) * uint32_t(K) * 4u;
        if (bytes == 0) return;
        if (count_only) { total += bytes; return; }
        const uint8_t* src = reinterpret_cast<const uint8_t*>(W + (size_t(l) * R + first) * K);
        for (uint32_t done = 0; done < bytes; done += PK_COPY_CHUNK)
          ptx::bulk_load(ptx::smem_u32(dst + off + done), src + done, min(PK_COPY_CHUNK, bytes - done), bar);
        off += bytes;
      };
      for (int pass = 0; pass < 2; ++pass) {
        uint32_t off = 0, total = 0;
        const bool co = pass == 0;
        if (kind == 0) { vec(c.rms_att, off, total, co); one(a.wq, dim, dim, off, total, co); one(a.wk, kv, dim, off, total, co); one(a.wv, kv, dim, off, total, co); }
        if (kind == 2) one(a.wo, dim, dim, off, total, co);
        if (kind == 3) { vec(c.rms_ffn, off, total, co); one(a.w1, hd, dim, off, total, co); one(a.w3, hd, dim, off, total, co); }
        if (kind == 4) one(a.w2, dim, hd, off, total, co);
        if (co) {
          if (total == 0) { ptx::mbar_arrive(bar); return; }   // empty slice
          ptx::mbar_arrive_expect_tx(bar, total);
        }
      }
      outstanding |= 1 << kind;
      parity = (parity & ~(1 << kind)) | ((l & 1) << kind);
    };
    bool ok = true;
    for (int l = 0; l < c.n_layers && ok; ++l)
      for (int kind = 0; kind < 5 && ok; ++kind) {
        if (kind == 1) continue;
        if (l > 0) ok = ptx::mbar_wait(ptx::smem_u32(&freeb[kind]), uint32_t((l - 1) & 1), &S.sh_abort, c.status, 40 + kind);
        if (ok) issue(l, kind);
      }
    // Before this warp leaves, its last requests must have landed (they have, unless the kernel is being
    // abandoned; then the bounded wait keeps copies from arriving in shared memory that is no longer ours).
    for (int k = 0; k < 5; ++k)
      if (outstanding & (1 << k))
        for (int spin = 0; spin < 400000; ++spin)
          if (ptx::mbar_try_wait(ptx::smem_u32(&full[k]), uint32_t((parity >> k) & 1))) break;
    *reinterpret_cast<volatile int*>(&S.prod_done) = 1;
    return;
  }

  // ================================================================== compute warps
  auto wait_weights = [&](int l, int kind) {
    return ptx::mbar_wait(ptx::smem_u32(&full[kind]), uint32_t(l & 1), &S.sh_abort, c.status, 20 + kind);
  };
  // Error exit: raise the abort flag for the producer and give it a bounded time to see its copies land.
  auto drain = [&]() {
    if (threadIdx.x == 0) {
      *reinterpret_cast<volatile int*>(&S.sh_abort) = 1;
      for (int spin = 0; spin < 4000000 && *reinterpret_cast<volatile int*>(&S.prod_done) == 0; ++spin) {}
    }
    csync();
  };

  // ---- embedding: x = table[token] (each block copies a slice), then everyone may read x
  {
    const int64_t token = c.ctl[0];
    for (int i = b * PK_THREADS + threadIdx.x; i < dim; i += G * PK_THREADS) c.x[i] = c.tok_emb[token * dim + i];
  }
  if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, 0)) { drain(); return; }
  const int pos = c.ctl[1];

  for (int l = 0; l < c.n_layers; ++l) {
    // ------------------------------------------------------------------ phase 0: q/k/v
    {
      constexpr int kind = 0;
      const float r = stage_x_rms(c.x, xs, dim, S.red);
      if (!wait_weights(l, kind)) { drain(); return; }
      finish_rmsnorm(xs, reinterpret_cast<const float*>(smem + a.koff[kind]), r, dim);
      const int nq = n_dim, nk = n_kv, q0 = r0_dim, k0 = r0_kv;
      const float4* w = reinterpret_cast<const float4*>(smem + a.koff[kind] + size_t(dim) * 4);
      const float4* xv = reinterpret_cast<const float4*>(xs);
      const int k4 = dim >> 2;
      const int nt = nq + 2 * nk;
      auto put = [&](int r, float v) {
        if (r < nq) c.q[q0 + r] = v;
        else if (r < nq + nk) c.k[k0 + r - nq] = v;
        else c.v[k0 + r - nq - nk] = v;
      };
      for (int r = 2 * warp; r < nt; r += 2 * PK_WARPS) {
        if (r + 1 < nt) {
          float v0, v1;
          row_dot2(w + size_t(r) * k4, w + size_t(r + 1) * k4, xv, k4, lane, v0, v1);
          if (lane == 0) { put(r, v0); put(r + 1, v1); }
        } else {
          const float v = row_dot(w + size_t(r) * k4, xv, k4, lane);
          if (lane == 0) put(r, v);
        }
      }
      // the barrier's leading block-wide sync also releases this kind's buffer to the producer warp
      if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, ptx::smem_u32(&freeb[kind]))) { drain(); return; }
    }
    // ------------------------------------------------------------------ phase 1: attention
    {
      pk_attention(c, S, sm_acc, l, pos);
      if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, 0)) { drain(); return; }
    }
    // ------------------------------------------------------------------ phase 2: wo + residual
    {
      constexpr int kind = 2;
      pk_merge_heads(c, xs);
      csync();
      if (!wait_weights(l, kind)) { drain(); return; }
      const int n = n_dim, r0 = r0_dim;
      const float4* w = reinterpret_cast<const float4*>(smem + a.koff[kind]);
      const int k4 = dim >> 2;
      const float4* xv = reinterpret_cast<const float4*>(xs);
      for (int r = 2 * warp; r < n; r += 2 * PK_WARPS) {
        const float xr0 = __ldcg(c.x + r0 + r), xr1 = r + 1 < n ? __ldcg(c.x + r0 + r + 1) : 0.0f;
        if (r + 1 < n) {
          float v0, v1;
          row_dot2(w + size_t(r) * k4, w + size_t(r + 1) * k4, xv, k4, lane, v0, v1);
          if (lane == 0) { c.x[r0 + r] = xr0 + v0; c.x[r0 + r + 1] = xr1 + v1; }
        } else {
          const float v = row_dot(w + size_t(r) * k4, xv, k4, lane);
          if (lane == 0) c.x[r0 + r] = xr0 + v;
        }
      }
      // the barrier's leading block-wide sync also releases this kind's buffer to the producer warp
      if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, ptx::smem_u32(&freeb[kind]))) { drain(); return; }
    }
    // ------------------------------------------------------------------ phase 3: gate / up, silu * mul
    {
      constexpr int kind = 3;
      const float r = stage_x_rms(c.x, xs, dim, S.red);
      if (!wait_weights(l, kind)) { drain(); return; }
      finish_rmsnorm(xs, reinterpret_cast<const float*>(smem + a.koff[kind]), r, dim);
      const int n = n_hd, r0 = r0_hd;
      const float4* w = reinterpret_cast<const float4*>(smem + a.koff[kind] + size_t(dim) * 4);
      const int k4 = dim >> 2;
      for (int r = warp; r < n; r += PK_WARPS) {
        float g, u;
        row_dot2(w + size_t(r) * k4, w + size_t(n + r) * k4, reinterpret_cast<const float4*>(xs), k4, lane, g, u);
        if (lane == 0) c.hb[r0 + r] = (g / (1.0f + expf(-g))) * u;
      }
      // the barrier's leading block-wide sync also releases this kind's buffer to the producer warp
      if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, ptx::smem_u32(&freeb[kind]))) { drain(); return; }
    }
    // ------------------------------------------------------------------ phase 4: down + residual
    {
      constexpr int kind = 4;
      for (int i = threadIdx.x; i < (hd >> 2); i += PK_THREADS)
        reinterpret_cast<float4*>(xs)[i] = __ldcg(reinterpret_cast<const float4*>(c.hb) + i);
      csync();
      if (!wait_weights(l, kind)) { drain(); return; }
      const int n = n_dim, r0 = r0_dim;
      const float4* w = reinterpret_cast<const float4*>(smem + a.koff[kind]);
      const int k4 = hd >> 2;
      const float4* xv = reinterpret_cast<const float4*>(xs);
      for (int r = 2 * warp; r < n; r += 2 * PK_WARPS) {
        const float xr0 = __ldcg(c.x + r0 + r), xr1 = r + 1 < n ? __ldcg(c.x + r0 + r + 1) : 0.0f;
        if (r + 1 < n) {
          float v0, v1;
          row_dot2(w + size_t(r) * k4, w + size_t(r + 1) * k4, xv, k4, lane, v0, v1);
          if (lane == 0) { c.x[r0 + r] = xr0 + v0; c.x[r0 + r + 1] = xr1 + v1; }
        } else {
          const float v = row_dot(w + size_t(r) * k4, xv, k4, lane);
          if (lane == 0) c.x[r0 + r] = xr0 + v;
        }
      }
      // the barrier's leading block-wide sync also releases this kind's buffer to the producer warp
      if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, ptx::smem_u32(&freeb[kind]))) { drain(); return; }
    }
  }

  // ---------------------------------------------------------------------- classifier + argmax
  {
    const float r = stage_x_rms(c.x, xs, dim, S.red);
    finish_rmsnorm(xs, c.rms_final, r, dim);
  }
  pk_classifier(c, S, xs);
  if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, 0)) { drain(); return; }
  pk_advance(c, pos);
}

// ---------------------------------------------------------------------------------------------
// Shared-memory plan: one buffer per phase kind (sized for the largest row slice any block owns) followed by
// the staged-vector buffer, which doubles as the attention scratch.
struct PersistPlan {
  uint32_t koff[5];
  uint32_t xs_off;
  size_t total;
};
static PersistPlan persist_plan(const LlamaModel& m, int G) {
  const size_t dim = m.cfg.dim, hd = m.cfg.hidden_dim, kv = m.kv_dim;
  auto up = [&](size_t R) { return (R + G - 1) / G; };
  auto al = [](size_t v) { return (v + 127) & ~size_t(127); };
  const size_t bytes[5] = {(up(dim) + 2 * up(kv) + 1) * dim * 4, 0, up(dim) * dim * 4, (2 * up(hd) + 1) * dim * 4,
                           up(dim) * hd * 4};
  PersistPlan p{};
  size_t off = 0;
  for (int k = 0; k < 5; ++k) {
    p.koff[k] = uint32_t(off);
    off += al(bytes[k]);
  }
  p.xs_off = uint32_t(off);
  off += al(std::max<size_t>(std::max(dim, hd) * 4, size_t(PK_WARPS) * 128 * 4));
  p.total = off;
  return p;
}
static size_t persist_smem_bytes(const LlamaModel& m, int G) { return persist_plan(m, G).total; }

bool pk_device_ok(const LlamaModel& m);
bool persistent_f32_supported(const LlamaModel& m) {
  return !m.cfg.w4 && pk_device_ok(m) && persist_smem_bytes(m, ctx().sm_count) <= PK_MAX_DYN_SMEM;
}

int pk_fill_common(LlamaModel& m, PkCommon& a) {
  const int G = ctx().sm_count;
  SIMP_REQUIRE(m.pk_bar && m.pk_best_val && m.pk_best_idx, SIMP_ERR_STATE, "persistent decode: model scratch missing");
  const simp_llama_config& c = m.cfg;
  a.dim = int(c.dim); a.hd = int(c.hidden_dim); a.kv = int(m.kv_dim); a.hs = int(m.head_size);
  a.n_heads = int(c.n_heads); a.kv_mul = int(c.n_heads / c.n_kv_heads); a.n_layers = int(c.n_layers);
  a.vocab = int(c.vocab_size); a.seq_len = int(c.seq_len);
  a.nsplit = 4;   // sequence splits of the attention phase: one (head, split) item per block, at most 4
  while (a.nsplit > 1 && a.n_heads * a.nsplit > G) a.nsplit >>= 1;
  a.tok_emb = m.tok_emb; a.rms_att = m.rms_att; a.rms_ffn = m.rms_ffn; a.rms_final = m.rms_final; a.wcls = m.wcls;
  a.x = m.x; a.hb = m.hb; a.q = m.q; a.k = m.k; a.v = m.v; a.logits = m.logits; a.kc = m.kc; a.vc = m.vc;
  a.part = m.attn_part;
  a.ctl = m.ctl; a.prompt = m.prompt; a.out_tokens = m.out_tokens;
  a.bar = m.pk_bar; a.best_val = m.pk_best_val; a.best_idx = m.pk_best_idx;
  a.status = ctx().dev_status;
  return SIMP_OK;
}

// Zeroes the barrier words and launches `kernel` cooperatively: one block per SM, all co-resident.
int pk_launch(const void* kernel, void* args_struct, unsigned* bar, size_t smem, cudaStream_t st) {
  SIMP_CUDA(cudaMemsetAsync(bar, 0, 8, st));
  void* params[1] = {args_struct};
  SIMP_CUDA(cudaLaunchCooperativeKernel(kernel, dim3(unsigned(ctx().sm_count)), dim3(PK_BLOCK), params, smem, st));
  return SIMP_OK;
}

bool pk_device_ok(const LlamaModel& m) {
  if (m.tp > 1 || !ctx().ready) return false;
  if (m.cfg.n_heads > ctx().sm_count) return false;        // one (head, split) item per block
  if (m.head_size > 128 || m.head_size % 4 || m.cfg.dim % 4 || m.cfg.hidden_dim % 4) return false;
  int coop = 0;
  return cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, ctx().device) == cudaSuccess && coop;
}

int enqueue_token_persistent_f32(LlamaModel& m, cudaStream_t st) {
  PersistArgs a{};
  if (int rc = pk_fill_common(m, a.c)) return rc;
  a.wq = m.wq; a.wk = m.wk; a.wv = m.wv; a.wo = m.wo; a.w1 = m.w1; a.w2 = m.w2; a.w3 = m.w3;
  const PersistPlan plan = persist_plan(m, ctx().sm_count);
  for (int k = 0; k < 5; ++k) a.koff[k] = plan.koff[k];
  a.xs_off = plan.xs_off;
  if (!m.pk_attr_done) {   // first (eager) pass of this model, outside any stream capture
    SIMP_CUDA(cudaFuncSetAttribute(llama_f32_token_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(PK_MAX_DYN_SMEM)));
    m.pk_attr_done = true;
  }
  return pk_launch(reinterpret_cast<const void*>(llama_f32_token_kernel), &a, a.c.bar, plan.total, st);
}

}  // namespace simp
