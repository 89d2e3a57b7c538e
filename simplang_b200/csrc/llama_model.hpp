// llama_model.hpp -- device-resident state of one LLaMA decoder (shared by the per-op graph path in
// llama.cu and the persistent per-token kernel of the f32 model in llama_persistent.cu).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "simp_gpu.h"

namespace simp {

struct LlamaModel {
  simp_llama_config cfg;
  int64_t kv_dim, head_size;
  // weights (device)
  float *tok_emb = nullptr, *rms_att = nullptr, *rms_ffn = nullptr, *rms_final = nullptr, *wcls = nullptr;
  float *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr, *w1 = nullptr, *w2 = nullptr, *w3 = nullptr;
  uint8_t* qweights = nullptr;
  float *scales = nullptr, *zeros = nullptr;
  int64_t off[7] = {0, 0, 0, 0, 0, 0, 0};   // wq wk wv wo w1 w2 w3 element offsets in the caller's arrays (W4)
  int64_t loff[7] = {0, 0, 0, 0, 0, 0, 0};  // the same for the device copy (differs under tensor parallelism)
  bool offsets_set = false;
  int tp = 1, rank = 0;                      // tensor-parallel degree and this rank
  void* tp_arena = nullptr;                  // tp > 1: symmetric buffer holding x | xb | hb (tagged words) | logits
  uint8_t* tp_peer[8] = {};                  // the arena of every rank as seen from this process
  float* tp_xn = nullptr;                    // tp > 1: normalised x for the classifier (plain floats)
  // state (device)
  float *x = nullptr, *xb = nullptr, *hb = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *logits = nullptr;
  float *kc = nullptr, *vc = nullptr, *attn_part = nullptr;
  int* attn_cnt = nullptr;  // per-head arrival counters of the attention kernel (zero between launches)
  int* ctl = nullptr;     // [0] token, [1] pos, [2] n_prompt, [3] step, [4] next (argmax)
  int32_t *prompt = nullptr, *out_tokens = nullptr;
  int64_t prompt_cap = 0, out_cap = 0;
  int nsplit = 1;
  // tensor maps of the key / value caches for the attention kernel's tiled loads: [n_layers * seq_len rows, kv_dim]
  // f32, boxes of 16 rows x head_size (valid when head_size % 4 == 0)
  CUtensorMap kmap, vmap;
  bool kv_tma = false;
  // scratch of the persistent per-token kernels: grid-barrier words, per-block argmax candidates
  unsigned* pk_bar = nullptr;
  float* pk_best_val = nullptr;
  int* pk_best_idx = nullptr;
  bool pk_attr_done = false;   // the kernel's shared-memory attribute was set on this model's device
  cudaGraphExec_t graph = nullptr;
  int graph_kernels = 0;       // kernel nodes of the captured token graph
  bool loaded_any = false;
};

// One token of the f32 model as a single persistent cooperative kernel (llama_persistent.cu).
int enqueue_token_persistent_f32(LlamaModel& m, cudaStream_t st);
bool persistent_f32_supported(const LlamaModel& m);

}  // namespace simp
