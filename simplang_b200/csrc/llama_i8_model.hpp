// llama_i8_model.hpp -- device-resident state of the int8 LLaMA-3.2-1B-style model (llama_i8.cu).
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <vector>

#include "simp_gpu.h"

namespace simp {

struct LlamaI8Model {
  simp_llama_i8_config cfg;
  int64_t kv_dim;
  float *rms_att = nullptr, *rms_ffn = nullptr, *rms_final = nullptr, *wcls = nullptr;
  int8_t *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr, *w1 = nullptr, *w2 = nullptr, *w3 = nullptr;
  // state
  int8_t *x_i8 = nullptr, *xb_i8 = nullptr, *ffn_hb = nullptr, *kc = nullptr, *vc = nullptr;
  float *x = nullptr, *xb = nullptr, *logits = nullptr;
  int32_t *q = nullptr, *k = nullptr, *v = nullptr;
  int* ctl = nullptr;   // [0] pos
  float* attn_part = nullptr;   // [n_heads, nsplit, head_dim + 2] split partials of the attention
  int* attn_cnt = nullptr;      // per-head arrival counters (zero between launches)
  int nsplit = 1;
  cudaGraphExec_t graph = nullptr;
  // prefill: scratch and one captured graph per sequence length that has been used
  struct PrefillPlan {
    int64_t M = 0;
    float* x = nullptr;
    int8_t *x_i8 = nullptr, *xb_i8 = nullptr, *hb = nullptr;
    int32_t *acc0 = nullptr, *acc1 = nullptr;
    cudaGraphExec_t graph = nullptr;
  };
  std::vector<PrefillPlan> plans;
};

}  // namespace simp
