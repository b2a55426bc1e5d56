// Host API of the sequence-mixing kernels (see seqmix.cu).  Pointers are device pointers; `bf16` selects the activation type
// (__nv_bfloat16, else float).  Functions returning bool report false for sizes no kernel instance covers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200seq {

struct DeltaArgs {
  const void *q, *k, *v;          // [T, KH, d], [T, KH, d], [T, H, dv] with row strides ldq / ldk / ldv (elements)
  int64_t ldq, ldk, ldv;
  const float* log_decay;         // [T, H, d]
  const float* beta;              // [T, H]
  const int *cu, *rows;
  float* state;                   // [rows, H, d, dv]
  float* out;                     // [T, H, dv]
  int H, KH, d, dv;
  int max_len;                    // the longest sequence of the step (0: unknown)
  float unit_eps, q_scale;        // unit_eps < 0: q / k are used as given
};

struct MlstmArgs {
  const void *q, *k, *v;          // [T, H, d], [T, H, d], [T, H, dv]
  int64_t ldq, ldk, ldv;
  const float *log_i, *log_f;     // [T, H]
  const int *cu, *rows;
  float *state, *norm_state, *max_state;
  float* out;
  int H, d, dv;
  int max_len;                    // the longest sequence of the step (0: unknown)
  float q_scale, denom_eps;
};

struct LatentAttnArgs {
  const void* q;                  // [T, H, r]
  const void* cache;              // [slots, r]
  const int *block_table, *tok_req, *tok_len;
  float* out;                     // [T, H, r]
  float* ws;                      // [T, H, n_splits, r + 2] when n_splits > 1
  int H, r, block_size, max_blocks, n_splits;
  int vec_ok;                     // rows of the cache may be copied 16 bytes at a time
  float scale;
};

void add_rms_norm(float* x, const void* delta, const void* w, void* y, int rows, int cols, float eps, bool bf16, cudaStream_t s);
void gated_head_rms_norm(const float* o, const void* w, const void* gate, void* y, int n_tok, int H, int dv, bool w_per_head,
                         float eps, bool bf16, cudaStream_t s);
void causal_conv_silu(const void* x, int64_t ldx, const void* w, const int* cu, const int* rows, const int* tok_seq, void* window,
                      void* y, int n_tok, int R, int C, int taps, int max_len, bool bf16, cudaStream_t s);
bool delta_rule_scan(const DeltaArgs& p, int R, bool bf16, cudaStream_t s);
bool mlstm_scan(const MlstmArgs& p, int R, bool bf16, cudaStream_t s);
bool latent_attention_paged(const LatentAttnArgs& p, int n_tok, bool bf16, cudaStream_t s);
// key splits per query token for a batch of n_tok tokens whose longest context is max_len
int latent_attention_splits(int H, int r, int n_tok, int max_len);
bool group_limited_router(const float* logits, float* probs, bool* rmap, int n_tok, int E, int topk, int G, int keep, bool renorm,
                          cudaStream_t s);

}  // namespace b200seq
