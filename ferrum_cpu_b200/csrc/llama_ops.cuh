// Launch wrappers of the Llama / Qwen row kernels (llama_ops.cu).
#pragma once
#include "fc_common.cuh"

namespace fc {

int launch_llama_embed_rows(const QMat& tok, const int* ids, int R, float* x, int* error_flag, cudaStream_t st);
// Rotation of window rows with the result written as bf16 hi / lo planes [R][ld] (the f32 rows stay as they were).
int launch_llama_rope_planes(const float* qkv, int R, int ld, int T, int n_q, int n_kv, int k_off, int hd, int rope_dim, int neox,
                             const float2* ftab, float inv_linear, void* hi, void* lo, cudaStream_t st);
int launch_llama_embed_step(const QMat& tok, int ctx, const int* queue, StepState* state, float* x, cudaStream_t st);
int launch_llama_rmsnorm(const float* x, const float* w, float eps, int rows, int d, float* y, const StepState* state,
                         cudaStream_t st);
// ftab[i] = {base^(-2i/rope_dim) as f32, freq_factor_i or 1}; inv_linear = 1 / linear_factor.
int launch_llama_rope_rows(float* qkv, int R, int ld, int T, int n_q, int n_kv, int k_off, int hd, int rope_dim, int neox,
                           const float2* ftab, float inv_linear, cudaStream_t st);
// Rows [R] of a fused, rotated q | k | v buffer -> the first R rows of a layer's caches.
int launch_llama_store_kv_rows(const float* qkv, int R, int ld, int q_dim, int kv_dim, float* kc, float* vc, cudaStream_t st);
// Rotation, cache append and single-query grouped attention in one kernel: q | k | v fused row
// in, attention output [n_q * hd] out.
int launch_llama_attn_decode(const float* qkv, int n_q, int n_kv, int hd, int rope_dim, int neox, const float2* ftab, float inv_linear,
                             float* kc, float* vc, int ctx, const StepState* state, float* out, cudaStream_t st);
// RMSNorm written as the bf16 hi / lo planes [rows][d] of the tensor-core GEMM.
int launch_llama_rmsnorm_planes(const float* x, const float* w, float eps, int rows, int d, void* hi, void* lo, cudaStream_t st);
int launch_llama_swiglu(const float* gu, int rows, int F, float* h, const StepState* state, cudaStream_t st);
int launch_llama_score_rows(const float* logits, int ldl, int V, const int* targets, int R, double* logprob, uint8_t* is_greedy,
                            cudaStream_t st);
int launch_llama_pick(const float* logits, int V, int* queue, int queue_cap, StepState* state, cudaStream_t st);

}  // namespace fc
