// Host-side launch functions implemented by the kernel translation units and called by the
// extern "C" layer in api.cu.  All return JB200_OK / JB200_ERR_ARG / JB200_ERR_CUDA.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace jb {

size_t pack_ternary_scratch_bytes(int out_features, int in_features);
int launch_pack_ternary(const float* w, int out_features, int in_features, const float* alpha_in, uint8_t* packed,
                        float* alpha_out, void* scratch, cudaStream_t stream);
int launch_pack_codes(const float* w_ternary, size_t n_elems, uint8_t* packed, cudaStream_t stream);
int launch_unpack_ternary(const uint8_t* packed, size_t n_bytes, int out_dtype, void* out, cudaStream_t stream);

// Extra arguments of the JB200_EPI_QK_ROPE_BF16 epilogue (q/k/v projection fused with the attention prologue).
struct GemmRope {
  const float* cos_tab;   // [n_pos][32]
  const float* sin_tab;
  const int32_t* pos0;    // [M / T] or null
  int pos0_scalar, n_pos, T, rope_feats;
};
int launch_ternary_gemm(const void* x_bf16, int M, int K, const uint8_t* w_packed, const float* alpha,
                        int alpha_rows, int N, int G, const int32_t* seg_offsets, int epilogue, void* out,
                        int bn_override, int w_layout, cudaStream_t stream, const GemmRope* rope = nullptr);
int launch_prepare_weights(const uint8_t* packed, size_t n_bytes, uint8_t* prepared, cudaStream_t stream);
void decode16_host(uint32_t w, uint32_t* out8);
void decode16_prepared_host(uint32_t w_canonical, uint32_t* out8);

int launch_rmsnorm(const void* x, int x_dtype, const float* w, float eps, void* y, int y_dtype, int n_rows, int C,
                   cudaStream_t stream);
int launch_embedding(const int64_t* idx, const float* table, int vocab, float* out, int n_rows, int C,
                     cudaStream_t stream);

int launch_router_top2(const void* x_bf16, const float* w_router, int n_tokens, int C, int E, int64_t* topk_idx,
                       float* gates, float* probs_out, double* probs_sum, int* top1_hist, cudaStream_t stream);
int launch_rmsnorm_router(const float* x, const float* w_norm, float eps, void* xn_bf16, const float* w_router,
                          int n_tokens, int C, int E, int64_t* topk_idx, float* gates, double* probs_sum,
                          int* top1_hist, cudaStream_t stream);
size_t moe_metadata_scratch_bytes(int n_tokens, int K, int E);
int launch_moe_metadata(const int64_t* topk_idx, int n_tokens, int K, int E, int* expert_counts, int* expert_offsets,
                        int* scatter_map, int* gather_map, int* gate_idx_map, void* scratch, cudaStream_t stream);
int moe_metadata_static_max_assignments();
int launch_moe_metadata_static(const int64_t* topk_idx, int n_tokens, int K, int E, int* expert_counts,
                               int* expert_offsets, int* scatter_map, int* gather_map, int* gate_idx_map,
                               cudaStream_t stream);
int launch_dispatch_gather(const void* x_bf16, const int* gather_map, int M, int n_tokens, int C, void* dispatched,
                           cudaStream_t stream);
int launch_scatter_combine(const void* y_bf16, const float* gates, const int* scatter_map, int n_tokens, int K, int C,
                           void* out, int out_dtype, double* stats, cudaStream_t stream);
int launch_moe_finalize(const double* stats, const double* probs_sum, const int* top1_hist, int E, long long n_tokens,
                        long long n_elems, float balance_alpha, float* scalars, cudaStream_t stream);

int launch_lsf_scan(const void* m, int m_dtype, const void* alpha_tensor, const float* alpha_scalar,
                    const float* act_var, const float* var_scale, float alpha_min, float alpha_max, const float* h0,
                    float* resid, void* out, int out_dtype, float* h_last, void* scratch, int B, int T, int D,
                    cudaStream_t stream);
size_t lsf_scan_scratch_bytes(int B, int T, int D);
int launch_lsf_step_norm(const void* m_bf16, const double* stats, const double* probs_sum, const int* top1_hist, int E,
                         long long n_tokens, long long n_elems, float balance_alpha, float* scalars,
                         const float* var_scale, float alpha_min, float alpha_max, const float* h_in, float* h_out,
                         float* x, const float* w_norm, float eps, void* xn_bf16, int B, int C, cudaStream_t stream);

int launch_attn_scan(const void* q, const void* k, const void* v, int ld_qkv, const float* gamma,
                     const float* cos_tab, const float* sin_tab, int n_pos, const int32_t* pos0, int pos0_scalar,
                     const float* s_in, void* o, int ld_o, float* s_out, void* scratch, int B, int T, int H,
                     int head_dim, int flags, cudaStream_t stream);
size_t attn_scan_scratch_bytes(int B, int T, int H);

int launch_peer_barrier(const void* const* peer_flags, int world, int rank, cudaStream_t stream);
int launch_ep_pull_gather(const void* const* peer_offs, const void* const* peer_gmap, const void* const* peer_xn,
                          int world, int rank, int E, int C, int K, int n_max, int max_rows, void* dispatched,
                          int32_t* seg_offsets, int32_t* meta, cudaStream_t stream);
int launch_ep_pull_combine(const void* const* peer_y, const void* const* peer_meta, const int32_t* offs_local,
                           const int64_t* topk_idx, const float* gates, const int32_t* scatter_map, int world, int rank,
                           int E, int C, int K, int n_tokens, int max_rows, void* out, int out_dtype, double* stats,
                           cudaStream_t stream);
int launch_sample(const void* logits, int logits_dtype, int ld, int n_rows, int V, float temperature, int top_k,
                  float top_p, const float* u, int64_t* out_token, float* out_prob, cudaStream_t stream);

}  // namespace jb
