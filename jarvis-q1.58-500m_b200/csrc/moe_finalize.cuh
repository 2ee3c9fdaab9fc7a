// The scalar outputs of the MoE layer from its accumulated statistics (jarvis_engine/jarvis_model.py:244-250):
// shared by moe_finalize_kernel and the fused single-token tail kernel, so that both derive the same bits.
#pragma once

namespace jb {

#if defined(__CUDACC__)

// torch.var (unbiased) of the layer output from its sum and sum of squares; a single element gives NaN as torch does.
__device__ __forceinline__ float moe_act_mean(const double* stats, long long n_elems) {
  return float(stats[0] / double(n_elems));
}
__device__ __forceinline__ float moe_act_var(const double* stats, long long n_elems) {
  const double mean = stats[0] / double(n_elems);
  const double var = (stats[1] - stats[0] * mean) / double(n_elems - 1);
  return n_elems > 1 ? float(var > 0.0 ? var : 0.0) : __int_as_float(0x7fc00000);
}

// scalars[0] = l_balance, [1] = act_mean, [2] = act_var, all f32; one thread.
__device__ __forceinline__ void moe_finalize_scalars(const double* stats, const double* probs_sum, const int* top1_hist,
                                                     int E, long long n_tokens, long long n_elems, float balance_alpha,
                                                     float* scalars) {
  if (probs_sum && top1_hist) {
    double acc = 0.0;
    for (int e = 0; e < E; ++e)
      acc += (double(top1_hist[e]) / double(n_tokens)) * (probs_sum[e] / double(n_tokens));
    scalars[0] = float(double(balance_alpha) * double(E) * acc);
  }
  if (stats) {
    scalars[1] = moe_act_mean(stats, n_elems);
    scalars[2] = moe_act_var(stats, n_elems);
  }
}

// The decay of one LSF call from the variance of the MoE output (jarvis_model.py:297-298).
__device__ __forceinline__ float lsf_alpha_from_var(float alpha_min, float alpha_max, float var_scale, float act_var) {
  return alpha_min + (alpha_max - alpha_min) * (1.0f / (1.0f + expf(var_scale * act_var)));
}

// One membrane update h <- alpha h + (1 - alpha) m with the roundings spelled out, so that every kernel that
// takes a single step produces the same bits.
__device__ __forceinline__ float lsf_step(float alpha, float h, float m) {
  return __fmaf_rn(alpha, h, __fmul_rn(1.0f - alpha, m));
}

#endif

}  // namespace jb
