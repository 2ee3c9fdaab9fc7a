// Top-2 MoE routing and token movement.
//
//   router      softmax(x W_r^T) -> top-2 ids + renormalised gates           jarvis_model.py:218-224
//   metadata    stable partition of assignments m = token*K + k by expert    sparse_model.cu:23-90 (M1)
//   gather      dispatched_x[slot] = x[gather_map[slot]]                     sparse_model.cu:95-112 (M2)
//   combine     out[i] = sum_k gate[i,k] * y[scatter_map[i,k]]  (+ sum, sum^2 of out)
//                                                                            sparse_model.cu:117-165 (M3),
//                                                                            jarvis_model.py:249-250
//   finalize    l_balance, act_mean, act_var                                 jarvis_model.py:244-250
//
// The reference builds the dispatch order with ONE thread walking all N*K assignments; here it
// is a parallel stable counting sort: per-chunk histograms, a scan over (chunk, expert), and a
// ballot-ranked scatter.  The order is a pure function of the ids and is bit-exact.
// All of it is HBM/latency-bound integer and copy work: no tensor cores.
#include "common.cuh"
#include "moe_finalize.cuh"
#include "launchers.h"

namespace jb {

namespace {

constexpr int MAX_E = 16;
constexpr int ROUTER_THREADS = 256;                 // 8 warps, one token per warp at a time
constexpr int ROUTER_TOKENS_PER_CTA = 32;             // 512 CTAs at 16k tokens: four resident per SM (64 registers)
constexpr int META_CHUNK = 256;                     // assignments per CTA of the metadata kernels

// ---------------------------------------------------------------------------------------------
// router
// ---------------------------------------------------------------------------------------------
// logits of one token (already warp-reduced, identical in every lane) -> softmax, top-2 with ties going
// to the lower expert id, gates, and the per-warp accumulators of P and the top-1 histogram.
template <int E>
__device__ __forceinline__ void router_finish(const float (&acc)[E], int lane, int tok, int64_t* topk_idx,
                                              float* gates, float* probs_out, int* h_acc, float (&p_local)[E]) {
  float mx = acc[0];
#pragma unroll
  for (int e = 1; e < E; ++e) mx = fmaxf(mx, acc[e]);
  float p[E], den = 0.f;
#pragma unroll
  for (int e = 0; e < E; ++e) { p[e] = expf(acc[e] - mx); den += p[e]; }
  const float inv = 1.0f / den;
  int i0 = 0, i1 = -1;
  float p0 = -1.f, p1 = -1.f;
#pragma unroll
  for (int e = 0; e < E; ++e) {
    p[e] *= inv;
    if (p[e] > p0) { p1 = p0; i1 = i0; p0 = p[e]; i0 = e; }
    else if (p[e] > p1) { p1 = p[e]; i1 = e; }
  }
  if (lane == 0) {
    topk_idx[size_t(tok) * 2 + 0] = i0;
    topk_idx[size_t(tok) * 2 + 1] = i1;
    const float g = p0 + p1 + 1e-8f;
    gates[size_t(tok) * 2 + 0] = p0 / g;
    gates[size_t(tok) * 2 + 1] = p1 / g;
    if (probs_out) {
#pragma unroll
      for (int e = 0; e < E; ++e) probs_out[size_t(tok) * E + e] = p[e];
    }
    atomicAdd(&h_acc[i0], 1);
#pragma unroll
    for (int e = 0; e < E; ++e) p_local[e] += p[e];
  }
}

// Router weights in shared memory: [E][C] with the 4-float groups of every row swizzled (group g of a row
// sits at g ^ ((g >> 3) & 1)).  A lane reads the two groups of its 8 consecutive channels, so lanes are
// 32 bytes apart and, unswizzled, lanes l and l + 4 of each 8-lane phase would hit the same banks.
__device__ __forceinline__ int router_w_index(int c) {   // c: channel, any value; returns the swizzled column
  const int g = c >> 2;
  return ((g ^ ((g >> 3) & 1)) << 2) | (c & 3);
}

// 8 consecutive activations times the matching router weights of every expert
template <int E>
__device__ __forceinline__ void router_dot8(const float (&xv)[8], const float* w_s, int C, int c, float (&acc)[E]) {
  const int ca = router_w_index(c), cb = router_w_index(c + 4);
#pragma unroll
  for (int e = 0; e < E; ++e) {
    const float4 wa = *reinterpret_cast<const float4*>(w_s + e * C + ca);
    const float4 wb = *reinterpret_cast<const float4*>(w_s + e * C + cb);
    acc[e] += xv[0] * wa.x + xv[1] * wa.y + xv[2] * wa.z + xv[3] * wa.w + xv[4] * wb.x + xv[5] * wb.y +
              xv[6] * wb.z + xv[7] * wb.w;
  }
}

template <int E>
__global__ void __launch_bounds__(ROUTER_THREADS)
router_top2_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w_router, int n_tokens, int C,
                   int tokens_per_cta,
                   int64_t* __restrict__ topk_idx, float* __restrict__ gates, float* __restrict__ probs_out,
                   double* __restrict__ probs_sum, int* __restrict__ top1_hist) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float w_s[];  // [E][C]
  __shared__ float p_acc[ROUTER_THREADS / 32][E];
  __shared__ int h_acc[E];
  for (int i = threadIdx.x; i < E * C; i += ROUTER_THREADS) w_s[(i / C) * C + router_w_index(i % C)] = __ldg(w_router + i);
  if (threadIdx.x < E) h_acc[threadIdx.x] = 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float p_local[E];
#pragma unroll
  for (int e = 0; e < E; ++e) p_local[e] = 0.f;
  const int tok0 = blockIdx.x * tokens_per_cta;
  for (int tt = warp; tt < tokens_per_cta; tt += ROUTER_THREADS / 32) {
    const int tok = tok0 + tt;
    if (tok >= n_tokens) break;
    const __nv_bfloat16* xr = x + size_t(tok) * C;
    float acc[E];
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] = 0.f;
    for (int c = lane * 8; c < C; c += 256) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(xr + c));
      const float xv[8] = {bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y),
                           bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w)};
      router_dot8<E>(xv, w_s, C, c, acc);
    }
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] = warp_sum(acc[e]);
    router_finish<E>(acc, lane, tok, topk_idx, gates, probs_out, h_acc, p_local);
  }
  if (lane == 0) {
#pragma unroll
    for (int e = 0; e < E; ++e) p_acc[warp][e] = p_local[e];
  }
  __syncthreads();
  if (threadIdx.x < E) {
    float s = 0.f;
    for (int w = 0; w < ROUTER_THREADS / 32; ++w) s += p_acc[w][threadIdx.x];
    if (probs_sum) atomicAdd(&probs_sum[threadIdx.x], double(s));
    if (top1_hist && h_acc[threadIdx.x]) atomicAdd(&top1_hist[threadIdx.x], h_acc[threadIdx.x]);
  }
}

// RMSNorm (norm2 of the block, jarvis_model.py:25-26, :431) fused with the router: the normalised row
// is rounded to bf16 and stored for the expert GEMMs, and the SAME rounded values feed the router
// logits in the same summation order as router_top2_kernel, so routing is bit-identical to running
// the two kernels separately while the row is read from HBM once.
template <int E>
__global__ void __launch_bounds__(ROUTER_THREADS, 2)
rmsnorm_router_kernel(const float* __restrict__ x, const float* __restrict__ w_norm, float eps,
                      __nv_bfloat16* __restrict__ xn, const float* __restrict__ w_router, int n_tokens, int C,
                      int64_t* __restrict__ topk_idx, float* __restrict__ gates,
                      double* __restrict__ probs_sum, int* __restrict__ top1_hist) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float w_s[];  // [E][C]
  __shared__ float p_acc[ROUTER_THREADS / 32][E];
  __shared__ int h_acc[E];
  for (int i = threadIdx.x; i < E * C; i += ROUTER_THREADS) w_s[(i / C) * C + router_w_index(i % C)] = __ldg(w_router + i);
  if (threadIdx.x < E) h_acc[threadIdx.x] = 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float p_local[E];
#pragma unroll
  for (int e = 0; e < E; ++e) p_local[e] = 0.f;
  // A warp takes TWO tokens per pass: their loads are in flight together, the two dependency chains interleave,
  // and the router weights read from shared memory serve both.  The CTAs are persistent (two per SM) and stride
  // over the token pairs, so the router matrix is staged once per CTA.
  const int n_pairs = (n_tokens + 1) >> 1;
  for (int pair = blockIdx.x * (ROUTER_THREADS / 32) + warp; pair < n_pairs; pair += gridDim.x * (ROUTER_THREADS / 32)) {
    const int tok = 2 * pair;
    const bool two = tok + 1 < n_tokens;
    const float* xr0 = x + size_t(tok) * C;
    const float* xr1 = x + size_t(two ? tok + 1 : tok) * C;     // a lone last token is processed twice, stored once
    float v[2][4][8];
    float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = (i * 32 + lane) * 8;
      if (c < C) {
        const float4 a0 = __ldg(reinterpret_cast<const float4*>(xr0 + c)), b0 = __ldg(reinterpret_cast<const float4*>(xr0 + c) + 1);
        const float4 a1 = __ldg(reinterpret_cast<const float4*>(xr1 + c)), b1 = __ldg(reinterpret_cast<const float4*>(xr1 + c) + 1);
        v[0][i][0] = a0.x; v[0][i][1] = a0.y; v[0][i][2] = a0.z; v[0][i][3] = a0.w;
        v[0][i][4] = b0.x; v[0][i][5] = b0.y; v[0][i][6] = b0.z; v[0][i][7] = b0.w;
        v[1][i][0] = a1.x; v[1][i][1] = a1.y; v[1][i][2] = a1.z; v[1][i][3] = a1.w;
        v[1][i][4] = b1.x; v[1][i][5] = b1.y; v[1][i][6] = b1.z; v[1][i][7] = b1.w;
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if ((i * 32 + lane) * 8 < C) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { ss0 = __fmaf_rn(v[0][i][j], v[0][i][j], ss0); ss1 = __fmaf_rn(v[1][i][j], v[1][i][j], ss1); }
      }
    }
    ss0 = warp_sum(ss0);
    ss1 = warp_sum(ss1);
    const float r0 = rsqrtf(ss0 / float(C) + eps), r1 = rsqrtf(ss1 / float(C) + eps);
    float acc0[E], acc1[E];
#pragma unroll
    for (int e = 0; e < E; ++e) { acc0[e] = 0.f; acc1[e] = 0.f; }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = (i * 32 + lane) * 8;
      if (c < C) {
        const float4 wa = __ldg(reinterpret_cast<const float4*>(w_norm + c));
        const float4 wb = __ldg(reinterpret_cast<const float4*>(w_norm + c) + 1);
        const uint4 pk0 = make_uint4(pack_bf16x2(v[0][i][0] * r0 * wa.x, v[0][i][1] * r0 * wa.y),
                                     pack_bf16x2(v[0][i][2] * r0 * wa.z, v[0][i][3] * r0 * wa.w),
                                     pack_bf16x2(v[0][i][4] * r0 * wb.x, v[0][i][5] * r0 * wb.y),
                                     pack_bf16x2(v[0][i][6] * r0 * wb.z, v[0][i][7] * r0 * wb.w));
        const uint4 pk1 = make_uint4(pack_bf16x2(v[1][i][0] * r1 * wa.x, v[1][i][1] * r1 * wa.y),
                                     pack_bf16x2(v[1][i][2] * r1 * wa.z, v[1][i][3] * r1 * wa.w),
                                     pack_bf16x2(v[1][i][4] * r1 * wb.x, v[1][i][5] * r1 * wb.y),
                                     pack_bf16x2(v[1][i][6] * r1 * wb.z, v[1][i][7] * r1 * wb.w));
        *reinterpret_cast<uint4*>(xn + size_t(tok) * C + c) = pk0;
        if (two) *reinterpret_cast<uint4*>(xn + size_t(tok + 1) * C + c) = pk1;
        const float xv0[8] = {bf16_lo(pk0.x), bf16_hi(pk0.x), bf16_lo(pk0.y), bf16_hi(pk0.y),
                              bf16_lo(pk0.z), bf16_hi(pk0.z), bf16_lo(pk0.w), bf16_hi(pk0.w)};
        const float xv1[8] = {bf16_lo(pk1.x), bf16_hi(pk1.x), bf16_lo(pk1.y), bf16_hi(pk1.y),
                              bf16_lo(pk1.z), bf16_hi(pk1.z), bf16_lo(pk1.w), bf16_hi(pk1.w)};
        router_dot8<E>(xv0, w_s, C, c, acc0);     // the same shared-memory words: the compiler loads them once
        router_dot8<E>(xv1, w_s, C, c, acc1);
      }
    }
#pragma unroll
    for (int e = 0; e < E; ++e) { acc0[e] = warp_sum(acc0[e]); acc1[e] = warp_sum(acc1[e]); }
    router_finish<E>(acc0, lane, tok, topk_idx, gates, nullptr, h_acc, p_local);
    if (two) router_finish<E>(acc1, lane, tok + 1, topk_idx, gates, nullptr, h_acc, p_local);
  }
  if (lane == 0) {
#pragma unroll
    for (int e = 0; e < E; ++e) p_acc[warp][e] = p_local[e];
  }
  __syncthreads();
  if (threadIdx.x < E) {
    float s = 0.f;
    for (int w = 0; w < ROUTER_THREADS / 32; ++w) s += p_acc[w][threadIdx.x];
    if (probs_sum) atomicAdd(&probs_sum[threadIdx.x], double(s));
    if (top1_hist && h_acc[threadIdx.x]) atomicAdd(&top1_hist[threadIdx.x], h_acc[threadIdx.x]);
  }
}

// ---------------------------------------------------------------------------------------------
// dispatch metadata: stable counting sort of M = N*K assignments by expert id
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int clamp_expert(long long e, int E) { return e < 0 ? 0 : (e >= E ? E - 1 : int(e)); }

__global__ void __launch_bounds__(META_CHUNK)
meta_hist_kernel(const int64_t* __restrict__ flat_idx, int M, int E, int* __restrict__ chunk_counts) {
  pdl_wait();
  pdl_trigger();
  __shared__ int h[MAX_E];
  if (threadIdx.x < MAX_E) h[threadIdx.x] = 0;
  __syncthreads();
  const int m = blockIdx.x * META_CHUNK + threadIdx.x;
  if (m < M) atomicAdd(&h[clamp_expert(flat_idx[m], E)], 1);
  __syncthreads();
  if (threadIdx.x < E) chunk_counts[blockIdx.x * E + threadIdx.x] = h[threadIdx.x];
}

// One CTA, one warp per expert: exclusive scan of the per-chunk counts of that expert, then the
// expert offsets.  chunk_base[c][e] = offsets[e] + sum_{c' < c} counts[c'][e].
__global__ void __launch_bounds__(32 * MAX_E)
meta_scan_kernel(const int* __restrict__ chunk_counts, int n_chunks, int E, int* __restrict__ chunk_base,
                 int* __restrict__ expert_counts, int* __restrict__ expert_offsets) {
  pdl_wait();
  pdl_trigger();
  __shared__ int totals[MAX_E];
  __shared__ int offs[MAX_E + 1];
  const int e = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (e < E) {
    int running = 0;
    for (int c0 = 0; c0 < n_chunks; c0 += 32) {
      const int c = c0 + lane;
      const int v = c < n_chunks ? chunk_counts[c * E + e] : 0;
      int incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      if (c < n_chunks) chunk_base[c * E + e] = running + incl - v;  // offsets[e] added below
      running += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) totals[e] = running;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int i = 0; i < E; ++i) { offs[i] = acc; acc += totals[i]; }
    offs[E] = acc;
    for (int i = 0; i < E; ++i) { expert_counts[i] = totals[i]; expert_offsets[i] = offs[i]; }
    expert_offsets[E] = acc;
  }
  __syncthreads();
  if (e < E) {
    const int add = offs[e];
    for (int c = lane; c < n_chunks; c += 32) chunk_base[c * E + e] += add;
  }
}

__global__ void __launch_bounds__(META_CHUNK)
meta_assign_kernel(const int64_t* __restrict__ flat_idx, int M, int K, int E, const int* __restrict__ chunk_base,
                   int* __restrict__ scatter_map, int* __restrict__ gather_map, int* __restrict__ gate_idx_map) {
  pdl_wait();
  pdl_trigger();
  __shared__ int warp_cnt[META_CHUNK / 32][MAX_E];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x * META_CHUNK + threadIdx.x;
  const int e = m < M ? clamp_expert(flat_idx[m], E) : -1;
  int rank = 0;  // assignments of the same expert earlier in this warp
  for (int q = 0; q < E; ++q) {
    const unsigned mask = __ballot_sync(0xffffffffu, e == q);
    if (e == q) rank = __popc(mask & ((1u << lane) - 1u));
    if (lane == 0) warp_cnt[warp][q] = __popc(mask);
  }
  __syncthreads();
  if (m < M) {
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_cnt[w][e];
    const int slot = chunk_base[blockIdx.x * E + e] + before + rank;
    scatter_map[m] = slot;
    gather_map[slot] = m / K;
    gate_idx_map[slot] = m % K;
  }
}

// Small batches (single-token decode steps): the three kernels above in one CTA of up to 1024 threads, one
// assignment per thread.  Same stable order: earlier assignments of the same expert come first.
constexpr int META_SMALL_MAX = 1024;
__global__ void __launch_bounds__(META_SMALL_MAX)
meta_small_kernel(const int64_t* __restrict__ flat_idx, int M, int K, int E, int* __restrict__ expert_counts,
                  int* __restrict__ expert_offsets, int* __restrict__ scatter_map, int* __restrict__ gather_map,
                  int* __restrict__ gate_idx_map) {
  pdl_wait();
  pdl_trigger();
  __shared__ int warp_cnt[META_SMALL_MAX / 32][MAX_E];
  __shared__ int offs[MAX_E + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_warps = (blockDim.x + 31) >> 5;
  const int m = threadIdx.x;
  const int e = m < M ? clamp_expert(flat_idx[m], E) : -1;
  int rank = 0;
  for (int q = 0; q < E; ++q) {
    const unsigned mask = __ballot_sync(0xffffffffu, e == q);
    if (e == q) rank = __popc(mask & ((1u << lane) - 1u));
    if (lane == 0) warp_cnt[warp][q] = __popc(mask);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int q = 0; q < E; ++q) {
      int c = 0;
      for (int w = 0; w < n_warps; ++w) c += warp_cnt[w][q];
      offs[q] = acc;
      expert_counts[q] = c;
      expert_offsets[q] = acc;
      acc += c;
    }
    offs[E] = acc;
    expert_offsets[E] = acc;
  }
  __syncthreads();
  if (m < M) {
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_cnt[w][e];
    const int slot = offs[e] + before + rank;
    scatter_map[m] = slot;
    gather_map[slot] = m / K;
    gate_idx_map[slot] = m % K;
  }
}

// ---------------------------------------------------------------------------------------------
// gather / combine
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
dispatch_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ gather_map, int M, int n_tokens,
                       int C, __nv_bfloat16* __restrict__ dispatched) {
  pdl_wait();
  pdl_trigger();
  const int slot = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (slot >= M) return;
  const int lane = threadIdx.x & 31;
  int tok = gather_map[slot];
  tok = tok < 0 ? 0 : (tok >= n_tokens ? n_tokens - 1 : tok);
  const uint4* src = reinterpret_cast<const uint4*>(x + size_t(tok) * C);
  uint4* dst = reinterpret_cast<uint4*>(dispatched + size_t(slot) * C);
  for (int c = lane; c < C / 8; c += 32) dst[c] = __ldg(src + c);
}

template <typename TOut>
__global__ void __launch_bounds__(256)
scatter_combine_kernel(const __nv_bfloat16* __restrict__ y, const float* __restrict__ gates,
                       const int* __restrict__ scatter_map, int n_tokens, int K, int M, int C,
                       TOut* __restrict__ out, double* __restrict__ stats) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red[2][8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tok = blockIdx.x * 8 + warp;
  float s1 = 0.f, s2 = 0.f;
  if (tok < n_tokens) {
    for (int c = lane * 8; c < C; c += 256) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int k = 0; k < K; ++k) {
        int slot = scatter_map[size_t(tok) * K + k];
        slot = slot < 0 ? 0 : (slot >= M ? M - 1 : slot);
        const float g = gates[size_t(tok) * K + k];
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(y + size_t(slot) * C + c));
        acc[0] += g * bf16_lo(v.x); acc[1] += g * bf16_hi(v.x); acc[2] += g * bf16_lo(v.y); acc[3] += g * bf16_hi(v.y);
        acc[4] += g * bf16_lo(v.z); acc[5] += g * bf16_hi(v.z); acc[6] += g * bf16_lo(v.w); acc[7] += g * bf16_hi(v.w);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) { s1 += acc[j]; s2 += acc[j] * acc[j]; }
      if constexpr (sizeof(TOut) == 2) {
        *reinterpret_cast<uint4*>(out + size_t(tok) * C + c) =
            make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                       pack_bf16x2(acc[6], acc[7]));
      } else {
        float4* o = reinterpret_cast<float4*>(out + size_t(tok) * C + c);
        o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
      }
    }
  }
  if (stats) {
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    if (lane == 0) { red[0][warp] = s1; red[1][warp] = s2; }
    __syncthreads();
    if (threadIdx.x == 0) {
      double a = 0.0, b = 0.0;
      for (int w = 0; w < 8; ++w) { a += double(red[0][w]); b += double(red[1][w]); }
      atomicAdd(&stats[0], a);
      atomicAdd(&stats[1], b);
    }
  }
}

// scalars[0] = l_balance, [1] = act_mean, [2] = act_var (unbiased), all f32.
__global__ void moe_finalize_kernel(const double* __restrict__ stats, const double* __restrict__ probs_sum,
                                    const int* __restrict__ top1_hist, int E, long long n_tokens, long long n_elems,
                                    float balance_alpha, float* __restrict__ scalars) {
  pdl_wait();
  pdl_trigger();
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  moe_finalize_scalars(stats, probs_sum, top1_hist, E, n_tokens, n_elems, balance_alpha, scalars);
}

}  // namespace

int launch_router_top2(const void* x_bf16, const float* w_router, int n_tokens, int C, int E, int64_t* topk_idx,
                       float* gates, float* probs_out, double* probs_sum, int* top1_hist, cudaStream_t stream) {
  JB_REQUIRE(n_tokens >= 0 && C > 0, "router_top2: bad shape");
  JB_REQUIRE(E == 4 || E == 8, "router_top2: num_experts (%d) must be 4 or 8", E);
  JB_REQUIRE(C % 8 == 0 && size_t(E) * C * 4 <= 160 * 1024, "router_top2: d_model (%d) must be a multiple of 8 and fit shared memory", C);
  if (n_tokens == 0) return JB200_OK;
  JB_REQUIRE(x_bf16 && w_router && topk_idx && gates, "router_top2: null pointer");
  JB_REQUIRE(aligned16(x_bf16) && aligned16(w_router), "router_top2: pointers must be 16-byte aligned");
  if (n_tokens == 0) return JB200_OK;
  // small batches (decode steps): one token per warp so that more than a handful of CTAs exist
  const int tpc = n_tokens <= 4096 ? ROUTER_THREADS / 32 : ROUTER_TOKENS_PER_CTA;
  const int blocks = (n_tokens + tpc - 1) / tpc;
  const size_t smem = size_t(E) * C * sizeof(float);
  if (E == 4) {
    JB_CUDA(cudaFuncSetAttribute(router_top2_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    launch_dep(router_top2_kernel<4>, blocks, ROUTER_THREADS, smem, stream,
        reinterpret_cast<const __nv_bfloat16*>(x_bf16), w_router, n_tokens, C, tpc, topk_idx, gates, probs_out, probs_sum,
        top1_hist);
  } else {
    JB_CUDA(cudaFuncSetAttribute(router_top2_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    launch_dep(router_top2_kernel<8>, blocks, ROUTER_THREADS, smem, stream,
        reinterpret_cast<const __nv_bfloat16*>(x_bf16), w_router, n_tokens, C, tpc, topk_idx, gates, probs_out, probs_sum,
        top1_hist);
  }
  JB_LAUNCH_CHECK("router_top2_kernel");
  return JB200_OK;
}

int launch_rmsnorm_router(const float* x, const float* w_norm, float eps, void* xn_bf16, const float* w_router,
                          int n_tokens, int C, int E, int64_t* topk_idx, float* gates, double* probs_sum,
                          int* top1_hist, cudaStream_t stream) {
  JB_REQUIRE(n_tokens >= 0 && C > 0, "rmsnorm_router: bad shape");
  JB_REQUIRE(E == 4 || E == 8, "rmsnorm_router: num_experts (%d) must be 4 or 8", E);
  JB_REQUIRE(C % 8 == 0 && C <= 1024, "rmsnorm_router: d_model (%d) must be a multiple of 8 and at most 1024", C);
  if (n_tokens == 0) return JB200_OK;
  JB_REQUIRE(x && w_norm && xn_bf16 && w_router && topk_idx && gates, "rmsnorm_router: null pointer");
  JB_REQUIRE(aligned16(x) && aligned16(w_norm) && aligned16(xn_bf16) && aligned16(w_router),
             "rmsnorm_router: pointers must be 16-byte aligned");
  if (n_tokens == 0) return JB200_OK;
  // persistent CTAs, two per SM, striding over the token pairs (one pair per warp and pass)
  const int sms = sm_count();
  if (sms <= 0) return JB200_ERR_CUDA;
  const int pair_blocks = ((n_tokens + 1) / 2 + ROUTER_THREADS / 32 - 1) / (ROUTER_THREADS / 32);
  const int blocks = pair_blocks < 2 * sms ? pair_blocks : 2 * sms;
  const size_t smem = size_t(E) * C * sizeof(float);
  __nv_bfloat16* xn = reinterpret_cast<__nv_bfloat16*>(xn_bf16);
  if (E == 4)
    launch_dep(rmsnorm_router_kernel<4>, blocks, ROUTER_THREADS, smem, stream, x, w_norm, eps, xn, w_router, n_tokens, C,
               topk_idx, gates, probs_sum, top1_hist);
  else
    launch_dep(rmsnorm_router_kernel<8>, blocks, ROUTER_THREADS, smem, stream, x, w_norm, eps, xn, w_router, n_tokens, C,
               topk_idx, gates, probs_sum, top1_hist);
  JB_LAUNCH_CHECK("rmsnorm_router_kernel");
  return JB200_OK;
}

size_t moe_metadata_scratch_bytes(int n_tokens, int K, int E) {
  if (n_tokens <= 0 || K <= 0 || E <= 0) return 0;
  const size_t chunks = (size_t(n_tokens) * K + META_CHUNK - 1) / META_CHUNK;
  return 2 * chunks * size_t(E) * sizeof(int);
}

int launch_moe_metadata(const int64_t* topk_idx, int n_tokens, int K, int E, int* expert_counts, int* expert_offsets,
                        int* scatter_map, int* gather_map, int* gate_idx_map, void* scratch, cudaStream_t stream) {
  JB_REQUIRE(n_tokens >= 0 && K >= 1 && K <= 8, "moe_metadata: bad shape (N=%d, K=%d)", n_tokens, K);
  JB_REQUIRE(E >= 1 && E <= MAX_E, "moe_metadata: num_experts (%d) must be in 1..%d", E, MAX_E);
  JB_REQUIRE(size_t(n_tokens) * K < (size_t(1) << 31), "moe_metadata: too many assignments");
  JB_REQUIRE(expert_counts && expert_offsets, "moe_metadata: null pointer");
  const int M = n_tokens * K;
  const int chunks = (M + META_CHUNK - 1) / META_CHUNK;
  JB_REQUIRE(M == 0 || (topk_idx && scatter_map && gather_map && gate_idx_map && scratch), "moe_metadata: null pointer");
  if (M > 0 && M <= META_SMALL_MAX) {
    launch_dep(meta_small_kernel, 1, (M + 31) / 32 * 32, 0, stream, topk_idx, M, K, E, expert_counts, expert_offsets, scatter_map,
                                                            gather_map, gate_idx_map);
    JB_LAUNCH_CHECK("meta_small_kernel");
    return JB200_OK;
  }
  int* chunk_counts = reinterpret_cast<int*>(scratch);
  int* chunk_base = chunk_counts + size_t(chunks) * E;
  if (M > 0) {
    launch_dep(meta_hist_kernel, chunks, META_CHUNK, 0, stream, topk_idx, M, E, chunk_counts);
    JB_LAUNCH_CHECK("meta_hist_kernel");
  }
  launch_dep(meta_scan_kernel, 1, 32 * MAX_E, 0, stream, chunk_counts, chunks, E, chunk_base, expert_counts, expert_offsets);
  JB_LAUNCH_CHECK("meta_scan_kernel");
  if (M > 0) {
    launch_dep(meta_assign_kernel, chunks, META_CHUNK, 0, stream, topk_idx, M, K, E, chunk_base, scatter_map, gather_map,
                                                          gate_idx_map);
    JB_LAUNCH_CHECK("meta_assign_kernel");
  }
  return JB200_OK;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the dispatch metadata: the two work arrays live in a fixed array
// that is part of the library image, so the caller never has to provide (or allocate) scratch.
// ---------------------------------------------------------------------------------------------
constexpr int STATIC_META_MAX_ASSIGNMENTS = 1 << 18;                                 // N*K <= 262144
constexpr int STATIC_META_MAX_CHUNKS = STATIC_META_MAX_ASSIGNMENTS / META_CHUNK;     // 1024
static __device__ __align__(256) int g_meta_scratch[2 * STATIC_META_MAX_CHUNKS * MAX_E];  // 128 KiB per GPU
static int* g_meta_scratch_ptr[64] = {nullptr};   // device address of the array, one per device ordinal

int moe_metadata_static_max_assignments() { return STATIC_META_MAX_ASSIGNMENTS; }

int launch_moe_metadata_static(const int64_t* topk_idx, int n_tokens, int K, int E, int* expert_counts,
                               int* expert_offsets, int* scatter_map, int* gather_map, int* gate_idx_map,
                               cudaStream_t stream) {
  JB_REQUIRE(n_tokens >= 0 && K >= 1 && K <= 8, "moe_metadata_static: bad shape (N=%d, K=%d)", n_tokens, K);
  JB_REQUIRE(size_t(n_tokens) * size_t(K) <= size_t(STATIC_META_MAX_ASSIGNMENTS),
             "moe_metadata_static: N*K = %zu exceeds the built-in scratch limit of %d assignments; "
             "use jb200_moe_metadata with caller-provided scratch",
             size_t(n_tokens) * size_t(K), STATIC_META_MAX_ASSIGNMENTS);
  int dev = 0;
  JB_CUDA(cudaGetDevice(&dev));
  JB_REQUIRE(dev >= 0 && dev < 64, "moe_metadata_static: device ordinal %d out of range", dev);
  if (!g_meta_scratch_ptr[dev]) {
    // First call on this device: resolve the array's DEVICE address.  In host code the name
    // g_meta_scratch is only a handle for the runtime, not something a kernel may dereference.
    int* ptr = nullptr;
    JB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_meta_scratch));
    g_meta_scratch_ptr[dev] = ptr;
  }
  // Every entry the scan and assign kernels read is written by the histogram kernel of the same
  // call first, so nothing left over from an earlier call needs clearing.
  return launch_moe_metadata(topk_idx, n_tokens, K, E, expert_counts, expert_offsets, scatter_map, gather_map,
                             gate_idx_map, g_meta_scratch_ptr[dev], stream);
}

int launch_dispatch_gather(const void* x_bf16, const int* gather_map, int M, int n_tokens, int C, void* dispatched,
                           cudaStream_t stream) {
  JB_REQUIRE(M >= 0 && n_tokens >= 0 && C > 0 && C % 8 == 0, "dispatch_gather: bad shape");
  if (M == 0) return JB200_OK;
  JB_REQUIRE(n_tokens > 0 && x_bf16 && gather_map && dispatched, "dispatch_gather: null pointer");
  JB_REQUIRE(aligned16(x_bf16) && aligned16(dispatched), "dispatch_gather: pointers must be 16-byte aligned");
  launch_dep(dispatch_gather_kernel, (M + 7) / 8, 256, 0, stream, reinterpret_cast<const __nv_bfloat16*>(x_bf16), gather_map, M,
                                                          n_tokens, C, reinterpret_cast<__nv_bfloat16*>(dispatched));
  JB_LAUNCH_CHECK("dispatch_gather_kernel");
  return JB200_OK;
}

int launch_scatter_combine(const void* y_bf16, const float* gates, const int* scatter_map, int n_tokens, int K, int C,
                           void* out, int out_dtype, double* stats, cudaStream_t stream) {
  JB_REQUIRE(n_tokens >= 0 && K >= 1 && K <= 8 && C > 0 && C % 8 == 0, "scatter_combine: bad shape");
  JB_REQUIRE(out_dtype == 0 || out_dtype == 1, "scatter_combine: out_dtype must be 0 (f32) or 1 (bf16)");
  if (n_tokens == 0) return JB200_OK;
  JB_REQUIRE(y_bf16 && gates && scatter_map && out, "scatter_combine: null pointer");
  JB_REQUIRE(aligned16(y_bf16) && aligned16(out), "scatter_combine: pointers must be 16-byte aligned");
  const int blocks = (n_tokens + 7) / 8;
  const int M = n_tokens * K;
  if (out_dtype == 1)
    launch_dep(scatter_combine_kernel<__nv_bfloat16>, blocks, 256, 0, stream,
        reinterpret_cast<const __nv_bfloat16*>(y_bf16), gates, scatter_map, n_tokens, K, M, C,
        reinterpret_cast<__nv_bfloat16*>(out), stats);
  else
    launch_dep(scatter_combine_kernel<float>, blocks, 256, 0, stream, reinterpret_cast<const __nv_bfloat16*>(y_bf16), gates,
                                                              scatter_map, n_tokens, K, M, C,
                                                              reinterpret_cast<float*>(out), stats);
  JB_LAUNCH_CHECK("scatter_combine_kernel");
  return JB200_OK;
}

int launch_moe_finalize(const double* stats, const double* probs_sum, const int* top1_hist, int E, long long n_tokens,
                        long long n_elems, float balance_alpha, float* scalars, cudaStream_t stream) {
  JB_REQUIRE(scalars != nullptr, "moe_finalize: null output");
  JB_REQUIRE(n_tokens > 0 && n_elems > 0, "moe_finalize: empty batch");
  launch_dep(moe_finalize_kernel, 1, 32, 0, stream, stats, probs_sum, top1_hist, E, n_tokens, n_elems, balance_alpha, scalars);
  JB_LAUNCH_CHECK("moe_finalize_kernel");
  return JB200_OK;
}

}  // namespace jb
