// Liquid State Fusion decay scan:  h_t = a_t * h_{t-1} + (1 - a_t) * m_t  per (batch, channel).
//
// Two flavours behind one kernel:
//   * model semantics (LiquidStateFusion.forward, jarvis_engine/jarvis_model.py:281-314): ONE scalar
//     decay per call, alpha = alpha_min + (alpha_max - alpha_min) * sigmoid(-var_scale * act_var),
//     read from device memory so the stream never waits for the host.  The reference evaluates it as
//     a dense T x T decay-matrix product (2*T^2*C flop per sequence); here it is a single streaming
//     pass: 2 bytes read + (optionally) the fused residual update per element.
//   * extension semantics (LiquidStateFusionFunction.forward, liquid_fusion_cuda/liquid_state_fusion.py
//     :49-70; kernel L9 liquid_state_fusion_cuda.cu:412-453): a per-element decay tensor (B, T, D).
//
// Parallel in T inside a CTA: each of the 8 warps scans a run of TPW consecutive tokens with a zero
// carry-in, publishes (product of decays, end value) in shared memory, the carries are combined in
// warp order (the recurrence is an associative affine map), and every thread fixes its values up
// with  h_t = local_t + P_t * carry_in.  A CTA owns 64 channels of one sequence and walks T tile by
// tile.  When B*D/64 CTAs cannot fill the GPU, T is also cut into segments.  A first launch (ENDS_ONLY)
// then computes, with ONE CTA PER TILE of the non-final segments (all tiles in parallel, nothing
// sequential), each tile's end value (and decay product) from a zero carry, reading m once more (it was
// just written by the MoE combine and is normally still in L2); the main launch folds the ends of all
// earlier tiles into its carry-in, which is exact because the recurrence is an affine map.
//
// The two forms the model and the scan sweep run (one scalar decay, bf16 input, and either the fused f32
// residual update or a bf16 output) take lsf_tma_kernel: the same scan, but the [128 tokens x 64 channels] tiles
// travel by TMA (cp.async.bulk.tensor) through a ring of shared-memory stages - loads complete on mbarriers
// (bounded waits), results are written into the tile in place and leave by a TMA store - so the bytes in flight
// no longer depend on how many registers a thread can spare for outstanding loads.
#include "common.cuh"
#include "gemm_shared.cuh"
#include "moe_finalize.cuh"
#include "launchers.h"

namespace jb {

namespace {

constexpr int LSF_WARPS = 8;
constexpr int LSF_THREADS = LSF_WARPS * 32;
constexpr int LSF_CH = 64;  // channels per CTA (2 per lane)

struct LsfParams {
  const void* m;           // [B][T][D]  TM
  const void* alpha_t;     // [B][T][D]  TM   (tensor mode)
  const float* alpha_s;    // scalar decay on the device, or null
  const float* act_var;    // scalar on the device (used when alpha_s is null)
  const float* var_scale;  // scalar on the device
  float alpha_min, alpha_max;
  const float* h0;         // [B][D] f32 or null
  float* resid;            // [B][T][D] f32 in/out or null:  resid += h
  void* out;               // [B][T][D] TOut or null
  float* h_last;           // [B][D] f32 or null
  int B, T, D;
  int seg_len, nseg;       // tokens per segment (multiple of the tile), number of segments (grid.z)
  int n_pre_tiles;         // tiles in the non-final segments = (nseg - 1) * seg_len / tile
  float* seg_end;          // [B][n_pre_tiles][D] end value of each of those tiles from a zero carry
  float* seg_prod;         // [B][n_pre_tiles][D] product of its decays (tensor mode)
};

template <typename T>
__device__ __forceinline__ float2 ld2(const T* p);
template <>
__device__ __forceinline__ float2 ld2<float>(const float* p) { return __ldg(reinterpret_cast<const float2*>(p)); }
template <>
__device__ __forceinline__ float2 ld2<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(p));
  return make_float2(bf16_lo(w), bf16_hi(w));
}
template <typename T>
__device__ __forceinline__ void st2(T* p, float a, float b);
template <>
__device__ __forceinline__ void st2<float>(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
template <>
__device__ __forceinline__ void st2<__nv_bfloat16>(__nv_bfloat16* p, float a, float b) {
  *reinterpret_cast<uint32_t*>(p) = pack_bf16x2(a, b);
}

template <bool TENSOR_ALPHA, typename TM, typename TOut, int TPW, bool ENDS_ONLY>
__global__ void __launch_bounds__(LSF_THREADS, TENSOR_ALPHA ? 1 : 2) lsf_scan_kernel(const LsfParams p) {
  pdl_wait();
  pdl_trigger();
  __shared__ float2 s_end[2][LSF_WARPS][32];   // end value of each warp's run
  __shared__ float2 s_prod[2][LSF_WARPS][32];  // product of decays over the run (tensor mode)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.y;
  const int ch = blockIdx.x * LSF_CH + lane * 2;
  const bool ch_ok = ch < p.D;
  const size_t seq_base = size_t(b) * p.T * p.D + ch;
  const TM* m = reinterpret_cast<const TM*>(p.m);
  const TM* at = reinterpret_cast<const TM*>(p.alpha_t);
  TOut* out = reinterpret_cast<TOut*>(p.out);

  float alpha = 0.f, pw[TPW];  // scalar mode: pw[i] = alpha^(i+1)
  if (!TENSOR_ALPHA) {
    if (p.alpha_s) {
      alpha = __ldg(p.alpha_s);
    } else {
      const float z = -__ldg(p.var_scale) * __ldg(p.act_var);
      alpha = p.alpha_min + (p.alpha_max - p.alpha_min) * (1.0f / (1.0f + expf(-z)));
    }
    float a = alpha;
#pragma unroll
    for (int i = 0; i < TPW; ++i) { pw[i] = a; a *= alpha; }
  }
  constexpr int TILE = LSF_WARPS * TPW;
  const int seg = blockIdx.z;                                    // ENDS_ONLY: the tile's index instead
  const int t_begin = ENDS_ONLY ? seg * TILE : seg * p.seg_len;
  const int t_end = ENDS_ONLY ? t_begin + TILE : min(p.T, t_begin + p.seg_len);
  float2 carry = make_float2(0.f, 0.f);
  float2 pcarry = make_float2(1.f, 1.f);   // running decay product of the segment (ENDS_ONLY, tensor mode)
  if (!ENDS_ONLY) {
    if (p.h0 && ch_ok) carry = __ldg(reinterpret_cast<const float2*>(p.h0 + size_t(b) * p.D + ch));
    if (seg > 0 && ch_ok) {
      const float a_seg = TENSOR_ALPHA ? 0.f : expf(float(TILE) * logf(alpha));   // decay over one tile
      const size_t e0 = (size_t(b) * p.n_pre_tiles) * p.D + ch;
      const int n_before = seg * (p.seg_len / TILE);
      for (int s2 = 0; s2 < n_before; ++s2) {
        const float2 e = __ldg(reinterpret_cast<const float2*>(p.seg_end + e0 + size_t(s2) * p.D));
        if (TENSOR_ALPHA) {
          const float2 q = __ldg(reinterpret_cast<const float2*>(p.seg_prod + e0 + size_t(s2) * p.D));
          carry.x = q.x * carry.x + e.x;
          carry.y = q.y * carry.y + e.y;
        } else {
          carry.x = a_seg * carry.x + e.x;
          carry.y = a_seg * carry.y + e.y;
        }
      }
    }
  }

  int buf = 0;
  for (int tile0 = t_begin; tile0 < t_end; tile0 += LSF_WARPS * TPW, buf ^= 1) {
    const int t0 = tile0 + warp * TPW;
    float2 loc[TPW];
    float2 prod[TENSOR_ALPHA ? TPW : 1];
    float2 mv[TPW], av[TENSOR_ALPHA ? TPW : 1];
#pragma unroll
    for (int i = 0; i < TPW; ++i) {
      const bool ok = ch_ok && (t0 + i) < p.T;
      mv[i] = ok ? ld2<TM>(m + seq_base + size_t(t0 + i) * p.D) : make_float2(0.f, 0.f);
      if (TENSOR_ALPHA) av[i] = ok ? ld2<TM>(at + seq_base + size_t(t0 + i) * p.D) : make_float2(1.f, 1.f);
    }
    // the residual values do not depend on the scan: their loads go out together with those of m, so
    // both streams are in flight at once and the read-modify-write never serialises
    float2 rold[(!ENDS_ONLY) ? TPW : 1];
    if (!ENDS_ONLY && p.resid) {
#pragma unroll
      for (int i = 0; i < TPW; ++i) {
        const int t = t0 + i;
        rold[i] = (ch_ok && t < p.T) ? *reinterpret_cast<const float2*>(p.resid + seq_base + size_t(t) * p.D)
                                     : make_float2(0.f, 0.f);
      }
    }
    float2 h = make_float2(0.f, 0.f), pr = make_float2(1.f, 1.f);
#pragma unroll
    for (int i = 0; i < TPW; ++i) {
      if (TENSOR_ALPHA) {
        // out-of-range tokens carry a = 1, m = 0: the identity map
        h.x = av[i].x * h.x + (1.0f - av[i].x) * mv[i].x;
        h.y = av[i].y * h.y + (1.0f - av[i].y) * mv[i].y;
        pr.x *= av[i].x;
        pr.y *= av[i].y;
        prod[i] = pr;
      } else {
        h.x = alpha * h.x + (1.0f - alpha) * mv[i].x;
        h.y = alpha * h.y + (1.0f - alpha) * mv[i].y;
      }
      loc[i] = h;
    }
    s_end[buf][warp][lane] = h;
    if (TENSOR_ALPHA) s_prod[buf][warp][lane] = pr;
    __syncthreads();
    // carry into this warp's run, and the carry out of the whole tile
    float2 c = carry, cn;
    const float a_run = TENSOR_ALPHA ? 0.f : pw[TPW - 1];
#pragma unroll
    for (int w = 0; w < LSF_WARPS; ++w) {
      if (w == warp) cn = c;
      const float2 e = s_end[buf][w][lane];
      if (TENSOR_ALPHA) {
        const float2 q = s_prod[buf][w][lane];
        c.x = q.x * c.x + e.x;
        c.y = q.y * c.y + e.y;
        if (ENDS_ONLY) { pcarry.x *= q.x; pcarry.y *= q.y; }
      } else {
        c.x = a_run * c.x + e.x;
        c.y = a_run * c.y + e.y;
      }
    }
    carry = c;
    c = cn;
    if (ENDS_ONLY) continue;
#pragma unroll
    for (int i = 0; i < TPW; ++i) {
      const int t = t0 + i;
      if (ch_ok && t < p.T) {
        const float fx = TENSOR_ALPHA ? prod[i].x : pw[i];
        const float fy = TENSOR_ALPHA ? prod[i].y : pw[i];
        const float hx = loc[i].x + fx * c.x;
        const float hy = loc[i].y + fy * c.y;
        const size_t o = seq_base + size_t(t) * p.D;
        if (out) st2<TOut>(out + o, hx, hy);
        if (p.resid) *reinterpret_cast<float2*>(p.resid + o) = make_float2(rold[i].x + hx, rold[i].y + hy);
        if (t == p.T - 1 && p.h_last) *reinterpret_cast<float2*>(p.h_last + size_t(b) * p.D + ch) = make_float2(hx, hy);
      }
    }
  }
  if (ENDS_ONLY && ch_ok && warp == 0) {
    const size_t e = (size_t(b) * p.n_pre_tiles + seg) * p.D + ch;
    *reinterpret_cast<float2*>(p.seg_end + e) = carry;
    if (TENSOR_ALPHA) *reinterpret_cast<float2*>(p.seg_prod + e) = pcarry;
  }
}

// Short sequences (decode steps): one thread per channel pair walks the few tokens itself.
template <bool TENSOR_ALPHA, typename TM, typename TOut>
__global__ void __launch_bounds__(256) lsf_short_kernel(const LsfParams p) {
  pdl_wait();
  pdl_trigger();
  const size_t pair = size_t(blockIdx.x) * 256 + threadIdx.x;
  const int half_d = p.D / 2;
  if (pair >= size_t(p.B) * half_d) return;
  const int b = int(pair / half_d), ch = int(pair % half_d) * 2;
  const TM* m = reinterpret_cast<const TM*>(p.m);
  const TM* at = reinterpret_cast<const TM*>(p.alpha_t);
  TOut* out = reinterpret_cast<TOut*>(p.out);
  float alpha = 0.f;
  if (!TENSOR_ALPHA) {
    if (p.alpha_s) alpha = __ldg(p.alpha_s);
    else alpha = lsf_alpha_from_var(p.alpha_min, p.alpha_max, __ldg(p.var_scale), __ldg(p.act_var));
  }
  float2 h = p.h0 ? *reinterpret_cast<const float2*>(p.h0 + size_t(b) * p.D + ch) : make_float2(0.f, 0.f);
  for (int t = 0; t < p.T; ++t) {
    const size_t o = (size_t(b) * p.T + t) * p.D + ch;
    const float2 mv = ld2<TM>(m + o);
    float2 a = make_float2(alpha, alpha);
    if (TENSOR_ALPHA) a = ld2<TM>(at + o);
    h.x = lsf_step(a.x, h.x, mv.x);
    h.y = lsf_step(a.y, h.y, mv.y);
    if (out) st2<TOut>(out + o, h.x, h.y);
    if (p.resid) {
      float2* r = reinterpret_cast<float2*>(p.resid + o);
      const float2 rv = *r;
      *r = make_float2(rv.x + h.x, rv.y + h.y);
    }
  }
  if (p.h_last) *reinterpret_cast<float2*>(p.h_last + size_t(b) * p.D + ch) = h;
}

// Single-token tail of a block (decode steps), three launches in one: the MoE layer's scalars from its accumulated
// statistics (moe_finalize_kernel), the LSF step with the fused residual (lsf_short_kernel at T = 1: the decay comes
// from act_var, h <- alpha h + (1 - alpha) m, x += h) and the RMSNorm that follows (norm1 of the next block or the
// final norm; rmsnorm_kernel<float, bf16>).  One warp per sequence, lanes on the channels of rmsnorm_kernel with its
// summation order, every rounding as in the three kernels: the results are theirs bit for bit.
struct LsfStepParams {
  const __nv_bfloat16* m;      // [B][C] MoE output
  const double* stats;         // [2] sum, sum of squares of the MoE output
  const double* probs_sum;     // [E] or null
  const int* top1_hist;        // [E] or null
  int E;
  long long n_tokens, n_elems;
  float balance_alpha;
  float* scalars;              // [3] out: l_balance, act_mean, act_var
  const float* var_scale;
  float alpha_min, alpha_max;
  const float* h_in;           // [B][C] or null (zero membrane)
  float* h_out;                // [B][C] (may alias h_in)
  float* x;                    // [B][C] residual stream, in/out
  const float* w_norm;         // [C] or null: no norm wanted
  float eps;
  __nv_bfloat16* xn;           // [B][C] out (with w_norm)
  int B, C;
};

__global__ void __launch_bounds__(256) lsf_step_norm_kernel(const LsfStepParams p) {
  pdl_wait();
  pdl_trigger();
  if (blockIdx.x == 0 && threadIdx.x == 0)
    moe_finalize_scalars(p.stats, p.probs_sum, p.top1_hist, p.E, p.n_tokens, p.n_elems, p.balance_alpha, p.scalars);
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= p.B) return;
  const float alpha = lsf_alpha_from_var(p.alpha_min, p.alpha_max, __ldg(p.var_scale), moe_act_var(p.stats, p.n_elems));
  const size_t base = size_t(row) * p.C;
  float v[4][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = (i * 32 + lane) * 8;
    if (c < p.C) {
      const uint4 mw = __ldg(reinterpret_cast<const uint4*>(p.m + base + c));
      const float mv[8] = {bf16_lo(mw.x), bf16_hi(mw.x), bf16_lo(mw.y), bf16_hi(mw.y),
                           bf16_lo(mw.z), bf16_hi(mw.z), bf16_lo(mw.w), bf16_hi(mw.w)};
      float h[8];
      if (p.h_in) {
        const float4 a = *reinterpret_cast<const float4*>(p.h_in + base + c), b = *reinterpret_cast<const float4*>(p.h_in + base + c + 4);
        h[0] = a.x; h[1] = a.y; h[2] = a.z; h[3] = a.w; h[4] = b.x; h[5] = b.y; h[6] = b.z; h[7] = b.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = 0.f;
      }
      const float4 xa = *reinterpret_cast<const float4*>(p.x + base + c), xb = *reinterpret_cast<const float4*>(p.x + base + c + 4);
      const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        h[j] = lsf_step(alpha, h[j], mv[j]);
        v[i][j] = xv[j] + h[j];
        ss = __fmaf_rn(v[i][j], v[i][j], ss);
      }
      *reinterpret_cast<float4*>(p.h_out + base + c) = make_float4(h[0], h[1], h[2], h[3]);
      *reinterpret_cast<float4*>(p.h_out + base + c + 4) = make_float4(h[4], h[5], h[6], h[7]);
      *reinterpret_cast<float4*>(p.x + base + c) = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
      *reinterpret_cast<float4*>(p.x + base + c + 4) = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
    }
  }
  if (!p.w_norm) return;
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / float(p.C) + p.eps);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = (i * 32 + lane) * 8;
    if (c < p.C) {
      const float4 wa = __ldg(reinterpret_cast<const float4*>(p.w_norm + c)), wb = __ldg(reinterpret_cast<const float4*>(p.w_norm + c + 4));
      *reinterpret_cast<uint4*>(p.xn + base + c) =
          make_uint4(pack_bf16x2(v[i][0] * r * wa.x, v[i][1] * r * wa.y), pack_bf16x2(v[i][2] * r * wa.z, v[i][3] * r * wa.w),
                     pack_bf16x2(v[i][4] * r * wb.x, v[i][5] * r * wb.y), pack_bf16x2(v[i][6] * r * wb.z, v[i][7] * r * wb.w));
    }
  }
}

constexpr int LSF_TPW = 16;                       // tokens per warp per tile
constexpr int LSF_TILE = LSF_WARPS * LSF_TPW;     // 128 tokens

template <bool TA, typename TM, typename TOut>
int launch_t(const LsfParams& p, cudaStream_t stream) {
  if (p.T <= 8) {
    const size_t pairs = size_t(p.B) * (p.D / 2);
    launch_dep(lsf_short_kernel<TA, TM, TOut>, unsigned((pairs + 255) / 256), 256, 0, stream, p);
    JB_LAUNCH_CHECK("lsf_short_kernel");
    return JB200_OK;
  }
  if (p.nseg > 1) {
    dim3 grid_a((p.D + LSF_CH - 1) / LSF_CH, p.B, p.n_pre_tiles);
    launch_dep(lsf_scan_kernel<TA, TM, TOut, LSF_TPW, true>, grid_a, LSF_THREADS, 0, stream, p);
    JB_LAUNCH_CHECK("lsf_scan_kernel<ends>");
  }
  dim3 grid((p.D + LSF_CH - 1) / LSF_CH, p.B, p.nseg);
  launch_dep(lsf_scan_kernel<TA, TM, TOut, LSF_TPW, false>, grid, LSF_THREADS, 0, stream, p);
  JB_LAUNCH_CHECK("lsf_scan_kernel");
  return JB200_OK;
}


// ------------------------------------------------------------------------------------------------------------
// TMA-staged scan (scalar decay, bf16 m).  FUSED: resid (f32) += h, no other output.  Otherwise: out (bf16) = h.
// Tensor maps are 3-D (channels, tokens, sequences), so tiles are clipped at the end of a sequence: loads past T
// read zeros (m = 0 leaves the recurrence a pure decay), stores past T are dropped.
// ------------------------------------------------------------------------------------------------------------
constexpr int LT_TOK = LSF_WARPS * 16;       // 128 tokens per tile (= LSF_TILE: the ends pre-pass uses the same tiles)
constexpr int LT_M_BYTES = LT_TOK * LSF_CH * 2;    // 16 KiB
constexpr int LT_R_BYTES = LT_TOK * LSF_CH * 4;    // 32 KiB

template <bool FUSED>
struct LsfTma {
  static constexpr int STAGE_BYTES = LT_M_BYTES + (FUSED ? LT_R_BYTES : 0);
  static constexpr size_t CTL_BYTES = 128 + 2 * LSF_WARPS * 32 * sizeof(float2);   // barriers + flag, run ends
  static constexpr size_t smem_bytes(int stages) { return size_t(stages) * STAGE_BYTES + CTL_BYTES + 128 /* alignment slack */; }
  // Stages: enough CTAs to put two (fused) or three (plain) on every SM -> a short ring each; a grid that leaves
  // SMs with one CTA -> that CTA gets a ring of four stages (and sequences are not cut into segments).
  static constexpr int STAGES_SHARED = FUSED ? 2 : 3;   // plain: four CTAs per SM (64 registers), so 512 CTAs (B=32 x 16 channel tiles) are one wave
  static constexpr int STAGES_ALONE = 4;
};

template <bool FUSED>
__global__ void __launch_bounds__(LSF_THREADS, FUSED ? 2 : 4)
lsf_tma_kernel(const __grid_constant__ CUtensorMap tm_m, const __grid_constant__ CUtensorMap tm_io, const LsfParams p,
               const int n_stages, unsigned int* status) {
  pdl_wait();
  pdl_trigger();
  using Cfg = LsfTma<FUSED>;
  constexpr int TPW = LT_TOK / LSF_WARPS;    // 16 (sixteen warps of 8 tokens were measured: slower)
  extern __shared__ uint8_t lsf_smem_raw[];
  const uint32_t raw_addr = smem_u32(lsf_smem_raw);
  const uint32_t base = (raw_addr + 127u) & ~127u;
  uint8_t* tiles = lsf_smem_raw + (base - raw_addr);
  uint8_t* ctl = tiles + size_t(n_stages) * Cfg::STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(ctl);                       // [STAGES]
  uint32_t* abort_flag = reinterpret_cast<uint32_t*>(ctl + 64);
  float2 (*s_end)[LSF_WARPS][32] = reinterpret_cast<float2 (*)[LSF_WARPS][32]>(ctl + 128);   // [2][8][32]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.y, seg = blockIdx.z;
  const int ch0 = blockIdx.x * LSF_CH;
  const int ch = ch0 + lane * 2;
  const bool ch_ok = ch < p.D;
  const int t_begin = seg * p.seg_len;
  const int t_end = min(p.T, t_begin + p.seg_len);
  const int n_tiles = (t_end - t_begin + LT_TOK - 1) / LT_TOK;

  float alpha;
  if (p.alpha_s) {
    alpha = __ldg(p.alpha_s);
  } else {
    const float z = -__ldg(p.var_scale) * __ldg(p.act_var);
    alpha = p.alpha_min + (p.alpha_max - p.alpha_min) * (1.0f / (1.0f + expf(-z)));
  }
  float pw[TPW];   // alpha^(i+1)
  {
    float a = alpha;
#pragma unroll
    for (int i = 0; i < TPW; ++i) { pw[i] = a; a *= alpha; }
  }
  float2 carry = make_float2(0.f, 0.f);
  if (p.h0 && ch_ok) carry = __ldg(reinterpret_cast<const float2*>(p.h0 + size_t(b) * p.D + ch));
  if (seg > 0 && ch_ok) {   // fold the ends of all earlier tiles (left by the ends pre-pass) into the carry-in
    const float a_tile = expf(float(LT_TOK) * logf(alpha));
    const size_t e0 = (size_t(b) * p.n_pre_tiles) * p.D + ch;
    const int n_before = seg * (p.seg_len / LT_TOK);
    for (int s2 = 0; s2 < n_before; ++s2) {
      const float2 e = __ldg(reinterpret_cast<const float2*>(p.seg_end + e0 + size_t(s2) * p.D));
      carry.x = a_tile * carry.x + e.x;
      carry.y = a_tile * carry.y + e.y;
    }
  }

  auto issue = [&](int i) {      // thread 0 only
    const int s = i % n_stages;
    const uint32_t bar = smem_u32(&full[s]);
    const uint32_t dst = smem_u32(tiles + size_t(s) * Cfg::STAGE_BYTES);
    mbar_arrive_expect_tx(bar, Cfg::STAGE_BYTES);
    tma_load_3d(dst, &tm_m, ch0, t_begin + i * LT_TOK, b, bar);
    if (FUSED) tma_load_3d(dst + LT_M_BYTES, &tm_io, ch0, t_begin + i * LT_TOK, b, bar);
  };
  if (threadIdx.x == 0) {
    for (int s = 0; s < n_stages; ++s) mbar_init(smem_u32(&full[s]), 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_m);
    tma_prefetch_desc(&tm_io);
    for (int i = 0; i < n_stages && i < n_tiles; ++i) issue(i);
  }
  __syncthreads();

  bool ok = true;
  for (int i = 0; i < n_tiles; ++i) {
    const int s = i % n_stages;
    const int buf = i & 1;
    uint8_t* m_tile = tiles + size_t(s) * Cfg::STAGE_BYTES;
    uint8_t* r_tile = m_tile + LT_M_BYTES;
    if (!mbar_wait(smem_u32(&full[s]), uint32_t(i / n_stages) & 1u, abort_flag, status, JB200_STATUS_LSF_LOAD)) ok = false;
    const int tl0 = warp * TPW;                          // first token of this warp's run inside the tile
    const int t0 = t_begin + i * LT_TOK + tl0;
    float2 loc[TPW];
    float2 h = make_float2(0.f, 0.f);
    if (ok) {
#pragma unroll
      for (int j = 0; j < TPW; ++j) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(m_tile + size_t(tl0 + j) * (LSF_CH * 2) + lane * 4);
        h.x = alpha * h.x + (1.0f - alpha) * bf16_lo(w);
        h.y = alpha * h.y + (1.0f - alpha) * bf16_hi(w);
        loc[j] = h;
      }
    }
    s_end[buf][warp][lane] = h;
    if (__syncthreads_or(!ok)) { ok = false; break; }
    // carry into this warp's run, and the carry out of the whole tile (the recurrence is an affine map)
    float2 c = carry, cn = carry;
#pragma unroll
    for (int w = 0; w < LSF_WARPS; ++w) {
      if (w == warp) cn = c;
      const float2 e = s_end[buf][w][lane];
      c.x = pw[TPW - 1] * c.x + e.x;
      c.y = pw[TPW - 1] * c.y + e.y;
    }
    carry = c;
#pragma unroll
    for (int j = 0; j < TPW; ++j) {
      const float hx = loc[j].x + pw[j] * cn.x, hy = loc[j].y + pw[j] * cn.y;
      if (FUSED) {
        float2* r = reinterpret_cast<float2*>(r_tile + size_t(tl0 + j) * (LSF_CH * 4) + lane * 8);
        const float2 old = *r;
        *r = make_float2(old.x + hx, old.y + hy);
      } else {
        *reinterpret_cast<uint32_t*>(m_tile + size_t(tl0 + j) * (LSF_CH * 2) + lane * 4) = pack_bf16x2(hx, hy);
      }
      if (t0 + j == p.T - 1 && p.h_last && ch_ok)
        *reinterpret_cast<float2*>(p.h_last + size_t(b) * p.D + ch) = make_float2(hx, hy);
    }
    fence_proxy_async_smem();        // the tile's new contents -> visible to the TMA store
    __syncthreads();
    if (threadIdx.x == 0) {
      tma_store_3d(&tm_io, ch0, t_begin + i * LT_TOK, b, smem_u32(FUSED ? r_tile : m_tile));
      bulk_commit_group();
      if (n_stages >= 4) {
        // deep ring: refill the stage of the tile BEFORE this one, whose store has had a whole tile's time to read
        // it, so that this thread does not sit out the latency of the store it has just issued
        if (i >= 1 && i - 1 + n_stages < n_tiles) {
          bulk_wait_group_read<1>();
          issue(i - 1 + n_stages);
        }
      } else if (i + n_stages < n_tiles) {
        bulk_wait_group_read<0>();   // the store has read the stage: it may be filled again
        issue(i + n_stages);
      }
    }
  }
  if (threadIdx.x == 0) bulk_wait_group<0>();   // every store has landed before the CTA gives up its shared memory
}

int make_lsf_map(CUtensorMap* tm, const void* ptr, CUtensorMapDataType dt, int elem, int B, int T, int D) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) {
    set_error("lsf_scan: cuTensorMapEncodeTiled entry point not available");
    return JB200_ERR_CUDA;
  }
  const cuuint64_t gdim[3] = {cuuint64_t(D), cuuint64_t(T), cuuint64_t(B)};
  const cuuint64_t gstride[2] = {cuuint64_t(D) * elem, cuuint64_t(T) * D * elem};
  const cuuint32_t box[3] = {cuuint32_t(LSF_CH), cuuint32_t(LT_TOK), 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult cr = fn(tm, dt, 3, const_cast<void*>(ptr), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) {
    set_error("lsf_scan: cuTensorMapEncodeTiled failed (%d)", int(cr));
    return JB200_ERR_CUDA;
  }
  return JB200_OK;
}

template <bool FUSED>
int launch_tma(LsfParams p, cudaStream_t stream) {
  using Cfg = LsfTma<FUSED>;
  const int sms = sm_count();
  if (sms <= 0) return JB200_ERR_CUDA;
  const long ctas = long((p.D + LSF_CH - 1) / LSF_CH) * p.B;
  int stages = Cfg::STAGES_SHARED;
  if (2 * ctas >= sms && ctas <= 2L * sms) {
    // between half a wave and two CTAs per SM: one uncut CTA per (sequence, 64 channels) with a deep ring keeps
    // the SM's loads in flight by itself; cutting T would cost the ends pre-pass (a second read of m, a launch)
    stages = Cfg::STAGES_ALONE;
    p.nseg = 1;
    p.seg_len = (p.T + LT_TOK - 1) / LT_TOK * LT_TOK;
    p.n_pre_tiles = 0;
  }
  CUtensorMap tm_m, tm_io;
  int rc;
  if ((rc = make_lsf_map(&tm_m, p.m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.B, p.T, p.D)) != JB200_OK) return rc;
  if (FUSED) rc = make_lsf_map(&tm_io, p.resid, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.B, p.T, p.D);
  else rc = make_lsf_map(&tm_io, p.out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.B, p.T, p.D);
  if (rc != JB200_OK) return rc;
  unsigned int* status = device_status_ptr();
  if (!status) return JB200_ERR_CUDA;
  if (p.nseg > 1) {
    dim3 grid_a((p.D + LSF_CH - 1) / LSF_CH, p.B, p.n_pre_tiles);
    launch_dep(lsf_scan_kernel<false, __nv_bfloat16, __nv_bfloat16, LSF_TPW, true>, grid_a, LSF_THREADS, 0, stream, p);
    JB_LAUNCH_CHECK("lsf_scan_kernel<ends>");
  }
  dim3 grid((p.D + LSF_CH - 1) / LSF_CH, p.B, p.nseg);
  JB_CUDA(cudaFuncSetAttribute(lsf_tma_kernel<FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               int(Cfg::smem_bytes(Cfg::STAGES_ALONE))));
  launch_dep(lsf_tma_kernel<FUSED>, grid, LSF_THREADS, Cfg::smem_bytes(stages), stream, tm_m, tm_io, p, stages, status);
  JB_LAUNCH_CHECK("lsf_tma_kernel");
  return JB200_OK;
}

// Segments so that about two CTAs per SM exist, each at least four tiles long.
void pick_lsf_segments(int B, int T, int D, int sms, int* seg_len, int* nseg) {
  const long ctas = long((D + LSF_CH - 1) / LSF_CH) * B;
  long want = (2L * sms) / ctas;   // rounded down: all CTAs resident at once, no partial second wave
  const long max_seg = T / (4 * LSF_TILE);
  if (want > max_seg) want = max_seg;
  if (want < 1) want = 1;
  long len = (T + want - 1) / want;
  len = (len + LSF_TILE - 1) / LSF_TILE * LSF_TILE;
  *seg_len = int(len);
  *nseg = int((T + len - 1) / len);
}

}  // namespace

size_t lsf_scan_scratch_bytes(int B, int T, int D) {
  if (B <= 0 || T <= 0 || D <= 0) return 0;
  const int sms = sm_count();
  int len, ns;
  pick_lsf_segments(B, T, D, sms > 0 ? sms : 148, &len, &ns);
  return size_t(2) * B * size_t(ns - 1) * size_t(len / LSF_TILE) * D * sizeof(float);
}

int launch_lsf_scan(const void* m, int m_dtype, const void* alpha_tensor, const float* alpha_scalar,
                    const float* act_var, const float* var_scale, float alpha_min, float alpha_max, const float* h0,
                    float* resid, void* out, int out_dtype, float* h_last, void* scratch, int B, int T, int D,
                    cudaStream_t stream) {
  JB_REQUIRE(B >= 0 && T >= 0 && D > 0, "lsf_scan: bad shape (%d, %d, %d)", B, T, D);
  JB_REQUIRE(D % 2 == 0, "lsf_scan: channel count (%d) must be even", D);
  JB_REQUIRE(B <= 65535, "lsf_scan: batch (%d) exceeds 65535", B);
  JB_REQUIRE((m_dtype == 0 || m_dtype == 1) && (out_dtype == 0 || out_dtype == 1), "lsf_scan: dtype must be 0 (f32) or 1 (bf16)");
  if (B == 0 || T == 0) return JB200_OK;
  JB_REQUIRE(m != nullptr, "lsf_scan: null input");
  JB_REQUIRE(alpha_tensor || alpha_scalar || (act_var && var_scale), "lsf_scan: no decay given");
  JB_REQUIRE(out || resid || h_last, "lsf_scan: no output requested");
  const uintptr_t a8 = 7u, a4 = 3u;
  JB_REQUIRE((reinterpret_cast<uintptr_t>(m) & (m_dtype == 0 ? a8 : a4)) == 0, "lsf_scan: input pointer misaligned");
  JB_REQUIRE(!alpha_tensor || (reinterpret_cast<uintptr_t>(alpha_tensor) & (m_dtype == 0 ? a8 : a4)) == 0, "lsf_scan: alpha pointer misaligned");
  JB_REQUIRE(!out || (reinterpret_cast<uintptr_t>(out) & (out_dtype == 0 ? a8 : a4)) == 0, "lsf_scan: output pointer misaligned");
  JB_REQUIRE(!resid || (reinterpret_cast<uintptr_t>(resid) & a8) == 0, "lsf_scan: residual pointer misaligned");
  JB_REQUIRE((!h0 || (reinterpret_cast<uintptr_t>(h0) & a8) == 0) && (!h_last || (reinterpret_cast<uintptr_t>(h_last) & a8) == 0),
             "lsf_scan: state pointer misaligned");
  LsfParams p;
  p.m = m; p.alpha_t = alpha_tensor; p.alpha_s = alpha_scalar; p.act_var = act_var; p.var_scale = var_scale;
  p.alpha_min = alpha_min; p.alpha_max = alpha_max; p.h0 = h0; p.resid = resid; p.out = out; p.h_last = h_last;
  p.B = B; p.T = T; p.D = D;
  p.seg_len = (T + LSF_TILE - 1) / LSF_TILE * LSF_TILE;
  p.nseg = 1;
  p.n_pre_tiles = 0;
  p.seg_end = p.seg_prod = nullptr;
  if (scratch) {
    JB_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & a8) == 0, "lsf_scan: scratch pointer misaligned");
    const int sms = sm_count();
    if (sms <= 0) return JB200_ERR_CUDA;
    pick_lsf_segments(B, T, D, sms, &p.seg_len, &p.nseg);
    p.n_pre_tiles = (p.nseg - 1) * (p.seg_len / LSF_TILE);
    p.seg_end = reinterpret_cast<float*>(scratch);
    p.seg_prod = p.seg_end + size_t(B) * p.n_pre_tiles * D;
  }
  JB_REQUIRE(p.nseg <= 65535 && p.n_pre_tiles <= 65535, "lsf_scan: too many segments");
  const bool ta = alpha_tensor != nullptr;
  using bf = __nv_bfloat16;
  // the forms the model and the scan sweep run: tiles by TMA (3-D maps need 16-byte aligned rows)
  if (!ta && m_dtype == 1 && T > 8 && D % 8 == 0 && aligned16(m) && B * long(T) * D < (1L << 40)) {
    if (resid && !out && aligned16(resid)) return launch_tma<true>(p, stream);
    if (out && !resid && out_dtype == 1 && aligned16(out)) return launch_tma<false>(p, stream);
  }
  if (!ta) {
    if (m_dtype == 1 && out_dtype == 1) return launch_t<false, bf, bf>(p, stream);
    if (m_dtype == 1 && out_dtype == 0) return launch_t<false, bf, float>(p, stream);
    if (m_dtype == 0 && out_dtype == 0) return launch_t<false, float, float>(p, stream);
    return launch_t<false, float, bf>(p, stream);
  }
  if (m_dtype == 1 && out_dtype == 1) return launch_t<true, bf, bf>(p, stream);
  if (m_dtype == 1 && out_dtype == 0) return launch_t<true, bf, float>(p, stream);
  if (m_dtype == 0 && out_dtype == 0) return launch_t<true, float, float>(p, stream);
  return launch_t<true, float, bf>(p, stream);
}

int launch_lsf_step_norm(const void* m_bf16, const double* stats, const double* probs_sum, const int* top1_hist, int E,
                         long long n_tokens, long long n_elems, float balance_alpha, float* scalars,
                         const float* var_scale, float alpha_min, float alpha_max, const float* h_in, float* h_out,
                         float* x, const float* w_norm, float eps, void* xn_bf16, int B, int C, cudaStream_t stream) {
  JB_REQUIRE(B >= 0 && C > 0, "lsf_step_norm: bad shape (%d, %d)", B, C);
  JB_REQUIRE(C % 8 == 0 && C <= 1024, "lsf_step_norm: d_model (%d) must be a multiple of 8 and at most 1024", C);
  JB_REQUIRE(E >= 0 && E <= 64 && n_tokens > 0 && n_elems > 0, "lsf_step_norm: bad counts");
  if (B == 0) return JB200_OK;
  JB_REQUIRE(m_bf16 && stats && scalars && var_scale && h_out && x, "lsf_step_norm: null pointer");
  JB_REQUIRE((w_norm == nullptr) == (xn_bf16 == nullptr), "lsf_step_norm: norm weight and normalised output come together");
  JB_REQUIRE(aligned16(m_bf16) && aligned16(h_out) && aligned16(x) && (!h_in || aligned16(h_in)) &&
                 (!w_norm || (aligned16(w_norm) && aligned16(xn_bf16))),
             "lsf_step_norm: pointers must be 16-byte aligned");
  LsfStepParams p;
  p.m = reinterpret_cast<const __nv_bfloat16*>(m_bf16);
  p.stats = stats; p.probs_sum = probs_sum; p.top1_hist = top1_hist; p.E = E;
  p.n_tokens = n_tokens; p.n_elems = n_elems; p.balance_alpha = balance_alpha; p.scalars = scalars;
  p.var_scale = var_scale; p.alpha_min = alpha_min; p.alpha_max = alpha_max;
  p.h_in = h_in; p.h_out = h_out; p.x = x; p.w_norm = w_norm; p.eps = eps;
  p.xn = reinterpret_cast<__nv_bfloat16*>(xn_bf16);
  p.B = B; p.C = C;
  launch_dep(lsf_step_norm_kernel, (B + 7) / 8, 256, 0, stream, p);
  JB_LAUNCH_CHECK("lsf_step_norm_kernel");
  return JB200_OK;
}

}  // namespace jb
