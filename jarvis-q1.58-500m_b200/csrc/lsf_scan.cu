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
#include "common.cuh"
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
    else alpha = p.alpha_min + (p.alpha_max - p.alpha_min) * (1.0f / (1.0f + expf(__ldg(p.var_scale) * __ldg(p.act_var))));
  }
  float2 h = p.h0 ? *reinterpret_cast<const float2*>(p.h0 + size_t(b) * p.D + ch) : make_float2(0.f, 0.f);
  for (int t = 0; t < p.T; ++t) {
    const size_t o = (size_t(b) * p.T + t) * p.D + ch;
    const float2 mv = ld2<TM>(m + o);
    float2 a = make_float2(alpha, alpha);
    if (TENSOR_ALPHA) a = ld2<TM>(at + o);
    h.x = a.x * h.x + (1.0f - a.x) * mv.x;
    h.y = a.y * h.y + (1.0f - a.y) * mv.y;
    if (out) st2<TOut>(out + o, h.x, h.y);
    if (p.resid) {
      float2* r = reinterpret_cast<float2*>(p.resid + o);
      const float2 rv = *r;
      *r = make_float2(rv.x + h.x, rv.y + h.y);
    }
  }
  if (p.h_last) *reinterpret_cast<float2*>(p.h_last + size_t(b) * p.D + ch) = h;
}

constexpr int LSF_TPW = 16;                       // tokens per warp per tile
constexpr int LSF_TILE = LSF_WARPS * LSF_TPW;     // 128 tokens

template <bool TA, typename TM, typename TOut>
int launch_t(const LsfParams& p, cudaStream_t stream) {
  if (p.T <= 8) {
    const size_t pairs = size_t(p.B) * (p.D / 2);
    lsf_short_kernel<TA, TM, TOut><<<unsigned((pairs + 255) / 256), 256, 0, stream>>>(p);
    JB_LAUNCH_CHECK("lsf_short_kernel");
    return JB200_OK;
  }
  if (p.nseg > 1) {
    dim3 grid_a((p.D + LSF_CH - 1) / LSF_CH, p.B, p.n_pre_tiles);
    lsf_scan_kernel<TA, TM, TOut, LSF_TPW, true><<<grid_a, LSF_THREADS, 0, stream>>>(p);
    JB_LAUNCH_CHECK("lsf_scan_kernel<ends>");
  }
  dim3 grid((p.D + LSF_CH - 1) / LSF_CH, p.B, p.nseg);
  lsf_scan_kernel<TA, TM, TOut, LSF_TPW, false><<<grid, LSF_THREADS, 0, stream>>>(p);
  JB_LAUNCH_CHECK("lsf_scan_kernel");
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

}  // namespace jb
