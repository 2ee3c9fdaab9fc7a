// Scalar-decay associative linear-attention causal scan, fused with its prologue.
//
//   q <- (ELU(q)+1)/sqrt(D),  k <- ELU(k)+1,  half-split RoPE on both   (jarvis_model.py:124-128, :29-71;
//                                                                      fused kernel A1, associative_attention_cuda.cu:28-112)
//   S_t = gamma*S_{t-1} + v_t (x) k_t,   o_t = S_t q_t                  (jarvis_model.py:131-190)
//   optional initial state S_in and final state S_out (B, H, D_v, D_k)  (associative_attention.py:126-152, :273-308;
//                                                                      kernel A3, associative_attention_cuda.cu:218-265)
//
// One CTA per (sequence, head, segment) walks its part of the sequence in 64-token chunks.  The state S never leaves
// the SM: it is carried in fp32 accumulator registers (one 16-row band per warp) and mirrored
// as bf16 in shared memory for the cross-chunk product, so HBM traffic is the algorithmic
// q, k, v in / o out (512 B per token-head) plus one optional state load/store per sequence-head.
// The reference's chunk-parallel path instead materialises per-chunk states (B,H,T/64,64,64) twice.
//
// Per chunk (c <= 64 tokens, decay tables for the actual c):
//   TMA (128B-swizzled boxes; one stage, four CTAs per SM cover each other's latency)  ->  q, k, v tiles in smem
//   all threads: feature map + RoPE in place on q, k;  Vw = v * gamma^(c-1-j)
//   warp w (query rows 16w..16w+15), tensor cores via mma.sync m16n8k16 bf16 -> fp32:
//     O  = (Q S^T) * gamma^(i+1)                 cross-chunk
//     A  = (Q K^T) o gamma^(i-j) [j <= i]         only the causal n-tiles are computed
//     O += A V                                    intra-chunk
//   warp w (state rows dv 16w..16w+15):  S = gamma^c S + Vw^T K
//
// Sequence segments: when B*H alone cannot fill the GPU (prefill of a few long sequences), T is cut
// into segments.  A first launch (STATE_ONLY) runs only the k/v half of the work for every non-final
// segment from a zero state and stores its contribution D_s; the main launch starts segment s from
// S = fold_{s' < s}(gamma^L S + D_s'), which is exact because the recurrence is linear in S.
// Extra HBM traffic: k and v are read twice (the second time mostly from L2).
#include "common.cuh"
#include "launchers.h"

namespace jb {

namespace {

constexpr int D = 64;             // head dim (fixed by the path: 16 heads x 64)
constexpr int CH = 64;            // chunk length, AssociativeLinearAttention.CHUNK_SIZE
constexpr int STAGES = 1;             // 49 KiB of shared memory and 128 registers per CTA -> four CTAs per SM, which cover each other's load latency
constexpr int TILE_BYTES = CH * D * 2;          // 8 KiB
constexpr int STAGE_BYTES = 3 * TILE_BYTES;     // q, k, v
constexpr int ATTN_THREADS = 128;

struct AttnParams {
  const float* gamma;      // [H] decay in (0,1)
  const float* cos_tab;    // [n_pos][32]
  const float* sin_tab;    // [n_pos][32]
  const int32_t* pos0;     // [B] first position of each sequence, or null (use pos0_scalar)
  int pos0_scalar;
  int n_pos;
  const float* s_in;       // [B][H][64][64] or null
  float* s_out;            // [B][H][64][64] or null
  __nv_bfloat16* o;        // [B*T][ld_o], head h at columns h*64
  int ld_o;
  int B, T, H;
  int seg_chunks;          // chunks per sequence segment (grid.z walks the segments)
  int nseg;
  float* seg_state;        // [B][H][nseg-1][64][64]: state contribution of each non-final segment
  int n_pieces;            // state contributions stored per (sequence, head): nseg - 1, or nseg in a state-only call
  int qk_prepared;         // q, k already hold phi(.) + RoPE with the head dim interleaved (d, d+32 adjacent)
  unsigned int* status;
};

struct Smem {
  uint8_t tiles[STAGES][STAGE_BYTES];  // [stage][q|k|v][64 rows x 128 B, 128B-swizzled]
  uint8_t vw[TILE_BYTES];              // v * gamma^(c-1-j)
  uint8_t s_bf16[2][TILE_BYTES];       // state mirror [dv][dk], double buffered
  float pw[CH + 1];                    // gamma^n
  float4 mf[8][32];                    // decay-mask factors of one 16x8 score tile, by (2*warp - key_tile + 1, lane)
  uint64_t full[STAGES];
  uint64_t full_b;                     // k/v-only pass: barrier of its second stage (the state-mirror buffers)
  uint32_t abort_flag;
};

constexpr size_t ATTN_SMEM_BYTES = sizeof(Smem) + 1024;

__device__ __forceinline__ uint32_t swz(int row, int chunk16) {  // byte offset inside a swizzled 64x128B tile
  return uint32_t(row) * 128u + (uint32_t(chunk16 ^ (row & 7)) << 4);
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ELU(x)+1 = x+1 for x > 0, exp(x) otherwise; branch-free, exp through ex2.approx (rel. error 2^-22,
// far below the bf16 rounding of the result).  For large positive x the unused exp is +inf, never NaN.
__device__ __forceinline__ float elu1(float x) { return x > 0.f ? x + 1.0f : __expf(x); }

template <bool STATE_ONLY>
__global__ void __launch_bounds__(ATTN_THREADS, 4)
attn_scan_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  Smem* sm = reinterpret_cast<Smem*>(smem_raw + (base - raw_addr));

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.x, b = blockIdx.y;
  const int T = p.T;
  const int n_chunks = (T + CH - 1) / CH;
  const int seg = blockIdx.z;
  const int ck_begin = seg * p.seg_chunks;
  const int ck_end = min(n_chunks, ck_begin + p.seg_chunks);
  const int row0 = b * T;                       // first row of this sequence in the (B*T, ld) matrices
  const int pos_base = p.pos0 ? p.pos0[b] : p.pos0_scalar;
  const float gamma = __ldg(p.gamma + h);
  const float log_g = logf(gamma);

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) mbar_init(smem_u32(&sm->full[s]), 1);
    mbar_init(smem_u32(&sm->full_b), 1);
    sm->abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  for (int n = tid; n <= CH; n += ATTN_THREADS) sm->pw[n] = expf(log_g * float(n));
  for (int e = tid; e < 8 * 32; e += ATTN_THREADS) {
    const int d = e >> 5, ln = e & 31;
    const int diff0 = 8 * (d - 1) + (ln >> 2) - 2 * (ln & 3);   // query row - key column of c0
    // gamma^(i-j) / sqrt(D): the 1/8 of the query feature map is a power of two, so applying it to the scores
    // (here and in the cross-chunk factor below) instead of to every element of q gives the same bits
    auto fac = [&](int x) { return x >= 0 ? 0.125f * expf(log_g * float(x)) : 0.f; };
    sm->mf[d][ln] = make_float4(fac(diff0), fac(diff0 - 1), fac(diff0 + 8), fac(diff0 + 7));
  }

  // state: fp32 accumulators, rows dv = 16*warp + lane/4 (+8), cols dk = 8*nt + 2*(lane%4) (+1)
  float S[8][4];
  {
    const int r = 16 * warp + (lane >> 2);
    const int cb = 2 * (lane & 3);
    const float* sin_p = (!STATE_ONLY && p.s_in) ? p.s_in + (size_t(b) * p.H + h) * D * D : nullptr;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int c = nt * 8 + cb;
      if (sin_p && p.qk_prepared) {
        // the kernel's dk axis is the interleaved one (column 2i = feature i, 2i + 1 = feature i + 32);
        // states cross the API in the natural order
        const int d = c >> 1;
        S[nt][0] = __ldg(sin_p + r * D + d);        S[nt][1] = __ldg(sin_p + r * D + d + 32);
        S[nt][2] = __ldg(sin_p + (r + 8) * D + d);  S[nt][3] = __ldg(sin_p + (r + 8) * D + d + 32);
      } else if (sin_p) {
        const float2 lo = __ldg(reinterpret_cast<const float2*>(sin_p + r * D + c));
        const float2 hi = __ldg(reinterpret_cast<const float2*>(sin_p + (r + 8) * D + c));
        S[nt][0] = lo.x; S[nt][1] = lo.y; S[nt][2] = hi.x; S[nt][3] = hi.y;
      } else {
        S[nt][0] = S[nt][1] = S[nt][2] = S[nt][3] = 0.f;
      }
      if (!STATE_ONLY && seg > 0) {
        // state entering this segment: fold the earlier segments' contributions, oldest first
        const float gL = expf(log_g * float(p.seg_chunks * CH));
        const float* dp = p.seg_state + (size_t(b) * p.H + h) * p.n_pieces * D * D;
        for (int s2 = 0; s2 < seg; ++s2, dp += D * D) {
          const float2 lo = __ldg(reinterpret_cast<const float2*>(dp + r * D + c));
          const float2 hi = __ldg(reinterpret_cast<const float2*>(dp + (r + 8) * D + c));
          S[nt][0] = gL * S[nt][0] + lo.x; S[nt][1] = gL * S[nt][1] + lo.y;
          S[nt][2] = gL * S[nt][2] + hi.x; S[nt][3] = gL * S[nt][3] + hi.y;
        }
      }
      if (!STATE_ONLY) {
        *reinterpret_cast<uint32_t*>(sm->s_bf16[0] + swz(r, c >> 3) + (c & 7) * 2) = pack_bf16x2(S[nt][0], S[nt][1]);
        *reinterpret_cast<uint32_t*>(sm->s_bf16[0] + swz(r + 8, c >> 3) + (c & 7) * 2) = pack_bf16x2(S[nt][2], S[nt][3]);
      }
    }
  }
  __syncthreads();

  // The k/v-only pass has no use for the q tile and the state mirror, so it runs two stages: k, v of odd
  // chunks land in the two mirror buffers (16 KiB, 1024-byte aligned like the tiles) under their own barrier.
  constexpr int N_ST = STATE_ONLY ? 2 : STAGES;
  auto issue_chunk = [&](int ck) {  // called by thread 0 only
    const int s = (ck - ck_begin) % N_ST;
    const bool second = STATE_ONLY && s == 1;
    const uint32_t bar = smem_u32(second ? &sm->full_b : &sm->full[STATE_ONLY ? 0 : s]);
    mbar_arrive_expect_tx(bar, STATE_ONLY ? 2 * TILE_BYTES : STAGE_BYTES);
    const uint32_t dst = smem_u32(sm->tiles[STATE_ONLY ? 0 : s]);
    const int r = row0 + ck * CH;
    if (!STATE_ONLY) tma_load_2d(dst, &tm_q, h * D, r, bar);
    tma_load_2d(second ? smem_u32(sm->s_bf16[0]) : dst + TILE_BYTES, &tm_k, h * D, r, bar);
    tma_load_2d(second ? smem_u32(sm->s_bf16[1]) : dst + 2 * TILE_BYTES, &tm_v, h * D, r, bar);
  };
  if (tid == 0) {
    for (int ck = ck_begin; ck < ck_begin + N_ST && ck < ck_end; ++ck) issue_chunk(ck);
  }

  const uint32_t vw_a = smem_u32(sm->vw);
  bool ok = true;
  for (int ck = ck_begin; ck < ck_end; ++ck) {
    const int lc = ck - ck_begin;
    const int s = lc % N_ST;
    const bool second = STATE_ONLY && s == 1;
    const int c_len = min(CH, T - ck * CH);
    uint8_t* q_p = sm->tiles[STATE_ONLY ? 0 : s];
    uint8_t* k_p = second ? sm->s_bf16[0] : q_p + TILE_BYTES;
    uint8_t* v_p = second ? sm->s_bf16[1] : q_p + 2 * TILE_BYTES;
    const uint32_t q_a = smem_u32(q_p), k_a = smem_u32(k_p), v_a = smem_u32(v_p);
    const uint32_t sb_a = smem_u32(sm->s_bf16[lc & 1]);
    uint8_t* sb_next = sm->s_bf16[(lc + 1) & 1];

    if (!mbar_wait(smem_u32(second ? &sm->full_b : &sm->full[STATE_ONLY ? 0 : s]), uint32_t(lc / N_ST) & 1u,
                   &sm->abort_flag, p.status, JB200_STATUS_ATTN_LOAD)) {
      ok = false;
    }
    if (__syncthreads_or(!ok)) break;   // leave together if any thread's wait ran out

    // ---- prologue: feature map + RoPE on q and k (pairs d, d+32), Vw = v * gamma^(c-1-j) ----------
    // 64 rows x 4 column groups of 8; 2 items per thread
#pragma unroll
    for (int it = 0; it < (p.qk_prepared ? 0 : 2); ++it) {
      const int item = tid + it * ATTN_THREADS;
      const int r = item >> 2, cg = item & 3;   // token row, 16-byte chunk in the first half
      int pos = pos_base + ck * CH + r;
      pos = pos < 0 ? 0 : (pos >= p.n_pos ? p.n_pos - 1 : pos);
      float cs[8], sn[8];
      {
        const float4* cp = reinterpret_cast<const float4*>(p.cos_tab + size_t(pos) * 32 + cg * 8);
        const float4* sp = reinterpret_cast<const float4*>(p.sin_tab + size_t(pos) * 32 + cg * 8);
        const float4 c0 = __ldg(cp), c1 = __ldg(cp + 1), s0 = __ldg(sp), s1 = __ldg(sp + 1);
        cs[0] = c0.x; cs[1] = c0.y; cs[2] = c0.z; cs[3] = c0.w; cs[4] = c1.x; cs[5] = c1.y; cs[6] = c1.z; cs[7] = c1.w;
        sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
      }
#pragma unroll
      for (int which = STATE_ONLY ? 1 : 0; which < 2; ++which) {  // 0: q, 1: k
        uint8_t* tp = which == 0 ? q_p : k_p;
        uint4* lo_p = reinterpret_cast<uint4*>(tp + swz(r, cg));
        uint4* hi_p = reinterpret_cast<uint4*>(tp + swz(r, cg + 4));
        const uint4 lo = *lo_p, hi = *hi_p;
        const uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w}, hw[4] = {hi.x, hi.y, hi.z, hi.w};
        uint32_t ol[4], oh[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float a0 = elu1(bf16_lo(lw[j])), a1 = elu1(bf16_hi(lw[j]));   // d
          const float b0 = elu1(bf16_lo(hw[j])), b1 = elu1(bf16_hi(hw[j]));   // d + 32
          // x*cos + rotate_half(x)*sin:  out[d] = x[d]cos - x[d+32]sin,  out[d+32] = x[d+32]cos + x[d]sin
          ol[j] = pack_bf16x2(a0 * cs[2 * j] - b0 * sn[2 * j], a1 * cs[2 * j + 1] - b1 * sn[2 * j + 1]);
          oh[j] = pack_bf16x2(b0 * cs[2 * j] + a0 * sn[2 * j], b1 * cs[2 * j + 1] + a1 * sn[2 * j + 1]);
        }
        *lo_p = make_uint4(ol[0], ol[1], ol[2], ol[3]);
        *hi_p = make_uint4(oh[0], oh[1], oh[2], oh[3]);
      }
    }
    // Vw: 64 rows x 8 chunks = 512 items, 4 per thread
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int item = tid + it * ATTN_THREADS;
      const int r = item >> 3, cg = item & 7;
      const float w = r < c_len ? sm->pw[c_len - 1 - r] : 0.f;   // rows past the end contribute nothing
      const uint4 v = *reinterpret_cast<const uint4*>(v_p + swz(r, cg));
      *reinterpret_cast<uint4*>(sm->vw + swz(r, cg)) =
          make_uint4(pack_bf16x2(bf16_lo(v.x) * w, bf16_hi(v.x) * w), pack_bf16x2(bf16_lo(v.y) * w, bf16_hi(v.y) * w),
                     pack_bf16x2(bf16_lo(v.z) * w, bf16_hi(v.z) * w), pack_bf16x2(bf16_lo(v.w) * w, bf16_hi(v.w) * w));
    }
    __syncthreads();

    if (!STATE_ONLY) {
    // ---- Q fragments of this warp's 16 rows (A operand, 4 k-steps over d) ---------------------------
    uint32_t qf[4][4];
    {
      const int r = 16 * warp + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) ldsm_x4(q_a + swz(r, 2 * ks + (lane >> 4)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }
    const int i_lo = 16 * warp + (lane >> 2);   // query row of c0,c1 ; c2,c3 are row i_lo + 8
    const int i_hi = i_lo + 8;

    // ---- cross-chunk: O = (Q S^T) * gamma^(i+1);  B[k=dk][n=dv] = S[dv][dk] -------------------------
    float O[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      O[nt][0] = O[nt][1] = O[nt][2] = O[nt][3] = 0.f;
      uint32_t bfr[8];
      const int r = nt * 8 + (lane & 7);
      ldsm_x4(sb_a + swz(r, (lane >> 3)), bfr[0], bfr[1], bfr[2], bfr[3]);       // dk 0..31
      ldsm_x4(sb_a + swz(r, 4 + (lane >> 3)), bfr[4], bfr[5], bfr[6], bfr[7]);   // dk 32..63
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) mma16816(O[nt], qf[ks], bfr[2 * ks], bfr[2 * ks + 1]);
    }
    {
      const float g_lo = 0.125f * sm->pw[min(i_lo + 1, CH)], g_hi = 0.125f * sm->pw[min(i_hi + 1, CH)];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) { O[nt][0] *= g_lo; O[nt][1] *= g_lo; O[nt][2] *= g_hi; O[nt][3] *= g_hi; }
    }

    // ---- intra-chunk: scores over the causal key tiles, decay mask, then P V ---------------------------
    uint32_t pf[4][4];              // P as A fragments: k-step kj covers keys 16kj..16kj+15
#pragma unroll
    for (int kj = 0; kj < 4; ++kj) {
      if (kj <= warp) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int jt = 2 * kj + half;
          float sc[4] = {0.f, 0.f, 0.f, 0.f};
          uint32_t bfr[8];
          const int r = jt * 8 + (lane & 7);
          ldsm_x4(k_a + swz(r, (lane >> 3)), bfr[0], bfr[1], bfr[2], bfr[3]);
          ldsm_x4(k_a + swz(r, 4 + (lane >> 3)), bfr[4], bfr[5], bfr[6], bfr[7]);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) mma16816(sc, qf[ks], bfr[2 * ks], bfr[2 * ks + 1]);
          const float4 f = sm->mf[2 * warp - jt + 1][lane];   // gamma^(i-j) for j <= i, else 0
          sc[0] *= f.x; sc[1] *= f.y; sc[2] *= f.z; sc[3] *= f.w;
          pf[kj][2 * half + 0] = pack_bf16x2(sc[0], sc[1]);
          pf[kj][2 * half + 1] = pack_bf16x2(sc[2], sc[3]);
        }
      }
    }

    // O += P V ;  B[k=j][n=dv] = V[j][dv]  (transposed load)
#pragma unroll
    for (int kj = 0; kj < 4; ++kj) {
      if (kj <= warp) {
        const int r = 16 * kj + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
        for (int np = 0; np < 4; ++np) {  // pairs of dv n-tiles
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(v_a + swz(r, 2 * np + (lane >> 4)), b0, b1, b2, b3);
          mma16816(O[2 * np], pf[kj], b0, b1);
          mma16816(O[2 * np + 1], pf[kj], b2, b3);
        }
      }
    }

    // ---- output: stage this warp's 16 rows in its own (already consumed) q rows, then 16-byte stores ------
    __syncwarp();
    {
      const int r = 16 * warp + (lane >> 2);
      const int cb = 2 * (lane & 3);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int c = nt * 8 + cb;
        *reinterpret_cast<uint32_t*>(q_p + swz(r, c >> 3) + (c & 7) * 2) = pack_bf16x2(O[nt][0], O[nt][1]);
        *reinterpret_cast<uint32_t*>(q_p + swz(r + 8, c >> 3) + (c & 7) * 2) = pack_bf16x2(O[nt][2], O[nt][3]);
      }
    }
    __syncwarp();
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int rr = 16 * warp + it * 4 + (lane >> 3), cg = lane & 7;
      if (rr < c_len) {
        const uint4 v = *reinterpret_cast<const uint4*>(q_p + swz(rr, cg));
        *reinterpret_cast<uint4*>(p.o + size_t(row0 + ck * CH + rr) * p.ld_o + h * D + cg * 8) = v;
      }
    }
    }  // !STATE_ONLY

    // ---- state update: S = gamma^c S + Vw^T K ;  A[m=dv][k=j] = Vw[j][dv], B[k=j][n=dk] = K[j][dk] -------
    {
      const float gc = sm->pw[c_len];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) { S[nt][0] *= gc; S[nt][1] *= gc; S[nt][2] *= gc; S[nt][3] *= gc; }
#pragma unroll
      for (int kj = 0; kj < 4; ++kj) {
        uint32_t af[4];
        {
          const int r = 16 * kj + (lane & 7) + 8 * (lane >> 4);
          ldsm_x4_t(vw_a + swz(r, 2 * warp + ((lane >> 3) & 1)), af[0], af[1], af[2], af[3]);
        }
        const int r = 16 * kj + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(k_a + swz(r, 2 * np + (lane >> 4)), b0, b1, b2, b3);
          mma16816(S[2 * np], af, b0, b1);
          mma16816(S[2 * np + 1], af, b2, b3);
        }
      }
      // publish the bf16 mirror for the next chunk's cross term (a k/v-only pass has none)
      if (!STATE_ONLY) {
        const int r = 16 * warp + (lane >> 2);
        const int cb = 2 * (lane & 3);
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          const int c = nt * 8 + cb;
          *reinterpret_cast<uint32_t*>(sb_next + swz(r, c >> 3) + (c & 7) * 2) = pack_bf16x2(S[nt][0], S[nt][1]);
          *reinterpret_cast<uint32_t*>(sb_next + swz(r + 8, c >> 3) + (c & 7) * 2) = pack_bf16x2(S[nt][2], S[nt][3]);
        }
      }
    }

    fence_proxy_async_smem();  // order this thread's generic accesses to stage s before the next TMA write into it
    __syncthreads();  // tiles of stage s and vw are free; the new state mirror is complete
    if (tid == 0 && ck + N_ST < ck_end) issue_chunk(ck + N_ST);
  }

  float* so = nullptr;
  if (STATE_ONLY) so = p.seg_state + ((size_t(b) * p.H + h) * p.n_pieces + seg) * D * D;
  else if (p.s_out && seg == p.nseg - 1) so = p.s_out + (size_t(b) * p.H + h) * D * D;
  if (ok && so) {
    const int r = 16 * warp + (lane >> 2);
    const int cb = 2 * (lane & 3);
    const bool natural = !STATE_ONLY && p.qk_prepared;   // segment contributions stay in the kernel's own order
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int c = nt * 8 + cb;
      if (natural) {
        const int d = c >> 1;
        so[r * D + d] = S[nt][0];        so[r * D + d + 32] = S[nt][1];
        so[(r + 8) * D + d] = S[nt][2];  so[(r + 8) * D + d + 32] = S[nt][3];
      } else {
        *reinterpret_cast<float2*>(so + r * D + c) = make_float2(S[nt][0], S[nt][1]);
        *reinterpret_cast<float2*>(so + (r + 8) * D + c) = make_float2(S[nt][2], S[nt][3]);
      }
    }
  }
}

// State-only calls (no output rows wanted): every piece of the sequence has left its contribution D_s, scanned
// from a zero state, in seg_state; the state after the whole sequence is
//   S = gamma^T S_in + sum_s gamma^(T - end_s) D_s,      end_s = last token of piece s + 1.
// One CTA per (head, sequence), 16 elements per thread.  The pieces are in the kernel's own column order
// (interleaved when q/k were prepared); s_in / s_out use the natural one.
__global__ void __launch_bounds__(256) attn_fold_states_kernel(const AttnParams p) {
  const int h = blockIdx.x, b = blockIdx.y;
  const float log_g = logf(__ldg(p.gamma + h));
  const int L = p.seg_chunks * CH;
  const size_t bh = size_t(b) * p.H + h;
  for (int e = threadIdx.x; e < D * D; e += 256) {
    const int r = e >> 6, d = e & 63;
    const int col = p.qk_prepared ? (2 * (d & 31) + (d >> 5)) : d;
    float acc = p.s_in ? expf(log_g * float(p.T)) * __ldg(p.s_in + bh * D * D + e) : 0.f;
    for (int s2 = 0; s2 < p.n_pieces; ++s2) {
      const int end = min((s2 + 1) * L, p.T);
      acc += expf(log_g * float(p.T - end)) * __ldg(p.seg_state + (bh * p.n_pieces + s2) * D * D + r * D + col);
    }
    p.s_out[bh * D * D + e] = acc;
  }
}

// One-token step (decode): S <- gamma*S + v (x) k', o = S q' for every (sequence, head).  Pure state
// streaming: 2 x 16 KiB of fp32 state per (sequence, head) against 384 B of q, k, v, so the kernel is a
// coalesced read-modify-write of S with the feature map + RoPE of the single token done in shared memory.
// Thread t owns state row t/4, columns 16*(t%4)..+15; s_out may alias s_in.
__global__ void __launch_bounds__(256)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                   const __nv_bfloat16* __restrict__ v, int ld_qkv, const AttnParams p) {
  __shared__ float sq[D], sk[D], sv[D], rq[D], rk[D];
  const int h = blockIdx.x, b = blockIdx.y, t = threadIdx.x;
  const float gamma = __ldg(p.gamma + h);
  if (t < D) {
    const size_t off = size_t(b) * ld_qkv + h * D + t;
    sq[t] = elu1(__bfloat162float(q[off])) * 0.125f;
    sk[t] = elu1(__bfloat162float(k[off]));
    sv[t] = __bfloat162float(v[off]);
  }
  __syncthreads();
  if (t < D / 2) {
    int pos = p.pos0 ? p.pos0[b] : p.pos0_scalar;
    pos = pos < 0 ? 0 : (pos >= p.n_pos ? p.n_pos - 1 : pos);
    const float c = __ldg(p.cos_tab + size_t(pos) * 32 + t), sn = __ldg(p.sin_tab + size_t(pos) * 32 + t);
    rq[t] = sq[t] * c - sq[t + 32] * sn;  rq[t + 32] = sq[t + 32] * c + sq[t] * sn;
    rk[t] = sk[t] * c - sk[t + 32] * sn;  rk[t + 32] = sk[t + 32] * c + sk[t] * sn;
  }
  __syncthreads();
  const int row = t >> 2, c0 = (t & 3) * 16;
  const size_t so = (size_t(b) * p.H + h) * D * D + size_t(row) * D + c0;
  const float vr = sv[row];
  float acc = 0.f;
  float4 st[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    st[i] = p.s_in ? *reinterpret_cast<const float4*>(p.s_in + so + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
    const int c = c0 + 4 * i;
    st[i].x = gamma * st[i].x + vr * rk[c];      st[i].y = gamma * st[i].y + vr * rk[c + 1];
    st[i].z = gamma * st[i].z + vr * rk[c + 2];  st[i].w = gamma * st[i].w + vr * rk[c + 3];
    acc += st[i].x * rq[c] + st[i].y * rq[c + 1] + st[i].z * rq[c + 2] + st[i].w * rq[c + 3];
  }
  if (p.s_out) {
#pragma unroll
    for (int i = 0; i < 4; ++i) *reinterpret_cast<float4*>(p.s_out + so + 4 * i) = st[i];
  }
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  if ((t & 3) == 0) p.o[size_t(b) * p.ld_o + h * D + row] = __float2bfloat16_rn(acc);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_map(CUtensorMap* tm, const void* ptr, int rows, int cols, int ld) {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      set_error("attn_scan: cuTensorMapEncodeTiled entry point not available");
      return JB200_ERR_CUDA;
    }
    fn = reinterpret_cast<EncodeTiledFn>(f);
  }
  const cuuint64_t gdim[2] = {cuuint64_t(cols), cuuint64_t(rows)};
  const cuuint64_t gstride[1] = {cuuint64_t(ld) * 2};
  const cuuint32_t box[2] = {cuuint32_t(D), cuuint32_t(CH)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult cr = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) {
    set_error("attn_scan: cuTensorMapEncodeTiled failed (%d)", int(cr));
    return JB200_ERR_CUDA;
  }
  return JB200_OK;
}

}  // namespace

// Segments: enough CTAs to fill three per SM, each segment at least four chunks long.
static void pick_segments(int B, int T, int H, int sms, int* seg_chunks, int* nseg) {
  const int n_chunks = (T + CH - 1) / CH;
  long want = (long(sms) * 4) / (long(B) * H);
  if (want < 1) want = 1;
  if (want > n_chunks / 4) want = n_chunks / 4 > 0 ? n_chunks / 4 : 1;
  int sc = int((n_chunks + want - 1) / want);
  *seg_chunks = sc;
  *nseg = (n_chunks + sc - 1) / sc;
}

size_t attn_scan_scratch_bytes(int B, int T, int H) {
  if (B <= 0 || T <= 0 || H <= 0) return 0;
  const int sms = sm_count();
  int sc, ns;
  pick_segments(B, T, H, sms > 0 ? sms : 148, &sc, &ns);
  return size_t(B) * H * size_t(ns) * D * D * sizeof(float);   // ns - 1 pieces for a full call, ns for a state-only one
}

int launch_attn_scan(const void* q, const void* k, const void* v, int ld_qkv, const float* gamma,
                     const float* cos_tab, const float* sin_tab, int n_pos, const int32_t* pos0, int pos0_scalar,
                     const float* s_in, void* o, int ld_o, float* s_out, void* scratch, int B, int T, int H,
                     int head_dim, int flags, cudaStream_t stream) {
  JB_REQUIRE((flags & ~JB200_ATTN_QK_PREPARED) == 0, "attn_scan: unknown flags %d", flags);
  JB_REQUIRE(!(flags & JB200_ATTN_QK_PREPARED) || T > 1, "attn_scan: prepared q/k is for T > 1 (single-token steps take raw q, k)");
  JB_REQUIRE(head_dim == D, "attn_scan: head_dim (%d) must be %d", head_dim, D);
  JB_REQUIRE(B >= 0 && T >= 0 && H > 0, "attn_scan: bad shape (B=%d, T=%d, H=%d)", B, T, H);
  JB_REQUIRE(B <= 65535, "attn_scan: batch (%d) exceeds 65535", B);
  if (B == 0 || T == 0) return JB200_OK;
  JB_REQUIRE(k && v && gamma && cos_tab && sin_tab, "attn_scan: null pointer");
  JB_REQUIRE(o ? (q != nullptr) : (s_out && scratch && T > 1),
             "attn_scan: a call without output rows (state only) needs s_out, scratch and T > 1; any other call needs q and o");
  if (!q) q = k;     // state only: the tensor map of q is built but never used
  JB_REQUIRE(ld_qkv >= H * D && ld_qkv % 8 == 0 && (!o || (ld_o >= H * D && ld_o % 8 == 0)),
             "attn_scan: row strides must cover H*64 columns and be multiples of 8 elements");
  JB_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && (!o || aligned16(o)) && aligned16(cos_tab) && aligned16(sin_tab),
             "attn_scan: pointers must be 16-byte aligned");
  JB_REQUIRE(!s_in || (reinterpret_cast<uintptr_t>(s_in) & 7u) == 0, "attn_scan: state pointer misaligned");
  JB_REQUIRE(!s_out || (reinterpret_cast<uintptr_t>(s_out) & 7u) == 0, "attn_scan: state pointer misaligned");
  JB_REQUIRE(size_t(B) * T < (size_t(1) << 31), "attn_scan: too many rows");
  JB_REQUIRE(n_pos >= 1, "attn_scan: empty RoPE table");
  if (!pos0) JB_REQUIRE(pos0_scalar >= 0 && pos0_scalar + T <= n_pos, "attn_scan: RoPE table (%d rows) too short for positions %d..%d", n_pos, pos0_scalar, pos0_scalar + T - 1);
  if (T == 1) {
    JB_REQUIRE(!s_in || aligned16(s_in), "attn_scan: state pointer must be 16-byte aligned for single-token steps");
    JB_REQUIRE(!s_out || aligned16(s_out), "attn_scan: state pointer must be 16-byte aligned for single-token steps");
    AttnParams dp;
    dp.gamma = gamma; dp.cos_tab = cos_tab; dp.sin_tab = sin_tab; dp.pos0 = pos0; dp.pos0_scalar = pos0_scalar;
    dp.n_pos = n_pos; dp.s_in = s_in; dp.s_out = s_out; dp.o = reinterpret_cast<__nv_bfloat16*>(o); dp.ld_o = ld_o;
    dp.B = B; dp.T = 1; dp.H = H; dp.seg_chunks = 1; dp.nseg = 1; dp.seg_state = nullptr; dp.n_pieces = 0; dp.qk_prepared = 0; dp.status = nullptr;
    attn_decode_kernel<<<dim3(H, B), 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(q),
                                                        reinterpret_cast<const __nv_bfloat16*>(k),
                                                        reinterpret_cast<const __nv_bfloat16*>(v), ld_qkv, dp);
    JB_LAUNCH_CHECK("attn_decode_kernel");
    return JB200_OK;
  }
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_map(&tq, q, B * T, H * D, ld_qkv)) != JB200_OK) return rc;
  if ((rc = make_map(&tk, k, B * T, H * D, ld_qkv)) != JB200_OK) return rc;
  if ((rc = make_map(&tv, v, B * T, H * D, ld_qkv)) != JB200_OK) return rc;
  AttnParams p;
  p.gamma = gamma; p.cos_tab = cos_tab; p.sin_tab = sin_tab; p.pos0 = pos0; p.pos0_scalar = pos0_scalar;
  p.n_pos = n_pos; p.s_in = s_in; p.s_out = s_out; p.o = reinterpret_cast<__nv_bfloat16*>(o); p.ld_o = ld_o;
  p.B = B; p.T = T; p.H = H;
  p.qk_prepared = (flags & JB200_ATTN_QK_PREPARED) ? 1 : 0;
  p.n_pieces = 0;
  p.status = device_status_ptr();
  if (!p.status) return JB200_ERR_CUDA;
  const int sms = sm_count();
  if (sms <= 0) return JB200_ERR_CUDA;
  p.seg_chunks = (T + CH - 1) / CH;
  p.nseg = 1;
  p.seg_state = reinterpret_cast<float*>(scratch);
  if (scratch) pick_segments(B, T, H, sms, &p.seg_chunks, &p.nseg);   // without scratch: one segment per sequence
  JB_REQUIRE(p.nseg <= 65535, "attn_scan: too many segments");
  JB_REQUIRE(!scratch || (reinterpret_cast<uintptr_t>(scratch) & 7u) == 0, "attn_scan: scratch pointer misaligned");
  p.n_pieces = o ? p.nseg - 1 : p.nseg;
  if (!o) {
    // state only: the k/v pass over every piece, then the fold
    JB_CUDA(cudaFuncSetAttribute(attn_scan_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(ATTN_SMEM_BYTES)));
    attn_scan_kernel<true><<<dim3(H, B, p.nseg), ATTN_THREADS, ATTN_SMEM_BYTES, stream>>>(tq, tk, tv, p);
    JB_LAUNCH_CHECK("attn_scan_kernel<state>");
    attn_fold_states_kernel<<<dim3(H, B), 256, 0, stream>>>(p);
    JB_LAUNCH_CHECK("attn_fold_states_kernel");
    return JB200_OK;
  }
  JB_CUDA(cudaFuncSetAttribute(attn_scan_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(ATTN_SMEM_BYTES)));
  if (p.nseg > 1) {
    JB_CUDA(cudaFuncSetAttribute(attn_scan_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(ATTN_SMEM_BYTES)));
    attn_scan_kernel<true><<<dim3(H, B, p.nseg - 1), ATTN_THREADS, ATTN_SMEM_BYTES, stream>>>(tq, tk, tv, p);
    JB_LAUNCH_CHECK("attn_scan_kernel<state>");
  }
  attn_scan_kernel<false><<<dim3(H, B, p.nseg), ATTN_THREADS, ATTN_SMEM_BYTES, stream>>>(tq, tk, tv, p);
  JB_LAUNCH_CHECK("attn_scan_kernel");
  return JB200_OK;
}

}  // namespace jb
