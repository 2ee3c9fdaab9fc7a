// Device helpers shared by the one-CTA and the CTA-pair ternary GEMM kernels: the 2-bit decoders for
// both weight layouts, the one-time re-encoding, and the GELU of the expert hidden layer.
#pragma once
#include "common.cuh"

namespace jb {

// 16 two-bit codes (one 32-bit word) -> 16 bf16 values (8 words), codes 0/1/2/3 -> 0/+1/-1/0.
// The codes are first spread to one per nibble; the nibbles then act as PRMT selectors
// into 4-byte tables of the high (00 3F BF 00) and low (00 80 80 00) bf16 bytes.
__host__ __device__ __forceinline__ uint32_t byte_perm_sw(uint32_t x, uint32_t y, uint32_t s) {
#if defined(__CUDA_ARCH__)
  return __byte_perm(x, y, s);
#else
  uint64_t pool = (uint64_t(y) << 32) | x;
  uint32_t r = 0;
  for (int i = 0; i < 4; ++i) r |= uint32_t((pool >> (8 * ((s >> (4 * i)) & 7))) & 0xFF) << (8 * i);
  return r;
#endif
}

__host__ __device__ __forceinline__ void decode16(uint32_t w, uint32_t* out) {
  constexpr uint32_t POOL_HI = 0x00BF3F00u;
  constexpr uint32_t POOL_LO = 0x00808000u;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    uint32_t x = (w >> (16 * half)) & 0xFFFFu;
    x = (x | (x << 8)) & 0x00FF00FFu;
    x = (x | (x << 4)) & 0x0F0F0F0Fu;
    x = (x | (x << 2)) & 0x33333333u;  // code j of this half sits in nibble j
    const uint32_t h03 = byte_perm_sw(POOL_HI, 0u, x);
    const uint32_t l03 = byte_perm_sw(POOL_LO, 0u, x);
    const uint32_t h47 = byte_perm_sw(POOL_HI, 0u, x >> 16);
    const uint32_t l47 = byte_perm_sw(POOL_LO, 0u, x >> 16);
    out[half * 4 + 0] = byte_perm_sw(l03, h03, 0x5140u);
    out[half * 4 + 1] = byte_perm_sw(l03, h03, 0x7362u);
    out[half * 4 + 2] = byte_perm_sw(l47, h47, 0x5140u);
    out[half * 4 + 3] = byte_perm_sw(l47, h47, 0x7362u);
  }
}

// Prepared layout: canonical word -> prepared word (host + device; the one-time re-encoding).
__host__ __device__ __forceinline__ uint32_t prepare_word(uint32_t w) {
  uint32_t out = 0;
  for (int k = 0; k < 16; ++k) {
    const uint32_t c = (w >> (2 * k)) & 3u;
    const uint32_t f = c == 1u ? 1u : (c == 2u ? 3u : 0u);          // (sign << 1) | nonzero
    out |= f << ((k & 1) * 16 + (k >> 1) * 2);
  }
  return out;
}
// Prepared word -> 8 bf16 pairs holding 2 * {-1, 0, +1}.
__host__ __device__ __forceinline__ void decode16_prepared(uint32_t w, uint32_t* out) {
#pragma unroll
  for (int j = 0; j < 8; ++j) out[j] = (w << (14 - 2 * j)) & 0xC000C000u;
}

// GELU for the expert hidden layer.  The reference uses the exact-erf form (F.gelu default,
// jarvis_model.py:236); here 0.5 x (1 + tanh(x (a + b x^2 + c x^4))) with a, b, c fitted to the erf
// form: |difference| < 2.6e-5 everywhere (plus tanh.approx's 2^-11 relative error), an order of
// magnitude below the bf16 rounding of the stored result, at 9 instructions instead of ~25 for erff
// in an epilogue that is issue-bound.
__device__ __forceinline__ float gelu_erf(float v) {
  const float xc = fminf(fmaxf(v, -8.0f), 8.0f);     // keeps the fitted polynomial in its monotone range
  const float x2 = xc * xc;
  float pz = fmaf(-0.0003515195915898722f, x2, 0.03700566448133039f);
  pz = fmaf(pz, x2, 0.797507862407347f);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(pz * xc));
  const float hv = 0.5f * v;
  return fmaf(hv, t, hv);
}


constexpr int MAX_GROUPS = 16;

struct GemmParams {
  const uint8_t* w_packed;   // [G][N][K/4]
  const float* alpha;        // [G][N / alpha_rows]
  const int32_t* seg_offsets;  // device [G+1] or nullptr (single segment [0, M))
  void* out;                 // bf16 [M][N] or f32 [M][N]
  int M, N, K, G;
  int alpha_rows;            // out-feature rows sharing one alpha (N for per-tensor)
  int bn;                    // token tile
  int epilogue;
  int w_layout;              // 0 canonical weight_packing.py layout, 1 prepared layout
  unsigned int* status;
  // JB200_EPI_RESID_F32: 8 staging tiles of [32 tokens][32 features] f32 in shared memory (one per epilogue warp),
  // from which the tile is ADDED to the residual stream by a TMA reduction; 0 = plain read-modify-write from registers
  uint32_t resid_stage_smem;
  // JB200_EPI_QK_ROPE_BF16 only: attention feature map + rotary embedding applied to out-features < rope_feats
  const float* cos_tab;      // [n_pos][32]
  const float* sin_tab;      // [n_pos][32]
  const int32_t* pos0;       // [rows / T] first position of every sequence, or null (pos0_scalar)
  int pos0_scalar, n_pos, T;
  int rope_feats;            // out-features [0, rope_feats) are q and k heads (64 features each), the rest plain
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}


// Residual epilogue: the old values of a tile (128 KiB) are what its epilogue waits for longest.  Called by
// an epilogue warp BEFORE it waits for the tile's accumulator, i.e. while the tile's MMAs still run: every
// lane asks L2 for the 128-byte line (32 f32 features) of one token row of each chunk the warp will handle.
__device__ __forceinline__ void prefetch_residual_rows(const GemmParams& p, int tok0, int tok_end, int f0, int half,
                                                       int bn, int lane) {
  const float* o = reinterpret_cast<const float*>(p.out);
  for (int c0 = half * 32; c0 < bn; c0 += 64) {
    const int row = tok0 + c0 + lane;
    if (row < tok_end) prefetch_l2(o + size_t(row) * p.N + f0);
  }
}

// One [32 out-features (TMEM lanes)] x [32 tokens (columns)] accumulator chunk -> alpha / GELU / residual ->
// global memory, straight from registers.  Lane = out-feature and register = token, and memory wants token
// rows, so lanes first trade values by shuffles: pairs for bf16 outputs (every lane stores a bf16x2 word, an
// instruction covers two 64-byte row segments), quads for f32 outputs (every lane loads / stores a float4,
// an instruction covers four 128-byte row segments).  Nothing is staged in shared memory,
// whose bandwidth the tensor core's operand reads, the TMA writes and the decoders already use up.
// Called by a whole epilogue warp.
__device__ __forceinline__ void store_acc_chunk(const GemmParams& p, uint32_t taddr, float alpha, size_t row0, int f0,
                                                int ntok, int lane, const CUtensorMap* tmap_out = nullptr,
                                                uint32_t stage_smem = 0) {
  uint32_t v[32];
  if (p.epilogue == JB200_EPI_RESID_F32 && stage_smem != 0) {
    // x[token][feature] += alpha * acc through the memory system: lane = feature, register = token, so writing
    // register t to stage[t][lane] is one conflict-free 128-byte row per instruction - no shuffles, no loads of
    // the old values, nothing waits on global memory.  The tile then leaves as one TMA reduce-add (f32), which
    // clips token rows past the end of the matrix.
    tmem_ld_32x32(taddr, v);
    tmem_ld_wait();
    if (lane == 0) bulk_wait_group_read<0>();     // the previous reduction has finished reading this warp's stage
    __syncwarp();
    const uint32_t dst = stage_smem + uint32_t(lane) * 4u;
#pragma unroll
    for (int t = 0; t < 32; ++t)
      asm volatile("st.shared.f32 [%0], %1;" ::"r"(dst + uint32_t(t) * 128u), "f"(alpha * __uint_as_float(v[t])) : "memory");
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_reduce_add_2d(tmap_out, f0, int(row0), stage_smem);
      bulk_commit_group();
    }
    return;
  }
  if (p.epilogue == JB200_EPI_QK_ROPE_BF16 && f0 < p.rope_feats) {
    // q / k heads whose weight rows were interleaved so that features d and d + 32 of a head are neighbouring
    // out-features (2i, 2i + 1): the lane pair that already swaps values for the bf16x2 store holds exactly
    // the two RoPE partners.  phi(x) = ELU(x) + 1 in f32 on the accumulator, then
    //   out[d] = phi(x[d]) cos - phi(x[d+32]) sin,   out[d+32] = phi(x[d+32]) cos + phi(x[d]) sin
    // (jarvis_model.py:124-128, :29-71), rounded to bf16 once.  The 1/sqrt(D) of the queries is left to the
    // attention kernel's score factors (a power of two: same bits).
    const int odd = lane & 1;
    const int pair = ((f0 & 32) >> 1) + (lane >> 1);              // rotary pair index i of this lane pair, 0..31
    const int n_seq = p.M / p.T;
    const int seq0 = int(row0) / p.T;                             // sequence and offset of the chunk's first row
    const int t0 = int(row0) - seq0 * p.T;
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (row0 + size_t(odd)) * p.N + f0 + (lane & ~1);
    const size_t step = size_t(p.N) * 2;
    const int base_pos = (p.pos0 ? __ldg(p.pos0 + min(seq0, n_seq - 1)) : p.pos0_scalar) + t0;
    // Fast path (warp-uniform): the 32 rows lie in one sequence and inside the table.  The angle of pair i grows
    // by the same amount from one position to the next, so only the lane's first (cos, sin) and the rotation by
    // two positions (table row 2) are loaded, before the accumulator wait; the other 15 come from the angle
    // addition formulas (error ~1e-6 after 15 steps, three orders below the bf16 rounding of the result).
    const bool fast = t0 + 32 <= p.T && base_pos >= 0 && base_pos + 32 <= p.n_pos && p.n_pos > 2;
    float cs = 1.f, sn = 0.f, c2 = 1.f, s2 = 0.f;
    if (fast) {
      cs = __ldg(p.cos_tab + size_t(base_pos + odd) * 32 + pair);
      sn = __ldg(p.sin_tab + size_t(base_pos + odd) * 32 + pair);
      c2 = __ldg(p.cos_tab + 2 * 32 + pair);
      s2 = __ldg(p.sin_tab + 2 * 32 + pair);
    }
    tmem_ld_32x32(taddr, v);
    tmem_ld_wait();
    int seq = seq0, t = t0 + odd;                                 // this lane's tokens: row0 + odd + 2 jj
    while (t >= p.T) { t -= p.T; ++seq; }
#pragma unroll
    for (int jj = 0; jj < 16; ++jj) {
      if (!fast) {
        int pos = (p.pos0 ? __ldg(p.pos0 + min(seq, n_seq - 1)) : p.pos0_scalar) + t;   // rows past M are not stored
        pos = pos < 0 ? 0 : (pos >= p.n_pos ? p.n_pos - 1 : pos);
        cs = __ldg(p.cos_tab + size_t(pos) * 32 + pair);
        sn = __ldg(p.sin_tab + size_t(pos) * 32 + pair);
        t += 2;
        while (t >= p.T) { t -= p.T; ++seq; }   // next sequence of the batch
      }
      float a = alpha * __uint_as_float(v[2 * jj]);       // token 2jj:     x[d] on even lanes, x[d+32] on odd lanes
      float b = alpha * __uint_as_float(v[2 * jj + 1]);   // token 2jj + 1
      a = a > 0.f ? a + 1.0f : __expf(a);
      b = b > 0.f ? b + 1.0f : __expf(b);
      // even lanes finish token 2jj (they need the partner's a), odd lanes token 2jj + 1 (the partner's b)
      const float got = __shfl_xor_sync(0xffffffffu, odd ? a : b, 1);
      const float lo = odd ? got : a;      // phi(x[d])
      const float hi = odd ? b : got;      // phi(x[d+32])
      const uint32_t w2 = pack_bf16x2(lo * cs - hi * sn, hi * cs + lo * sn);
      if (2 * jj + odd < ntok) *reinterpret_cast<uint32_t*>(o) = w2;
      o += step;
      if (fast) {                           // advance the angle by two positions
        const float cn = cs * c2 - sn * s2;
        sn = sn * c2 + cs * s2;
        cs = cn;
      }
    }
  } else if (p.epilogue == JB200_EPI_BF16 || p.epilogue == JB200_EPI_GELU_BF16 || p.epilogue == JB200_EPI_QK_ROPE_BF16) {
    const bool gelu = p.epilogue == JB200_EPI_GELU_BF16;
    tmem_ld_32x32(taddr, v);
    tmem_ld_wait();
    const int odd = lane & 1;
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (row0 + size_t(odd)) * p.N + f0 + (lane & ~1);
    const size_t step = size_t(p.N) * 2;   // two token rows
#pragma unroll
    for (int jj = 0; jj < 16; ++jj) {
      float a = alpha * __uint_as_float(v[2 * jj]);
      float b = alpha * __uint_as_float(v[2 * jj + 1]);
      if (gelu) { a = gelu_erf(a); b = gelu_erf(b); }
      const float got = __shfl_xor_sync(0xffffffffu, odd ? a : b, 1);
      const uint32_t w2 = odd ? pack_bf16x2(got, b) : pack_bf16x2(a, got);   // features (f & ~1, f | 1)
      if (2 * jj + odd < ntok) *reinterpret_cast<uint32_t*>(o) = w2;       // token 2jj (even lanes) / 2jj+1 (odd)
      o += step;
    }
  } else {
    // f32 outputs: 4x4 transposes inside lane quads (two shuffle rounds) turn "lane = feature, 4 registers =
    // 4 tokens" into "lane = token (row0 + 4g + lane % 4), float4 = 4 features", so that loads of the old
    // residual values and stores are 16 bytes per lane and cover four 128-byte row segments per instruction.
    const bool resid = p.epilogue == JB200_EPI_RESID_F32;
    const int sub = lane & 3;
    float* o = reinterpret_cast<float*>(p.out) + (row0 + size_t(sub)) * p.N + f0 + (lane >> 2) * 4;
    const size_t step = size_t(p.N) * 4;   // four token rows
    float4 old[8];
    if (resid) {
      // start the loads of the old values before waiting for the accumulator
#pragma unroll
      for (int g = 0; g < 8; ++g)
        old[g] = 4 * g + sub < ntok ? __ldcs(reinterpret_cast<const float4*>(o + size_t(g) * step))
                                    : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    tmem_ld_32x32(taddr, v);
    tmem_ld_wait();
    const bool up = (lane & 2) != 0, odd = (lane & 1) != 0;
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      float v0 = alpha * __uint_as_float(v[4 * g + 0]), v1 = alpha * __uint_as_float(v[4 * g + 1]);
      float v2 = alpha * __uint_as_float(v[4 * g + 2]), v3 = alpha * __uint_as_float(v[4 * g + 3]);
      // swap the off-diagonal 2x2 blocks between lanes l and l ^ 2 ...
      float r0 = __shfl_xor_sync(0xffffffffu, up ? v0 : v2, 2);
      float r1 = __shfl_xor_sync(0xffffffffu, up ? v1 : v3, 2);
      if (up) { v0 = r0; v1 = r1; } else { v2 = r0; v3 = r1; }
      // ... then transpose inside every 2x2 block between lanes l and l ^ 1
      r0 = __shfl_xor_sync(0xffffffffu, odd ? v0 : v1, 1);
      r1 = __shfl_xor_sync(0xffffffffu, odd ? v2 : v3, 1);
      if (odd) { v0 = r0; v2 = r1; } else { v1 = r0; v3 = r1; }
      float4 w4 = make_float4(v0, v1, v2, v3);
      if (resid) {
        w4.x = __fadd_rn(w4.x, old[g].x); w4.y = __fadd_rn(w4.y, old[g].y);
        w4.z = __fadd_rn(w4.z, old[g].z); w4.w = __fadd_rn(w4.w, old[g].w);
      }
      if (4 * g + sub < ntok) *reinterpret_cast<float4*>(o + size_t(g) * step) = w4;
    }
  }
}

}  // namespace jb
