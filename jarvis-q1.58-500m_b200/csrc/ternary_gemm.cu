// Ternary linear layers on the 5th-generation tensor cores (tcgen05 + TMEM).
//
//   Y[tok, f] = epilogue( alpha * sum_k X[tok, k] * Wq[f, k] ),   Wq in {-1, 0, +1}
//
// replaces TernaryLinear.forward (jarvis_engine/utils/ternary_ops.py:51-53) and the
// packed prototype packed_ternary_gemm_kernel
// (experiments/architecture_matrix/ternary_packed/packed_kernel.cu:25-73).  Weights
// stay in the 2-bit layout of runtime/weight_packing.py:22-51 (4 codes per byte along
// the in-feature axis, code 0 -> 0, 1 -> +1, 2 -> -1) all the way into shared memory,
// where they are expanded to bf16 {-1,0,+1} in the 128-byte-swizzled K-major layout that
// a tcgen05.mma shared-memory descriptor reads.
//
// Orientation: the weight tile is the UMMA "A" operand (M = 128 out-features) and the
// activation tile is the "B" operand (N = BN tokens, 32..256), so one 16-byte load of
// packed codes (64 weights) per thread per K-block feeds up to 256 token columns.  The
// accumulator D lives in TMEM with lane = out-feature, column = token.
//
// One persistent CTA per SM, 576 threads:
//   warp 0       TMA producer for the activation tiles (+ TMEM allocation)
//   warp 1       MMA issuer (one elected lane)
//   warps 2-9    weight decoders, two groups of four taking alternate K-blocks (one warp's own
//                instruction latency per K-block exceeds the 512 cycles its MMAs take); thread r of a
//                group owns weight row r of the tile
//   warps 10-17  epilogue (two warps per TMEM lane quadrant, alternate 32-token chunks): TMEM -> registers -> alpha / GELU -> smem transpose -> 16-byte row stores / residual add
// Two accumulator buffers (2 x 256 TMEM columns) let the epilogue of tile i overlap the
// main loop of tile i+1.  Token rows may be split into segments (one per expert), each
// with its own weight matrix and alpha: the grouped form used by the MoE experts.
//
// Two 2-bit weight layouts are accepted (w_layout):
//   0  canonical, exactly runtime/weight_packing.py (code k of a row at bits 2*(k%4) of byte k/4,
//      0 -> 0, 1 -> +1, 2 -> -1): decoded with a nibble spread + PRMT byte tables (~8 ops / 2 weights);
//   1  prepared (jb200_prepare_weights, a one-time re-encoding of the same 2 bits per weight): inside
//      every 32-bit word the even in-features sit in the low half and the odd ones in the high half,
//      each as (sign << 1 | nonzero), so (w << (14 - 2j)) & 0xC000C000 IS the bf16 pair
//      {0, +2.0, -2.0} for in-features (2j, 2j+1): 2 ops / 2 weights; the factor 2 is folded into alpha.
// The decoders share the SM's issue slots with the epilogue, and the kernel is issue-bound, so the
// instruction count of the decode is what sets the tensor-pipe utilisation.
#include "common.cuh"

namespace jb {

namespace {

constexpr int BM = 128;         // out-feature rows per tile  (UMMA M)
constexpr int BK = 64;          // k elements per stage (= one 128-byte swizzle row of bf16)
constexpr int STAGES = 4;
constexpr int BN_MAX = 256;     // token columns per tile (UMMA N), runtime 32..256
constexpr int A_STAGE_BYTES = BM * BK * 2;       // 16 KiB
constexpr int B_STAGE_BYTES = BN_MAX * BK * 2;   // 32 KiB
constexpr int MAX_GROUPS = 16;
constexpr int NUM_THREADS = 576;
constexpr int DEC_WARP0 = 2, EPI_WARP0 = 10;
constexpr int TMEM_COLS = 512;

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
};

struct SmemCtl {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
  int32_t seg[MAX_GROUPS + 1];
};

constexpr int STAGE_OUT_BYTES = 32 * 32 * 4;     // one epilogue warp's [32 tokens][32 features] f32 block
constexpr size_t SMEM_BYTES = 1024 /*alignment slack*/ + size_t(STAGES) * (A_STAGE_BYTES + B_STAGE_BYTES) +
                              ((sizeof(SmemCtl) + 127) / 128) * 128 + 8 * STAGE_OUT_BYTES;

struct TileCoord {
  int group;     // segment / expert
  int ft;        // out-feature tile
  int tok0;      // first token row of the tile (absolute row in X / Y)
  int tok_end;   // end of the segment (rows >= tok_end are not stored)
};

// Tile t -> coordinates.  Out-feature tiles vary fastest so that CTAs running at the
// same time share activation tiles through L2.
__device__ __forceinline__ bool tile_coord(const SmemCtl* ctl, int t, int n_ft, int G, int bn, TileCoord* c) {
  int tt = t / n_ft;
  c->ft = t - tt * n_ft;
  for (int g = 0; g < G; ++g) {
    const int beg = ctl->seg[g], end = ctl->seg[g + 1];
    const int tiles = (end - beg + bn - 1) / bn;
    if (tt < tiles) {
      c->group = g;
      c->tok0 = beg + tt * bn;
      c->tok_end = end;
      return true;
    }
    tt -= tiles;
  }
  return false;
}

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

__global__ void __launch_bounds__(NUM_THREADS, 1)
ternary_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const uint32_t a_base = base;
  const uint32_t b_base = base + STAGES * A_STAGE_BYTES;
  SmemCtl* ctl = reinterpret_cast<SmemCtl*>(smem + size_t(STAGES) * (A_STAGE_BYTES + B_STAGE_BYTES));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int bn = p.bn;
  const int n_ft = p.N / BM;
  const int n_kb = p.K / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1 + 128);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl->tmem_full[a]), 1);
      mbar_init(smem_u32(&ctl->tmem_empty[a]), 256);
    }
    ctl->abort_flag = 0;
    if (p.seg_offsets) {
      for (int g = 0; g <= p.G; ++g) ctl->seg[g] = min(max(p.seg_offsets[g], 0), p.M);
    } else {
      ctl->seg[0] = 0;
      ctl->seg[1] = p.M;
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&ctl->tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile uint32_t* abort_flag = &ctl->abort_flag;

  int total_tiles = 0;
  for (int g = 0; g < p.G; ++g) total_tiles += (ctl->seg[g + 1] - ctl->seg[g] + bn - 1) / bn;
  total_tiles *= n_ft;

  if (warp == 0) {
    // ---------------- TMA producer: activation tiles ----------------
    if (lane == 0) {
      uint32_t it = 0;
      TileCoord tc;
      for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
        if (!tile_coord(ctl, t, n_ft, p.G, bn, &tc)) break;
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(smem_u32(&ctl->empty[s]), ph ^ 1u, abort_flag, p.status, JB200_STATUS_GEMM_PRODUCER))
            goto done;
          mbar_arrive_expect_tx(smem_u32(&ctl->full[s]), uint32_t(bn) * BK * 2);
          tma_load_2d(b_base + s * B_STAGE_BYTES, &tmap_x, kb * BK, tc.tok0, smem_u32(&ctl->full[s]));
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(BM, bn);
      uint32_t it = 0, tile_n = 0;
      for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++tile_n) {
        const uint32_t acc = tile_n & 1u;
        const uint32_t acc_ph = (tile_n >> 1) & 1u;
        if (!mbar_wait(smem_u32(&ctl->tmem_empty[acc]), acc_ph ^ 1u, abort_flag, p.status, JB200_STATUS_GEMM_MMA))
          goto done;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN_MAX;
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(smem_u32(&ctl->full[s]), ph, abort_flag, p.status, JB200_STATUS_GEMM_MMA)) goto done;
          tc_fence_after_sync();
          const uint64_t adesc = umma_desc_k_sw128(a_base + s * A_STAGE_BYTES);
          const uint64_t bdesc = umma_desc_k_sw128(b_base + s * B_STAGE_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            // 16 bf16 = 32 bytes further along K inside the swizzle atom: +2 in the >>4 address field
            umma_bf16_ss(d_tmem, adesc + uint64_t(kk * 2), bdesc + uint64_t(kk * 2), idesc,
                         (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&ctl->empty[s]));
        }
        umma_commit(smem_u32(&ctl->tmem_full[acc]));
      }
    }
  } else if (warp < EPI_WARP0) {
    // ---------------- weight decoders ----------------
    const int grp = (warp - DEC_WARP0) >> 2;                      // K-blocks with (it & 1) == grp
    const int r = ((warp - DEC_WARP0) & 3) * 32 + lane;            // weight row inside the tile
    const size_t row_bytes = size_t(p.K) / 4;
    const uint32_t swz = uint32_t(r & 7);
    uint32_t it = 0;
    TileCoord tc;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      if (!tile_coord(ctl, t, n_ft, p.G, bn, &tc)) break;
      const uint8_t* wrow = p.w_packed + (size_t(tc.group) * p.N + size_t(tc.ft) * BM + r) * row_bytes;
      // this group's first K-block of the tile: kb0 = 0 or 1 depending on the running parity
      const int kb0 = int((it ^ uint32_t(grp)) & 1u);
      uint4 cur = make_uint4(0u, 0u, 0u, 0u);
      if (kb0 < n_kb) cur = __ldg(reinterpret_cast<const uint4*>(wrow + size_t(kb0) * 16));
      for (int kb = 0; kb < n_kb; ++kb, ++it) {
        if (((it ^ uint32_t(grp)) & 1u) != 0u) continue;    // the other group's K-block
        uint4 nxt = cur;
        if (kb + 2 < n_kb) nxt = __ldg(reinterpret_cast<const uint4*>(wrow + size_t(kb + 2) * 16));
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1u;
        if (!mbar_wait(smem_u32(&ctl->empty[s]), ph ^ 1u, abort_flag, p.status, JB200_STATUS_GEMM_DECODE)) goto done;
        uint8_t* arow = smem + size_t(s) * A_STAGE_BYTES + size_t(r) * 128;
        const uint32_t words[4] = {cur.x, cur.y, cur.z, cur.w};
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
          uint32_t v[8];
          if (p.w_layout) decode16_prepared(words[wi], v); else decode16(words[wi], v);
          const uint32_t c0 = uint32_t(2 * wi), c1 = uint32_t(2 * wi + 1);
          *reinterpret_cast<uint4*>(arow + ((c0 ^ swz) << 4)) = make_uint4(v[0], v[1], v[2], v[3]);
          *reinterpret_cast<uint4*>(arow + ((c1 ^ swz) << 4)) = make_uint4(v[4], v[5], v[6], v[7]);
        }
        fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core's async proxy
        mbar_arrive(smem_u32(&ctl->full[s]));
        cur = nxt;
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int q = warp & 3;                 // TMEM lane quadrant this warp may read
    const int half = (warp - EPI_WARP0) >> 2; // which of the alternating 32-token chunks
    uint8_t* stage_base = reinterpret_cast<uint8_t*>(ctl) + ((sizeof(SmemCtl) + 127) / 128) * 128;
    uint32_t tile_n = 0;
    TileCoord tc;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++tile_n) {
      if (!tile_coord(ctl, t, n_ft, p.G, bn, &tc)) break;
      const uint32_t acc = tile_n & 1u;
      const uint32_t acc_ph = (tile_n >> 1) & 1u;
      if (!mbar_wait(smem_u32(&ctl->tmem_full[acc]), acc_ph, abort_flag, p.status, JB200_STATUS_GEMM_EPILOGUE))
        goto done;
      tc_fence_after_sync();
      const int feat = tc.ft * BM + q * 32 + lane;
      uint8_t* stage = stage_base + (warp - EPI_WARP0) * STAGE_OUT_BYTES;
      const float alpha = __ldg(p.alpha + size_t(tc.group) * (p.N / p.alpha_rows) + feat / p.alpha_rows) *
                          (p.w_layout ? 0.5f : 1.0f);   // prepared weights decode to +-2
      const uint32_t t_lane = tmem_base + (uint32_t(q * 32) << 16) + acc * BN_MAX;
      for (int c0 = half * 32; c0 < bn; c0 += 64) {
        if (tc.tok0 + c0 >= tc.tok_end) break;   // warp-uniform
        const int ntok = min(32, tc.tok_end - (tc.tok0 + c0));
        // residual epilogue: start the loads of the old values before waiting for the accumulator
        float4 old[8];
        if (p.epilogue == JB200_EPI_RESID_F32) {
          const float* o = reinterpret_cast<const float*>(p.out);
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int idx = it * 32 + lane, r = idx >> 3, c16 = idx & 7;
            old[it] = r < ntok ? __ldcs(reinterpret_cast<const float4*>(
                                     o + size_t(tc.tok0 + c0 + r) * p.N + tc.ft * BM + q * 32 + c16 * 4))
                               : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
        uint32_t v[32];
        tmem_ld_32x32(t_lane + c0, v);
        tmem_ld_wait();
        // The accumulator chunk is lane = out-feature, register = token; HBM wants token rows.  Turn
        // it through this warp's staging block in shared memory ([32 tokens][32 features]) so that
        // global memory sees 16-byte accesses on whole 64 B / 128 B row segments.
        const int f0 = tc.ft * BM + q * 32;
        const size_t row0 = size_t(tc.tok0 + c0);
        if (p.epilogue == JB200_EPI_BF16 || p.epilogue == JB200_EPI_GELU_BF16) {
          const bool gelu = p.epilogue == JB200_EPI_GELU_BF16;
          __nv_bfloat16* st = reinterpret_cast<__nv_bfloat16*>(stage);
          // lane pairs (features f, f+1) swap one value per token pair, so each lane writes a bf16x2 word:
          // 16 four-byte staging stores per chunk instead of 32 two-byte ones (shared-memory bandwidth is
          // what the tensor core's operand reads, the decoders and this epilogue compete for)
          const bool odd = lane & 1;
          uint32_t* stw = reinterpret_cast<uint32_t*>(st);
#pragma unroll
          for (int jj = 0; jj < 16; ++jj) {
            float a = alpha * __uint_as_float(v[2 * jj]);
            float b = alpha * __uint_as_float(v[2 * jj + 1]);
            if (gelu) { a = gelu_erf(a); b = gelu_erf(b); }
            const float got = __shfl_xor_sync(0xffffffffu, odd ? a : b, 1);
            const uint32_t w2 = odd ? pack_bf16x2(got, b) : pack_bf16x2(a, got);
            stw[(2 * jj + (odd ? 1 : 0)) * 16 + (lane >> 1)] = w2;   // [token][feature pair]
          }
          __syncwarp();
          __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out);
#pragma unroll
          for (int it = 0; it < 4; ++it) {
            const int idx = it * 32 + lane, r = idx >> 2, c16 = idx & 3;
            const uint4 w4 = *reinterpret_cast<const uint4*>(st + r * 32 + c16 * 8);
            if (r < ntok) *reinterpret_cast<uint4*>(o + (row0 + r) * p.N + f0 + c16 * 8) = w4;
          }
        } else {
          const bool resid = p.epilogue == JB200_EPI_RESID_F32;
          float* st = reinterpret_cast<float*>(stage);
#pragma unroll
          for (int j = 0; j < 32; ++j) st[j * 32 + lane] = alpha * __uint_as_float(v[j]);
          __syncwarp();
          float* o = reinterpret_cast<float*>(p.out);
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int idx = it * 32 + lane, r = idx >> 3, c16 = idx & 7;
            float4 w4 = *reinterpret_cast<const float4*>(st + r * 32 + c16 * 4);
            if (resid) { w4.x += old[it].x; w4.y += old[it].y; w4.z += old[it].z; w4.w += old[it].w; }
            if (r < ntok) *reinterpret_cast<float4*>(o + (row0 + r) * p.N + f0 + c16 * 4) = w4;
          }
        }
        __syncwarp();   // staging block is reused by the next chunk
      }
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&ctl->tmem_empty[acc]));
    }
  }

done:
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
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

int pick_bn(int M, int G, int n_ft, int sms) {
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128) return 128;
  // 256-token tiles run ~1.5x faster per flop than 128-token ones (half the decode and half the A-tile
  // traffic per MMA column), so they win unless their last wave is far emptier.
  auto eff = [&](int bn) {
    const long tiles = long((M + bn - 1) / bn + (G - 1)) * n_ft;
    const long waves = (tiles + sms - 1) / sms;
    return double(tiles) / double(waves * sms);
  };
  return (eff(256) >= 0.70 * eff(128)) ? 256 : 128;
}

}  // namespace

int launch_ternary_gemm(const void* x_bf16, int M, int K, const uint8_t* w_packed, const float* alpha,
                        int alpha_rows, int N, int G, const int32_t* seg_offsets, int epilogue, void* out,
                        int bn_override, int w_layout, cudaStream_t stream) {
  JB_REQUIRE(M >= 0 && N > 0 && K > 0, "ternary_linear: bad sizes M=%d N=%d K=%d", M, N, K);
  JB_REQUIRE(N % BM == 0, "ternary_linear: out_features (%d) must be a multiple of %d", N, BM);
  JB_REQUIRE(K % BK == 0, "ternary_linear: in_features (%d) must be a multiple of %d", K, BK);
  JB_REQUIRE(G >= 1 && G <= MAX_GROUPS, "ternary_linear: groups (%d) must be in 1..%d", G, MAX_GROUPS);
  JB_REQUIRE(G == 1 || seg_offsets != nullptr, "ternary_linear: grouped call needs segment offsets");
  JB_REQUIRE(alpha_rows > 0 && alpha_rows % BM == 0 && N % alpha_rows == 0,
             "ternary_linear: alpha_rows (%d) must be a multiple of %d dividing out_features", alpha_rows, BM);
  JB_REQUIRE(epilogue >= JB200_EPI_BF16 && epilogue <= JB200_EPI_F32, "ternary_linear: unknown epilogue %d", epilogue);
  JB_REQUIRE(w_layout == 0 || w_layout == 1, "ternary_linear: weight layout must be 0 (canonical) or 1 (prepared)");
  JB_REQUIRE(x_bf16 && w_packed && alpha && out, "ternary_linear: null pointer");
  JB_REQUIRE(aligned16(x_bf16) && aligned16(w_packed) && aligned16(out), "ternary_linear: pointers must be 16-byte aligned");
  if (M == 0) return JB200_OK;
  const int sms = sm_count();
  if (sms <= 0) return JB200_ERR_CUDA;
  const int n_ft = N / BM;
  int bn = bn_override > 0 ? bn_override : pick_bn(M, G, n_ft, sms);
  JB_REQUIRE(bn == 32 || bn == 64 || bn == 128 || bn == 256, "ternary_linear: token tile %d not in {32,64,128,256}", bn);

  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) {
    set_error("ternary_linear: cuTensorMapEncodeTiled entry point not available");
    return JB200_ERR_CUDA;
  }
  CUtensorMap tmap;
  const cuuint64_t gdim[2] = {cuuint64_t(K), cuuint64_t(M)};
  const cuuint64_t gstride[1] = {cuuint64_t(K) * 2};
  const cuuint32_t box[2] = {cuuint32_t(BK), cuuint32_t(bn)};
  const cuuint32_t estr[2] = {1, 1};
  CUresult cr = enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x_bf16), gdim, gstride, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) {
    set_error("ternary_linear: cuTensorMapEncodeTiled failed (%d)", int(cr));
    return JB200_ERR_CUDA;
  }

  GemmParams p;
  p.w_packed = w_packed;
  p.alpha = alpha;
  p.seg_offsets = seg_offsets;
  p.out = out;
  p.M = M; p.N = N; p.K = K; p.G = G;
  p.alpha_rows = alpha_rows;
  p.bn = bn;
  p.epilogue = epilogue;
  p.w_layout = w_layout;
  p.status = device_status_ptr();
  if (!p.status) return JB200_ERR_CUDA;

  // per device and cheap: set on every call rather than remembering which devices have seen it
  JB_CUDA(cudaFuncSetAttribute(ternary_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM_BYTES)));
  const long max_tiles = long((M + bn - 1) / bn + (G - 1)) * n_ft;
  const int grid = int(max_tiles < sms ? max_tiles : sms);
  ternary_gemm_kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmap, p);
  JB_LAUNCH_CHECK("ternary_gemm_kernel");
  return JB200_OK;
}

// Host-side views of the in-kernel decodes, for the CPU unit test of the bit manipulation.
void decode16_host(uint32_t w, uint32_t* out8) { decode16(w, out8); }
void decode16_prepared_host(uint32_t w_canonical, uint32_t* out8) { decode16_prepared(prepare_word(w_canonical), out8); }

namespace {
__global__ void prepare_weights_kernel(const uint32_t* __restrict__ in, size_t n_words, uint32_t* __restrict__ out) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n_words; i += size_t(gridDim.x) * blockDim.x)
    out[i] = prepare_word(__ldg(in + i));
}
}  // namespace

int launch_prepare_weights(const uint8_t* packed, size_t n_bytes, uint8_t* prepared, cudaStream_t stream) {
  JB_REQUIRE(n_bytes % 4 == 0, "prepare_weights: byte count must be a multiple of 4 (16 weights per word)");
  JB_REQUIRE(packed && prepared, "prepare_weights: null pointer");
  JB_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 3u) == 0 && (reinterpret_cast<uintptr_t>(prepared) & 3u) == 0,
             "prepare_weights: pointers must be 4-byte aligned");
  if (n_bytes == 0) return JB200_OK;
  const size_t n_words = n_bytes / 4;
  size_t blocks = (n_words + 255) / 256;
  if (blocks > 4096) blocks = 4096;
  prepare_weights_kernel<<<unsigned(blocks), 256, 0, stream>>>(reinterpret_cast<const uint32_t*>(packed), n_words,
                                                              reinterpret_cast<uint32_t*>(prepared));
  JB_LAUNCH_CHECK("prepare_weights_kernel");
  return JB200_OK;
}

}  // namespace jb
