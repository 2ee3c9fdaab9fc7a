// Ternary linear layers on CTA pairs: two SMs drive their tensor cores as one (tcgen05 cta_group::2).
//
// Same contract as ternary_gemm_kernel (TernaryLinear.forward, jarvis_engine/utils/ternary_ops.py:51-53;
// weights in the 2-bit layout of runtime/weight_packing.py:22-51), different tiling: a tile is
// 256 out-features x BN tokens, computed by the two CTAs of a 2-CTA cluster.  Each CTA decodes ITS 128
// weight rows into its own shared memory and fetches only ITS half of the activation tile (BN/2 token
// rows) by TMA; one tcgen05.mma.cta_group::2 issued by the even CTA multiplies both halves, and each CTA
// ends up with the accumulator of its own 128 out-features (TMEM lanes) x BN tokens (columns).
//
// Why: per K-block of 64 the one-CTA kernel moves 32 KiB of activations into every SM's shared memory and
// the tensor core reads them back, on top of the 16 KiB decoded weight tile; shared-memory bandwidth is
// what limits that kernel.  In a pair every SM stages and reads half as many activation bytes for the
// same number of MMA cycles, and the smaller stage leaves room for seven pipeline stages instead of four.
//
// Roles inside each CTA are those of the one-CTA kernel (576 threads: TMA producer, MMA issuer - idle in
// the odd CTA -, 2 x 4 decoder warps, 8 epilogue warps).  Barriers that gate the MMA issuer (`full`,
// `tmem_empty`) live in the even CTA and are arrived on by both CTAs (one elected lane per warp, remote
// arrive through the shared::cluster window); barriers that the tensor core signals (`empty`,
// `tmem_full`) exist in both CTAs and one tcgen05.commit arrives on both copies.
#include "common.cuh"
#include "gemm_shared.cuh"

namespace jb {

namespace {

constexpr int BM = 128;          // out-feature rows per CTA (the pair's UMMA M is 256)
constexpr int BK = 64;
constexpr int STAGES = 7;
constexpr int BN_MAX = 256;      // token columns per tile (UMMA N): 128 or 256
constexpr int A_STAGE_BYTES = BM * BK * 2;             // 16 KiB
constexpr int B_STAGE_BYTES = (BN_MAX / 2) * BK * 2;   // 16 KiB: this CTA's half of the token rows
constexpr int NUM_THREADS = 576;
constexpr int DEC_WARP0 = 2, EPI_WARP0 = 10;
constexpr int TMEM_COLS = 512;

struct PairCtl {
  uint64_t full[STAGES];       // used in the even CTA: 1 expect_tx arrival + 8 decoder warps (4 per CTA)
  uint64_t empty[STAGES];      // per CTA: one tcgen05.commit
  uint64_t tmem_full[2];       // per CTA: one tcgen05.commit
  uint64_t tmem_empty[2];      // used in the even CTA: 16 epilogue warps (8 per CTA)
  uint32_t tmem_base;
  uint32_t abort_flag;
  int32_t seg[MAX_GROUPS + 1];
};

constexpr size_t CTL_BYTES = ((sizeof(PairCtl) + 127) / 128) * 128;
constexpr size_t SMEM_BYTES = 1024 /*alignment slack*/ + size_t(STAGES) * (A_STAGE_BYTES + B_STAGE_BYTES) + CTL_BYTES;
static_assert(SMEM_BYTES <= 227 * 1024, "pair GEMM shared memory exceeds the per-CTA limit");

struct PairTile {
  int group, ft2, tok0, tok_end;
};

// Tile t -> coordinates; 256-feature tiles vary fastest so that pairs running together share activations in L2.
__device__ __forceinline__ bool pair_tile(const PairCtl* ctl, int t, int n_ft2, int G, int bn, PairTile* c) {
  int tt = t / n_ft2;
  c->ft2 = t - tt * n_ft2;
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

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
ternary_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const uint32_t a_base = base;
  const uint32_t b_base = base + STAGES * A_STAGE_BYTES;
  PairCtl* ctl = reinterpret_cast<PairCtl*>(smem + size_t(STAGES) * (A_STAGE_BYTES + B_STAGE_BYTES));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();       // 0 = even CTA (issues the MMAs), 1 = odd CTA
  const int pair = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;
  const int bn = p.bn;
  const int half_bn = bn >> 1;
  const int n_ft2 = p.N / (2 * BM);
  const int n_kb = p.K / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1 + 8);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl->tmem_full[a]), 1);
      mbar_init(smem_u32(&ctl->tmem_empty[a]), 16);
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
    tmem_alloc_pair(smem_u32(&ctl->tmem_base), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  // both CTAs' barriers are initialised before either touches the other's
  cluster_arrive_release();
  cluster_wait_acquire();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile uint32_t* abort_flag = &ctl->abort_flag;

  int total_tiles = 0;
  for (int g = 0; g < p.G; ++g) total_tiles += (ctl->seg[g + 1] - ctl->seg[g] + bn - 1) / bn;
  total_tiles *= n_ft2;

  if (warp == 0) {
    // ---------------- TMA producer: this CTA's half of the activation tile ----------------
    if (lane == 0) {
      uint32_t it = 0;
      PairTile tc;
      for (int t = pair; t < total_tiles; t += n_pairs) {
        if (!pair_tile(ctl, t, n_ft2, p.G, bn, &tc)) break;
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(smem_u32(&ctl->empty[s]), ph ^ 1u, abort_flag, p.status, JB200_STATUS_GEMM_PRODUCER))
            goto done;
          // the even CTA's barrier counts the bytes of both halves
          if (rank == 0) mbar_arrive_expect_tx(smem_u32(&ctl->full[s]), uint32_t(bn) * BK * 2);
          tma_load_2d_pair(b_base + s * B_STAGE_BYTES, &tmap_x, kb * BK, tc.tok0 + int(rank) * half_bn,
                           smem_u32(&ctl->full[s]));
        }
      }
      // tail: the partner's tensor-core commits still arrive on this CTA's `empty` barriers; stay until
      // the last use of every stage has been released
      for (uint32_t j = it > uint32_t(STAGES) ? it - STAGES : 0u; j < it; ++j) {
        if (!mbar_wait(smem_u32(&ctl->empty[j % STAGES]), (j / STAGES) & 1u, abort_flag, p.status,
                       JB200_STATUS_GEMM_PRODUCER))
          goto done;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (even CTA only) ----------------
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_idesc_bf16(2 * BM, bn);
      uint32_t it = 0, tile_n = 0;
      for (int t = pair; t < total_tiles; t += n_pairs, ++tile_n) {
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
            umma_bf16_ss_pair(d_tmem, adesc + uint64_t(kk * 2), bdesc + uint64_t(kk * 2), idesc,
                              (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit_pair(smem_u32(&ctl->empty[s]));   // the stage is free in both CTAs once these MMAs retire
        }
        umma_commit_pair(smem_u32(&ctl->tmem_full[acc]));
      }
    }
  } else if (warp < EPI_WARP0) {
    // ---------------- weight decoders: this CTA's 128 rows of the 256-row tile ----------------
    const int grp = (warp - DEC_WARP0) >> 2;
    const int r = ((warp - DEC_WARP0) & 3) * 32 + lane;
    const size_t row_bytes = size_t(p.K) / 4;
    const uint32_t swz = uint32_t(r & 7);
    const uint32_t full0 = mapa_u32(smem_u32(&ctl->full[0]), 0u);   // the even CTA's `full` barriers
    uint32_t it = 0;
    PairTile tc;
    for (int t = pair; t < total_tiles; t += n_pairs) {
      if (!pair_tile(ctl, t, n_ft2, p.G, bn, &tc)) break;
      const uint8_t* wrow =
          p.w_packed + (size_t(tc.group) * p.N + size_t(tc.ft2) * (2 * BM) + size_t(rank) * BM + r) * row_bytes;
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
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(full0 + uint32_t(s) * 8u);
        cur = nxt;
      }
    }
  } else {
    // ---------------- epilogue: this CTA's 128 out-features ----------------
    const int q = warp & 3;
    const int half = (warp - EPI_WARP0) >> 2;
    const uint32_t tmem_empty0 = mapa_u32(smem_u32(&ctl->tmem_empty[0]), 0u);
    uint32_t tile_n = 0;
    PairTile tc;
    for (int t = pair; t < total_tiles; t += n_pairs, ++tile_n) {
      if (!pair_tile(ctl, t, n_ft2, p.G, bn, &tc)) break;
      const uint32_t acc = tile_n & 1u;
      const uint32_t acc_ph = (tile_n >> 1) & 1u;
      if (p.epilogue == JB200_EPI_RESID_F32)
        prefetch_residual_rows(p, tc.tok0, tc.tok_end, tc.ft2 * (2 * BM) + int(rank) * BM + q * 32, half, bn, lane);
      if (!mbar_wait(smem_u32(&ctl->tmem_full[acc]), acc_ph, abort_flag, p.status, JB200_STATUS_GEMM_EPILOGUE))
        goto done;
      tc_fence_after_sync();
      const int f0 = tc.ft2 * (2 * BM) + int(rank) * BM + q * 32;
      const float alpha = __ldg(p.alpha + size_t(tc.group) * (p.N / p.alpha_rows) + (f0 + lane) / p.alpha_rows) *
                          (p.w_layout ? 0.5f : 1.0f);   // prepared weights decode to +-2
      const uint32_t t_lane = tmem_base + (uint32_t(q * 32) << 16) + acc * BN_MAX;
      for (int c0 = half * 32; c0 < bn; c0 += 64) {
        if (tc.tok0 + c0 >= tc.tok_end) break;   // warp-uniform
        const int ntok = min(32, tc.tok_end - (tc.tok0 + c0));
        store_acc_chunk(p, t_lane + c0, alpha, size_t(tc.tok0 + c0), f0, ntok, lane);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tmem_empty0 + acc * 8u);
    }
  }

done:
  tc_fence_before_sync();
  __syncthreads();
  // neither CTA may leave (or free tensor memory) while its partner can still arrive on its barriers,
  // have MMAs of the pair in flight or read its accumulator
  cluster_arrive_release();
  cluster_wait_acquire();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace

// Token tile for the pair kernel (0 = not applicable: out-features not a multiple of 256, or a tile it lacks).
int pair_token_tile(int M, int N, int G, int bn_override, int sms) {
  if (N % (2 * BM) != 0 || sms < 2) return 0;
  if (bn_override > 0) return (bn_override == 128 || bn_override == 256) ? bn_override : 0;
  if (M <= 128) return 128;
  const int n_ft2 = N / (2 * BM);
  const int pairs = sms / 2;
  auto eff = [&](int bn) {
    const long tiles = long((M + bn - 1) / bn + (G - 1)) * n_ft2;
    const long waves = (tiles + pairs - 1) / pairs;
    return double(tiles) / double(waves * pairs);
  };
  return (eff(256) >= 0.70 * eff(128)) ? 256 : 128;
}

int launch_ternary_gemm_pair(const void* x_bf16, const GemmParams& p, cudaStream_t stream) {
  const int sms = sm_count();
  if (sms <= 0) return JB200_ERR_CUDA;
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) {
    set_error("ternary_linear: cuTensorMapEncodeTiled entry point not available");
    return JB200_ERR_CUDA;
  }
  CUtensorMap tmap;
  const cuuint64_t gdim[2] = {cuuint64_t(p.K), cuuint64_t(p.M)};
  const cuuint64_t gstride[1] = {cuuint64_t(p.K) * 2};
  const cuuint32_t box[2] = {cuuint32_t(BK), cuuint32_t(p.bn / 2)};
  const cuuint32_t estr[2] = {1, 1};
  CUresult cr = enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x_bf16), gdim, gstride, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) {
    set_error("ternary_linear: cuTensorMapEncodeTiled failed (%d)", int(cr));
    return JB200_ERR_CUDA;
  }
  JB_CUDA(cudaFuncSetAttribute(ternary_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM_BYTES)));
  const long max_tiles = long((p.M + p.bn - 1) / p.bn + (p.G - 1)) * (p.N / (2 * BM));
  const long pairs = sms / 2;
  const int grid = 2 * int(max_tiles < pairs ? max_tiles : pairs);
  ternary_gemm_pair_kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmap, p);
  JB_LAUNCH_CHECK("ternary_gemm_pair_kernel");
  return JB200_OK;
}

}  // namespace jb
