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
//   warps 10-17  epilogue (two warps per TMEM lane quadrant, alternate 32-token chunks): TMEM -> registers ->
//                alpha / GELU -> row-segment stores straight from registers.  The f32 residual epilogue
//                (x += alpha * acc) sends every other chunk through a [32 tokens][32 features] staging tile and a
//                TMA reduce-add (cp.reduce.async.bulk.tensor .add.f32: no load of the old values, no shuffles)
//                and the rest through a read-modify-write from registers, so that the L2's reduction path and
//                the load/store path each carry half of the tile
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
//   2  dense bf16 weights [N][K] (the lm_head, jarvis_model.py:535, which the reference keeps as nn.Linear): nothing to
//      decode, the weight tile is a second TMA load into the same swizzled stage buffer and the decoder warps retire.
// The decoders, the TMA writes, the tensor core's operand reads and the epilogue all go through the same
// shared memory and issue slots; per-role cycle counters put the MMA issue interval at 126 cycles (of 128) for
// K = 4096 and 154 for K = 1024, so the cheap decode and an epilogue that never touches shared memory are what
// keep the tensor pipe fed.
#include "common.cuh"
#include "gemm_shared.cuh"
#include "launchers.h"

namespace jb {

namespace {

constexpr int BM = 128;         // out-feature rows per tile  (UMMA M)
constexpr int BK = 64;          // k elements per stage (= one 128-byte swizzle row of bf16)
constexpr int STAGES = 4;
constexpr int BN_MAX = 256;     // token columns per tile (UMMA N), runtime 32..256
constexpr int A_STAGE_BYTES = BM * BK * 2;       // 16 KiB
constexpr int B_STAGE_BYTES = BN_MAX * BK * 2;   // 32 KiB
constexpr int NUM_THREADS = 576;
constexpr int DEC_WARP0 = 2, EPI_WARP0 = 10;
constexpr int TMEM_COLS = 512;

struct SmemCtl {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
  int32_t seg[MAX_GROUPS + 1];
};

constexpr size_t CTL_BYTES = ((sizeof(SmemCtl) + 127) / 128) * 128;
constexpr int RESID_STAGE_BYTES = 32 * 32 * 4;                   // one [32 tokens][32 features] f32 tile per epilogue warp
constexpr size_t SMEM_BYTES = 1024 /*alignment slack*/ + size_t(STAGES) * (A_STAGE_BYTES + B_STAGE_BYTES) + CTL_BYTES;
constexpr size_t SMEM_BYTES_RESID = SMEM_BYTES + 8 * RESID_STAGE_BYTES;

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

__global__ void __launch_bounds__(NUM_THREADS, 1)
ternary_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                    const __grid_constant__ CUtensorMap tmap_out, const GemmParams p) {
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
  const bool dense_w = p.w_layout == 2;     // weight tiles come by TMA: only the producer arrives on `full`

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), dense_w ? 1 : 1 + 128);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl->tmem_full[a]), 1);
      mbar_init(smem_u32(&ctl->tmem_empty[a]), 256);
    }
    ctl->abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_x);
    if (dense_w) tma_prefetch_desc(&tmap_w);
  }
  if (warp == 0) {
    __syncwarp();                 // tcgen05.alloc is warp-collective: lane 0 rejoins from the barrier set-up first
    tmem_alloc(smem_u32(&ctl->tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  // The set-up above overlaps the tail of the kernel before this one on the stream; nothing before this line reads
  // or writes global memory.
  pdl_wait();
  pdl_trigger();
  if (threadIdx.x == 0) {
    if (p.seg_offsets) {
      for (int g = 0; g <= p.G; ++g) ctl->seg[g] = min(max(p.seg_offsets[g], 0), p.M);
    } else {
      ctl->seg[0] = 0;
      ctl->seg[1] = p.M;
    }
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
          mbar_arrive_expect_tx(smem_u32(&ctl->full[s]), uint32_t(bn) * BK * 2 + (dense_w ? uint32_t(A_STAGE_BYTES) : 0u));
          tma_load_2d(b_base + s * B_STAGE_BYTES, &tmap_x, kb * BK, tc.tok0, smem_u32(&ctl->full[s]));
          if (dense_w)
            tma_load_2d(a_base + s * A_STAGE_BYTES, &tmap_w, kb * BK, tc.group * p.N + tc.ft * BM, smem_u32(&ctl->full[s]));
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
    if (dense_w) goto done;
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
          if (p.w_layout == 1) decode16_prepared(words[wi], v); else decode16(words[wi], v);
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
    // residual epilogue through TMA reductions: this warp's staging tile sits behind the control block
    const uint32_t stage_smem = p.resid_stage_smem
                                    ? base + uint32_t(STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + CTL_BYTES) +
                                          uint32_t(warp - EPI_WARP0) * RESID_STAGE_BYTES
                                    : 0u;
    if (stage_smem && lane == 0) tma_prefetch_desc(&tmap_out);
    uint32_t tile_n = 0;
    TileCoord tc;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++tile_n) {
      if (!tile_coord(ctl, t, n_ft, p.G, bn, &tc)) break;
      const uint32_t acc = tile_n & 1u;
      const uint32_t acc_ph = (tile_n >> 1) & 1u;
      if (p.epilogue == JB200_EPI_RESID_F32)
        prefetch_residual_rows(p, tc.tok0, tc.tok_end, tc.ft * BM + q * 32, half, bn, lane);
      if (!mbar_wait(smem_u32(&ctl->tmem_full[acc]), acc_ph, abort_flag, p.status, JB200_STATUS_GEMM_EPILOGUE))
        goto done;
      tc_fence_after_sync();
      const int feat = tc.ft * BM + q * 32 + lane;
      const float alpha = dense_w ? 1.0f
                                  : __ldg(p.alpha + size_t(tc.group) * (p.N / p.alpha_rows) + feat / p.alpha_rows) *
                                        (p.w_layout ? 0.5f : 1.0f);   // prepared weights decode to +-2
      const uint32_t t_lane = tmem_base + (uint32_t(q * 32) << 16) + acc * BN_MAX;
      for (int c0 = half * 32; c0 < bn; c0 += 64) {
        if (tc.tok0 + c0 >= tc.tok_end) break;   // warp-uniform
        const int ntok = min(32, tc.tok_end - (tc.tok0 + c0));
        // the reductions go through the L2's atomic units, the register read-modify-write through the load/store
        // path: alternate chunks use one and the other, so both carry half of the tile
        store_acc_chunk(p, t_lane + c0, alpha, size_t(tc.tok0 + c0), tc.ft * BM + q * 32, ntok, lane, &tmap_out,
                        ((c0 >> 6) & 1) ? 0u : stage_smem);
      }
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&ctl->tmem_empty[acc]));
    }
    if (stage_smem && lane == 0) bulk_wait_group<0>();   // every reduction has landed before the CTA ends
  }

done:
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

int pick_bn(int M, int G, int n_ft, int sms) {
  if (M <= 32) return 32;
  // decode-size batches: the launch is latency-bound (16-32 K-blocks of one tile per CTA), and 64-token tiles
  // spread it over more SMs with shorter MMA and epilogue phases per CTA (measured 2 us less per launch)
  if (M <= 512) return 64;
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
                        int bn_override, int w_layout, cudaStream_t stream, const GemmRope* rope) {
  JB_REQUIRE(M >= 0 && N > 0 && K > 0, "ternary_linear: bad sizes M=%d N=%d K=%d", M, N, K);
  JB_REQUIRE(N % BM == 0, "ternary_linear: out_features (%d) must be a multiple of %d", N, BM);
  JB_REQUIRE(K % BK == 0, "ternary_linear: in_features (%d) must be a multiple of %d", K, BK);
  JB_REQUIRE(G >= 1 && G <= MAX_GROUPS, "ternary_linear: groups (%d) must be in 1..%d", G, MAX_GROUPS);
  JB_REQUIRE(G == 1 || seg_offsets != nullptr, "ternary_linear: grouped call needs segment offsets");
  JB_REQUIRE(alpha_rows > 0 && alpha_rows % BM == 0 && N % alpha_rows == 0,
             "ternary_linear: alpha_rows (%d) must be a multiple of %d dividing out_features", alpha_rows, BM);
  JB_REQUIRE(epilogue >= JB200_EPI_BF16 && epilogue <= JB200_EPI_QK_ROPE_BF16, "ternary_linear: unknown epilogue %d", epilogue);
  JB_REQUIRE((epilogue == JB200_EPI_QK_ROPE_BF16) == (rope != nullptr), "ternary_linear: the q/k RoPE epilogue needs its tables (use jb200_qkv_linear_rope)");
  if (rope) {
    JB_REQUIRE(G == 1, "qkv_linear_rope: no grouped form");
    JB_REQUIRE(rope->cos_tab && rope->sin_tab && rope->n_pos >= 1, "qkv_linear_rope: RoPE tables missing");
    JB_REQUIRE(rope->T >= 1 && M % rope->T == 0, "qkv_linear_rope: rows (%d) must be a multiple of the sequence length (%d)", M, rope->T);
    JB_REQUIRE(rope->rope_feats >= 0 && rope->rope_feats <= N && rope->rope_feats % 64 == 0,
               "qkv_linear_rope: rotated features (%d) must be whole 64-wide heads within out_features", rope->rope_feats);
  }
  JB_REQUIRE(w_layout >= 0 && w_layout <= 2, "ternary_linear: weight layout must be 0 (canonical), 1 (prepared) or 2 (dense bf16)");
  JB_REQUIRE(w_layout != 2 || (G == 1 && !rope && (epilogue == JB200_EPI_BF16 || epilogue == JB200_EPI_F32)),
             "dense_linear: one weight matrix, plain bf16 or f32 output");
  if (M == 0) return JB200_OK;   // nothing to do: an empty batch may come with null row pointers
  JB_REQUIRE(x_bf16 && w_packed && (alpha || w_layout == 2) && out, "ternary_linear: null pointer");
  JB_REQUIRE(aligned16(x_bf16) && aligned16(w_packed) && aligned16(out), "ternary_linear: pointers must be 16-byte aligned");
  if (M == 0) return JB200_OK;
  const int sms = sm_count();
  if (sms <= 0) return JB200_ERR_CUDA;
  const int n_ft = N / BM;
  JB_REQUIRE(bn_override == 0 || bn_override == 32 || bn_override == 64 || bn_override == 128 || bn_override == 256,
             "ternary_linear: token tile %d not in {32,64,128,256}", bn_override);
  const int bn = bn_override > 0 ? bn_override : pick_bn(M, G, n_ft, sms);

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
  p.cos_tab = rope ? rope->cos_tab : nullptr;
  p.sin_tab = rope ? rope->sin_tab : nullptr;
  p.pos0 = rope ? rope->pos0 : nullptr;
  p.pos0_scalar = rope ? rope->pos0_scalar : 0;
  p.n_pos = rope ? rope->n_pos : 0;
  p.T = rope ? rope->T : 1;
  p.rope_feats = rope ? rope->rope_feats : 0;
  p.status = device_status_ptr();
  if (!p.status) return JB200_ERR_CUDA;

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


  CUtensorMap tmap_w = tmap;     // packed weights: the decoders read them with plain loads, the map is not used
  if (w_layout == 2) {
    const cuuint64_t wdim[2] = {cuuint64_t(K), cuuint64_t(N)};
    const cuuint32_t wbox[2] = {cuuint32_t(BK), cuuint32_t(BM)};
    cr = enc(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint8_t*>(w_packed), wdim, gstride, wbox, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) {
      set_error("dense_linear: cuTensorMapEncodeTiled failed for the weights (%d)", int(cr));
      return JB200_ERR_CUDA;
    }
  }

  // Residual epilogue of a single matrix: the tile is added to the f32 stream by TMA reductions (needs 16-byte
  // aligned rows); grouped calls and odd strides keep the read-modify-write from registers.
  CUtensorMap tmap_out = tmap;
  p.resid_stage_smem = 0;
  if (epilogue == JB200_EPI_RESID_F32 && G == 1 && N % 4 == 0 && aligned16(out)) {
    const cuuint64_t odim[2] = {cuuint64_t(N), cuuint64_t(M)};
    const cuuint64_t ostride[1] = {cuuint64_t(N) * 4};
    const cuuint32_t obox[2] = {32, 32};
    cr = enc(&tmap_out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, out, odim, ostride, obox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) {
      set_error("ternary_linear: cuTensorMapEncodeTiled failed for the residual stream (%d)", int(cr));
      return JB200_ERR_CUDA;
    }
    p.resid_stage_smem = 1;
  }
  const size_t smem_bytes = p.resid_stage_smem ? SMEM_BYTES_RESID : SMEM_BYTES;

  // per device and cheap: set on every call rather than remembering which devices have seen it
  JB_CUDA(cudaFuncSetAttribute(ternary_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM_BYTES_RESID)));
  const long max_tiles = long((M + bn - 1) / bn + (G - 1)) * n_ft;
  const int grid = int(max_tiles < sms ? max_tiles : sms);
  launch_dep(ternary_gemm_kernel, grid, NUM_THREADS, smem_bytes, stream, tmap, tmap_w, tmap_out, p);
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
