// Scalar-decay associative linear-attention causal scan on the 5th-generation tensor cores, fused with its prologue.
//
//   q <- (ELU(q)+1)/sqrt(D),  k <- ELU(k)+1,  half-split RoPE on both   (jarvis_model.py:124-128, :29-71;
//                                                                      fused kernel A1, associative_attention_cuda.cu:28-112)
//   S_t = gamma*S_{t-1} + v_t (x) k_t,   o_t = S_t q_t                  (jarvis_model.py:131-190)
//   optional initial state S_in and final state S_out (B, H, D_v, D_k)  (associative_attention.py:126-152, :273-308;
//                                                                      kernel A3, associative_attention_cuda.cu:218-265)
//
// The reference's chunk-parallel path does the four chunk products as batched library GEMMs over materialised
// per-chunk states (associative_attention.py:242-266).  Here one CTA per (sequence, head, segment) walks its part
// of the sequence in 128-token chunks and issues the same four products as tcgen05.mma (bf16 operands from shared
// memory, fp32 accumulators in tensor memory); the state S never leaves the SM (fp32 master copy in registers,
// bf16 copy in shared memory as an MMA operand), so HBM traffic is q, k, v in / o out (512 B per token-head)
// plus one optional state load / store per (sequence, head).  Chunk length is free: the chunked form equals
// the recurrence for any length, only rounding differs.
//
// Per chunk of c <= 128 tokens (i, j: query / key token inside the chunk; g = gamma):
//   TMA (128B-swizzled [128 tokens][64] boxes)                        ->  q, k, v tiles in shared memory
//   all threads: feature map + RoPE in place on q and k;  kw[j] = k'[j] * g^(c-1-j)
//   MMA  A:  scores = Q' K'^T       (M=128 i, N=128 j, K=64; both operands K-major)             -> TMEM [0,128)
//            O2     = Q' S^T        (M=128 i, N=64 dv, K=64; S bf16 [dv][dk] is K-major)        -> TMEM [128,192)
//   MMA  S:  dS     = V^T Kw        (M=dv, N=dk, K=128 j; both operands are the [token][64] tiles read
//                                    MN-major; M is padded to 128 by reading the 64 dv twice)    -> TMEM [192,256)
//   all threads: P[i][j] = scores * g^(i-j) / 8 for j <= i, else 0      (TMEM -> registers -> bf16 tile in smem)
//   MMA  B:  O1     = P V           (M=128 i, N=64 dv, K=128 j; V read MN-major from its raw tile) -> TMEM [0,64)
//   all threads: S = g^c S + dS (registers; bf16 copy to smem);   o[i] = O1 + g^(i+1)/8 * O2  -> global
// One thread issues the TMA loads and the MMAs; every wait (TMA arrival, MMA completion) is an mbarrier wait
// bounded in time.  256 TMEM columns, 105 KiB of shared memory and <= 128 registers per thread let two CTAs
// share an SM and cover each other's latencies.
//
// Sequence segments: when B*H alone cannot fill the GPU (prefill of a few long sequences), T is cut into
// segments.  A first launch (STATE_ONLY) runs only the k/v half of the work for every non-final segment from a
// zero state and stores its contribution D_s; the main launch starts segment s from
// S = fold_{s' < s}(gamma^L S + D_s'), which is exact because the recurrence is linear in S.
// Extra HBM traffic: k and v of the non-final segments are read twice (the second time mostly from L2).
#include <type_traits>

#include "common.cuh"
#include "launchers.h"

namespace jb {

namespace {

constexpr int D = 64;             // head dim (fixed by the path: 16 heads x 64)
constexpr int CH = 128;           // tokens per chunk = rows of one MMA tile
constexpr int TILE_BYTES = CH * D * 2;          // 16 KiB: [128 tokens][64 bf16], 128B-swizzled
constexpr int S_BYTES = D * D * 2;              // 8 KiB: bf16 state [dv][dk]

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
  float* seg_state;        // [B][H][n_pieces][64][64]: state contribution of each piece
  int n_pieces;            // pieces stored per (sequence, head): nseg - 1, or nseg in a state-only call
  int qk_prepared;         // q, k already hold phi(.) + RoPE with the head dim interleaved (d, d+32 adjacent)
  int wide_store;          // output rows are 32-byte aligned: 256-bit stores
  // Balanced launch (more sequence-heads than SMs, a partly filled last wave): the first n_split sequence-heads are
  // cut in two at chunk split_chunk.  CTAs take tickets from ctrl[0]; tickets [0, n_split) are the first parts,
  // [n_split, B*H) whole sequence-heads, [B*H, B*H + n_split) the second parts, which find the state after the
  // first part in handoff[unit] once ctrl[1 + unit] has counted the eight consumer warps that wrote it.
  int n_split, split_chunk;
  float* handoff;          // [n_split][64][64] f32
  int* ctrl;               // [1 + n_split], zeroed before the launch
  unsigned int* status;
};

__device__ __forceinline__ uint32_t swz(int row, int chunk16) {  // byte offset inside a swizzled [rows][128 B] tile
  return uint32_t(row) * 128u + (uint32_t(chunk16 ^ (row & 7)) << 4);
}

// Shared-memory matrix descriptor, 128-byte swizzle.  K-major operands (rows of 64 K-elements): lbo is unused
// (16), sbo = 1024 is the distance between 8-row groups.  MN-major operands (a [K rows][64 MN-elements] tile):
// sbo = 1024 is the distance between groups of 8 K rows, lbo the distance between blocks of 64 MN-elements.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// kind::f16 instruction descriptor: bf16 operands, fp32 accumulator; a_mn / b_mn = 1 reads that operand MN-major.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n, int a_mn, int b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(a_mn) << 15) | (uint32_t(b_mn) << 16) |
         (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void st_global_256(void* p, const uint32_t* w) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}

// ELU(x)+1 = max(x, 0) + exp(min(x, 0)) = (x + |x|)/2 + 2^((x - |x|) * log2(e)/2): two adds, one multiply, one
// ex2.approx (flush-to-zero form: a single MUFU, rel. error 2^-22, far below the bf16 rounding of the result) and
// one fused multiply-add, all on the FMA / MUFU pipes - no compare, no select.  For x > 0 the exponent is exactly
// 0 and the result is x + 1 rounded once; for x <= 0 the first term is exactly 0.
__device__ __forceinline__ float elu1(float x) {
  const float ax = fabsf(x);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"((x - ax) * 0.72134752044448170368f));
  return fmaf(x + ax, 0.5f, e);
}

// ------------------------------------------------------------------------------------------------------------
// k/v-only pass: the state contribution of one piece of a sequence from a zero state (pieces = the non-final
// segments of a full call, or all pieces of a state-only call).  One CTA per (sequence, head, piece), 256 threads,
// two CTAs per SM.  Per chunk: TMA k, v (two stages) -> kw = phi(k) with RoPE, times gamma^(c-1-j) ->
// dS = V^T Kw as tcgen05.mma (accumulator in TMEM) -> S = gamma^c S + dS in registers.  The feature map, the
// angles and the rounding of kw are instruction for instruction those of the pipeline kernel's prologue, so a
// segmented call and an unsegmented one see the same bf16 operands.
// ------------------------------------------------------------------------------------------------------------
constexpr int STATE_THREADS = 256;
constexpr uint32_t STATE_TMEM_COLS = 64;

struct StateSmem {
  uint8_t k[2][TILE_BYTES];
  uint8_t v[2][TILE_BYTES];
  uint8_t kw[TILE_BYTES];
  float pw[CH + 1];            // gamma^n
  uint64_t full[2], bar_s;
  uint32_t tmem_base;
  uint32_t abort_flag;
};
constexpr size_t STATE_SMEM_BYTES = sizeof(StateSmem) + 1024;

__global__ void __launch_bounds__(STATE_THREADS, 2)
attn_state_pass_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                       const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  StateSmem* sm = reinterpret_cast<StateSmem*>(smem_raw + (base - raw_addr));

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qd = warp & 3;          // TMEM lane quarter this warp may access
  const int hf = warp >> 2;
  const int h = blockIdx.x, b = blockIdx.y, seg = blockIdx.z;
  const int T = p.T;
  const int n_chunks = (T + CH - 1) / CH;
  const int ck_begin = seg * p.seg_chunks;
  const int ck_end = min(n_chunks, ck_begin + p.seg_chunks);
  const int row0 = b * T;

  if (tid == 0) {
    mbar_init(smem_u32(&sm->full[0]), 1);
    mbar_init(smem_u32(&sm->full[1]), 1);
    mbar_init(smem_u32(&sm->bar_s), 1);
    sm->abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 0) {
    __syncwarp();                 // tcgen05.alloc is warp-collective: lane 0 rejoins from the barrier set-up first
    tmem_alloc(smem_u32(&sm->tmem_base), STATE_TMEM_COLS);
    tmem_relinquish();
  }
  pdl_wait();        // everything above overlapped the kernel before this one; global memory is read from here on
  pdl_trigger();
  const int pos_base = p.pos0 ? p.pos0[b] : p.pos0_scalar;
  const float log_g = logf(__ldg(p.gamma + h));
  for (int n = tid; n <= CH; n += STATE_THREADS) sm->pw[n] = expf(log_g * float(n));
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tm = sm->tmem_base;
  const uint32_t tm_lane = tm + (uint32_t(32 * qd) << 16);

  auto issue = [&](int ck) {      // thread 0 only
    const int st = (ck - ck_begin) & 1;
    const uint32_t bar = smem_u32(&sm->full[st]);
    mbar_arrive_expect_tx(bar, 2 * TILE_BYTES);
    tma_load_2d(smem_u32(sm->k[st]), &tm_k, h * D, row0 + ck * CH, bar);
    tma_load_2d(smem_u32(sm->v[st]), &tm_v, h * D, row0 + ck * CH, bar);
  };
  if (tid == 0) {
    for (int ck = ck_begin; ck < ck_begin + 2 && ck < ck_end; ++ck) issue(ck);
  }

  // the thread's share of the state: row dv = 32*(qd&1) + lane, columns 16*cg .. 16*cg+15 (see the pipeline kernel)
  const int s_row = 32 * (qd & 1) + lane;
  const int s_cg = 2 * (qd >> 1) + hf;
  float S[16];
#pragma unroll
  for (int e = 0; e < 16; ++e) S[e] = 0.f;

  const int cg = tid & 3;
  const int r_lo = (tid >> 5) * 8 + ((tid >> 2) & 1) * 4 + ((tid >> 3) & 3);
  float c64[8], s64[8];
  {
    const int stp = 64 < p.n_pos ? 64 : p.n_pos - 1;
    const float4* cq = reinterpret_cast<const float4*>(p.cos_tab + size_t(stp) * 32 + cg * 8);
    const float4* sq = reinterpret_cast<const float4*>(p.sin_tab + size_t(stp) * 32 + cg * 8);
    const float4 d0 = __ldg(cq), d1 = __ldg(cq + 1), e0 = __ldg(sq), e1 = __ldg(sq + 1);
    c64[0] = d0.x; c64[1] = d0.y; c64[2] = d0.z; c64[3] = d0.w; c64[4] = d1.x; c64[5] = d1.y; c64[6] = d1.z; c64[7] = d1.w;
    s64[0] = e0.x; s64[1] = e0.y; s64[2] = e0.z; s64[3] = e0.w; s64[4] = e1.x; s64[5] = e1.y; s64[6] = e1.z; s64[7] = e1.w;
  }

  bool ok = true;
  for (int ck = ck_begin; ck < ck_end; ++ck) {
    const int lc = ck - ck_begin;
    const int st = lc & 1;
    const int c_len = min(CH, T - ck * CH);
    const uint8_t* k_p = sm->k[st];
    float cs[8], sn[8];
    if (!p.qk_prepared) {         // angles of the thread's first row (in flight during the wait below)
      int pos = pos_base + ck * CH + r_lo;
      pos = pos < 0 ? 0 : (pos >= p.n_pos ? p.n_pos - 1 : pos);
      const float4* cp = reinterpret_cast<const float4*>(p.cos_tab + size_t(pos) * 32 + cg * 8);
      const float4* sp = reinterpret_cast<const float4*>(p.sin_tab + size_t(pos) * 32 + cg * 8);
      const float4 a0 = __ldg(cp), a1 = __ldg(cp + 1), b0 = __ldg(sp), b1 = __ldg(sp + 1);
      cs[0] = a0.x; cs[1] = a0.y; cs[2] = a0.z; cs[3] = a0.w; cs[4] = a1.x; cs[5] = a1.y; cs[6] = a1.z; cs[7] = a1.w;
      sn[0] = b0.x; sn[1] = b0.y; sn[2] = b0.z; sn[3] = b0.w; sn[4] = b1.x; sn[5] = b1.y; sn[6] = b1.z; sn[7] = b1.w;
    }
    if (!mbar_wait(smem_u32(&sm->full[st]), uint32_t(lc >> 1) & 1u, &sm->abort_flag, p.status, JB200_STATUS_ATTN_LOAD)) ok = false;
    if (ok) {
#pragma unroll
      for (int it = 0; it < 2; ++it) {
        const int r = r_lo + 64 * it;
        const float w = r < c_len ? sm->pw[c_len - 1 - r] : 0.f;   // rows past the end contribute nothing
        const uint4 lo = *reinterpret_cast<const uint4*>(k_p + swz(r, cg));
        const uint4 hi = *reinterpret_cast<const uint4*>(k_p + swz(r, cg + 4));
        const uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w}, hw[4] = {hi.x, hi.y, hi.z, hi.w};
        uint32_t wl[4], wh[4];
        if (p.qk_prepared) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            wl[j] = pack_bf16x2(bf16_lo(lw[j]) * w, bf16_hi(lw[j]) * w);
            wh[j] = pack_bf16x2(bf16_lo(hw[j]) * w, bf16_hi(hw[j]) * w);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float a0 = elu1(bf16_lo(lw[j])), a1 = elu1(bf16_hi(lw[j]));   // d
            const float b0 = elu1(bf16_lo(hw[j])), b1 = elu1(bf16_hi(hw[j]));   // d + 32
            const float l0 = a0 * cs[2 * j] - b0 * sn[2 * j], l1 = a1 * cs[2 * j + 1] - b1 * sn[2 * j + 1];
            const float h0 = b0 * cs[2 * j] + a0 * sn[2 * j], h1 = b1 * cs[2 * j + 1] + a1 * sn[2 * j + 1];
            wl[j] = pack_bf16x2(l0 * w, l1 * w);
            wh[j] = pack_bf16x2(h0 * w, h1 * w);
          }
          if (it == 0) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float cn = cs[e] * c64[e] - sn[e] * s64[e];
              sn[e] = sn[e] * c64[e] + cs[e] * s64[e];
              cs[e] = cn;
            }
          }
        }
        *reinterpret_cast<uint4*>(sm->kw + swz(r, cg)) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
        *reinterpret_cast<uint4*>(sm->kw + swz(r, cg + 4)) = make_uint4(wh[0], wh[1], wh[2], wh[3]);
      }
    }
    fence_proxy_async_smem();   // kw -> visible to the tensor core; orders the reads of k before the next TMA write
    tc_fence_before_sync();
    if (__syncthreads_or(!ok)) { ok = false; break; }
    tc_fence_after_sync();
    if (tid == 0) {
      constexpr uint32_t id_ds = umma_idesc(128, 64, 1, 1);
      const uint32_t v_a = smem_u32(sm->v[st]), kw_a = smem_u32(sm->kw);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma_bf16_ss(tm, umma_desc(v_a + ks * 2048, 0, 1024), umma_desc(kw_a + ks * 2048, 1024, 1024), id_ds, ks != 0);
      umma_commit(smem_u32(&sm->bar_s));
    }
    if (!mbar_wait(smem_u32(&sm->bar_s), uint32_t(lc) & 1u, &sm->abort_flag, p.status, JB200_STATUS_ATTN_MMA)) ok = false;
    tc_fence_after_sync();
    if (tid == 0 && ok && ck + 2 < ck_end) issue(ck + 2);     // this chunk's k and v buffers are free again
    __syncwarp();
    if (ok) {
      uint32_t r[16];
      tmem_ld_32x16(tm_lane + 16 * s_cg, r);
      tmem_ld_wait();
      const float gc = sm->pw[c_len];
#pragma unroll
      for (int e = 0; e < 16; ++e) S[e] = gc * S[e] + __uint_as_float(r[e]);
    }
  }

  if (ok) {       // pieces stay in the kernel's own column order (interleaved when q/k were prepared)
    float* sp = p.seg_state + ((size_t(b) * p.H + h) * p.n_pieces + seg) * D * D + s_row * D + 16 * s_cg;
#pragma unroll
    for (int e4 = 0; e4 < 4; ++e4)
      *reinterpret_cast<float4*>(sp + 4 * e4) = make_float4(S[4 * e4], S[4 * e4 + 1], S[4 * e4 + 2], S[4 * e4 + 3]);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tm, STATE_TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------------------------
// The full pass as a warp-specialised pipeline: one CTA per SM, 576 threads, several chunks in flight.
//   warp 0       TMA producer: q, k, v tiles of chunk c+2 as soon as the MMAs that read stage c%2 have retired
//   warp 1       MMA issuer (one thread), per chunk c in this order:
//                  S(c)  dS = V^T Kw                 -> TMEM DS        (needs the prologue of c, v of c)
//                  A2(c) O2 = Q' S^T                  -> TMEM O2[c%2]   (needs the state after chunk c-1 in smem)
//                  B(c)  O1 = P V                     -> TMEM SC[c%2] columns 0-63 (needs P of c)
//                  A1(c+1) scores = Q' K'^T of the NEXT chunk -> TMEM SC[(c+1)%2]
//                so the scores of chunk c+1 are computed while the consumers finish chunk c
//   warps 2-9    prologue: feature map + RoPE in place on q and k of a stage, kw = k' * gamma^(c-1-j)
//   warps 10-17  consumers (two per TMEM lane quarter): decay mask scores -> P, state update, output rows
// Double-buffered: q/k/kw/v stages, score and O2 accumulators, the bf16 state copy.  Single: P (its reader,
// MMA B, has retired before the next mask step starts, because the output rows of a chunk wait for it).
// ------------------------------------------------------------------------------------------------------------
// Per-role cycle counters of one CTA (block 0,0,0), compiled in with -DJB_ATTN_TIMING only: every role adds the
// cycles it spends in each of its waits and work phases; a harness reads g_attn_timing after the launch.
#ifdef JB_ATTN_TIMING
__device__ long long g_attn_timing[18 * 8];
#define JB_T_DECL long long t_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long t_last = clock64();
#define JB_T_MARK(k) { const long long t_now = clock64(); t_acc[k] += t_now - t_last; t_last = t_now; }
#define JB_T_FLUSH(w) if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0) { for (int kk = 0; kk < 8; ++kk) g_attn_timing[(w) * 8 + kk] = t_acc[kk]; }
#else
#define JB_T_DECL
#define JB_T_MARK(k)
#define JB_T_FLUSH(w)
#endif

constexpr int PIPE_THREADS = 576;
constexpr int PRO_WARP0 = 2, CON_WARP0 = 10;
constexpr int NST = 3;                                       // stages of the q / k / kw / v tiles
constexpr uint32_t PIPE_TMEM_COLS = 512;
constexpr uint32_t PT_SC = 0, PT_O2 = 256, PT_DS = 384, PT_P = 448;   // SC[2] x 128, O2[2] x 64, DS x 64, P x 64

struct PipeSmem {
  uint8_t q[NST][TILE_BYTES];
  uint8_t k[NST][TILE_BYTES];
  uint8_t kw[NST][TILE_BYTES];
  uint8_t v[NST][TILE_BYTES];
  uint8_t s[2][S_BYTES];       // bf16 state copy, [n & 1] = state after n chunks of this CTA
  float pwm[2 * CH];           // pwm[x + CH] = gamma^x / 8 for x >= 0, 0 for x < 0: the decay mask by (i - j)
  float pw[CH + 1];            // gamma^n
  uint64_t full_qk[NST], full_v[NST], empty_qk[NST], empty_v[NST], pro_done[NST];
  uint64_t bar_sc[2], bar_b[2], o_done[2];
  uint64_t bar_s, s_done, p_done;
  uint32_t tmem_base;
  uint32_t abort_flag;
  int ticket;
};
constexpr size_t PIPE_SMEM_BYTES = sizeof(PipeSmem) + 1024;

__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__global__ void __launch_bounds__(PIPE_THREADS, 1)
attn_scan_pipe_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  PipeSmem* sm = reinterpret_cast<PipeSmem*>(smem_raw + (base - raw_addr));

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = p.T;
  const int n_chunks = (T + CH - 1) / CH;

  if (tid == 0) {
    for (int s = 0; s < NST; ++s) {
      mbar_init(smem_u32(&sm->full_qk[s]), 1);
      mbar_init(smem_u32(&sm->full_v[s]), 1);
      mbar_init(smem_u32(&sm->empty_qk[s]), 1);
      mbar_init(smem_u32(&sm->empty_v[s]), 1);
      mbar_init(smem_u32(&sm->pro_done[s]), 256);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&sm->bar_sc[s]), 1);
      mbar_init(smem_u32(&sm->bar_b[s]), 1);
      mbar_init(smem_u32(&sm->o_done[s]), 256);
    }
    mbar_init(smem_u32(&sm->bar_s), 1);
    mbar_init(smem_u32(&sm->s_done), 256);
    mbar_init(smem_u32(&sm->p_done), 256);
    sm->abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 0) {
    __syncwarp();                 // tcgen05.alloc is warp-collective: lane 0 rejoins from the barrier set-up first
    tmem_alloc(smem_u32(&sm->tmem_base), PIPE_TMEM_COLS);
    tmem_relinquish();
  }
  pdl_wait();        // everything above overlapped the kernel before this one; global memory is read from here on
  pdl_trigger();
  // Which chunks of which sequence-head this CTA scans.  piece: 0 a whole sequence-head or a pre-passed segment,
  // 1 the first part of a cut one (leaves its end state in handoff), 2 the second part (starts from it).
  int h = blockIdx.x, b = blockIdx.y, seg = blockIdx.z, piece = 0;
  int ck_begin = seg * p.seg_chunks, ck_end = min(n_chunks, ck_begin + p.seg_chunks);
  if (p.n_split > 0) {
    // a ticket instead of the block index: whoever holds a second part started after every first part was taken
    if (tid == 0) sm->ticket = atomicAdd(p.ctrl, 1);
    __syncthreads();
    const int t = sm->ticket, U = p.B * p.H;
    seg = 0;
    int unit = t;                                     // = b * H + h
    if (t < p.n_split) { piece = 1; ck_begin = 0; ck_end = p.split_chunk; }
    else if (t < U) { ck_begin = 0; ck_end = n_chunks; }
    else { unit = t - U; piece = 2; ck_begin = p.split_chunk; ck_end = n_chunks; }
    b = unit / p.H;
    h = unit - b * p.H;
  }
  const int n_loc = ck_end - ck_begin;
  const int row0 = b * T;
  const float log_g = logf(__ldg(p.gamma + h));
  for (int n = tid; n <= CH; n += PIPE_THREADS) sm->pw[n] = expf(log_g * float(n));
  for (int n = tid; n < 2 * CH; n += PIPE_THREADS) {
    // gamma^(i-j) / sqrt(D): the 1/8 of the query feature map is a power of two, so applying it to the scores
    // (and to the cross-chunk factor) instead of to every element of q gives the same bits
    const int x = n - CH;
    sm->pwm[n] = x >= 0 ? 0.125f * expf(log_g * float(x)) : 0.f;
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tm = sm->tmem_base;
  volatile uint32_t* abort_flag = &sm->abort_flag;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      JB_T_DECL
      int s = 0;
      uint32_t prev = 1u;                       // parity of the PREVIOUS use of the stage
      for (int lc = 0; lc < n_loc; ++lc) {
        const int r = row0 + (ck_begin + lc) * CH;
        JB_T_MARK(0)
        if (lc >= NST && !mbar_wait(smem_u32(&sm->empty_qk[s]), prev, abort_flag, p.status, JB200_STATUS_ATTN_LOAD)) break;
        JB_T_MARK(1)
        mbar_arrive_expect_tx(smem_u32(&sm->full_qk[s]), 2 * TILE_BYTES);
        tma_load_2d(smem_u32(sm->q[s]), &tm_q, h * D, r, smem_u32(&sm->full_qk[s]));
        tma_load_2d(smem_u32(sm->k[s]), &tm_k, h * D, r, smem_u32(&sm->full_qk[s]));
        JB_T_MARK(0)
        if (lc >= NST && !mbar_wait(smem_u32(&sm->empty_v[s]), prev, abort_flag, p.status, JB200_STATUS_ATTN_LOAD)) break;
        JB_T_MARK(2)
        mbar_arrive_expect_tx(smem_u32(&sm->full_v[s]), TILE_BYTES);
        tma_load_2d(smem_u32(sm->v[s]), &tm_v, h * D, r, smem_u32(&sm->full_v[s]));
        if (++s == NST) { s = 0; prev ^= 1u; }
      }
      JB_T_MARK(0)
      JB_T_FLUSH(0)
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t id_sc = umma_idesc(128, 128, 0, 0), id_o2 = umma_idesc(128, 64, 0, 0);
      constexpr uint32_t id_ds = umma_idesc(128, 64, 1, 1), id_o1 = umma_idesc(128, 64, 0, 1);
      // Operand descriptors of stage 0; stage s is +s*TILE_BYTES (+1024 in the address field).  A K-step of 16
      // elements is +32 bytes (+2) inside a K-major row, +2048 bytes (+128: two 8-row groups) in the MN-major
      // [token][64] tiles.
      constexpr uint64_t STG = TILE_BYTES >> 4;
      const uint64_t d_q0 = umma_desc(smem_u32(sm->q[0]), 16, 1024), d_k0 = umma_desc(smem_u32(sm->k[0]), 16, 1024);
      const uint64_t d_kw0 = umma_desc(smem_u32(sm->kw[0]), 1024, 1024);
      const uint64_t d_va0 = umma_desc(smem_u32(sm->v[0]), 0, 1024);      // as the M operand of dS: the 64 dv read twice
      const uint64_t d_vb0 = umma_desc(smem_u32(sm->v[0]), 1024, 1024);   // as the N operand of P V
      const uint64_t d_s0 = umma_desc(smem_u32(sm->s[0]), 16, 1024);
      auto issue_scores = [&](int stage, int buf) {
        const uint64_t dq = d_q0 + uint64_t(stage) * STG, dk = d_k0 + uint64_t(stage) * STG;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_bf16_ss(tm + PT_SC + 128 * buf, dq + uint64_t(ks * 2), dk + uint64_t(ks * 2), id_sc, ks != 0);
        umma_commit(smem_u32(&sm->bar_sc[buf]));
      };
      JB_T_DECL
      bool ok = n_loc > 0 && mbar_wait(smem_u32(&sm->pro_done[0]), 0u, abort_flag, p.status, JB200_STATUS_ATTN_MMA);
      JB_T_MARK(4)
      if (ok) {
        tc_fence_after_sync();
        issue_scores(0, 0);
      }
      int s = 0;                                 // stage of chunk lc
      uint32_t sp = 0u;                          // parity of this use of the stage
      for (int lc = 0; ok && lc < n_loc; ++lc) {
        const int buf = lc & 1;                  // accumulator buffers SC / O2 and the state copy alternate
        const uint32_t u = uint32_t(lc >> 1) & 1u;
        const int s1 = s + 1 == NST ? 0 : s + 1; // stage and parity of chunk lc + 1
        const uint32_t sp1 = s + 1 == NST ? sp ^ 1u : sp;
        const uint64_t dq = d_q0 + uint64_t(s) * STG, dkw = d_kw0 + uint64_t(s) * STG;
        const uint64_t dva = d_va0 + uint64_t(s) * STG, dvb = d_vb0 + uint64_t(s) * STG;
        const uint64_t ds = d_s0 + uint64_t(buf) * (S_BYTES >> 4);
        // S(lc): needs v of the chunk, and the consumers to be done with the previous dS (completion #lc of s_done,
        // which also says that s[lc & 1] holds the state after lc chunks)
        JB_T_MARK(0)
        if (!mbar_wait(smem_u32(&sm->full_v[s]), sp, abort_flag, p.status, JB200_STATUS_ATTN_LOAD)) break;
        JB_T_MARK(1)
        if (!mbar_wait(smem_u32(&sm->s_done), uint32_t(lc) & 1u, abort_flag, p.status, JB200_STATUS_ATTN_MMA)) break;
        JB_T_MARK(2)
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_bf16_ss(tm + PT_DS, dva + uint64_t(ks * 128), dkw + uint64_t(ks * 128), id_ds, ks != 0);
        umma_commit(smem_u32(&sm->bar_s));
        // A2(lc): O2 = Q' S^T.  O2[buf] was read by the output rows of chunk lc - 2, which the scores of this chunk
        // (issued into SC[buf] earlier) already waited for.
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_bf16_ss(tm + PT_O2 + 64 * buf, dq + uint64_t(ks * 2), ds + uint64_t(ks * 2), id_o2, ks != 0);
        umma_commit(smem_u32(&sm->empty_qk[s]));       // q, k, kw of this stage: every MMA that reads them is issued
        // A1(lc + 1): scores of the next chunk into the other accumulator, ahead of B(lc) when the next chunk's
        // prologue is already done (then the consumers find them ready when they finish this chunk)
        bool scores_issued = lc + 1 >= n_loc;
        if (!scores_issued && mbar_try_wait(smem_u32(&sm->pro_done[s1]), sp1) &&
            (lc + 1 < 2 || mbar_try_wait(smem_u32(&sm->o_done[buf ^ 1]), (uint32_t((lc + 1) >> 1) - 1u) & 1u))) {
          tc_fence_after_sync();
          issue_scores(s1, buf ^ 1);
          scores_issued = true;
        }
        // B(lc): O1 = P V into the score columns the mask step has fully read; P (bf16 pairs) is read from TMEM
        JB_T_MARK(0)
        if (!mbar_wait(smem_u32(&sm->p_done), uint32_t(lc) & 1u, abort_flag, p.status, JB200_STATUS_ATTN_MMA)) break;
        JB_T_MARK(3)
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_bf16_ts(tm + PT_SC + 128 * buf, tm + PT_P + ks * 8, dvb + uint64_t(ks * 128), id_o1, ks != 0);
        umma_commit(smem_u32(&sm->bar_b[buf]));
        umma_commit(smem_u32(&sm->empty_v[s]));
        if (!scores_issued) {
          JB_T_MARK(0)
          if (!mbar_wait(smem_u32(&sm->pro_done[s1]), sp1, abort_flag, p.status, JB200_STATUS_ATTN_MMA)) break;
          JB_T_MARK(4)
          if (lc + 1 >= 2 && !mbar_wait(smem_u32(&sm->o_done[buf ^ 1]), (uint32_t((lc + 1) >> 1) - 1u) & 1u, abort_flag,
                                        p.status, JB200_STATUS_ATTN_MMA)) break;
          JB_T_MARK(5)
          tc_fence_after_sync();
          issue_scores(s1, buf ^ 1);
        }
        (void)u;
        s = s1;
        sp = sp1;
      }
      JB_T_MARK(0)
      JB_T_FLUSH(1)
    }
  } else if (warp < CON_WARP0) {
    // ---------------- prologue warps ----------------
    const int ptid = tid - PRO_WARP0 * 32;
    const int pos_base = p.pos0 ? p.pos0[b] : p.pos0_scalar;
    // 128 rows x 4 column groups of 8 rotary pairs = 512 items per chunk, two per thread: (row r, group cg) and
    // (row r + 64, group cg).  Eight consecutive lanes take 4 groups of two rows that are 4 apart, so that their
    // 16-byte accesses to the swizzled tiles fall into different banks.
    const int cg = ptid & 3;
    const int r_lo = (ptid >> 5) * 8 + ((ptid >> 2) & 1) * 4 + ((ptid >> 3) & 3);
    // RoPE angles: the thread's 8 frequencies are fixed.  The angles of its first row come from the table (the
    // loads for the NEXT chunk are issued when a chunk is finished, so their latency passes during the wait for
    // that chunk's tiles); its second row is 64 positions further, one fixed rotation by (cos, sin)(64 theta_i)
    // away (angle addition in f32: error ~1e-7 against the 4e-3 of the bf16 result).  Every chunk starts from
    // the table again, so results do not depend on how a sequence is cut into segments or calls.
    float cs[8], sn[8], c64[8], s64[8];
    auto load_angles = [&](int ck) {
      int pos = pos_base + ck * CH + r_lo;
      pos = pos < 0 ? 0 : (pos >= p.n_pos ? p.n_pos - 1 : pos);
      const float4* cp = reinterpret_cast<const float4*>(p.cos_tab + size_t(pos) * 32 + cg * 8);
      const float4* sp = reinterpret_cast<const float4*>(p.sin_tab + size_t(pos) * 32 + cg * 8);
      const float4 a0 = __ldg(cp), a1 = __ldg(cp + 1), b0 = __ldg(sp), b1 = __ldg(sp + 1);
      cs[0] = a0.x; cs[1] = a0.y; cs[2] = a0.z; cs[3] = a0.w; cs[4] = a1.x; cs[5] = a1.y; cs[6] = a1.z; cs[7] = a1.w;
      sn[0] = b0.x; sn[1] = b0.y; sn[2] = b0.z; sn[3] = b0.w; sn[4] = b1.x; sn[5] = b1.y; sn[6] = b1.z; sn[7] = b1.w;
    };
    {
      const int stp = 64 < p.n_pos ? 64 : p.n_pos - 1;     // tables shorter than 65 rows: rows >= 64 are past the end anyway
      const float4* cq = reinterpret_cast<const float4*>(p.cos_tab + size_t(stp) * 32 + cg * 8);
      const float4* sq = reinterpret_cast<const float4*>(p.sin_tab + size_t(stp) * 32 + cg * 8);
      const float4 d0 = __ldg(cq), d1 = __ldg(cq + 1), e0 = __ldg(sq), e1 = __ldg(sq + 1);
      c64[0] = d0.x; c64[1] = d0.y; c64[2] = d0.z; c64[3] = d0.w; c64[4] = d1.x; c64[5] = d1.y; c64[6] = d1.z; c64[7] = d1.w;
      s64[0] = e0.x; s64[1] = e0.y; s64[2] = e0.z; s64[3] = e0.w; s64[4] = e1.x; s64[5] = e1.y; s64[6] = e1.z; s64[7] = e1.w;
      load_angles(ck_begin);
    }
    JB_T_DECL
    int s = 0;
    uint32_t sp = 0u;
    for (int lc = 0; lc < n_loc; ++lc) {
      const int ck = ck_begin + lc;
      const int c_len = min(CH, T - ck * CH);
      uint8_t* q_p = sm->q[s];
      uint8_t* k_p = sm->k[s];
      uint8_t* kw_p = sm->kw[s];
      JB_T_MARK(0)
      if (!mbar_wait(smem_u32(&sm->full_qk[s]), sp, abort_flag, p.status, JB200_STATUS_ATTN_LOAD)) break;
      JB_T_MARK(1)
#pragma unroll
      for (int it = 0; it < 2; ++it) {
        const int r = r_lo + 64 * it;
        const float w = r < c_len ? sm->pw[c_len - 1 - r] : 0.f;   // rows past the end contribute nothing
        if (p.qk_prepared) {
          // q', k' came out of the projection's epilogue: only the decay-weighted copy of k is made here
          const uint4 lo = *reinterpret_cast<const uint4*>(k_p + swz(r, cg));
          const uint4 hi = *reinterpret_cast<const uint4*>(k_p + swz(r, cg + 4));
          *reinterpret_cast<uint4*>(kw_p + swz(r, cg)) =
              make_uint4(pack_bf16x2(bf16_lo(lo.x) * w, bf16_hi(lo.x) * w), pack_bf16x2(bf16_lo(lo.y) * w, bf16_hi(lo.y) * w),
                         pack_bf16x2(bf16_lo(lo.z) * w, bf16_hi(lo.z) * w), pack_bf16x2(bf16_lo(lo.w) * w, bf16_hi(lo.w) * w));
          *reinterpret_cast<uint4*>(kw_p + swz(r, cg + 4)) =
              make_uint4(pack_bf16x2(bf16_lo(hi.x) * w, bf16_hi(hi.x) * w), pack_bf16x2(bf16_lo(hi.y) * w, bf16_hi(hi.y) * w),
                         pack_bf16x2(bf16_lo(hi.z) * w, bf16_hi(hi.z) * w), pack_bf16x2(bf16_lo(hi.w) * w, bf16_hi(hi.w) * w));
          continue;
        }
        // all four 16-byte pieces of the row pair first, so that their latencies overlap
        uint4* ql_p = reinterpret_cast<uint4*>(q_p + swz(r, cg));
        uint4* qh_p = reinterpret_cast<uint4*>(q_p + swz(r, cg + 4));
        uint4* kl_p = reinterpret_cast<uint4*>(k_p + swz(r, cg));
        uint4* kh_p = reinterpret_cast<uint4*>(k_p + swz(r, cg + 4));
        const uint4 ql = *ql_p, qh = *qh_p, kl = *kl_p, kh = *kh_p;
#pragma unroll
        for (int which = 0; which < 2; ++which) {  // 0: q, 1: k
          const uint4 lo = which == 0 ? ql : kl, hi = which == 0 ? qh : kh;
          const uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w}, hw[4] = {hi.x, hi.y, hi.z, hi.w};
          uint32_t ol[4], oh[4], wl[4], wh[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float a0 = elu1(bf16_lo(lw[j])), a1 = elu1(bf16_hi(lw[j]));   // d
            const float b0 = elu1(bf16_lo(hw[j])), b1 = elu1(bf16_hi(hw[j]));   // d + 32
            // x*cos + rotate_half(x)*sin:  out[d] = x[d]cos - x[d+32]sin,  out[d+32] = x[d+32]cos + x[d]sin
            const float l0 = a0 * cs[2 * j] - b0 * sn[2 * j], l1 = a1 * cs[2 * j + 1] - b1 * sn[2 * j + 1];
            const float h0 = b0 * cs[2 * j] + a0 * sn[2 * j], h1 = b1 * cs[2 * j + 1] + a1 * sn[2 * j + 1];
            ol[j] = pack_bf16x2(l0, l1);
            oh[j] = pack_bf16x2(h0, h1);
            if (which == 1) {
              wl[j] = pack_bf16x2(l0 * w, l1 * w);
              wh[j] = pack_bf16x2(h0 * w, h1 * w);
            }
          }
          *(which == 0 ? ql_p : kl_p) = make_uint4(ol[0], ol[1], ol[2], ol[3]);
          *(which == 0 ? qh_p : kh_p) = make_uint4(oh[0], oh[1], oh[2], oh[3]);
          if (which == 1) {
            *reinterpret_cast<uint4*>(kw_p + swz(r, cg)) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
            *reinterpret_cast<uint4*>(kw_p + swz(r, cg + 4)) = make_uint4(wh[0], wh[1], wh[2], wh[3]);
          }
        }
        if (it == 0) {             // advance the angles by 64 positions: to the thread's second row
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float cn = cs[e] * c64[e] - sn[e] * s64[e];
            sn[e] = sn[e] * c64[e] + cs[e] * s64[e];
            cs[e] = cn;
          }
        }
      }
      if (!p.qk_prepared && lc + 1 < n_loc) load_angles(ck + 1);
      JB_T_MARK(2)
      fence_proxy_async_smem();                          // generic-proxy writes -> visible to the tensor core
      mbar_arrive(smem_u32(&sm->pro_done[s]));
      JB_T_MARK(3)
      if (++s == NST) { s = 0; sp ^= 1u; }
    }
    JB_T_FLUSH(warp)
  } else {
    // ---------------- consumers ----------------
    const int qd = warp & 3;                             // TMEM lane quarter of this warp
    const int hf = (warp - CON_WARP0) >> 2;              // which half of the columns it takes
    const uint32_t tm_lane = tm + (uint32_t(32 * qd) << 16);
    const int i = 32 * qd + lane;                        // query row = TMEM lane
    // fp32 state: row dv = 32*(qd&1) + lane, columns dk = 16*cg .. 16*cg+15 (the accumulator of MMA S holds the
    // 64 dv rows twice, lanes 0-63 and 64-127, so every consumer warp finds its share in its own lane quarter)
    const int s_row = 32 * (qd & 1) + lane;
    const int s_cg = 2 * (qd >> 1) + hf;
    const size_t bh = size_t(b) * p.H + h;
    // P lives in TMEM as bf16 pairs: lane = query row, column c = keys 2c, 2c+1.  32-key blocks above the diagonal
    // of this warp's rows are never written by the mask step: zero them once.
    {
      uint32_t z[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) z[e] = 0u;
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const int jb = 2 * hf + jj;
        if (jb > qd) tmem_st_32x16(tm_lane + PT_P + 16 * jb, z);
      }
      tmem_st_wait();
    }
    float S[16];
    if (piece == 2) {
      // second part of a cut sequence-head: the state after the first part, written by the eight consumer warps of
      // the CTA that scanned it (in this kernel's own element order).  Bounded wait on their count.
      int* flag = p.ctrl + 1 + bh;
      if (lane == 0) {
        const unsigned long long t0 = globaltimer_ns();
        int seen;
        for (;;) {
          asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
          if (seen >= 8 || *abort_flag) break;
          if (globaltimer_ns() - t0 > JB_WAIT_LIMIT_NS) {
            *abort_flag = 1u;
            atomicCAS(p.status, 0u, JB200_STATUS_ATTN_HANDOFF);
            break;
          }
          __nanosleep(200);
        }
      }
      __syncwarp();
      __threadfence();
      const float* hp = p.handoff + bh * D * D + s_row * D + 16 * s_cg;
#pragma unroll
      for (int e4 = 0; e4 < 4; ++e4) {
        const float4 v4 = __ldcg(reinterpret_cast<const float4*>(hp) + e4);
        S[4 * e4] = v4.x; S[4 * e4 + 1] = v4.y; S[4 * e4 + 2] = v4.z; S[4 * e4 + 3] = v4.w;
      }
    } else {
      const float* sin_p = p.s_in ? p.s_in + bh * D * D + s_row * D : nullptr;
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const int c = 16 * s_cg + e;
        const int d = p.qk_prepared ? (c >> 1) + 32 * (c & 1) : c;   // prepared q/k: the dk axis is interleaved
        S[e] = sin_p ? __ldg(sin_p + d) : 0.f;
      }
      if (seg > 0) {   // state entering this segment: fold the earlier segments' contributions, oldest first
        const float gL = expf(log_g * float(p.seg_chunks * CH));
        const float* dp = p.seg_state + bh * p.n_pieces * D * D + s_row * D + 16 * s_cg;
        for (int s2 = 0; s2 < seg; ++s2, dp += D * D) {
#pragma unroll
          for (int e4 = 0; e4 < 4; ++e4) {
            const float4 v4 = __ldg(reinterpret_cast<const float4*>(dp) + e4);
            S[4 * e4 + 0] = gL * S[4 * e4 + 0] + v4.x; S[4 * e4 + 1] = gL * S[4 * e4 + 1] + v4.y;
            S[4 * e4 + 2] = gL * S[4 * e4 + 2] + v4.z; S[4 * e4 + 3] = gL * S[4 * e4 + 3] + v4.w;
          }
        }
      }
    }
    auto publish_state = [&](int buf) {
      uint32_t w[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) w[e] = pack_bf16x2(S[2 * e], S[2 * e + 1]);
      *reinterpret_cast<uint4*>(sm->s[buf] + swz(s_row, 2 * s_cg)) = make_uint4(w[0], w[1], w[2], w[3]);
      *reinterpret_cast<uint4*>(sm->s[buf] + swz(s_row, 2 * s_cg + 1)) = make_uint4(w[4], w[5], w[6], w[7]);
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&sm->s_done));
    };
    publish_state(0);
    bool ok = true;
    JB_T_DECL
    for (int lc = 0; lc < n_loc; ++lc) {
      const int buf = lc & 1;
      const uint32_t u = uint32_t(lc >> 1) & 1u;
      const int ck = ck_begin + lc;
      const int c_len = min(CH, T - ck * CH);
      // ---- decay mask: scores -> P ----
      JB_T_MARK(0)
      if (!mbar_wait(smem_u32(&sm->bar_sc[buf]), u, abort_flag, p.status, JB200_STATUS_ATTN_MMA)) { ok = false; break; }
      JB_T_MARK(1)
      tc_fence_after_sync();
      __syncwarp();               // tcgen05.ld / st are warp-collective: rejoin after the per-thread wait
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const int jb = 2 * hf + jj;                      // 32-key block
        if (jb > qd) continue;                           // above the diagonal for all rows of this warp: stays zero
        uint32_t r[32];
        tmem_ld_32x32(tm_lane + PT_SC + 128 * buf + 32 * jb, r);
        tmem_ld_wait();
        const float* f = sm->pwm + (i - 32 * jb + CH);   // f[-c]: factor of key 32*jb + c
        uint32_t w[16];
#pragma unroll
        for (int c2 = 0; c2 < 16; ++c2)
          w[c2] = pack_bf16x2(__uint_as_float(r[2 * c2]) * f[-2 * c2], __uint_as_float(r[2 * c2 + 1]) * f[-2 * c2 - 1]);
        tmem_st_32x16(tm_lane + PT_P + 16 * jb, w);
      }
      tmem_st_wait();
      JB_T_MARK(2)
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&sm->p_done));
      JB_T_MARK(3)
      // ---- state update: S = gamma^c S + dS ----
      if (!mbar_wait(smem_u32(&sm->bar_s), uint32_t(lc) & 1u, abort_flag, p.status, JB200_STATUS_ATTN_MMA)) { ok = false; break; }
      JB_T_MARK(4)
      tc_fence_after_sync();
      __syncwarp();
      {
        uint32_t r[16];
        tmem_ld_32x16(tm_lane + PT_DS + 16 * s_cg, r);
        tmem_ld_wait();
        const float gc = sm->pw[c_len];
#pragma unroll
        for (int e = 0; e < 16; ++e) S[e] = gc * S[e] + __uint_as_float(r[e]);
      }
      publish_state((lc + 1) & 1);
      JB_T_MARK(5)
      // ---- output rows: o[i] = O1 + gamma^(i+1)/8 * O2 ----
      if (!mbar_wait(smem_u32(&sm->bar_b[buf]), u, abort_flag, p.status, JB200_STATUS_ATTN_MMA)) { ok = false; break; }
      JB_T_MARK(6)
      tc_fence_after_sync();
      __syncwarp();
      {
        uint32_t a[32], c2[32];
        tmem_ld_32x32(tm_lane + PT_SC + 128 * buf + 32 * hf, a);
        tmem_ld_32x32(tm_lane + PT_O2 + 64 * buf + 32 * hf, c2);
        tmem_ld_wait();
        tc_fence_before_sync();
        mbar_arrive(smem_u32(&sm->o_done[buf]));         // both accumulators are in registers now
        const float g = 0.125f * sm->pw[i + 1];
        uint32_t w[16];
#pragma unroll
        for (int e = 0; e < 16; ++e)
          w[e] = pack_bf16x2(fmaf(g, __uint_as_float(c2[2 * e]), __uint_as_float(a[2 * e])),
                             fmaf(g, __uint_as_float(c2[2 * e + 1]), __uint_as_float(a[2 * e + 1])));
        if (i < c_len) {
          __nv_bfloat16* op = p.o + size_t(row0 + ck * CH + i) * p.ld_o + h * D + 32 * hf;
          if (p.wide_store) {
            st_global_256(op, w);
            st_global_256(op + 16, w + 8);
          } else {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4)
              *reinterpret_cast<uint4*>(op + 8 * q4) = make_uint4(w[4 * q4], w[4 * q4 + 1], w[4 * q4 + 2], w[4 * q4 + 3]);
          }
        }
      }
      JB_T_MARK(7)
    }
    JB_T_FLUSH(warp)
    if (piece == 1) {
      // first part of a cut sequence-head: its end state for the CTA that takes the second part
      if (ok) {
        float* hp = p.handoff + bh * D * D + s_row * D + 16 * s_cg;
#pragma unroll
        for (int e4 = 0; e4 < 4; ++e4)
          __stcg(reinterpret_cast<float4*>(hp) + e4, make_float4(S[4 * e4], S[4 * e4 + 1], S[4 * e4 + 2], S[4 * e4 + 3]));
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(p.ctrl + 1 + bh, 1);
      }
    } else if (ok && p.s_out && seg == p.nseg - 1) {
      float* sp = p.s_out + bh * D * D + s_row * D;
      if (p.qk_prepared) {
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const int c = 16 * s_cg + e;
          sp[(c >> 1) + 32 * (c & 1)] = S[e];
        }
      } else {
#pragma unroll
        for (int e4 = 0; e4 < 4; ++e4)
          *reinterpret_cast<float4*>(sp + 16 * s_cg + 4 * e4) = make_float4(S[4 * e4], S[4 * e4 + 1], S[4 * e4 + 2], S[4 * e4 + 3]);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tm, PIPE_TMEM_COLS);
  }
}

// State-only calls (no output rows wanted): every piece of the sequence has left its contribution D_s, scanned
// from a zero state, in seg_state; the state after the whole sequence is
//   S = gamma^T S_in + sum_s gamma^(T - end_s) D_s,      end_s = last token of piece s + 1.
// One CTA per (head, sequence), 16 elements per thread.  The pieces are in the kernel's own column order
// (interleaved when q/k were prepared); s_in / s_out use the natural one.
__global__ void __launch_bounds__(256) attn_fold_states_kernel(const AttnParams p) {
  pdl_wait();
  pdl_trigger();
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

// One element of the single-token state update, S' = gamma S + v k', with its roundings spelled out so that both
// decode kernels below produce the same state bits.
__device__ __forceinline__ float decode_update(float gamma, float s, float v, float k) {
  return __fmaf_rn(gamma, s, __fmul_rn(v, k));
}

// One-token step (decode): S <- gamma*S + v (x) k', o = S q' for every (sequence, head).  Pure state
// streaming: 2 x 16 KiB of fp32 state per (sequence, head) against 384 B of q, k, v, so the kernel is a
// coalesced read-modify-write of S with the feature map + RoPE of the single token done in shared memory.
// Thread t owns state row t/4, columns 16*(t%4)..+15; s_out may alias s_in.
__global__ void __launch_bounds__(256)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                   const __nv_bfloat16* __restrict__ v, int ld_qkv, const AttnParams p) {
  __shared__ float sq[D], sk[D], sv[D], rq[D], rk[D];
  pdl_wait();
  pdl_trigger();
  const int h = blockIdx.x, b = blockIdx.y, t = threadIdx.x;
  // the thread's 64 bytes of state first: they are in flight during the feature map of the token below
  const int row = t >> 2, c0 = (t & 3) * 16;
  const size_t so = (size_t(b) * p.H + h) * D * D + size_t(row) * D + c0;
  float4 st[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    st[i] = p.s_in ? *reinterpret_cast<const float4*>(p.s_in + so + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
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
  const float vr = sv[row];
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = c0 + 4 * i;
    st[i].x = decode_update(gamma, st[i].x, vr, rk[c]);      st[i].y = decode_update(gamma, st[i].y, vr, rk[c + 1]);
    st[i].z = decode_update(gamma, st[i].z, vr, rk[c + 2]);  st[i].w = decode_update(gamma, st[i].w, vr, rk[c + 3]);
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

// The same step as a stream of 16 KiB state tiles through shared memory: a fixed grid of CTAs (two per SM), each
// walking its share of the (sequence, head) pairs with four tiles in flight as untiled bulk copies (global -> shared
// on an mbarrier, shared -> global as a bulk group), the update done in place in the tile.  Bytes in flight do not
// depend on registers or on CTA turnover, which is what holds attn_decode_kernel at ~0.6 of the HBM peak.  Needs
// both s_in and s_out (they may be the same buffer); the feature map of the NEXT pair's token is computed while the
// current tile is awaited.  Thread t of 256: columns 32*((t>>3)&1) + 4*(t&7) .. +3 of rows 16*i + (t>>4), i = 0..3, so
// a quarter-warp always touches 128 contiguous bytes of the tile (no bank conflicts).
constexpr int DEC_STAGES = 4;
constexpr int DEC_TILE_BYTES = D * D * 4;
struct DecodeSmem {
  float tile[DEC_STAGES][D * D];
  uint64_t full[DEC_STAGES];
  float rq[2][D], rk[2][D], sv[2][D];
  uint32_t abort_flag;
};
constexpr size_t DEC_SMEM_BYTES = sizeof(DecodeSmem) + 128;

__global__ void __launch_bounds__(256, 2)
attn_decode_stream_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                          const __nv_bfloat16* __restrict__ v, int ld_qkv, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  DecodeSmem* sm = reinterpret_cast<DecodeSmem*>(smem_raw + (((raw_addr + 127u) & ~127u) - raw_addr));
  const int t = threadIdx.x, lane = t & 31;
  if (t == 0) {
    for (int s = 0; s < DEC_STAGES; ++s) mbar_init(smem_u32(&sm->full[s]), 1);
    sm->abort_flag = 0;
    fence_mbar_init();
  }
  pdl_wait();
  pdl_trigger();
  __syncthreads();
  volatile uint32_t* abort_flag = &sm->abort_flag;
  const int n_units = p.B * p.H;
  const int n_my = (n_units - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x);   // units u = blockIdx.x + i * gridDim.x
  auto unit_of = [&](int i) { return int(blockIdx.x) + i * int(gridDim.x); };
  auto issue_load = [&](int i) {      // thread 0 only
    const int s = i % DEC_STAGES;
    mbar_arrive_expect_tx(smem_u32(&sm->full[s]), DEC_TILE_BYTES);
    bulk_load_1d(smem_u32(sm->tile[s]), p.s_in + size_t(unit_of(i)) * D * D, DEC_TILE_BYTES, smem_u32(&sm->full[s]));
  };
  if (t == 0) {
    for (int i = 0; i < DEC_STAGES && i < n_my; ++i) issue_load(i);
  }
  // feature map + RoPE of the token of unit i into buffer i & 1: threads 0..31 the q / k pairs (d, d + 32), 32..95 v
  auto token_features = [&](int i) {
    if (t >= 96) return;
    const int u = unit_of(i), b = u / p.H, h = u - b * p.H, buf = i & 1;
    const size_t off = size_t(b) * ld_qkv + h * D;
    if (t < 32) {
      const float q0 = elu1(__bfloat162float(q[off + t])) * 0.125f, q1 = elu1(__bfloat162float(q[off + t + 32])) * 0.125f;
      const float k0 = elu1(__bfloat162float(k[off + t])), k1 = elu1(__bfloat162float(k[off + t + 32]));
      int pos = p.pos0 ? p.pos0[b] : p.pos0_scalar;
      pos = pos < 0 ? 0 : (pos >= p.n_pos ? p.n_pos - 1 : pos);
      const float c = __ldg(p.cos_tab + size_t(pos) * 32 + t), sn = __ldg(p.sin_tab + size_t(pos) * 32 + t);
      sm->rq[buf][t] = q0 * c - q1 * sn;  sm->rq[buf][t + 32] = q1 * c + q0 * sn;
      sm->rk[buf][t] = k0 * c - k1 * sn;  sm->rk[buf][t + 32] = k1 * c + k0 * sn;
    } else {
      sm->sv[buf][t - 32] = __bfloat162float(v[off + t - 32]);
    }
  };
  if (n_my > 0) token_features(0);
  __syncthreads();
  const int col0 = 32 * ((t >> 3) & 1) + 4 * (t & 7), r0 = t >> 4;
  for (int i = 0; i < n_my; ++i) {
    const int s = i % DEC_STAGES, buf = i & 1;
    const int u = unit_of(i), b = u / p.H, h = u - b * p.H;
    if (i + 1 < n_my) token_features(i + 1);          // its loads overlap the wait for this unit's tile
    const float gamma = __ldg(p.gamma + h);
    const float4 kq = *reinterpret_cast<const float4*>(&sm->rk[buf][col0]);
    const float4 qq = *reinterpret_cast<const float4*>(&sm->rq[buf][col0]);
    if (!mbar_wait(smem_u32(&sm->full[s]), uint32_t(i / DEC_STAGES) & 1u, abort_flag, p.status, JB200_STATUS_ATTN_LOAD)) break;
    float acc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int row = 16 * j + r0;
      float4* cell = reinterpret_cast<float4*>(&sm->tile[s][row * D + col0]);
      const float vr = sm->sv[buf][row];
      float4 st = *cell;
      st.x = decode_update(gamma, st.x, vr, kq.x);  st.y = decode_update(gamma, st.y, vr, kq.y);
      st.z = decode_update(gamma, st.z, vr, kq.z);  st.w = decode_update(gamma, st.w, vr, kq.w);
      *cell = st;
      acc[j] = st.x * qq.x + st.y * qq.y + st.z * qq.z + st.w * qq.w;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int o = 1; o < 16; o <<= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
    }
    if ((lane & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j) p.o[size_t(b) * p.ld_o + h * D + 16 * j + r0] = __float2bfloat16_rn(acc[j]);
    }
    fence_proxy_async_smem();      // the updated tile goes out through the async proxy
    __syncthreads();               // tile complete; also orders this iteration's reads of rq/rk/sv before their reuse
    if (t == 0) {
      bulk_store_1d(p.s_out + size_t(u) * D * D, smem_u32(sm->tile[s]), DEC_TILE_BYTES);
      bulk_commit_group();
      if (i >= 1 && i - 1 + DEC_STAGES < n_my) {
        bulk_wait_group_read<1>();   // the store of unit i - 1 has read its tile: the stage takes unit i - 1 + DEC_STAGES
        issue_load(i - 1 + DEC_STAGES);
      }
    }
  }
  if (t == 0) bulk_wait_group<0>();
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

// Segments: the pipeline kernel runs one CTA per SM, so sequences are cut only when B*H leaves SMs idle;
// each segment is at least two chunks long.
static void pick_segments(int B, int T, int H, int sms, int* seg_chunks, int* nseg) {
  const int n_chunks = (T + CH - 1) / CH;
  long want = long(sms) / (long(B) * H);
  if (want < 1) want = 1;
  if (want > n_chunks / 2) want = n_chunks / 2 > 0 ? n_chunks / 2 : 1;
  int sc = int((n_chunks + want - 1) / want);
  *seg_chunks = sc;
  *nseg = (n_chunks + sc - 1) / sc;
}

// Balanced launch: with more sequence-heads than SMs and a last wave that is at most half full, that many
// sequence-heads are cut in two; the first parts run first, the second parts last, and the makespan drops by half
// a sequence (B=32 x 16 heads on 148 SMs: 64 -> 56 chunk times).  A sequence's chunks are serial, so nothing is to be
// gained when every SM holds at most one sequence-head.
static int pick_split(int B, int T, int H, int sms) {
  const long U = long(B) * H;
  const int n_chunks = (T + CH - 1) / CH;
  if (U <= sms || n_chunks < 8) return 0;      // short sequences: the ticket and the hand-off cost more than they save
  const int R = int(U % sms);
  return (R > 0 && 2 * R <= sms) ? R : 0;
}

size_t attn_scan_scratch_bytes(int B, int T, int H) {
  if (B <= 0 || T <= 0 || H <= 0) return 0;
  int sms = sm_count();
  if (sms <= 0) sms = 148;
  int sc, ns;
  pick_segments(B, T, H, sms, &sc, &ns);
  const size_t seg_bytes = size_t(B) * H * size_t(ns) * D * D * sizeof(float);   // ns - 1 pieces for a full call, ns for a state-only one
  const int n_split = pick_split(B, T, H, sms);
  const size_t split_bytes = n_split ? size_t(n_split) * D * D * sizeof(float) + (size_t(n_split) + 1) * sizeof(int) : 0;
  return seg_bytes > split_bytes ? seg_bytes : split_bytes;
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
  JB_REQUIRE(size_t(B) * T < (size_t(1) << 31), "attn_scan: too many rows");
  JB_REQUIRE(n_pos >= 1, "attn_scan: empty RoPE table");
  if (!pos0) JB_REQUIRE(pos0_scalar >= 0 && pos0_scalar + T <= n_pos, "attn_scan: RoPE table (%d rows) too short for positions %d..%d", n_pos, pos0_scalar, pos0_scalar + T - 1);
  JB_REQUIRE(!s_in || aligned16(s_in), "attn_scan: state pointers must be 16-byte aligned");
  JB_REQUIRE(!s_out || aligned16(s_out), "attn_scan: state pointers must be 16-byte aligned");
  if (T == 1) {
    AttnParams dp;
    dp.gamma = gamma; dp.cos_tab = cos_tab; dp.sin_tab = sin_tab; dp.pos0 = pos0; dp.pos0_scalar = pos0_scalar;
    dp.n_pos = n_pos; dp.s_in = s_in; dp.s_out = s_out; dp.o = reinterpret_cast<__nv_bfloat16*>(o); dp.ld_o = ld_o;
    dp.B = B; dp.T = 1; dp.H = H; dp.seg_chunks = 1; dp.nseg = 1; dp.seg_state = nullptr; dp.n_pieces = 0; dp.qk_prepared = 0;
    dp.wide_store = 0; dp.status = device_status_ptr();
    if (!dp.status) return JB200_ERR_CUDA;
    if (s_in && s_out && B * H >= 64) {
      // the state streams through shared memory as bulk copies: two CTAs per SM walk the (sequence, head) pairs
      const int sms = sm_count();
      if (sms <= 0) return JB200_ERR_CUDA;
      JB_CUDA(cudaFuncSetAttribute(attn_decode_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(DEC_SMEM_BYTES)));
      const int grid = B * H < 2 * sms ? B * H : 2 * sms;
      launch_dep(attn_decode_stream_kernel, grid, 256, DEC_SMEM_BYTES, stream, reinterpret_cast<const __nv_bfloat16*>(q),
                 reinterpret_cast<const __nv_bfloat16*>(k), reinterpret_cast<const __nv_bfloat16*>(v), ld_qkv, dp);
      JB_LAUNCH_CHECK("attn_decode_stream_kernel");
      return JB200_OK;
    }
    launch_dep(attn_decode_kernel, dim3(H, B), 256, 0, stream, reinterpret_cast<const __nv_bfloat16*>(q),
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
  p.wide_store = (o && (reinterpret_cast<uintptr_t>(o) & 31u) == 0 && ld_o % 16 == 0) ? 1 : 0;
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
  JB_REQUIRE(!scratch || aligned16(scratch), "attn_scan: scratch pointer must be 16-byte aligned");
  p.n_pieces = o ? p.nseg - 1 : p.nseg;
  p.n_split = 0; p.split_chunk = 0; p.handoff = nullptr; p.ctrl = nullptr;
  if (!o) {
    // state only: the k/v pass over every piece, then the fold
    JB_CUDA(cudaFuncSetAttribute(attn_state_pass_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(STATE_SMEM_BYTES)));
    launch_dep(attn_state_pass_kernel, dim3(H, B, p.nseg), STATE_THREADS, STATE_SMEM_BYTES, stream, tk, tv, p);
    JB_LAUNCH_CHECK("attn_state_pass_kernel");
    launch_dep(attn_fold_states_kernel, dim3(H, B), 256, 0, stream, p);
    JB_LAUNCH_CHECK("attn_fold_states_kernel");
    return JB200_OK;
  }
  JB_CUDA(cudaFuncSetAttribute(attn_scan_pipe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(PIPE_SMEM_BYTES)));
  if (p.nseg > 1) {
    JB_CUDA(cudaFuncSetAttribute(attn_state_pass_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(STATE_SMEM_BYTES)));
    launch_dep(attn_state_pass_kernel, dim3(H, B, p.nseg - 1), STATE_THREADS, STATE_SMEM_BYTES, stream, tk, tv, p);
    JB_LAUNCH_CHECK("attn_state_pass_kernel");
  }
  if (scratch && p.nseg == 1 && (p.n_split = pick_split(B, T, H, sms)) > 0) {
    p.split_chunk = ((T + CH - 1) / CH) / 2;
    p.handoff = reinterpret_cast<float*>(scratch);
    p.ctrl = reinterpret_cast<int*>(p.handoff + size_t(p.n_split) * D * D);
    JB_CUDA(cudaMemsetAsync(p.ctrl, 0, (size_t(p.n_split) + 1) * sizeof(int), stream));
    launch_dep(attn_scan_pipe_kernel, dim3(unsigned(long(B) * H + p.n_split)), PIPE_THREADS, PIPE_SMEM_BYTES, stream, tq, tk,
               tv, p);
    JB_LAUNCH_CHECK("attn_scan_pipe_kernel");
    return JB200_OK;
  }
  launch_dep(attn_scan_pipe_kernel, dim3(H, B, p.nseg), PIPE_THREADS, PIPE_SMEM_BYTES, stream, tq, tk, tv, p);
  JB_LAUNCH_CHECK("attn_scan_pipe_kernel");
  return JB200_OK;
}

#ifdef JB_ATTN_TIMING
// Timing builds only: copies the per-role cycle counters of the last pipeline launch to the host.
extern "C" int jb200_debug_attn_timing(long long* out) {
  return cudaMemcpyFromSymbol(out, g_attn_timing, sizeof(long long) * 18 * 8) == cudaSuccess ? 0 : 1;
}
#endif

}  // namespace jb
