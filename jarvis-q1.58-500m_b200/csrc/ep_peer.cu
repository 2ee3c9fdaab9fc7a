// Expert parallelism over peer memory: the dispatch and the return exchange of the top-2 MoE layer done by
// the gather / combine kernels themselves, with plain loads from the other GPUs' memory over NVLink, instead
// of an all-to-all followed by a local gather (and a local scatter followed by an all-to-all back).
//
// Every rank routes its own tokens (replicated router) and leaves, in buffers its peers can read:
//   xn     bf16 [n_tokens][C]   the rows the experts consume
//   gmap   i32  [n_tokens*K]    expert-sorted position -> token (gather_map of jb200_moe_metadata)
//   offs   i32  [E + 2]         expert_offsets of its own dispatch, then its n_tokens
// With world <= E rank r owns the experts [r*per, (r+1)*per), per = E / world.  With world > E every expert is
// served by shards = world / E consecutive ranks: rank r owns part r % shards of expert r / shards, i.e. of every
// source's cnt rows of that expert the slice [cnt*part/shards, cnt*(part+1)/shards) (the packed weights are 1 MiB
// per expert, so replicas are free).  Its pull-gather kernel builds, for each owned expert (part), the rows of
// every source rank in (source rank, local stable order) - the single-GPU dispatch order when ranks hold
// contiguous token ranges (moe_compute_metadata_kernel, sparse_model_cuda/sparse_model.cu:23-90) - by reading
// the peers' offs / gmap / xn directly, and publishes where each source's rows start (`meta`).  After the
// grouped GEMMs the home ranks pull their tokens' expert outputs back from the owners' `y` buffers with the
// gate-weighted sum of scatter_combine_kernel.  No host read of any count: grids are sized for the worst
// case and idle warps leave at once.  The caller separates the phases with a stream-ordered barrier over
// the ranks (any collective): peers' buffers are complete before they are read and not reused before
// everyone has read them.
#include "common.cuh"
#include "launchers.h"

namespace jb {

namespace {

constexpr int EP_MAX_WORLD = 16;
constexpr int EP_MAX_OWNED = 16;

struct PullGatherParams {
  const int32_t* const* offs;          // [world] -> peer offs arrays [E + 2]
  const int32_t* const* gmap;          // [world] -> peer gather maps
  const __nv_bfloat16* const* xn;      // [world] -> peer rows
  int world, rank, per, shards, E, C, K;
  int n_max;                           // capacity of every peer's xn buffer in tokens (its gmap holds n_max * K)
  int max_rows;                        // capacity of `dispatched` in rows
  __nv_bfloat16* dispatched;           // [max_rows][C]
  int32_t* seg_offsets;                // [per + 1] rows of each owned expert (device; read by the grouped GEMM)
  int32_t* meta;                       // [per][world + 1] start of every source's rows inside the expert segment,
                                       // then [per + 1] a copy of seg_offsets; read by the peers' combine
};

__global__ void __launch_bounds__(256)
ep_pull_gather_kernel(const PullGatherParams p) {
  __shared__ int s_pre[EP_MAX_OWNED][EP_MAX_WORLD + 1];   // prefix over sources inside one owned expert
  __shared__ int s_src_off[EP_MAX_OWNED][EP_MAX_WORLD];   // where that expert starts in the source's sorted order
  __shared__ int s_ntok[EP_MAX_WORLD];
  __shared__ int s_seg[EP_MAX_OWNED + 1];
  const int W = p.world, per = p.per;
  for (int i = threadIdx.x; i < per * W; i += blockDim.x) {
    const int el = i / W, s = i - el * W;
    const int e = p.shards > 1 ? p.rank / p.shards : p.rank * per + el;
    const int part = p.shards > 1 ? p.rank % p.shards : 0;
    const int32_t* o = p.offs[s];
    const int lo = o[e], cnt = max(o[e + 1] - lo, 0);
    const int plo = int(long(cnt) * part / p.shards), phi = int(long(cnt) * (part + 1) / p.shards);
    s_src_off[el][s] = lo + plo;
    s_pre[el][s + 1] = phi - plo;              // counts for now
    if (el == 0) s_ntok[s] = o[p.E + 1];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int total = 0;
    for (int el = 0; el < per; ++el) {
      s_seg[el] = total;
      s_pre[el][0] = 0;
      for (int s = 0; s < W; ++s) s_pre[el][s + 1] += s_pre[el][s];
      total += s_pre[el][W];
    }
    s_seg[per] = total;
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int i = threadIdx.x; i < per * (W + 1); i += blockDim.x) p.meta[i] = s_pre[i / (W + 1)][i % (W + 1)];
    for (int i = threadIdx.x; i <= per; i += blockDim.x) {
      const int v = min(s_seg[i], p.max_rows);
      p.meta[per * (W + 1) + i] = v;
      p.seg_offsets[i] = v;
    }
  }
  const int total = min(s_seg[per], p.max_rows);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Peer loads have a latency of microseconds, and a row costs two dependent ones (gather map entry, then the row):
  // a warp therefore works on four rows at once - lanes 0-3 look the four tokens up, then every lane has up to 16
  // independent 16-byte loads in flight before the first store.
  constexpr int RPW = 4;
  const int chunks = p.C / 8;                                    // 16-byte pieces per row
  for (int row0 = (blockIdx.x * 8 + warp) * RPW; row0 < total; row0 += gridDim.x * 8 * RPW) {
    int my_src = 0, my_tok = 0;
    if (lane < RPW && row0 + lane < total) {
      const int row = row0 + lane;
      int el = 0;
      while (el + 1 < per && row >= s_seg[el + 1]) ++el;
      const int within = row - s_seg[el];
      int s = 0;
      while (s + 1 < W && within >= s_pre[el][s + 1]) ++s;
      const int i = within - s_pre[el][s];
      const int ntok = min(max(s_ntok[s], 1), p.n_max);
      int slot = s_src_off[el][s] + i;
      slot = slot < 0 ? 0 : (slot >= ntok * p.K ? ntok * p.K - 1 : slot);   // never leave the peer's map
      int tok = p.gmap[s][slot];                                   // peer load
      tok = tok < 0 ? 0 : (tok >= ntok ? ntok - 1 : tok);          // never leave the peer's buffer
      my_src = s;
      my_tok = tok;
    }
    const uint4* src[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int s = __shfl_sync(0xffffffffu, my_src, r), tok = __shfl_sync(0xffffffffu, my_tok, r);
      src[r] = reinterpret_cast<const uint4*>(p.xn[s] + size_t(tok) * p.C);
    }
    for (int c0 = 0; c0 < chunks; c0 += 128) {                     // 128 pieces = 4 per lane
      uint4 v[RPW][4];
#pragma unroll
      for (int r = 0; r < RPW; ++r)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = c0 + j * 32 + lane;
          if (row0 + r < total && c < chunks) v[r][j] = src[r][c];   // peer loads, 16 B per lane
        }
#pragma unroll
      for (int r = 0; r < RPW; ++r)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = c0 + j * 32 + lane;
          if (row0 + r < total && c < chunks) reinterpret_cast<uint4*>(p.dispatched + size_t(row0 + r) * p.C)[c] = v[r][j];
        }
    }
  }
}

struct PullCombineParams {
  const __nv_bfloat16* const* y;       // [world] -> owners' output rows
  const int32_t* const* meta;          // [world] -> owners' meta (see above)
  const int32_t* offs_local;           // [E + 1] this rank's expert_offsets
  const int64_t* topk_idx;             // [n_tokens][K]
  const float* gates;                  // [n_tokens][K]
  const int32_t* scatter_map;          // [n_tokens][K] position in this rank's expert-sorted order
  int world, rank, per, shards, E, C, K, n_tokens, max_rows;
  double* stats;                       // [2] sum, sum of squares of the output (or null)
};

template <typename TOut>
__global__ void __launch_bounds__(256)
ep_pull_combine_kernel(const PullCombineParams p, TOut* __restrict__ out) {
  __shared__ int s_base[EP_MAX_WORLD * EP_MAX_OWNED];   // per (expert, part): first row of MY rows in the owner's y
  __shared__ int s_off[EP_MAX_WORLD * EP_MAX_OWNED + 1];
  __shared__ float red[2][8];
  const int W = p.world, per = p.per, SH = p.shards;
  for (int i = threadIdx.x; i < p.E * SH; i += blockDim.x) {
    const int e = i / SH, part = i - e * SH;
    const int owner = SH > 1 ? e * SH + part : e / per;
    const int el = SH > 1 ? 0 : e - owner * per;
    const int32_t* m = p.meta[owner];                              // peer loads
    s_base[i] = m[per * (W + 1) + el] + m[el * (W + 1) + p.rank];
  }
  for (int e = threadIdx.x; e <= p.E; e += blockDim.x) s_off[e] = p.offs_local[e];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tok = blockIdx.x * 8 + warp;
  float s1 = 0.f, s2 = 0.f;
  if (tok < p.n_tokens) {
    // the token's K rows and gates first (lanes 0..K-1 resolve one slot each), then all loads of a 1024-column
    // span (K x 4 pieces of 16 bytes per lane) are issued before the first is used
    int my_row = 0, my_owner = 0;
    float my_gate = 0.f;
    if (lane < p.K) {
      const int k = lane;
      long long e64 = p.topk_idx[size_t(tok) * p.K + k];
      const int e = e64 < 0 ? 0 : (e64 >= p.E ? p.E - 1 : int(e64));
      const int q = p.scatter_map[size_t(tok) * p.K + k] - s_off[e];    // position among MY rows of expert e
      int part = 0, plo = 0;
      if (SH > 1) {                       // which owner took that slice of my rows (same bounds as its gather)
        const int cnt = max(s_off[e + 1] - s_off[e], 0);
        while (part + 1 < SH && q >= int(long(cnt) * (part + 1) / SH)) ++part;
        plo = int(long(cnt) * part / SH);
      }
      my_owner = SH > 1 ? e * SH + part : e / per;
      int row = s_base[e * SH + part] + (q - plo);
      my_row = row < 0 ? 0 : (row >= p.max_rows ? p.max_rows - 1 : row);     // never leave the owner's buffer
      my_gate = p.gates[size_t(tok) * p.K + k];
    }
    int rows[8], owners[8];          // all lanes of the warp take part in the exchange, whatever their columns
    float gs[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      rows[k] = __shfl_sync(0xffffffffu, my_row, k);
      owners[k] = __shfl_sync(0xffffffffu, my_owner, k);
      gs[k] = k < p.K ? __shfl_sync(0xffffffffu, my_gate, k) : 0.f;
    }
    for (int c0 = lane * 8; c0 < p.C; c0 += 1024) {
      float acc[4][8];
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[j][i] = 0.f;
      for (int k0 = 0; k0 < p.K; k0 += 2) {           // two slots at a time: 8 loads in flight per lane
        uint4 v[2][4];
        float g[2];
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          const int k = k0 + kk < p.K ? k0 + kk : k0;
          int row = rows[0], owner = owners[0];
#pragma unroll
          for (int t = 1; t < 8; ++t)
            if (t == k) { row = rows[t]; owner = owners[t]; }
          float gk = gs[0];
#pragma unroll
          for (int t = 1; t < 8; ++t)
            if (t == k) gk = gs[t];
          g[kk] = k0 + kk < p.K ? gk : 0.f;
          const __nv_bfloat16* yr = p.y[owner] + size_t(row) * p.C;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int c = c0 + j * 256;
            v[kk][j] = c < p.C ? *reinterpret_cast<const uint4*>(yr + c) : make_uint4(0u, 0u, 0u, 0u);   // peer load
          }
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 w = v[kk][j];
            acc[j][0] += g[kk] * bf16_lo(w.x); acc[j][1] += g[kk] * bf16_hi(w.x); acc[j][2] += g[kk] * bf16_lo(w.y);
            acc[j][3] += g[kk] * bf16_hi(w.y); acc[j][4] += g[kk] * bf16_lo(w.z); acc[j][5] += g[kk] * bf16_hi(w.z);
            acc[j][6] += g[kk] * bf16_lo(w.w); acc[j][7] += g[kk] * bf16_hi(w.w);
          }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = c0 + j * 256;
        if (c >= p.C) continue;
#pragma unroll
        for (int i = 0; i < 8; ++i) { s1 += acc[j][i]; s2 += acc[j][i] * acc[j][i]; }
        if constexpr (sizeof(TOut) == 2) {
          *reinterpret_cast<uint4*>(out + size_t(tok) * p.C + c) =
              make_uint4(pack_bf16x2(acc[j][0], acc[j][1]), pack_bf16x2(acc[j][2], acc[j][3]), pack_bf16x2(acc[j][4], acc[j][5]),
                         pack_bf16x2(acc[j][6], acc[j][7]));
        } else {
          float4* o = reinterpret_cast<float4*>(out + size_t(tok) * p.C + c);
          o[0] = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
          o[1] = make_float4(acc[j][4], acc[j][5], acc[j][6], acc[j][7]);
        }
      }
    }
  }
  if (p.stats) {
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    if (lane == 0) { red[0][warp] = s1; red[1][warp] = s2; }
    __syncthreads();
    if (threadIdx.x == 0) {
      double a = 0.0, b = 0.0;
      for (int w = 0; w < 8; ++w) { a += double(red[0][w]); b += double(red[1][w]); }
      atomicAdd(&p.stats[0], a);
      atomicAdd(&p.stats[1], b);
    }
  }
}

// Barrier over the ranks through flags in peer memory.  Thread t < world writes this rank's barrier count into
// slot `rank` of rank t's flag block (release, system scope: everything this GPU wrote before is visible to a
// peer that reads the flag with acquire), then waits for slot t of its own block to reach the same count.
__global__ void __launch_bounds__(32) peer_barrier_kernel(int32_t* const* flags, int world, int rank, unsigned int* status) {
  __shared__ int epoch;
  int32_t* mine = flags[rank];
  if (threadIdx.x == 0) epoch = ++mine[JB200_PEER_FLAG_WORDS - 1];
  __syncwarp();
  const int e = epoch;
  const int t = threadIdx.x;
  if (t < world) {
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flags[t] + rank), "r"(e) : "memory");
    const unsigned long long t0 = globaltimer_ns();
    int v;
    for (;;) {
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine + t) : "memory");
      if (v - e >= 0) break;                       // counts only grow: a peer may already be one barrier ahead
      if (globaltimer_ns() - t0 > JB_WAIT_LIMIT_NS) {
        atomicCAS(status, 0u, JB200_STATUS_PEER_BARRIER);
        break;
      }
      __nanosleep(100);
    }
    __threadfence_system();
  }
}

bool ep_shape_ok(int world, int rank, int E, int C) {
  if (!(world >= 1 && world <= EP_MAX_WORLD && rank >= 0 && rank < world && E >= 1 && C > 0 && C % 8 == 0)) return false;
  if (world <= E) return E % world == 0 && E / world <= EP_MAX_OWNED && E <= EP_MAX_WORLD * EP_MAX_OWNED;
  return world % E == 0;        // every expert served by world / E ranks
}

}  // namespace

int launch_peer_barrier(const void* const* peer_flags, int world, int rank, cudaStream_t stream) {
  JB_REQUIRE(peer_flags && world >= 1 && world <= JB200_PEER_FLAG_WORDS - 1 && rank >= 0 && rank < world,
             "peer_barrier: bad arguments (world=%d, rank=%d)", world, rank);
  unsigned int* status = device_status_ptr();
  if (!status) return JB200_ERR_CUDA;
  peer_barrier_kernel<<<1, 32, 0, stream>>>(reinterpret_cast<int32_t* const*>(const_cast<void* const*>(
                                                reinterpret_cast<const void* const*>(peer_flags))), world, rank, status);
  JB_LAUNCH_CHECK("peer_barrier_kernel");
  return JB200_OK;
}

int launch_ep_pull_gather(const void* const* peer_offs, const void* const* peer_gmap, const void* const* peer_xn,
                          int world, int rank, int E, int C, int K, int n_max, int max_rows, void* dispatched,
                          int32_t* seg_offsets, int32_t* meta, cudaStream_t stream) {
  JB_REQUIRE(ep_shape_ok(world, rank, E, C), "ep_pull_gather: unsupported shape (world=%d, rank=%d, E=%d, C=%d)", world,
             rank, E, C);
  JB_REQUIRE(K >= 1 && K <= 8 && n_max > 0, "ep_pull_gather: bad K or token capacity");
  JB_REQUIRE(max_rows > 0 && peer_offs && peer_gmap && peer_xn && dispatched && seg_offsets && meta,
             "ep_pull_gather: null pointer or empty capacity");
  JB_REQUIRE(aligned16(dispatched), "ep_pull_gather: output rows must be 16-byte aligned");
  PullGatherParams p;
  p.offs = reinterpret_cast<const int32_t* const*>(peer_offs);
  p.gmap = reinterpret_cast<const int32_t* const*>(peer_gmap);
  p.xn = reinterpret_cast<const __nv_bfloat16* const*>(peer_xn);
  p.world = world; p.rank = rank; p.per = world <= E ? E / world : 1; p.shards = world <= E ? 1 : world / E;
  p.E = E; p.C = C; p.K = K; p.n_max = n_max; p.max_rows = max_rows;
  p.dispatched = reinterpret_cast<__nv_bfloat16*>(dispatched);
  p.seg_offsets = seg_offsets;
  p.meta = meta;
  const int sms = sm_count();
  if (sms <= 0) return JB200_ERR_CUDA;
  long blocks = (long(max_rows) + 7) / 8;
  if (blocks > long(sms) * 8) blocks = long(sms) * 8;     // every block reads the peers' tables once, then strides
  ep_pull_gather_kernel<<<unsigned(blocks), 256, 0, stream>>>(p);
  JB_LAUNCH_CHECK("ep_pull_gather_kernel");
  return JB200_OK;
}

int launch_ep_pull_combine(const void* const* peer_y, const void* const* peer_meta, const int32_t* offs_local,
                           const int64_t* topk_idx, const float* gates, const int32_t* scatter_map, int world, int rank,
                           int E, int C, int K, int n_tokens, int max_rows, void* out, int out_dtype, double* stats,
                           cudaStream_t stream) {
  JB_REQUIRE(ep_shape_ok(world, rank, E, C), "ep_pull_combine: unsupported shape (world=%d, rank=%d, E=%d, C=%d)", world,
             rank, E, C);
  JB_REQUIRE(K >= 1 && K <= 8 && n_tokens >= 0 && max_rows > 0, "ep_pull_combine: bad shape");
  JB_REQUIRE(out_dtype == 0 || out_dtype == 1, "ep_pull_combine: out_dtype must be 0 (f32) or 1 (bf16)");
  if (n_tokens == 0) return JB200_OK;
  JB_REQUIRE(peer_y && peer_meta && offs_local && topk_idx && gates && scatter_map && out, "ep_pull_combine: null pointer");
  JB_REQUIRE(aligned16(out), "ep_pull_combine: output must be 16-byte aligned");
  PullCombineParams p;
  p.y = reinterpret_cast<const __nv_bfloat16* const*>(peer_y);
  p.meta = reinterpret_cast<const int32_t* const*>(peer_meta);
  p.offs_local = offs_local; p.topk_idx = topk_idx; p.gates = gates; p.scatter_map = scatter_map;
  p.world = world; p.rank = rank; p.per = world <= E ? E / world : 1; p.shards = world <= E ? 1 : world / E;
  p.E = E; p.C = C; p.K = K; p.n_tokens = n_tokens;
  p.max_rows = max_rows; p.stats = stats;
  const int blocks = (n_tokens + 7) / 8;
  if (out_dtype == 1)
    ep_pull_combine_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(p, reinterpret_cast<__nv_bfloat16*>(out));
  else
    ep_pull_combine_kernel<float><<<blocks, 256, 0, stream>>>(p, reinterpret_cast<float*>(out));
  JB_LAUNCH_CHECK("ep_pull_combine_kernel");
  return JB200_OK;
}

}  // namespace jb
