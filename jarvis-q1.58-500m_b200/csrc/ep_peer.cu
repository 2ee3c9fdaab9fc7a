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
  for (int row = blockIdx.x * 8 + warp; row < total; row += gridDim.x * 8) {
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
    const uint4* src = reinterpret_cast<const uint4*>(p.xn[s] + size_t(tok) * p.C);
    uint4* dst = reinterpret_cast<uint4*>(p.dispatched + size_t(row) * p.C);
    for (int c = lane; c < p.C / 8; c += 32) dst[c] = src[c];     // peer loads, 16 B per lane
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
    for (int c = lane * 8; c < p.C; c += 256) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int k = 0; k < p.K; ++k) {
        long long e64 = p.topk_idx[size_t(tok) * p.K + k];
        const int e = e64 < 0 ? 0 : (e64 >= p.E ? p.E - 1 : int(e64));
        const int q = p.scatter_map[size_t(tok) * p.K + k] - s_off[e];    // position among MY rows of expert e
        int part = 0, plo = 0;
        if (SH > 1) {                       // which owner took that slice of my rows (same bounds as its gather)
          const int cnt = max(s_off[e + 1] - s_off[e], 0);
          while (part + 1 < SH && q >= int(long(cnt) * (part + 1) / SH)) ++part;
          plo = int(long(cnt) * part / SH);
        }
        const int owner = SH > 1 ? e * SH + part : e / per;
        int row = s_base[e * SH + part] + (q - plo);
        row = row < 0 ? 0 : (row >= p.max_rows ? p.max_rows - 1 : row);     // never leave the owner's buffer
        const float g = p.gates[size_t(tok) * p.K + k];
        const uint4 v = *reinterpret_cast<const uint4*>(p.y[owner] + size_t(row) * p.C + c);   // peer load
        acc[0] += g * bf16_lo(v.x); acc[1] += g * bf16_hi(v.x); acc[2] += g * bf16_lo(v.y); acc[3] += g * bf16_hi(v.y);
        acc[4] += g * bf16_lo(v.z); acc[5] += g * bf16_hi(v.z); acc[6] += g * bf16_lo(v.w); acc[7] += g * bf16_hi(v.w);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) { s1 += acc[j]; s2 += acc[j] * acc[j]; }
      if constexpr (sizeof(TOut) == 2) {
        *reinterpret_cast<uint4*>(out + size_t(tok) * p.C + c) =
            make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                       pack_bf16x2(acc[6], acc[7]));
      } else {
        float4* o = reinterpret_cast<float4*>(out + size_t(tok) * p.C + c);
        o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
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

bool ep_shape_ok(int world, int rank, int E, int C) {
  if (!(world >= 1 && world <= EP_MAX_WORLD && rank >= 0 && rank < world && E >= 1 && C > 0 && C % 8 == 0)) return false;
  if (world <= E) return E % world == 0 && E / world <= EP_MAX_OWNED && E <= EP_MAX_WORLD * EP_MAX_OWNED;
  return world % E == 0;        // every expert served by world / E ranks
}

}  // namespace

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
