// Next-token sampling for the decode driver: temperature, top-k and nucleus (top-p) filtering of one row of
// logits per sequence, then one draw.  Follows sample_next_token (jarvis_engine/evaluate_jarvis.py:158-185):
//   temperature <= 0          -> argmax
//   x = logits / max(temperature, 1e-5)
//   top-k: keep x >= (k-th largest x)            (ties with the k-th value are kept, as `logits < v[:, -1]` does)
//   top-p: sort kept x descending, p = softmax, c = cumsum(p); drop position i >= 1 when c[i-1] > top_p
//   draw from softmax over what is left
// The reference draws with torch.multinomial; here the caller supplies one uniform number u in [0, 1) per row
// and the draw is the inverse CDF over the kept tokens in descending order of x (ties: lower token id first),
// so that a given (logits, u) has one answer that a CPU restatement can check.
//
// One CTA per row.  The k-th largest value is found with a 4-pass byte-wise radix select over the row
// (the row, 100-200 KB, stays in L2 between passes); the <= 2048 survivors are sorted in shared memory with a
// bitonic network and the two cumulative sums run sequentially in one thread, in index order, like the
// reference's cumsum.
#include "common.cuh"
#include "launchers.h"

namespace jb {

namespace {

constexpr int SAMPLE_THREADS = 256;
constexpr int SAMPLE_CAP = 2048;       // candidates kept in shared memory (top_k <= 1024 plus ties)
constexpr int SAMPLE_MAX_K = 1024;

// order-preserving map float -> uint32 (larger float <=> larger key); NaN is treated as -inf
__device__ __forceinline__ uint32_t float_key(float x) {
  if (x != x) x = -INFINITY;
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

template <typename T>
__device__ __forceinline__ float load_logit(const T* row, int i);
template <>
__device__ __forceinline__ float load_logit<float>(const float* row, int i) { return __ldg(row + i); }
template <>
__device__ __forceinline__ float load_logit<__nv_bfloat16>(const __nv_bfloat16* row, int i) {
  return __bfloat162float(row[i]);
}

struct SampleSmem {
  float val[SAMPLE_CAP];
  int idx[SAMPLE_CAP];
  unsigned int hist[256];
  unsigned int prefix;       // key bits fixed so far
  unsigned int remaining;    // rank still to find inside the current bucket
  unsigned int count;        // candidates gathered
  unsigned int ties;         // elements whose key equals the k-th key
  float red_val[SAMPLE_THREADS / 32];
  int red_idx[SAMPLE_THREADS / 32];
};

template <typename T>
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const T* __restrict__ logits, int ld, int V, float temperature, int top_k, float top_p,
              const float* __restrict__ u, int64_t* __restrict__ out_token, float* __restrict__ out_prob) {
  pdl_wait();
  pdl_trigger();
  __shared__ SampleSmem sm;
  const int row_i = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* row = logits + size_t(row_i) * ld;

  if (temperature <= 0.f || top_k == 1) {
    // argmax, lowest index among equals
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
      float x = load_logit<T>(row, i);
      if (x != x) x = -INFINITY;
      if (x > best || (x == best && i < bi)) { best = x; bi = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { sm.red_val[warp] = best; sm.red_idx[warp] = bi; }
    __syncthreads();
    if (tid == 0) {
      for (int w = 1; w < SAMPLE_THREADS / 32; ++w)
        if (sm.red_val[w] > best || (sm.red_val[w] == best && sm.red_idx[w] < bi)) { best = sm.red_val[w]; bi = sm.red_idx[w]; }
      out_token[row_i] = bi == 0x7fffffff ? 0 : bi;
      if (out_prob) out_prob[row_i] = 1.0f;
    }
    return;
  }

  const float inv_t = 1.0f / fmaxf(temperature, 1e-5f);
  const unsigned int k = unsigned(min(top_k, V));

  // ---- radix select: key of the k-th largest scaled logit ---------------------------------------------
  if (tid == 0) { sm.prefix = 0u; sm.remaining = k; sm.count = 0u; }
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = tid; i < 256; i += SAMPLE_THREADS) sm.hist[i] = 0u;
    __syncthreads();
    const unsigned int prefix = sm.prefix;
    const unsigned int mask_hi = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
      const uint32_t key = float_key(load_logit<T>(row, i) * inv_t);
      if ((key & mask_hi) == prefix) atomicAdd(&sm.hist[(key >> shift) & 0xFFu], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      unsigned int rem = sm.remaining;
      int b = 255;
      for (; b > 0; --b) {               // walk buckets from the largest byte value down
        if (sm.hist[b] >= rem) break;
        rem -= sm.hist[b];
      }
      sm.prefix = prefix | (unsigned(b) << shift);
      sm.remaining = rem;
      sm.ties = sm.hist[b];              // after the last pass: the elements equal to the k-th value
    }
    __syncthreads();
  }
  const uint32_t kth_key = sm.prefix;

  // ---- gather the survivors (key >= k-th key) -------------------------------------------------------------
  // Strictly larger values number at most k - 1 <= 1023 and always fit.  When they and the values EQUAL to the
  // k-th one fit the buffer together, arrival order does not matter (the sort below fixes it).  When a long run
  // of equal values would overflow it (constant or degenerate rows), the larger values are taken first and the
  // equal ones follow in ascending token id until the buffer is full, so the result stays a function of
  // (logits, u) and the argmax can never be crowded out.
  const bool overflow = (k - sm.remaining) + sm.ties > unsigned(SAMPLE_CAP);
  for (int i = tid; i < V; i += SAMPLE_THREADS) {
    const float x = load_logit<T>(row, i) * inv_t;
    const uint32_t key = float_key(x);
    if (overflow ? key > kth_key : key >= kth_key) {
      const unsigned int slot = atomicAdd(&sm.count, 1u);
      if (slot < SAMPLE_CAP) { sm.val[slot] = (x != x) ? -INFINITY : x; sm.idx[slot] = i; }
    }
  }
  __syncthreads();
  if (overflow) {
    for (int i0 = 0; i0 < V; i0 += SAMPLE_THREADS) {
      const unsigned int base = sm.count;            // stable: written only between the barriers below
      if (base >= unsigned(SAMPLE_CAP)) break;
      const int i = i0 + tid;
      const float x = i < V ? load_logit<T>(row, i) * inv_t : 0.f;
      const bool tie = i < V && float_key(x) == kth_key;
      const unsigned int bal = __ballot_sync(0xffffffffu, tie);
      if (lane == 0) sm.red_idx[warp] = __popc(bal);
      __syncthreads();
      unsigned int before = 0, total = 0;
      for (int w = 0; w < SAMPLE_THREADS / 32; ++w) {
        if (w < warp) before += unsigned(sm.red_idx[w]);
        total += unsigned(sm.red_idx[w]);
      }
      const unsigned int slot = base + before + __popc(bal & ((1u << lane) - 1u));
      if (tie && slot < unsigned(SAMPLE_CAP)) { sm.val[slot] = x; sm.idx[slot] = i; }
      __syncthreads();
      if (tid == 0) sm.count = base + total;
      __syncthreads();
    }
  }
  const int n = int(min(sm.count, unsigned(SAMPLE_CAP)));
  int n2 = 1;
  while (n2 < n) n2 <<= 1;
  for (int i = n + tid; i < n2; i += SAMPLE_THREADS) { sm.val[i] = -INFINITY; sm.idx[i] = 0x7fffffff; }
  __syncthreads();

  // ---- bitonic sort: value descending, token id ascending among equals -----------------------------------
  for (int size = 2; size <= n2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = tid; t < (n2 >> 1); t += SAMPLE_THREADS) {
        const int lo = 2 * t - (t & (stride - 1));
        const int hi = lo + stride;
        const bool desc = (lo & size) == 0;    // this block ends up "best first"
        const float va = sm.val[lo], vb = sm.val[hi];
        const int ia = sm.idx[lo], ib = sm.idx[hi];
        const bool a_first = va > vb || (va == vb && ia < ib);   // a ranks before b
        if (a_first != desc) { sm.val[lo] = vb; sm.val[hi] = va; sm.idx[lo] = ib; sm.idx[hi] = ia; }
      }
      __syncthreads();
    }
  }

  // ---- nucleus cut and draw (sequential, index order) -----------------------------------------------------
  if (tid == 0) {
    const float x0 = sm.val[0];
    int m = n;
    if (top_p > 0.f && top_p < 1.f) {
      float z = 0.f;
      for (int i = 0; i < n; ++i) z += expf(sm.val[i] - x0);
      float c = 0.f;
      m = 1;
      for (int i = 0; i + 1 < n; ++i) {
        c += expf(sm.val[i] - x0) / z;
        if (c > top_p) break;             // position i + 1 is removed, and every later one with it
        m = i + 2;
      }
    }
    float zm = 0.f;
    for (int i = 0; i < m; ++i) zm += expf(sm.val[i] - x0);
    const float target = u[row_i] * zm;
    float c = 0.f;
    int pick = m - 1;
    for (int i = 0; i < m; ++i) {
      c += expf(sm.val[i] - x0);
      if (c > target) { pick = i; break; }
    }
    out_token[row_i] = sm.idx[pick];
    if (out_prob) out_prob[row_i] = expf(sm.val[pick] - x0) / zm;
  }
}

}  // namespace

int launch_sample(const void* logits, int logits_dtype, int ld, int n_rows, int V, float temperature, int top_k,
                  float top_p, const float* u, int64_t* out_token, float* out_prob, cudaStream_t stream) {
  JB_REQUIRE(n_rows >= 0 && V > 0 && ld >= V, "sample: bad shape (rows=%d, V=%d, ld=%d)", n_rows, V, ld);
  JB_REQUIRE(logits_dtype == 0 || logits_dtype == 1, "sample: logits dtype must be 0 (f32) or 1 (bf16)");
  if (n_rows == 0) return JB200_OK;
  JB_REQUIRE(logits && out_token, "sample: null pointer");
  const bool greedy = temperature <= 0.f;
  JB_REQUIRE(greedy || (top_k >= 1 && top_k <= SAMPLE_MAX_K),
             "sample: top_k (%d) must be in 1..%d (the nucleus cut works on the top-k survivors)", top_k, SAMPLE_MAX_K);
  JB_REQUIRE(greedy || top_k == 1 || u != nullptr, "sample: a uniform number per row is needed to draw");
  JB_REQUIRE(greedy || (top_p > 0.f && top_p <= 1.f) || top_p <= 0.f, "sample: top_p out of range");
  if (n_rows == 0) return JB200_OK;
  if (logits_dtype == 0)
    launch_dep(sample_kernel<float>, n_rows, SAMPLE_THREADS, 0, stream, reinterpret_cast<const float*>(logits), ld, V,
                                                                temperature, top_k, top_p, u, out_token, out_prob);
  else
    launch_dep(sample_kernel<__nv_bfloat16>, n_rows, SAMPLE_THREADS, 0, stream, 
        reinterpret_cast<const __nv_bfloat16*>(logits), ld, V, temperature, top_k, top_p, u, out_token, out_prob);
  JB_LAUNCH_CHECK("sample_kernel");
  return JB200_OK;
}

}  // namespace jb
