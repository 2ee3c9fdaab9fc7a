// Row-wise glue kernels of the block: RMSNorm (jarvis_engine/jarvis_model.py:25-26) and the
// token-embedding gather (nn.Embedding at jarvis_model.py:452, 498).  Both are pure HBM
// streaming: one warp per row, 16-byte accesses.
#include "common.cuh"
#include "launchers.h"

namespace jb {

namespace {

constexpr int ROW_THREADS = 256;  // 8 rows per CTA

template <typename TIn>
__device__ __forceinline__ void load8(const TIn* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
  v[0] = bf16_lo(a.x); v[1] = bf16_hi(a.x); v[2] = bf16_lo(a.y); v[3] = bf16_hi(a.y);
  v[4] = bf16_lo(a.z); v[5] = bf16_hi(a.z); v[6] = bf16_lo(a.w); v[7] = bf16_hi(a.w);
}
template <typename TOut>
__device__ __forceinline__ void store8(TOut* p, const float (&v)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&v)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                                            pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
}

// One warp per row; the row is kept in registers between the two passes when C <= 8*32*MAXV.
template <typename TIn, typename TOut, int MAXV>
__global__ void __launch_bounds__(ROW_THREADS) rmsnorm_kernel(const TIn* __restrict__ x, const float* __restrict__ w,
                                                              float eps, TOut* __restrict__ y, int n_rows, int C) {
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x * (ROW_THREADS / 32) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int lane = threadIdx.x & 31;
  const TIn* xr = x + size_t(row) * C;
  TOut* yr = y + size_t(row) * C;
  float v[MAXV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = (i * 32 + lane) * 8;
    if (c < C) {
      load8<TIn>(xr + c, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = __fmaf_rn(v[i][j], v[i][j], ss);
    }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / float(C) + eps);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = (i * 32 + lane) * 8;
    if (c < C) {
      float wv[8], o[8];
      load8<float>(w + c, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[i][j] * r * wv[j];
      store8<TOut>(yr + c, o);
    }
  }
}

__global__ void __launch_bounds__(ROW_THREADS) embedding_kernel(const int64_t* __restrict__ idx,
                                                                const float* __restrict__ table, int vocab,
                                                                float* __restrict__ out, int n_rows, int C) {
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x * (ROW_THREADS / 32) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int lane = threadIdx.x & 31;
  long long id = idx[row];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // clamp instead of faulting on a bad id
  const float4* src = reinterpret_cast<const float4*>(table + size_t(id) * C);
  float4* dst = reinterpret_cast<float4*>(out + size_t(row) * C);
  for (int c = lane; c < C / 4; c += 32) dst[c] = __ldg(src + c);
}

template <typename TIn, typename TOut>
int launch_rmsnorm_t(const void* x, const float* w, float eps, void* y, int n_rows, int C, cudaStream_t stream) {
  const int blocks = (n_rows + ROW_THREADS / 32 - 1) / (ROW_THREADS / 32);
  if (C <= 1024)
    launch_dep(rmsnorm_kernel<TIn, TOut, 4>, blocks, ROW_THREADS, 0, stream, reinterpret_cast<const TIn*>(x), w, eps,
               reinterpret_cast<TOut*>(y), n_rows, C);
  else
    launch_dep(rmsnorm_kernel<TIn, TOut, 16>, blocks, ROW_THREADS, 0, stream, reinterpret_cast<const TIn*>(x), w, eps,
               reinterpret_cast<TOut*>(y), n_rows, C);
  JB_LAUNCH_CHECK("rmsnorm_kernel");
  return JB200_OK;
}

}  // namespace

int launch_rmsnorm(const void* x, int x_dtype, const float* w, float eps, void* y, int y_dtype, int n_rows, int C,
                   cudaStream_t stream) {
  JB_REQUIRE(n_rows >= 0 && C > 0, "rmsnorm: bad shape (%d, %d)", n_rows, C);
  JB_REQUIRE(C % 8 == 0 && C <= 4096, "rmsnorm: row length (%d) must be a multiple of 8 and at most 4096", C);
  JB_REQUIRE((x_dtype == 0 || x_dtype == 1) && (y_dtype == 0 || y_dtype == 1), "rmsnorm: dtype must be 0 (f32) or 1 (bf16)");
  if (n_rows == 0) return JB200_OK;
  JB_REQUIRE(x && w && y, "rmsnorm: null pointer");
  JB_REQUIRE(aligned16(x) && aligned16(w) && aligned16(y), "rmsnorm: pointers must be 16-byte aligned");
  if (n_rows == 0) return JB200_OK;
  if (x_dtype == 0 && y_dtype == 1) return launch_rmsnorm_t<float, __nv_bfloat16>(x, w, eps, y, n_rows, C, stream);
  if (x_dtype == 0 && y_dtype == 0) return launch_rmsnorm_t<float, float>(x, w, eps, y, n_rows, C, stream);
  if (x_dtype == 1 && y_dtype == 1) return launch_rmsnorm_t<__nv_bfloat16, __nv_bfloat16>(x, w, eps, y, n_rows, C, stream);
  return launch_rmsnorm_t<__nv_bfloat16, float>(x, w, eps, y, n_rows, C, stream);
}

int launch_embedding(const int64_t* idx, const float* table, int vocab, float* out, int n_rows, int C,
                     cudaStream_t stream) {
  JB_REQUIRE(n_rows >= 0 && C > 0 && vocab > 0, "embedding: bad shape");
  JB_REQUIRE(C % 4 == 0, "embedding: row length (%d) must be a multiple of 4", C);
  if (n_rows == 0) return JB200_OK;
  JB_REQUIRE(idx && table && out, "embedding: null pointer");
  JB_REQUIRE(aligned16(table) && aligned16(out), "embedding: pointers must be 16-byte aligned");
  if (n_rows == 0) return JB200_OK;
  const int blocks = (n_rows + ROW_THREADS / 32 - 1) / (ROW_THREADS / 32);
  launch_dep(embedding_kernel, blocks, ROW_THREADS, 0, stream, idx, table, vocab, out, n_rows, C);
  JB_LAUNCH_CHECK("embedding_kernel");
  return JB200_OK;
}

}  // namespace jb
