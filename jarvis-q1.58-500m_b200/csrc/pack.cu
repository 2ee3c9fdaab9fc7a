// Absmean ternary quantisation and the 2-bit weight layout.
//
// Mirrors TernaryQuantizeSTE.forward (jarvis_engine/utils/ternary_ops.py:24-31) and
// pack_ternary_tensor / unpack_ternary_tensor (runtime/weight_packing.py:22-70):
// code 0 -> 0, 1 -> +1, 2 -> -1 (3 is never produced and decodes to 0), four codes per
// byte, lowest bits first, along the in-feature axis.  Integer work: results are exact.
#include "common.cuh"

namespace jb {

namespace {

constexpr int PACK_THREADS = 256;
constexpr int ABS_SUM_MAX_BLOCKS = 1024;

__global__ void __launch_bounds__(PACK_THREADS) abs_sum_kernel(const float* __restrict__ w, size_t n,
                                                               double* __restrict__ partial) {
  double acc = 0.0;
  const size_t n4 = n / 4;
  const float4* w4 = reinterpret_cast<const float4*>(w);
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += size_t(gridDim.x) * blockDim.x) {
    const float4 v = __ldg(w4 + i);
    acc += double(fabsf(v.x)) + double(fabsf(v.y)) + double(fabsf(v.z)) + double(fabsf(v.w));
  }
  __shared__ double red[PACK_THREADS / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double s = 0.0;
    for (int i = 0; i < PACK_THREADS / 32; ++i) s += red[i];
    partial[blockIdx.x] = s;
  }
}

__global__ void finalize_alpha_kernel(const double* __restrict__ partial, int nb, size_t n,
                                      const float* __restrict__ alpha_in, float* __restrict__ alpha_out) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  if (alpha_in) {
    *alpha_out = *alpha_in;
    return;
  }
  double s = 0.0;
  for (int i = 0; i < nb; ++i) s += partial[i];
  const float a = float(s / double(n));
  *alpha_out = fmaxf(a, 1e-8f);
}

__device__ __forceinline__ uint32_t quant_code(float w, float alpha) {
  float t = __fdiv_rn(w, alpha);
  t = t < -1.0f ? -1.0f : (t > 1.0f ? 1.0f : t);  // NaN stays NaN, as torch.clamp does
  const float q = rintf(t);                       // round half to even, as torch.round does
  return q == 1.0f ? 1u : (q == -1.0f ? 2u : 0u);
}

__device__ __forceinline__ uint32_t tern_code(float q) { return q == 1.0f ? 1u : (q == -1.0f ? 2u : 0u); }

// One thread -> 16 weights -> 4 packed bytes.
template <bool QUANT>
__global__ void __launch_bounds__(PACK_THREADS) pack_kernel(const float* __restrict__ w, size_t n16, size_t n_tail4,
                                                            const float* __restrict__ alpha_p,
                                                            uint8_t* __restrict__ packed) {
  const float alpha = QUANT ? *alpha_p : 1.0f;
  const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n16) {
    const float4* src = reinterpret_cast<const float4*>(w) + i * 4;
    uint32_t word = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const float4 v = __ldg(src + b);
      uint32_t c0, c1, c2, c3;
      if (QUANT) {
        c0 = quant_code(v.x, alpha); c1 = quant_code(v.y, alpha); c2 = quant_code(v.z, alpha); c3 = quant_code(v.w, alpha);
      } else {
        c0 = tern_code(v.x); c1 = tern_code(v.y); c2 = tern_code(v.z); c3 = tern_code(v.w);
      }
      word |= (c0 | (c1 << 2) | (c2 << 4) | (c3 << 6)) << (8 * b);
    }
    reinterpret_cast<uint32_t*>(packed)[i] = word;
  } else if (i < n16 + n_tail4) {
    // ragged tail: groups of 4 weights past the last full group of 16
    const size_t g = n16 * 4 + (i - n16);
    const float4 v = __ldg(reinterpret_cast<const float4*>(w) + g);
    uint32_t c0, c1, c2, c3;
    if (QUANT) {
      c0 = quant_code(v.x, alpha); c1 = quant_code(v.y, alpha); c2 = quant_code(v.z, alpha); c3 = quant_code(v.w, alpha);
    } else {
      c0 = tern_code(v.x); c1 = tern_code(v.y); c2 = tern_code(v.z); c3 = tern_code(v.w);
    }
    packed[g] = uint8_t(c0 | (c1 << 2) | (c2 << 4) | (c3 << 6));
  }
}

template <typename T>
__device__ __forceinline__ T tern_value(uint32_t c);
template <>
__device__ __forceinline__ float tern_value<float>(uint32_t c) { return c == 1u ? 1.0f : (c == 2u ? -1.0f : 0.0f); }
template <>
__device__ __forceinline__ __nv_bfloat16 tern_value<__nv_bfloat16>(uint32_t c) {
  return __float2bfloat16_rn(c == 1u ? 1.0f : (c == 2u ? -1.0f : 0.0f));
}

template <typename T>
__global__ void __launch_bounds__(PACK_THREADS) unpack_kernel(const uint8_t* __restrict__ packed, size_t n_bytes,
                                                              T* __restrict__ out) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n_bytes; i += size_t(gridDim.x) * blockDim.x) {
    const uint32_t b = packed[i];
    T* o = out + i * 4;
    o[0] = tern_value<T>(b & 3u);
    o[1] = tern_value<T>((b >> 2) & 3u);
    o[2] = tern_value<T>((b >> 4) & 3u);
    o[3] = tern_value<T>((b >> 6) & 3u);
  }
}

int abs_sum_blocks(size_t n) {
  size_t b = (n / 4 + PACK_THREADS * 8 - 1) / (PACK_THREADS * 8);
  if (b < 1) b = 1;
  if (b > ABS_SUM_MAX_BLOCKS) b = ABS_SUM_MAX_BLOCKS;
  return int(b);
}

}  // namespace

size_t pack_ternary_scratch_bytes(int out_features, int in_features) {
  if (out_features <= 0 || in_features <= 0) return 0;
  return size_t(abs_sum_blocks(size_t(out_features) * in_features)) * sizeof(double);
}

int launch_pack_ternary(const float* w, int out_features, int in_features, const float* alpha_in, uint8_t* packed,
                        float* alpha_out, void* scratch, cudaStream_t stream) {
  JB_REQUIRE(out_features > 0 && in_features > 0, "pack_ternary: bad shape (%d, %d)", out_features, in_features);
  JB_REQUIRE(in_features % 4 == 0, "pack_ternary: in_features (%d) must be divisible by 4", in_features);
  JB_REQUIRE(w && packed && alpha_out, "pack_ternary: null pointer");
  JB_REQUIRE(alpha_in || scratch, "pack_ternary: scratch is required when alpha is computed");
  JB_REQUIRE(aligned16(w), "pack_ternary: weight pointer must be 16-byte aligned");
  JB_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 3u) == 0, "pack_ternary: packed pointer must be 4-byte aligned");
  const size_t n = size_t(out_features) * in_features;
  const int nb = abs_sum_blocks(n);
  if (!alpha_in) {
    abs_sum_kernel<<<nb, PACK_THREADS, 0, stream>>>(w, n, reinterpret_cast<double*>(scratch));
    JB_LAUNCH_CHECK("abs_sum_kernel");
  }
  finalize_alpha_kernel<<<1, 32, 0, stream>>>(reinterpret_cast<const double*>(scratch), nb, n, alpha_in, alpha_out);
  JB_LAUNCH_CHECK("finalize_alpha_kernel");
  const size_t n16 = n / 16, tail4 = (n % 16) / 4;
  const size_t threads = n16 + tail4;
  pack_kernel<true><<<unsigned((threads + PACK_THREADS - 1) / PACK_THREADS), PACK_THREADS, 0, stream>>>(
      w, n16, tail4, alpha_out, packed);
  JB_LAUNCH_CHECK("pack_kernel<quant>");
  return JB200_OK;
}

int launch_pack_codes(const float* w_ternary, size_t n_elems, uint8_t* packed, cudaStream_t stream) {
  JB_REQUIRE(n_elems % 4 == 0, "pack_codes: element count must be divisible by 4");
  if (n_elems == 0) return JB200_OK;
  JB_REQUIRE(w_ternary && packed, "pack_codes: null pointer");
  JB_REQUIRE(aligned16(w_ternary), "pack_codes: input pointer must be 16-byte aligned");
  JB_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 3u) == 0, "pack_codes: packed pointer must be 4-byte aligned");
  if (n_elems == 0) return JB200_OK;
  const size_t n16 = n_elems / 16, tail4 = (n_elems % 16) / 4;
  const size_t threads = n16 + tail4;
  pack_kernel<false><<<unsigned((threads + PACK_THREADS - 1) / PACK_THREADS), PACK_THREADS, 0, stream>>>(
      w_ternary, n16, tail4, nullptr, packed);
  JB_LAUNCH_CHECK("pack_kernel<codes>");
  return JB200_OK;
}

int launch_unpack_ternary(const uint8_t* packed, size_t n_bytes, int out_dtype, void* out, cudaStream_t stream) {
  JB_REQUIRE(out_dtype == 0 || out_dtype == 1, "unpack_ternary: out_dtype must be 0 (f32) or 1 (bf16)");
  if (n_bytes == 0) return JB200_OK;
  JB_REQUIRE(packed && out, "unpack_ternary: null pointer");
  if (n_bytes == 0) return JB200_OK;
  size_t blocks = (n_bytes + PACK_THREADS - 1) / PACK_THREADS;
  if (blocks > 65535) blocks = 65535;
  if (out_dtype == 0)
    unpack_kernel<float><<<unsigned(blocks), PACK_THREADS, 0, stream>>>(packed, n_bytes, reinterpret_cast<float*>(out));
  else
    unpack_kernel<__nv_bfloat16><<<unsigned(blocks), PACK_THREADS, 0, stream>>>(packed, n_bytes,
                                                                              reinterpret_cast<__nv_bfloat16*>(out));
  JB_LAUNCH_CHECK("unpack_kernel");
  return JB200_OK;
}

}  // namespace jb
