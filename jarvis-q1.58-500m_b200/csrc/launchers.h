// Host-side launch functions implemented by the kernel translation units and called by the
// extern "C" layer in api.cu.  All return JB200_OK / JB200_ERR_ARG / JB200_ERR_CUDA.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace jb {

size_t pack_ternary_scratch_bytes(int out_features, int in_features);
int launch_pack_ternary(const float* w, int out_features, int in_features, const float* alpha_in, uint8_t* packed,
                        float* alpha_out, void* scratch, cudaStream_t stream);
int launch_pack_codes(const float* w_ternary, size_t n_elems, uint8_t* packed, cudaStream_t stream);
int launch_unpack_ternary(const uint8_t* packed, size_t n_bytes, int out_dtype, void* out, cudaStream_t stream);

int launch_ternary_gemm(const void* x_bf16, int M, int K, const uint8_t* w_packed, const float* alpha,
                        int alpha_rows, int N, int G, const int32_t* seg_offsets, int epilogue, void* out,
                        int bn_override, cudaStream_t stream);
void decode16_host(uint32_t w, uint32_t* out8);

}  // namespace jb
