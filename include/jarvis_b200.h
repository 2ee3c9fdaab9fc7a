/*
 * libjarvis_b200 -- C ABI of the B200 (sm_100a) Jarvis block-forward kernels.
 *
 * Every entry point is what a binding of the reference's native extensions would call for
 * the block-forward path; the comment above each one cites the reference interface it
 * replaces (paths are relative to the reference project root).
 *
 * Conventions
 *   - All tensor pointers are DEVICE pointers owned by the caller; nothing is allocated
 *     unless the entry point says so.  Row-major, innermost dimension contiguous.
 *   - `stream` is a cudaStream_t passed as void*; calls are asynchronous on it.
 *   - bf16 tensors are passed as `const void*` / `void*` (2 bytes per element).
 *   - Return value: JB200_OK, JB200_ERR_ARG (bad shape / alignment / null pointer, found on
 *     the host before any launch; nothing ran), JB200_ERR_CUDA (a CUDA call failed).
 *     jb200_last_error() returns the message of the calling thread's last failure.
 *   - Kernels never spin without a bound: a wait that runs out sets the device status word
 *     (jb200_device_status) and the kernel returns.
 */
#ifndef JARVIS_B200_H_
#define JARVIS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define JB200_OK 0
#define JB200_ERR_ARG (-1)
#define JB200_ERR_CUDA 1

/* epilogues of jb200_ternary_linear / jb200_ternary_linear_grouped */
#define JB200_EPI_BF16 0      /* out bf16 [M][N]  = alpha * acc                       */
#define JB200_EPI_GELU_BF16 1 /* out bf16 [M][N]  = gelu_erf(alpha * acc)             */
#define JB200_EPI_RESID_F32 2 /* out f32  [M][N] += alpha * acc   (residual stream)   */
#define JB200_EPI_F32 3       /* out f32  [M][N]  = alpha * acc                       */

/* device status codes (0 = no bounded wait ever ran out) */
#define JB200_STATUS_GEMM_PRODUCER 0x11u
#define JB200_STATUS_GEMM_MMA 0x12u
#define JB200_STATUS_GEMM_DECODE 0x13u
#define JB200_STATUS_GEMM_EPILOGUE 0x14u
#define JB200_STATUS_ATTN_LOAD 0x21u
#define JB200_STATUS_LSF_LOAD 0x31u
#define JB200_STATUS_SELFTEST_WAIT 0x7Fu

/* ---- library ----------------------------------------------------------------------- */

/* Message of this thread's last failed call ("" if none). */
const char* jb200_last_error(void);

/* ABI version of this library (bumped on any signature change). */
int jb200_abi_version(void);

/* Reads the current device's status word into *status (synchronises the device) and,
 * when `clear` is non-zero, resets it to 0. */
int jb200_device_status(unsigned int* status, int clear);

/* Launches a one-CTA kernel that waits on an mbarrier nothing ever arrives on; the wait
 * gives up after `limit_ms` and records JB200_STATUS_SELFTEST_WAIT.  Exercises the bounded
 * wait + status path that every pipelined kernel here relies on. */
int jb200_selftest_bounded_wait(int limit_ms, void* stream);

/* ---- ternary weights ---------------------------------------------------------------- */

/* Absmean quantisation + 2-bit packing of one weight matrix, done once at load time.
 * Replaces TernaryQuantizeSTE.forward (jarvis_engine/utils/ternary_ops.py:24-31, run by the
 * reference on every forward) followed by pack_ternary_tensor
 * (runtime/weight_packing.py:22-51):
 *   alpha = max(mean|W|, 1e-8);  q = rint(clamp(W/alpha, -1, 1));  code 0/1/2 for 0/+1/-1;
 *   byte = c0 | c1<<2 | c2<<4 | c3<<6 over 4 consecutive in-features.
 * w: f32 [out][in] (in % 4 == 0).  packed: u8 [out][in/4].  alpha_out: f32 [1].
 * alpha_in: optional f32 [1] on the device; when given it is used instead of the computed
 * mean (lets a caller reproduce another implementation's alpha bit for bit).
 * When alpha is computed, `scratch` holds the per-block partial sums of |W|
 * (jb200_pack_ternary_scratch_bytes bytes, 8-byte aligned); it may be NULL when alpha_in is given. */
size_t jb200_pack_ternary_scratch_bytes(int out_features, int in_features);
int jb200_pack_ternary(const float* w, int out_features, int in_features, const float* alpha_in,
                       uint8_t* packed, float* alpha_out, void* scratch, void* stream);

/* Packing of an already-ternary tensor with values in {-1, 0, +1}
 * (pack_ternary_tensor, runtime/weight_packing.py:22-51).  n_elems % 4 == 0. */
int jb200_pack_codes(const float* w_ternary, size_t n_elems, uint8_t* packed, void* stream);

/* unpack_ternary_tensor (runtime/weight_packing.py:53-70): codes -> {-1, 0, +1}.
 * out_dtype: 0 = f32, 1 = bf16.  n_bytes packed bytes produce 4*n_bytes values. */
int jb200_unpack_ternary(const uint8_t* packed, size_t n_bytes, int out_dtype, void* out, void* stream);

/* y = epilogue(alpha * x @ unpack(W)^T) on tcgen05 tensor cores, weights decoded from the
 * 2-bit layout in shared memory.  Replaces TernaryLinear.forward
 * (jarvis_engine/utils/ternary_ops.py:51-53) and packed_ternary_matmul
 * (experiments/architecture_matrix/ternary_packed/packed_kernel.cu:75-108).
 * x: bf16 [M][K].  packed: u8 [N][K/4].  alpha: f32 [N / alpha_rows] (alpha_rows = N for the
 * per-tensor scale; several matrices stacked along N, e.g. q/k/v, each keep their own).
 * N % 128 == 0, K % 64 == 0, alpha_rows % 128 == 0.  out: per `epilogue`.
 * token_tile: 0 = choose, else one of 32/64/128/256. */
int jb200_ternary_linear(const void* x, int M, int K, const uint8_t* packed, const float* alpha, int alpha_rows,
                         int N, int epilogue, void* out, int token_tile, void* stream);

/* Grouped form for the MoE experts: rows [seg_offsets[g], seg_offsets[g+1]) of x use weight
 * matrix g (packed: u8 [G][N][K/4], alpha: f32 [G]).  seg_offsets: i32 [G+1] on the DEVICE
 * (the expert_offsets of jb200_moe_metadata), so no host synchronisation is needed -- the
 * reference reads them back with .cpu() every layer (sparse_model_cuda/sparse_model.py:157)
 * and loops over experts on the host (:159-164). */
int jb200_ternary_linear_grouped(const void* x, int M, int K, const uint8_t* packed, const float* alpha, int N,
                                 int G, const int32_t* seg_offsets, int epilogue, void* out, int token_tile,
                                 void* stream);

/* Host-side copy of the bit manipulation the GEMM's decoder warps run: 16 two-bit codes
 * (one little-endian u32 of the packed layout) -> 16 bf16 values in out8[8] (two per u32,
 * lower in-feature in the low half).  Runs on the CPU; used by the unit tests. */
void jb200_host_decode16(uint32_t word, uint32_t* out8);

#ifdef __cplusplus
}
#endif
#endif /* JARVIS_B200_H_ */
