// extern "C" surface of libjarvis_b200: argument plumbing only, the kernels live in the
// other translation units.  Also owns the per-thread error message, the device status word
// that bounded waits report into, and the bounded-wait self test.
#include <stdarg.h>
#include <stdlib.h>
#include <atomic>
#include <string.h>

#include "common.cuh"
#include "launchers.h"

namespace jb {

namespace {
thread_local char g_err[512] = "";
__device__ unsigned int g_status_word = 0;
constexpr int MAX_DEVICES = 64;
unsigned int* g_status_ptr[MAX_DEVICES] = {nullptr};
int g_sm_count[MAX_DEVICES] = {0};
std::atomic<long long> g_launches{0};
}  // namespace

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

namespace {
// -1: not read yet; the environment variable JB200_DEPENDENT_LAUNCH=0 turns the attribute off for a process
std::atomic<int> g_dep_launch{-1};
}  // namespace
bool dependent_launch_enabled() {
  int v = g_dep_launch.load(std::memory_order_relaxed);
  if (v < 0) {
    const char* e = getenv("JB200_DEPENDENT_LAUNCH");
    v = (e && e[0] == '0') ? 0 : 1;
    g_dep_launch.store(v, std::memory_order_relaxed);
  }
  return v != 0;
}
int set_dependent_launch(int on) {
  const int before = dependent_launch_enabled() ? 1 : 0;
  g_dep_launch.store(on ? 1 : 0, std::memory_order_relaxed);
  return before;
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
  return JB200_ERR_CUDA;
}

unsigned int* device_status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
    set_error("device_status_ptr: cudaGetDevice failed");
    return nullptr;
  }
  if (!g_status_ptr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_status_word);
    if (e != cudaSuccess) {
      cuda_fail(e, "cudaGetSymbolAddress(status word)");
      return nullptr;
    }
    g_status_ptr[dev] = reinterpret_cast<unsigned int*>(p);
  }
  return g_status_ptr[dev];
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
    set_error("sm_count: cudaGetDevice failed");
    return -1;
  }
  if (!g_sm_count[dev]) {
    int n = 0;
    cudaError_t e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) {
      cuda_fail(e, "cudaDeviceGetAttribute(SM count)");
      return -1;
    }
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

namespace {

__global__ void selftest_wait_kernel(unsigned long long limit_ns, unsigned int* status) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
    // Nothing ever arrives on `bar`: the wait below must give up on its own.
    const unsigned long long t0 = globaltimer_ns();
    bool done = false;
    for (uint32_t it = 0; !done; ++it) {
      done = mbar_try_wait(smem_u32(&bar), 0u);
      if (!done && (it & 63u) == 0u && globaltimer_ns() - t0 > limit_ns) {
        atomicCAS(status, 0u, JB200_STATUS_SELFTEST_WAIT);
        break;
      }
    }
  }
}

}  // namespace
}  // namespace jb

using namespace jb;

extern "C" {

const char* jb200_last_error(void) { return g_err; }

int jb200_abi_version(void) { return 11; }

long long jb200_kernel_launches(int reset) {
  return reset ? g_launches.exchange(0) : g_launches.load();
}

int jb200_set_dependent_launch(int enable) { return jb::set_dependent_launch(enable); }

int jb200_device_status(unsigned int* status, int clear) {
  JB_REQUIRE(status != nullptr, "device_status: null output pointer");
  unsigned int* p = device_status_ptr();
  if (!p) return JB200_ERR_CUDA;
  JB_CUDA(cudaDeviceSynchronize());
  JB_CUDA(cudaMemcpy(status, p, sizeof(unsigned int), cudaMemcpyDeviceToHost));
  if (clear) JB_CUDA(cudaMemset(p, 0, sizeof(unsigned int)));
  return JB200_OK;
}

int jb200_selftest_bounded_wait(int limit_ms, void* stream) {
  JB_REQUIRE(limit_ms > 0 && limit_ms <= 2000, "selftest_bounded_wait: limit_ms (%d) must be in 1..2000", limit_ms);
  unsigned int* p = device_status_ptr();
  if (!p) return JB200_ERR_CUDA;
  selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(1000000ull * (unsigned long long)limit_ms, p);
  JB_LAUNCH_CHECK("selftest_wait_kernel");
  return JB200_OK;
}

size_t jb200_pack_ternary_scratch_bytes(int out_features, int in_features) {
  return pack_ternary_scratch_bytes(out_features, in_features);
}

int jb200_pack_ternary(const float* w, int out_features, int in_features, const float* alpha_in, uint8_t* packed,
                       float* alpha_out, void* scratch, void* stream) {
  return launch_pack_ternary(w, out_features, in_features, alpha_in, packed, alpha_out, scratch,
                             static_cast<cudaStream_t>(stream));
}

int jb200_pack_codes(const float* w_ternary, size_t n_elems, uint8_t* packed, void* stream) {
  return launch_pack_codes(w_ternary, n_elems, packed, static_cast<cudaStream_t>(stream));
}

int jb200_unpack_ternary(const uint8_t* packed, size_t n_bytes, int out_dtype, void* out, void* stream) {
  return launch_unpack_ternary(packed, n_bytes, out_dtype, out, static_cast<cudaStream_t>(stream));
}

int jb200_ternary_linear(const void* x, int M, int K, const uint8_t* packed, const float* alpha, int alpha_rows,
                         int N, int epilogue, void* out, int token_tile, int w_layout, void* stream) {
  return launch_ternary_gemm(x, M, K, packed, alpha, alpha_rows, N, 1, nullptr, epilogue, out, token_tile, w_layout,
                             static_cast<cudaStream_t>(stream));
}

int jb200_dense_linear(const void* x, int M, int K, const void* w, int N, int out_dtype, void* out, int token_tile,
                       void* stream) {
  JB_REQUIRE(out_dtype == 0 || out_dtype == 1, "dense_linear: out_dtype must be 0 (f32) or 1 (bf16)");
  return launch_ternary_gemm(x, M, K, static_cast<const uint8_t*>(w), nullptr, N, N, 1, nullptr,
                             out_dtype == 1 ? JB200_EPI_BF16 : JB200_EPI_F32, out, token_tile, 2,
                             static_cast<cudaStream_t>(stream));
}

int jb200_ternary_linear_grouped(const void* x, int M, int K, const uint8_t* packed, const float* alpha, int N,
                                 int G, const int32_t* seg_offsets, int epilogue, void* out, int token_tile,
                                 int w_layout, void* stream) {
  return launch_ternary_gemm(x, M, K, packed, alpha, N, N, G, seg_offsets, epilogue, out, token_tile, w_layout,
                             static_cast<cudaStream_t>(stream));
}

int jb200_qkv_linear_rope(const void* x, int M, int K, const uint8_t* packed, const float* alpha, int alpha_rows,
                          int N, int rope_feats, const float* cos_tab, const float* sin_tab, int n_pos,
                          const int32_t* pos0, int pos0_scalar, int T, void* out, int token_tile, int w_layout,
                          void* stream) {
  GemmRope r{cos_tab, sin_tab, pos0, pos0_scalar, n_pos, T, rope_feats};
  return launch_ternary_gemm(x, M, K, packed, alpha, alpha_rows, N, 1, nullptr, JB200_EPI_QK_ROPE_BF16, out, token_tile,
                             w_layout, static_cast<cudaStream_t>(stream), &r);
}

int jb200_peer_barrier(const void* const* peer_flags, int world, int rank, void* stream) {
  return launch_peer_barrier(peer_flags, world, rank, static_cast<cudaStream_t>(stream));
}

int jb200_peer_buffer_alloc(size_t bytes, void** ptr, unsigned char* handle64) {
  JB_REQUIRE(bytes > 0 && ptr && handle64, "peer_buffer_alloc: bad arguments");
  void* d = nullptr;
  JB_CUDA(cudaMalloc(&d, bytes));
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, d);
  if (e != cudaSuccess) {
    (void)cudaFree(d);
    JB_CUDA(e);
  }
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  *ptr = d;
  return JB200_OK;
}

int jb200_peer_buffer_open(const unsigned char* handle64, void** ptr) {
  JB_REQUIRE(handle64 && ptr, "peer_buffer_open: bad arguments");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* d = nullptr;
  // opened with the accessing device current: the mapping is made for this device, peer access included
  JB_CUDA(cudaIpcOpenMemHandle(&d, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr = d;
  return JB200_OK;
}

int jb200_peer_buffer_close(void* ptr) {
  if (ptr) JB_CUDA(cudaIpcCloseMemHandle(ptr));
  return JB200_OK;
}

int jb200_peer_buffer_free(void* ptr) {
  if (ptr) JB_CUDA(cudaFree(ptr));
  return JB200_OK;
}

int jb200_ep_pull_gather(const void* const* peer_offs, const void* const* peer_gmap, const void* const* peer_xn,
                         int world, int rank, int E, int C, int K, int n_max, int max_rows, void* dispatched,
                         int32_t* seg_offsets, int32_t* meta, void* stream) {
  return launch_ep_pull_gather(peer_offs, peer_gmap, peer_xn, world, rank, E, C, K, n_max, max_rows, dispatched,
                               seg_offsets, meta, static_cast<cudaStream_t>(stream));
}

int jb200_ep_pull_combine(const void* const* peer_y, const void* const* peer_meta, const int32_t* offs_local,
                          const int64_t* topk_idx, const float* gates, const int32_t* scatter_map, int world, int rank,
                          int E, int C, int K, int n_tokens, int max_rows, void* out, int out_dtype, double* stats,
                          void* stream) {
  return launch_ep_pull_combine(peer_y, peer_meta, offs_local, topk_idx, gates, scatter_map, world, rank, E, C, K,
                                n_tokens, max_rows, out, out_dtype, stats, static_cast<cudaStream_t>(stream));
}

int jb200_sample(const void* logits, int logits_dtype, int ld, int n_rows, int V, float temperature, int top_k,
                 float top_p, const float* u, int64_t* out_token, float* out_prob, void* stream) {
  return launch_sample(logits, logits_dtype, ld, n_rows, V, temperature, top_k, top_p, u, out_token, out_prob,
                       static_cast<cudaStream_t>(stream));
}

int jb200_rmsnorm(const void* x, int x_dtype, const float* w, float eps, void* y, int y_dtype, int n_rows, int C,
                  void* stream) {
  return launch_rmsnorm(x, x_dtype, w, eps, y, y_dtype, n_rows, C, static_cast<cudaStream_t>(stream));
}

int jb200_embedding(const int64_t* idx, const float* table, int vocab, float* out, int n_rows, int C, void* stream) {
  return launch_embedding(idx, table, vocab, out, n_rows, C, static_cast<cudaStream_t>(stream));
}

int jb200_attn_scan(const void* q, const void* k, const void* v, int ld_qkv, const float* gamma,
                    const float* cos_tab, const float* sin_tab, int n_pos, const int32_t* pos0, int pos0_scalar,
                    const float* s_in, void* o, int ld_o, float* s_out, void* scratch, int B, int T, int H,
                    int head_dim, int flags, void* stream) {
  return launch_attn_scan(q, k, v, ld_qkv, gamma, cos_tab, sin_tab, n_pos, pos0, pos0_scalar, s_in, o, ld_o, s_out,
                          scratch, B, T, H, head_dim, flags, static_cast<cudaStream_t>(stream));
}

size_t jb200_attn_scan_scratch_bytes(int B, int T, int H) { return attn_scan_scratch_bytes(B, T, H); }

int jb200_router_top2(const void* x, const float* w_router, int N, int C, int E, int64_t* topk_idx, float* gates,
                      float* probs, double* probs_sum, int32_t* top1_hist, void* stream) {
  return launch_router_top2(x, w_router, N, C, E, topk_idx, gates, probs, probs_sum, top1_hist,
                            static_cast<cudaStream_t>(stream));
}

int jb200_rmsnorm_router(const float* x, const float* w_norm, float eps, void* xn, const float* w_router, int N,
                         int C, int E, int64_t* topk_idx, float* gates, double* probs_sum, int32_t* top1_hist,
                         void* stream) {
  return launch_rmsnorm_router(x, w_norm, eps, xn, w_router, N, C, E, topk_idx, gates, probs_sum, top1_hist,
                               static_cast<cudaStream_t>(stream));
}

size_t jb200_moe_metadata_scratch_bytes(int N, int K, int E) { return moe_metadata_scratch_bytes(N, K, E); }

int jb200_moe_metadata(const int64_t* topk_idx, int N, int K, int E, int32_t* expert_counts,
                       int32_t* expert_offsets, int32_t* scatter_map, int32_t* gather_map, int32_t* gate_idx_map,
                       void* scratch, void* stream) {
  return launch_moe_metadata(topk_idx, N, K, E, expert_counts, expert_offsets, scatter_map, gather_map, gate_idx_map,
                             scratch, static_cast<cudaStream_t>(stream));
}

int jb200_moe_metadata_static_max_assignments(void) { return moe_metadata_static_max_assignments(); }

int jb200_moe_metadata_static(const int64_t* topk_idx, int N, int K, int E, int32_t* expert_counts,
                              int32_t* expert_offsets, int32_t* scatter_map, int32_t* gather_map,
                              int32_t* gate_idx_map, void* stream) {
  return launch_moe_metadata_static(topk_idx, N, K, E, expert_counts, expert_offsets, scatter_map, gather_map,
                                    gate_idx_map, static_cast<cudaStream_t>(stream));
}

int jb200_moe_dispatch_gather(const void* x, const int32_t* gather_map, int M, int N, int C, void* dispatched,
                              void* stream) {
  return launch_dispatch_gather(x, gather_map, M, N, C, dispatched, static_cast<cudaStream_t>(stream));
}

int jb200_moe_scatter_combine(const void* y, const float* gates, const int32_t* scatter_map, int N, int K, int C,
                              void* out, int out_dtype, double* stats, void* stream) {
  return launch_scatter_combine(y, gates, scatter_map, N, K, C, out, out_dtype, stats,
                                static_cast<cudaStream_t>(stream));
}

int jb200_moe_finalize(const double* stats, const double* probs_sum, const int32_t* top1_hist, int E,
                       long long n_tokens, long long n_elems, float balance_alpha, float* scalars, void* stream) {
  return launch_moe_finalize(stats, probs_sum, top1_hist, E, n_tokens, n_elems, balance_alpha, scalars,
                             static_cast<cudaStream_t>(stream));
}

int jb200_lsf_scan(const void* m, int m_dtype, const void* alpha_tensor, const float* alpha_scalar,
                   const float* act_var, const float* var_scale, float alpha_min, float alpha_max, const float* h0,
                   float* resid, void* out, int out_dtype, float* h_last, void* scratch, int B, int T, int D,
                   void* stream) {
  return launch_lsf_scan(m, m_dtype, alpha_tensor, alpha_scalar, act_var, var_scale, alpha_min, alpha_max, h0, resid,
                         out, out_dtype, h_last, scratch, B, T, D, static_cast<cudaStream_t>(stream));
}

size_t jb200_lsf_scan_scratch_bytes(int B, int T, int D) { return lsf_scan_scratch_bytes(B, T, D); }

int jb200_lsf_step_norm(const void* m_bf16, const double* stats, const double* probs_sum, const int32_t* top1_hist,
                        int E, long long n_tokens, long long n_elems, float balance_alpha, float* scalars,
                        const float* var_scale, float alpha_min, float alpha_max, const float* h_in, float* h_out,
                        float* x, const float* w_norm, float eps, void* xn_bf16, int B, int C, void* stream) {
  return launch_lsf_step_norm(m_bf16, stats, probs_sum, top1_hist, E, n_tokens, n_elems, balance_alpha, scalars,
                              var_scale, alpha_min, alpha_max, h_in, h_out, x, w_norm, eps, xn_bf16, B, C,
                              static_cast<cudaStream_t>(stream));
}

int jb200_prepare_weights(const uint8_t* packed, size_t n_bytes, uint8_t* prepared, void* stream) {
  return launch_prepare_weights(packed, n_bytes, prepared, static_cast<cudaStream_t>(stream));
}

void jb200_host_decode16(uint32_t word, uint32_t* out8) { decode16_host(word, out8); }
void jb200_host_decode16_prepared(uint32_t word, uint32_t* out8) { decode16_prepared_host(word, out8); }

}  // extern "C"
