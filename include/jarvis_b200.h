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
#define JB200_EPI_QK_ROPE_BF16 4 /* jb200_qkv_linear_rope only: bf16 out, attention prologue on the q/k heads */
#define JB200_ATTN_QK_PREPARED 1 /* jb200_attn_scan flag: q, k come from jb200_qkv_linear_rope */

/* device status codes (0 = no bounded wait ever ran out) */
#define JB200_STATUS_GEMM_PRODUCER 0x11u
#define JB200_STATUS_GEMM_MMA 0x12u
#define JB200_STATUS_GEMM_DECODE 0x13u
#define JB200_STATUS_GEMM_EPILOGUE 0x14u
#define JB200_STATUS_ATTN_LOAD 0x21u
#define JB200_STATUS_ATTN_MMA 0x22u
#define JB200_STATUS_ATTN_HANDOFF 0x23u   /* the second part of a cut sequence never saw the first part's state */
#define JB200_STATUS_LSF_LOAD 0x31u
#define JB200_STATUS_PEER_BARRIER 0x41u
#define JB200_STATUS_SELFTEST_WAIT 0x7Fu

/* ---- library ----------------------------------------------------------------------- */

/* Message of this thread's last failed call ("" if none). */
const char* jb200_last_error(void);

/* ABI version of this library (bumped on any signature change). */
int jb200_abi_version(void);

/* Number of kernels this library has launched in this process since the last reset
 * (returns the count before resetting when `reset` is non-zero). */
long long jb200_kernel_launches(int reset);

/* The kernels of the forward chain are launched with programmatic stream serialisation: each starts while the
 * kernel before it on the stream is still running and waits (griddepcontrol.wait) before it touches memory, so
 * launch latency and set-up overlap the predecessor; captured into CUDA graphs as programmatic edges.  No
 * reference counterpart (the reference launches each kernel fully serialised).  enable = 0 launches them fully
 * serialised again; returns the previous setting.  The environment variable JB200_DEPENDENT_LAUNCH=0 sets the
 * initial state. */
int jb200_set_dependent_launch(int enable);

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
 * token_tile: 0 = choose, else one of 32/64/128/256.
 * w_layout: 0 = `packed` is the canonical weight_packing.py layout; 1 = `packed` was re-encoded by
 * jb200_prepare_weights (same size, about 4x fewer decode instructions in the kernel). */
int jb200_ternary_linear(const void* x, int M, int K, const uint8_t* packed, const float* alpha, int alpha_rows,
                         int N, int epilogue, void* out, int token_tile, int w_layout, void* stream);

/* Dense bf16 linear layer without bias on the same tensor-core pipeline: Y = X W^T.  Replaces the one dense
 * projection of the path, lm_head = nn.Linear(d_model, vocab_size, bias=False) (jarvis_engine/jarvis_model.py:458, 535),
 * which the reference does not quantise.  x: bf16 [M][K]; w: bf16 [N][K] (N % 128 == 0: pad the vocabulary rows with
 * zeros; K % 64 == 0); out: [M][N] bf16 (out_dtype 1) or f32 (out_dtype 0), row stride N.  Weight tiles are loaded
 * by TMA next to the activation tiles; token_tile as in jb200_ternary_linear. */
int jb200_dense_linear(const void* x, int M, int K, const void* w, int N, int out_dtype, void* out, int token_tile,
                       void* stream);

/* The q/k/v projection fused with the prologue of the attention scan: as jb200_ternary_linear with a bf16
 * output, but out-features [0, rope_feats) (the q and k heads, 64 features each) come out as
 *   phi(x) = ELU(x) + 1, then half-split RoPE at position pos0[row / T] + row % T
 * (AssociativeLinearAttention.forward, jarvis_engine/jarvis_model.py:124-128; apply_rotary_emb :29-71; fused kernel
 * A1, associative_attention_cuda/associative_attention_cuda.cu:28-112), computed in f32 on the accumulator and
 * rounded to bf16 once.  The caller must have INTERLEAVED the weight rows of every q/k head: row 2i of a head
 * holds the head's feature i, row 2i+1 its feature i + 32 (i < 32); the output keeps that order, which
 * jb200_attn_scan reads with JB200_ATTN_QK_PREPARED.  The queries' 1/sqrt(64) is applied by the scan.
 * cos_tab / sin_tab: f32 [n_pos][32]; pos0: int32 [M / T] or NULL (then pos0_scalar); positions are clamped
 * to the table.  M % T == 0. */
int jb200_qkv_linear_rope(const void* x, int M, int K, const uint8_t* packed, const float* alpha, int alpha_rows,
                          int N, int rope_feats, const float* cos_tab, const float* sin_tab, int n_pos,
                          const int32_t* pos0, int pos0_scalar, int T, void* out, int token_tile, int w_layout,
                          void* stream);

/* One-time re-encoding of canonical packed weights for the GEMM's fast decode: still 2 bits per
 * weight and the same byte count; inside each aligned group of 16 in-features (one 32-bit word) the
 * even in-features move to the low half-word and the odd ones to the high half-word, each stored as
 * (sign << 1 | nonzero).  Works on any number of whole words (n_bytes % 4 == 0), so stacked matrices
 * can be converted in one call.  No counterpart in the reference (its prototype decodes byte by byte,
 * experiments/architecture_matrix/ternary_packed/packed_kernel.cu:46-68). */
int jb200_prepare_weights(const uint8_t* packed, size_t n_bytes, uint8_t* prepared, void* stream);

/* Grouped form for the MoE experts: rows [seg_offsets[g], seg_offsets[g+1]) of x use weight
 * matrix g (packed: u8 [G][N][K/4], alpha: f32 [G]).  seg_offsets: i32 [G+1] on the DEVICE
 * (the expert_offsets of jb200_moe_metadata), so no host synchronisation is needed -- the
 * reference reads them back with .cpu() every layer (sparse_model_cuda/sparse_model.py:157)
 * and loops over experts on the host (:159-164). */
int jb200_ternary_linear_grouped(const void* x, int M, int K, const uint8_t* packed, const float* alpha, int N,
                                 int G, const int32_t* seg_offsets, int epilogue, void* out, int token_tile,
                                 int w_layout, void* stream);

/* ---- block glue --------------------------------------------------------------------- */

/* RMSNorm.forward (jarvis_engine/jarvis_model.py:25-26): y = x * rsqrt(mean(x^2) + eps) * w.
 * x: [n_rows][C] f32 (dtype 0) or bf16 (dtype 1); w: f32 [C]; y: f32 or bf16.  C % 8 == 0, C <= 4096. */
int jb200_rmsnorm(const void* x, int x_dtype, const float* w, float eps, void* y, int y_dtype, int n_rows, int C,
                  void* stream);

/* Token embedding gather (nn.Embedding, jarvis_engine/jarvis_model.py:452, 498) into the f32
 * residual stream.  idx: i64 [n_rows]; table: f32 [vocab][C]; out: f32 [n_rows][C]. */
int jb200_embedding(const int64_t* idx, const float* table, int vocab, float* out, int n_rows, int C, void* stream);

/* ---- attention scan ----------------------------------------------------------------- */

/* Feature map + RoPE + chunkwise decayed scan, with the carried state in and out.  Replaces
 * fused_rope_elu_forward + the four bmm + recurrent_chunk_state_scan_forward of the CUDA drop-in
 * (associative_attention_cuda/associative_attention_cpp.cpp:36-57, associative_attention.py:232-266)
 * and the chunk loop of AssociativeLinearAttention.forward (jarvis_engine/jarvis_model.py:124-190).
 * q, k, v: bf16 rows [B*T] with row stride ld_qkv elements, head h at columns [64h, 64h+64) (the raw
 *   projection outputs: a fused q|k|v matrix is passed as three pointers into it);
 * gamma: f32 [H] = sigmoid(gamma_raw);  cos_tab/sin_tab: f32 [n_pos][32] (first half of the RoPE cache);
 * pos0: i32 [B] first position of each sequence, or NULL to use pos0_scalar for all (start_pos);
 * s_in / s_out: f32 [B][H][64][64] (D_v x D_k, the layout of h_prev / h_last), each may be NULL;
 * o: bf16 rows [B*T] with stride ld_o.  head_dim must be 64.
 * scratch: jb200_attn_scan_scratch_bytes(B, T, H) bytes (8-byte aligned) or NULL.  With scratch, long
 *   sequences are cut into segments that run in parallel (a first launch computes each segment's state
 *   contribution from k and v); with NULL every (sequence, head) is walked by one CTA.
 * o == NULL (then q may be NULL too; needs s_out, scratch, T > 1): state only - just the k/v half of the work,
 *   every piece of the sequence in parallel, and s_out = the state after the sequence (what a rank of a
 *   context-parallel group needs from its slice before it knows its incoming state).
 * flags: 0, or JB200_ATTN_QK_PREPARED when q and k were produced by jb200_qkv_linear_rope (feature map and
 * RoPE already applied, head dim interleaved): the scan then skips its own prologue; s_in / s_out keep the
 * natural (B, H, D_v, D_k) order either way.  T == 1 (decode step) takes raw q, k only.
 */
size_t jb200_attn_scan_scratch_bytes(int B, int T, int H);
int jb200_attn_scan(const void* q, const void* k, const void* v, int ld_qkv, const float* gamma,
                    const float* cos_tab, const float* sin_tab, int n_pos, const int32_t* pos0, int pos0_scalar,
                    const float* s_in, void* o, int ld_o, float* s_out, void* scratch, int B, int T, int H,
                    int head_dim, int flags, void* stream);

/* ---- MoE routing ---------------------------------------------------------------------- */

/* Eval-mode router of SparseMoELayer.forward (jarvis_engine/jarvis_model.py:218-224): logits in f32,
 * softmax, top-2 (equal probabilities: lower expert id first), gates = p / (p0 + p1 + 1e-8).
 * x: bf16 [N][C]; w_router: f32 [E][C] (E = 4 or 8, C % 8 == 0);
 * topk_idx: i64 [N][2]; gates: f32 [N][2]; probs: f32 [N][E] or NULL;
 * probs_sum: f64 [E] or NULL and top1_hist: i32 [E] or NULL are ACCUMULATED into (zero them first):
 * the P and f of the load-balance loss (jarvis_model.py:244-247). */
int jb200_router_top2(const void* x, const float* w_router, int N, int C, int E, int64_t* topk_idx, float* gates,
                      float* probs, double* probs_sum, int32_t* top1_hist, void* stream);

/* norm2 + router in one pass over the f32 residual stream (JarvisBlock.forward, jarvis_model.py:431:
 * self.moe(self.norm2(x)) with RMSNorm :25-26 and the router :218-224): writes xn = bf16(RMSNorm(x))
 * for the expert GEMMs and routes from those same rounded values, bit-identical to jb200_rmsnorm followed
 * by jb200_router_top2.  x: f32 [N][C] (C % 8 == 0, C <= 1024); other arguments as jb200_router_top2. */
int jb200_rmsnorm_router(const float* x, const float* w_norm, float eps, void* xn, const float* w_router, int N,
                         int C, int E, int64_t* topk_idx, float* gates, double* probs_sum, int32_t* top1_hist,
                         void* stream);

/* compute_metadata (sparse_model_cuda/sparse_model_cpp.cpp:83-90, kernel sparse_model.cu:23-90):
 * stable partition of assignments m = token*K + k by expert.  All outputs i32:
 * expert_counts [E], expert_offsets [E+1], scatter_map [N][K] (slot of m), gather_map [N*K]
 * (token of slot), gate_idx_map [N*K] (k of slot).  scratch: jb200_moe_metadata_scratch_bytes. */
size_t jb200_moe_metadata_scratch_bytes(int N, int K, int E);
int jb200_moe_metadata(const int64_t* topk_idx, int N, int K, int E, int32_t* expert_counts,
                       int32_t* expert_offsets, int32_t* scatter_map, int32_t* gather_map, int32_t* gate_idx_map,
                       void* scratch, void* stream);

/* Same result as jb200_moe_metadata, but without a scratch argument and without any allocation.
 * (No counterpart in the reference: its extension allocates its outputs and work buffers through
 * torch on every call.)  It is meant for hosts that cannot hand this library device memory on
 * demand -- for example an inference server that gives all device memory to its own arena at
 * start-up and gives plugins a fixed share of it, or a latency-critical loop that must not reach
 * cudaMalloc because that call stalls the whole device.  The work arrays live in a 128 KiB array
 * built into the library (every GPU that loads the library carries it until the process exits),
 * which limits N*K to jb200_moe_metadata_static_max_assignments() = 262144; larger inputs are
 * refused with JB200_ERR_ARG.  The first call on each device looks up the array's device address
 * (a host-side runtime query, nothing is allocated); make that first call during start-up, before
 * any stream capture is begun.  All calls on a device share the one array: two calls whose kernels
 * may overlap on the GPU (different streams, no ordering between them) race on it -- keep them on
 * one stream or order them with events.  The caller still owns all inputs and outputs. */
int jb200_moe_metadata_static_max_assignments(void);
int jb200_moe_metadata_static(const int64_t* topk_idx, int N, int K, int E, int32_t* expert_counts,
                              int32_t* expert_offsets, int32_t* scatter_map, int32_t* gather_map,
                              int32_t* gate_idx_map, void* stream);

/* dispatch_gather (sparse_model.cu:95-112): dispatched[slot][:] = x[gather_map[slot]][:], bf16 rows of C. */
int jb200_moe_dispatch_gather(const void* x, const int32_t* gather_map, int M, int N, int C, void* dispatched,
                              void* stream);

/* scatter_combine (sparse_model.cu:117-165): out[i] = sum_k gates[i][k] * y[scatter_map[i][k]] with f32
 * accumulation; y: bf16 [N*K][C]; out: f32 (0) or bf16 (1) [N][C].  stats: f64 [2] or NULL, ACCUMULATES
 * sum(out) and sum(out^2) of the unrounded values (for act_mean / act_var, jarvis_model.py:249-250). */
int jb200_moe_scatter_combine(const void* y, const float* gates, const int32_t* scatter_map, int N, int K, int C,
                              void* out, int out_dtype, double* stats, void* stream);

/* Side outputs of SparseMoELayer.forward (jarvis_model.py:244-250) from the accumulators above:
 * scalars[0] = l_balance = balance_alpha * E * sum_e f_e * P_e, scalars[1] = act_mean,
 * scalars[2] = act_var (unbiased).  Any accumulator may be NULL (its scalars are left untouched). */
int jb200_moe_finalize(const double* stats, const double* probs_sum, const int32_t* top1_hist, int E,
                       long long n_tokens, long long n_elems, float balance_alpha, float* scalars, void* stream);

/* ---- Liquid State Fusion ---------------------------------------------------------------- */

/* h_t = a*h_{t-1} + (1-a)*m_t along T for every (b, channel).
 * Model semantics (LiquidStateFusion.forward, jarvis_engine/jarvis_model.py:281-314): alpha_tensor NULL;
 *   the scalar decay is *alpha_scalar if given, else alpha_min + (alpha_max-alpha_min) *
 *   sigmoid(-(*var_scale) * (*act_var)) -- all device scalars.
 * Extension semantics (liquid_state_fusion_cuda.forward(alpha, M, h0),
 *   liquid_fusion_cuda/liquid_state_fusion_cpp.cpp:67-74): alpha_tensor [B][T][D] in m's dtype.
 * m: [B][T][D] f32 (0) or bf16 (1), D even;  h0: f32 [B][D] or NULL (zeros);
 * out: [B][T][D] f32/bf16 or NULL;  resid: f32 [B][T][D] or NULL, updated in place resid += h (the
 * block's residual add, jarvis_model.py:436);  h_last: f32 [B][D] or NULL.
 * scratch: jb200_lsf_scan_scratch_bytes(B, T, D) bytes (8-byte aligned) or NULL; with scratch, long
 * sequences are cut into segments that run in parallel (a first launch computes the segment ends). */
size_t jb200_lsf_scan_scratch_bytes(int B, int T, int D);
int jb200_lsf_scan(const void* m, int m_dtype, const void* alpha_tensor, const float* alpha_scalar,
                   const float* act_var, const float* var_scale, float alpha_min, float alpha_max, const float* h0,
                   float* resid, void* out, int out_dtype, float* h_last, void* scratch, int B, int T, int D,
                   void* stream);

/* Tail of a block for single-token steps (T = 1), three of the calls above in one launch with their results bit
 * for bit: jb200_moe_finalize (scalars from the accumulators; SparseMoELayer.forward, jarvis_model.py:244-250),
 * jb200_lsf_scan at T = 1 with the fused residual (decay from act_var; LiquidStateFusion.forward, jarvis_model.py:
 * 281-314, and the residual add :436: h_out = a*h_in + (1-a)*m, x += h_out) and, when w_norm is given, the
 * jb200_rmsnorm that follows (norm1 of the next block, jarvis_model.py:430, or the final norm :516) into xn_bf16.
 * m_bf16, xn_bf16: bf16 [B][C]; h_in (NULL = zeros), h_out (may alias h_in), x: f32 [B][C]; C a multiple of 8,
 * at most 1024.  n_tokens / n_elems as in jb200_moe_finalize. */
int jb200_lsf_step_norm(const void* m_bf16, const double* stats, const double* probs_sum, const int32_t* top1_hist,
                        int E, long long n_tokens, long long n_elems, float balance_alpha, float* scalars,
                        const float* var_scale, float alpha_min, float alpha_max, const float* h_in, float* h_out,
                        float* x, const float* w_norm, float eps, void* xn_bf16, int B, int C, void* stream);

/* ---- expert parallelism over peer memory (no counterpart: the reference is single-GPU) ------------------- */

/* Device buffers that other processes on the node can map (CUDA IPC).  alloc: cudaMalloc on the current device and
 * the 64-byte handle to send to the peers (by any host channel); open: maps a peer's buffer for kernels of the
 * CURRENT device (peer access over NVLink is switched on by the mapping); close / free undo them.  These are the
 * only entry points that allocate; call them at set-up time, never between kernels. */
int jb200_peer_buffer_alloc(size_t bytes, void** ptr, unsigned char* handle64);
int jb200_peer_buffer_open(const unsigned char* handle64, void** ptr);
int jb200_peer_buffer_close(void* ptr);
int jb200_peer_buffer_free(void* ptr);

/* Stream-ordered barrier over the ranks of one node through flags in peer-mapped memory (a few microseconds,
 * where a one-element collective costs a kernel launch of the communication library per rank).  peer_flags[r]:
 * a block of JB200_PEER_FLAG_WORDS i32 in rank r's peer-mapped buffer, zeroed once at set-up; word s is written by
 * rank s, the last word counts this rank's barriers.  The kernel (one warp) tells every rank that this rank's
 * earlier work on the stream has finished and waits until every rank has said so; kernels launched after it on the
 * stream see what the peers wrote before their call.  Every rank must call it the same number of times, one GPU
 * per rank (ranks sharing a GPU would wait for kernels that cannot start).  The wait is bounded (2 s): on expiry
 * the device status word gets JB200_STATUS_PEER_BARRIER and the kernel returns. */
#define JB200_PEER_FLAG_WORDS 32
int jb200_peer_barrier(const void* const* peer_flags, int world, int rank, void* stream);

/* The dispatch exchange of the MoE layer done by the gather itself: rank `rank` of `world` owns experts
 * [rank*E/world, (rank+1)*E/world) - or, when world > E (world % E == 0), part rank % (world/E) of expert
 * rank / (world/E): of every source's cnt rows of that expert the slice [cnt*part/shards, cnt*(part+1)/shards),
 * with E/world read as 1 in the sizes below - and builds their input rows by reading every rank's routing result and rows
 * directly from that rank's memory (plain loads over NVLink; all pointers in the three device arrays must be
 * mapped in this process, e.g. CUDA IPC handles of the peers' buffers):
 *   peer_offs[s]: i32 [E + 2] = rank s's expert_offsets (jb200_moe_metadata) followed by its n_tokens
 *   peer_gmap[s]: i32 [n_max * K] = its gather_map;   peer_xn[s]: bf16 [n_max][C] = its rows
 * Output: dispatched bf16 [max_rows][C], rows of owned expert 0 first, inside an expert ordered by (source rank,
 * local stable order) = the dispatch order of sparse_model_cuda/sparse_model.cu:23-90 when ranks hold contiguous
 * token ranges; seg_offsets i32 [E/world + 1] on the device for jb200_ternary_linear_grouped; meta i32
 * [(E/world) * (world + 1) + E/world + 1] (start of every source's rows inside each owned expert, then a copy of
 * seg_offsets), which the peers' jb200_ep_pull_combine reads.  Nothing is read back to the host; the caller
 * places a stream-ordered barrier over the ranks before this call (peers' buffers written), between the expert
 * GEMMs and jb200_ep_pull_combine (owners' outputs written), and before any of the buffers is reused. */
int jb200_ep_pull_gather(const void* const* peer_offs, const void* const* peer_gmap, const void* const* peer_xn,
                         int world, int rank, int E, int C, int K, int n_max, int max_rows, void* dispatched,
                         int32_t* seg_offsets, int32_t* meta, void* stream);

/* The return exchange fused with scatter_combine (sparse_model.cu:104-124): out[t] = sum_k gates[t][k] *
 * y_owner[row], the row read from the owner rank's output buffer peer_y[owner] (bf16 [max_rows][C]) at the
 * position its meta (peer_meta[owner]) gives for this rank's rows.  offs_local / topk_idx / gates / scatter_map are
 * this rank's own routing results; out f32 or bf16 [n_tokens][C]; stats as jb200_moe_scatter_combine. */
int jb200_ep_pull_combine(const void* const* peer_y, const void* const* peer_meta, const int32_t* offs_local,
                          const int64_t* topk_idx, const float* gates, const int32_t* scatter_map, int world, int rank,
                          int E, int C, int K, int n_tokens, int max_rows, void* out, int out_dtype, double* stats,
                          void* stream);

/* ---- decode driver: next-token sampling ------------------------------------------------------- */

/* One draw per row of logits, replacing sample_next_token (jarvis_engine/evaluate_jarvis.py:158-185):
 * temperature <= 0 -> argmax (lowest id among equals); else x = logits / max(temperature, 1e-5), keep
 * x >= the top_k-th largest x (ties kept), sort descending, softmax, drop position i >= 1 once the
 * cumulative probability before it exceeds top_p (0 < top_p < 1; other values: no nucleus cut), and draw
 * from the softmax over what is left.  The reference draws with torch.multinomial; here u[row] in [0, 1)
 * comes from the caller and the draw is the inverse CDF over the kept tokens in descending order of x
 * (equal x: lower id first).  logits: f32 (logits_dtype 0) or bf16 (1), row stride ld >= V elements.
 * top_k in 1..1024 (the reference's top_k=None, a nucleus cut over the full vocabulary, is not offered).
 * out_prob (optional, f32 [n_rows]): probability of the drawn token under the filtered distribution. */
int jb200_sample(const void* logits, int logits_dtype, int ld, int n_rows, int V, float temperature, int top_k,
                 float top_p, const float* u, int64_t* out_token, float* out_prob, void* stream);

/* Host-side copy of the bit manipulation the GEMM's decoder warps run: 16 two-bit codes
 * (one little-endian u32 of the packed layout) -> 16 bf16 values in out8[8] (two per u32,
 * lower in-feature in the low half).  Runs on the CPU; used by the unit tests. */
void jb200_host_decode16(uint32_t word, uint32_t* out8);
/* Same for the prepared layout: takes the CANONICAL word, re-encodes it as jb200_prepare_weights does and
 * decodes it as the kernel does; out8 holds 2 * {-1, 0, +1} as bf16 pairs. */
void jb200_host_decode16_prepared(uint32_t word, uint32_t* out8);

#ifdef __cplusplus
}
#endif
#endif /* JARVIS_B200_H_ */
