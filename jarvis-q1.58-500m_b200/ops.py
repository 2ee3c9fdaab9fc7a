"""Thin tensor-level wrappers over the C ABI (one function per entry point).

Every function takes CUDA tensors, checks dtype/contiguity, passes raw device pointers and
the current CUDA stream, and raises RuntimeError with the library's message on failure.
Output tensors are allocated here with torch (device memory plumbing only).
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import ATTN_QK_PREPARED, EPI_BF16, EPI_F32, EPI_GELU_BF16, EPI_RESID_F32  # noqa: F401


# torch's current stream of the current device as a raw cudaStream_t.  torch.cuda.current_stream() builds a Stream
# object behind several Python-level checks (~7 us); with ~340 launches per forward that is a third of the
# host time of a forward, so the two C accessors are used directly when this torch has them.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return None if t is None else t.data_ptr()


def _overlap(a: torch.Tensor, b: torch.Tensor) -> bool:
    """True when the memory of two contiguous tensors intersects (same tensor, views, slices of one buffer)."""
    a0, b0 = a.data_ptr(), b.data_ptr()
    return a0 < b0 + b.numel() * b.element_size() and b0 < a0 + a.numel() * a.element_size()


def _need(t: torch.Tensor, dtype, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise RuntimeError(f"{name}: expected a CUDA tensor (this path has no CPU fallback)")
    if t.dtype != dtype:
        raise RuntimeError(f"{name}: expected dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise RuntimeError(f"{name}: expected a contiguous tensor")
    return t


# --------------------------------------------------------------------------- ternary weights
def pack_ternary(w: torch.Tensor, alpha: torch.Tensor | None = None):
    """Absmean-quantise and pack one (out, in) fp32 weight matrix.

    Returns (packed uint8 (out, in/4), alpha fp32 (1,)).  Mirrors TernaryQuantizeSTE.forward
    (jarvis_engine/utils/ternary_ops.py:24-31) + pack_ternary_tensor
    (runtime/weight_packing.py:22-51)."""
    lib = _lib.load()
    _need(w, torch.float32, "pack_ternary.w")
    if w.dim() != 2:
        raise RuntimeError("pack_ternary: expected a 2-D weight")
    out_f, in_f = w.shape
    if in_f % 4 != 0:
        raise RuntimeError("pack_ternary: Last dimension must be divisible by 4")
    packed = torch.empty((out_f, in_f // 4), dtype=torch.uint8, device=w.device)
    alpha_out = torch.empty((1,), dtype=torch.float32, device=w.device)
    scratch = None
    if alpha is None:
        nbytes = lib.jb200_pack_ternary_scratch_bytes(out_f, in_f)
        scratch = torch.empty((max(nbytes, 8) // 8,), dtype=torch.float64, device=w.device)
    else:
        alpha = _need(alpha.reshape(1), torch.float32, "pack_ternary.alpha")
    _lib.check(
        lib.jb200_pack_ternary(_ptr(w), out_f, in_f, _ptr(alpha), _ptr(packed), _ptr(alpha_out), _ptr(scratch),
                               _stream()),
        "jb200_pack_ternary",
    )
    return packed, alpha_out


def pack_codes(w_ternary: torch.Tensor) -> torch.Tensor:
    """pack_ternary_tensor (runtime/weight_packing.py:22-51) for a tensor of {-1, 0, +1}."""
    lib = _lib.load()
    w = _need(w_ternary.float().contiguous(), torch.float32, "pack_codes.w")
    if w.shape[-1] % 4 != 0:
        raise RuntimeError("pack_codes: Last dimension must be divisible by 4")
    packed = torch.empty((*w.shape[:-1], w.shape[-1] // 4), dtype=torch.uint8, device=w.device)
    _lib.check(lib.jb200_pack_codes(_ptr(w), w.numel(), _ptr(packed), _stream()), "jb200_pack_codes")
    return packed


def unpack_ternary(packed: torch.Tensor, shape, dtype=torch.bfloat16) -> torch.Tensor:
    """unpack_ternary_tensor (runtime/weight_packing.py:53-70)."""
    lib = _lib.load()
    _need(packed, torch.uint8, "unpack_ternary.packed")
    if dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError("unpack_ternary: dtype must be float32 or bfloat16")
    out = torch.empty((packed.numel() * 4,), dtype=dtype, device=packed.device)
    _lib.check(
        lib.jb200_unpack_ternary(_ptr(packed), packed.numel(), 0 if dtype == torch.float32 else 1, _ptr(out),
                                 _stream()),
        "jb200_unpack_ternary",
    )
    return out.reshape(tuple(shape))


def prepare_weights(packed: torch.Tensor) -> torch.Tensor:
    """Canonical packed weights -> the GEMM's fast-decode layout (same shape and size)."""
    lib = _lib.load()
    _need(packed, torch.uint8, "prepare_weights.packed")
    out = torch.empty_like(packed)
    _lib.check(lib.jb200_prepare_weights(_ptr(packed), packed.numel(), _ptr(out), _stream()), "jb200_prepare_weights")
    return out


def ternary_linear(x: torch.Tensor, packed: torch.Tensor, alpha: torch.Tensor, *, epilogue: int = EPI_BF16,
                   out: torch.Tensor | None = None, alpha_rows: int | None = None, token_tile: int = 0,
                   prepared: bool = False):
    """epilogue(alpha * x @ unpack(packed)^T): x bf16 (M, K), packed uint8 (N, K/4) in the canonical
    layout, or in the prepare_weights layout when prepared=True."""
    lib = _lib.load()
    _need(x, torch.bfloat16, "ternary_linear.x")
    _need(packed, torch.uint8, "ternary_linear.packed")
    _need(alpha, torch.float32, "ternary_linear.alpha")
    M, K = x.shape
    N = packed.shape[0]
    if packed.shape[1] * 4 != K:
        raise RuntimeError(f"ternary_linear: packed weight has K={packed.shape[1] * 4}, x has K={K}")
    if alpha_rows is None:
        alpha_rows = N // alpha.numel()
    if out is None:
        odt = torch.bfloat16 if epilogue in (EPI_BF16, EPI_GELU_BF16) else torch.float32
        if epilogue == EPI_RESID_F32:
            raise RuntimeError("ternary_linear: the residual epilogue needs `out` (the f32 residual stream)")
        out = torch.empty((M, N), dtype=odt, device=x.device)
    else:
        _need(out, torch.bfloat16 if epilogue in (EPI_BF16, EPI_GELU_BF16) else torch.float32, "ternary_linear.out")
        if tuple(out.shape) != (M, N):
            raise RuntimeError("ternary_linear: out has the wrong shape")
    _lib.check(
        lib.jb200_ternary_linear(_ptr(x), M, K, _ptr(packed), _ptr(alpha), alpha_rows, N, epilogue, _ptr(out),
                                 token_tile, 1 if prepared else 0, _stream()),
        "jb200_ternary_linear",
    )
    return out


def ternary_linear_grouped(x: torch.Tensor, packed: torch.Tensor, alpha: torch.Tensor, seg_offsets: torch.Tensor, *,
                           epilogue: int = EPI_BF16, out: torch.Tensor | None = None, token_tile: int = 0,
                           prepared: bool = False):
    """Rows [seg_offsets[g], seg_offsets[g+1]) of x (bf16 (M, K)) go through weight g of
    packed (uint8 (G, N, K/4)) with scale alpha[g]."""
    lib = _lib.load()
    _need(x, torch.bfloat16, "ternary_linear_grouped.x")
    _need(packed, torch.uint8, "ternary_linear_grouped.packed")
    _need(alpha, torch.float32, "ternary_linear_grouped.alpha")
    _need(seg_offsets, torch.int32, "ternary_linear_grouped.seg_offsets")
    M, K = x.shape
    G, N, K4 = packed.shape
    if K4 * 4 != K or alpha.numel() != G or seg_offsets.numel() != G + 1:
        raise RuntimeError("ternary_linear_grouped: inconsistent shapes")
    if out is None:
        odt = torch.bfloat16 if epilogue in (EPI_BF16, EPI_GELU_BF16) else torch.float32
        out = torch.empty((M, N), dtype=odt, device=x.device)   # the segments cover every row
    _lib.check(
        lib.jb200_ternary_linear_grouped(_ptr(x), M, K, _ptr(packed), _ptr(alpha), N, G, _ptr(seg_offsets), epilogue,
                                         _ptr(out), token_tile, 1 if prepared else 0, _stream()),
        "jb200_ternary_linear_grouped",
    )
    return out


def dense_linear(x: torch.Tensor, w: torch.Tensor, *, out_dtype=torch.bfloat16, out: torch.Tensor | None = None,
                 token_tile: int = 0) -> torch.Tensor:
    """x @ w^T with dense bf16 weights on the tensor-core pipeline of the ternary GEMM (weight tiles by TMA instead
    of the 2-bit decode): the lm_head, nn.Linear(d_model, vocab, bias=False) (jarvis_engine/jarvis_model.py:458, 535).
    x: bf16 (M, K); w: bf16 (N, K) with N % 128 == 0 (pad the vocabulary with zero rows) -> (M, N)."""
    lib = _lib.load()
    _need(x, torch.bfloat16, "dense_linear.x")
    _need(w, torch.bfloat16, "dense_linear.w")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise RuntimeError(f"dense_linear: weight has K={w.shape[1]}, x has K={K}")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    else:
        _need(out, out_dtype, "dense_linear.out")
        if tuple(out.shape) != (M, N):
            raise RuntimeError("dense_linear: out has the wrong shape")
    _lib.check(lib.jb200_dense_linear(_ptr(x), M, K, _ptr(w), N, _dt(out), _ptr(out), token_tile, _stream()),
               "jb200_dense_linear")
    return out


def interleave_head_rows(packed_rows: torch.Tensor, n_heads: int) -> torch.Tensor:
    """Row permutation qkv_linear_rope expects for a q or k projection: inside every 64-row head, new row 2i is
    old row i and new row 2i + 1 is old row i + 32 (RoPE partners become neighbouring out-features).
    packed_rows: (n_heads * 64, ...) any dtype (applied to the PACKED rows, before prepare_weights)."""
    idx = torch.arange(64, device=packed_rows.device)
    src = (idx >> 1) + 32 * (idx & 1)
    full = (torch.arange(n_heads, device=packed_rows.device).view(-1, 1) * 64 + src.view(1, -1)).reshape(-1)
    return packed_rows.index_select(0, full).contiguous()


def qkv_linear_rope(x: torch.Tensor, packed: torch.Tensor, alpha: torch.Tensor, cos_tab: torch.Tensor,
                    sin_tab: torch.Tensor, T: int, rope_feats: int, *, start_pos=0, alpha_rows: int | None = None,
                    out: torch.Tensor | None = None, token_tile: int = 0, prepared: bool = False):
    """The fused q|k|v projection with the attention prologue in its epilogue: out-features [0, rope_feats)
    (q and k heads, rows interleaved with interleave_head_rows) get ELU+1 and RoPE at position
    start_pos[row // T] + row % T; the rest (v) is the plain bf16 output.  -> bf16 (M, N)."""
    lib = _lib.load()
    _need(x, torch.bfloat16, "qkv_linear_rope.x")
    _need(packed, torch.uint8, "qkv_linear_rope.packed")
    _need(alpha, torch.float32, "qkv_linear_rope.alpha")
    _need(cos_tab, torch.float32, "qkv_linear_rope.cos_tab")
    _need(sin_tab, torch.float32, "qkv_linear_rope.sin_tab")
    M, K = x.shape
    N = packed.shape[0]
    if packed.shape[1] * 4 != K:
        raise RuntimeError(f"qkv_linear_rope: packed weight has K={packed.shape[1] * 4}, x has K={K}")
    if cos_tab.shape[1] != 32 or sin_tab.shape != cos_tab.shape:
        raise RuntimeError("qkv_linear_rope: RoPE tables must be (n_pos, 32)")
    if alpha_rows is None:
        alpha_rows = N // alpha.numel()
    pos_t, pos_s = None, 0
    if torch.is_tensor(start_pos):
        pos_t = _need(start_pos, torch.int32, "qkv_linear_rope.start_pos")
        if pos_t.numel() * T != M:
            raise RuntimeError("qkv_linear_rope: one start position per sequence is needed")
    else:
        pos_s = int(start_pos)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    else:
        _need(out, torch.bfloat16, "qkv_linear_rope.out")
    _lib.check(
        lib.jb200_qkv_linear_rope(_ptr(x), M, K, _ptr(packed), _ptr(alpha), alpha_rows, N, rope_feats, _ptr(cos_tab),
                                  _ptr(sin_tab), cos_tab.shape[0], _ptr(pos_t), pos_s, T, _ptr(out), token_tile,
                                  1 if prepared else 0, _stream()),
        "jb200_qkv_linear_rope",
    )
    return out


def selftest_bounded_wait(limit_ms: int = 50) -> int:
    """Runs the wait-that-must-give-up kernel and returns the device status it left."""
    lib = _lib.load()
    _lib.device_status(clear=True)
    _lib.check(lib.jb200_selftest_bounded_wait(limit_ms, _stream()), "jb200_selftest_bounded_wait")
    return _lib.device_status(clear=True)


# --------------------------------------------------------------------------- glue
def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise RuntimeError(f"expected float32 or bfloat16, got {t.dtype}")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, out_dtype=torch.bfloat16) -> torch.Tensor:
    """RMSNorm.forward (jarvis_engine/jarvis_model.py:25-26) over the last axis."""
    lib = _lib.load()
    if not (x.is_cuda and x.is_contiguous()):
        raise RuntimeError("rmsnorm: expected a contiguous CUDA tensor")
    _need(weight, torch.float32, "rmsnorm.weight")
    C = x.shape[-1]
    y = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    _lib.check(lib.jb200_rmsnorm(_ptr(x), _dt(x), _ptr(weight), eps, _ptr(y), _dt(y), x.numel() // C, C, _stream()),
               "jb200_rmsnorm")
    return y


def embedding(idx: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """tok_emb gather into the f32 residual stream (jarvis_engine/jarvis_model.py:498)."""
    lib = _lib.load()
    _need(idx, torch.int64, "embedding.idx")
    _need(table, torch.float32, "embedding.table")
    out = torch.empty((*idx.shape, table.shape[1]), dtype=torch.float32, device=idx.device)
    _lib.check(lib.jb200_embedding(_ptr(idx), _ptr(table), table.shape[0], _ptr(out), idx.numel(), table.shape[1],
                                   _stream()), "jb200_embedding")
    return out


# --------------------------------------------------------------------------- attention scan
def attn_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gamma: torch.Tensor, cos_tab: torch.Tensor,
              sin_tab: torch.Tensor, B: int, T: int, H: int, *, start_pos=0, state_in: torch.Tensor | None = None,
              want_state: bool = False, out: torch.Tensor | None = None, segmented: bool = True,
              state_out: torch.Tensor | None = None, qk_prepared: bool = False, want_out: bool = True):
    """Feature map + RoPE + decayed causal scan (qk_prepared=True: q and k come from qkv_linear_rope, the
    scan skips its prologue; want_out=False: state only, returns (None, state) after a k/v-only pass).  q, k, v: bf16 2-D views (B*T, H*64) sharing one
    row stride (e.g. column slices of a fused q|k|v matrix).  start_pos: int, or int32 (B,) tensor of
    per-sequence first positions.  Returns (o bf16 (B*T, H*64), final state f32 (B,H,64,64) or None)."""
    lib = _lib.load()
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not (t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1):
            raise RuntimeError(f"attn_scan.{name}: expected a 2-D bf16 CUDA tensor with unit inner stride")
    ld = q.stride(0)
    if k.stride(0) != ld or v.stride(0) != ld or tuple(q.shape) != (B * T, H * 64):
        raise RuntimeError("attn_scan: q, k, v must share shape (B*T, H*64) and row stride")
    _need(gamma, torch.float32, "attn_scan.gamma")
    _need(cos_tab, torch.float32, "attn_scan.cos_tab")
    _need(sin_tab, torch.float32, "attn_scan.sin_tab")
    if cos_tab.shape[1] != 32 or sin_tab.shape != cos_tab.shape:
        raise RuntimeError("attn_scan: RoPE tables must be (n_pos, 32)")
    pos_t, pos_s = None, 0
    if torch.is_tensor(start_pos):
        pos_t = _need(start_pos, torch.int32, "attn_scan.start_pos")
    else:
        pos_s = int(start_pos)
    if state_in is not None:
        _need(state_in, torch.float32, "attn_scan.state_in")
        if tuple(state_in.shape) != (B, H, 64, 64):
            raise RuntimeError("attn_scan: state_in must be (B, H, 64, 64)")
    if not want_out:
        if T <= 1:
            raise RuntimeError("attn_scan: a state-only call needs T > 1")
        want_state, segmented, out = True, True, None
    elif out is None:
        out = torch.empty((B * T, H * 64), dtype=torch.bfloat16, device=q.device)
    if state_out is not None:
        # may alias state_in when the call runs one segment per sequence (every CTA reads its own
        # (sequence, head) state before it writes it): the decode step updates states in place
        s_out = _need(state_out, torch.float32, "attn_scan.state_out")
        if state_in is not None and _overlap(state_out, state_in):
            segmented = False      # also for two views of one buffer: segment CTAs would read what the last one writes
    else:
        s_out = torch.empty((B, H, 64, 64), dtype=torch.float32, device=q.device) if want_state else None
    scratch = None
    if segmented:
        nbytes = lib.jb200_attn_scan_scratch_bytes(B, T, H)
        if nbytes:
            scratch = torch.empty((nbytes // 4,), dtype=torch.float32, device=q.device)
    _lib.check(
        lib.jb200_attn_scan(_ptr(q), _ptr(k), _ptr(v), ld, _ptr(gamma), _ptr(cos_tab), _ptr(sin_tab), cos_tab.shape[0],
                            _ptr(pos_t), pos_s, _ptr(state_in), _ptr(out), out.stride(0) if out is not None else 0, _ptr(s_out),
                            _ptr(scratch),
                            B, T, H, 64, ATTN_QK_PREPARED if qk_prepared else 0, _stream()),
        "jb200_attn_scan",
    )
    return out, s_out


# --------------------------------------------------------------------------- MoE routing
def router_top2(x: torch.Tensor, w_router: torch.Tensor, *, want_probs: bool = False, probs_sum=None, top1_hist=None):
    """Returns (topk_idx int64 (N, 2), gates f32 (N, 2), probs f32 (N, E) or None)."""
    lib = _lib.load()
    _need(x, torch.bfloat16, "router_top2.x")
    _need(w_router, torch.float32, "router_top2.w_router")
    N, C = x.shape
    E = w_router.shape[0]
    idx = torch.empty((N, 2), dtype=torch.int64, device=x.device)
    gates = torch.empty((N, 2), dtype=torch.float32, device=x.device)
    probs = torch.empty((N, E), dtype=torch.float32, device=x.device) if want_probs else None
    _lib.check(lib.jb200_router_top2(_ptr(x), _ptr(w_router), N, C, E, _ptr(idx), _ptr(gates), _ptr(probs),
                                     _ptr(probs_sum), _ptr(top1_hist), _stream()), "jb200_router_top2")
    return idx, gates, probs


def rmsnorm_router(x: torch.Tensor, w_norm: torch.Tensor, eps: float, w_router: torch.Tensor, *, probs_sum=None,
                   top1_hist=None, xn_out: torch.Tensor | None = None):
    """Fused norm2 + router: x f32 (N, C) -> (xn bf16 (N, C), topk_idx int64 (N, 2), gates f32 (N, 2)).
    xn_out: where to write the normalised rows (e.g. a buffer other GPUs read) instead of a new tensor."""
    lib = _lib.load()
    _need(x, torch.float32, "rmsnorm_router.x")
    _need(w_norm, torch.float32, "rmsnorm_router.w_norm")
    _need(w_router, torch.float32, "rmsnorm_router.w_router")
    N, C = x.shape
    E = w_router.shape[0]
    if xn_out is None:
        xn = torch.empty((N, C), dtype=torch.bfloat16, device=x.device)
    else:
        xn = _need(xn_out, torch.bfloat16, "rmsnorm_router.xn_out")
        if tuple(xn.shape) != (N, C):
            raise RuntimeError("rmsnorm_router: xn_out has the wrong shape")
    idx = torch.empty((N, 2), dtype=torch.int64, device=x.device)
    gates = torch.empty((N, 2), dtype=torch.float32, device=x.device)
    _lib.check(lib.jb200_rmsnorm_router(_ptr(x), _ptr(w_norm), eps, _ptr(xn), _ptr(w_router), N, C, E, _ptr(idx),
                                        _ptr(gates), _ptr(probs_sum), _ptr(top1_hist), _stream()),
               "jb200_rmsnorm_router")
    return xn, idx, gates


def moe_metadata(topk_idx: torch.Tensor, num_experts: int, *, gather_out: torch.Tensor | None = None,
                 offsets_out: torch.Tensor | None = None):
    """compute_metadata(topk_idx, E) -> (counts, offsets, scatter_map, gather_map, gate_idx_map), int32.
    gather_out (N*K,) / offsets_out (E+1,): caller-owned int32 buffers to write those two maps into (the expert-
    parallel exchange publishes them to the other ranks from its own buffer)."""
    lib = _lib.load()
    _need(topk_idx, torch.int64, "moe_metadata.topk_idx")
    N, K = topk_idx.shape
    dev = topk_idx.device
    i32 = torch.int32
    counts = torch.empty((num_experts,), dtype=i32, device=dev)
    if offsets_out is not None:
        offsets = _need(offsets_out, i32, "moe_metadata.offsets_out")
        if offsets.numel() != num_experts + 1:
            raise RuntimeError("moe_metadata: offsets_out must hold E + 1 entries")
    else:
        offsets = torch.empty((num_experts + 1,), dtype=i32, device=dev)
    scatter = torch.empty((N, K), dtype=i32, device=dev)
    if gather_out is not None:
        gather = _need(gather_out, i32, "moe_metadata.gather_out")
        if gather.numel() != N * K:
            raise RuntimeError("moe_metadata: gather_out must hold N * K entries")
    else:
        gather = torch.empty((N * K,), dtype=i32, device=dev)
    gate_idx = torch.empty((N * K,), dtype=i32, device=dev)
    nbytes = lib.jb200_moe_metadata_scratch_bytes(N, K, num_experts)
    scratch = torch.empty((max(nbytes, 4) // 4,), dtype=i32, device=dev)
    _lib.check(lib.jb200_moe_metadata(_ptr(topk_idx), N, K, num_experts, _ptr(counts), _ptr(offsets), _ptr(scatter),
                                      _ptr(gather), _ptr(gate_idx), _ptr(scratch), _stream()), "jb200_moe_metadata")
    return counts, offsets, scatter, gather, gate_idx


def dispatch_gather(x: torch.Tensor, gather_map: torch.Tensor) -> torch.Tensor:
    lib = _lib.load()
    _need(x, torch.bfloat16, "dispatch_gather.x")
    _need(gather_map, torch.int32, "dispatch_gather.gather_map")
    N, C = x.shape
    M = gather_map.numel()
    out = torch.empty((M, C), dtype=torch.bfloat16, device=x.device)
    _lib.check(lib.jb200_moe_dispatch_gather(_ptr(x), _ptr(gather_map), M, N, C, _ptr(out), _stream()),
               "jb200_moe_dispatch_gather")
    return out


def scatter_combine(y: torch.Tensor, gates: torch.Tensor, scatter_map: torch.Tensor, *, out_dtype=torch.bfloat16,
                    stats: torch.Tensor | None = None) -> torch.Tensor:
    lib = _lib.load()
    _need(y, torch.bfloat16, "scatter_combine.y")
    _need(gates, torch.float32, "scatter_combine.gates")
    _need(scatter_map, torch.int32, "scatter_combine.scatter_map")
    N, K = scatter_map.shape
    C = y.shape[1]
    out = torch.empty((N, C), dtype=out_dtype, device=y.device)
    if stats is not None:
        _need(stats, torch.float64, "scatter_combine.stats")
    _lib.check(lib.jb200_moe_scatter_combine(_ptr(y), _ptr(gates), _ptr(scatter_map), N, K, C, _ptr(out), _dt(out),
                                             _ptr(stats), _stream()), "jb200_moe_scatter_combine")
    return out


def moe_finalize(stats, probs_sum, top1_hist, E: int, n_tokens: int, n_elems: int, balance_alpha: float,
                 scalars: torch.Tensor | None = None) -> torch.Tensor:
    """-> f32 (3,) = [l_balance, act_mean, act_var]."""
    lib = _lib.load()
    ref = stats if stats is not None else probs_sum
    if scalars is None:
        scalars = torch.zeros((3,), dtype=torch.float32, device=ref.device)
    _lib.check(lib.jb200_moe_finalize(_ptr(stats), _ptr(probs_sum), _ptr(top1_hist), E, n_tokens, n_elems,
                                      balance_alpha, _ptr(scalars), _stream()), "jb200_moe_finalize")
    return scalars


# --------------------------------------------------------------------------- LSF
def lsf_scan(m: torch.Tensor, *, alpha_tensor=None, alpha_scalar=None, act_var=None, var_scale=None,
             alpha_min: float = 0.1, alpha_max: float = 0.99, h0=None, resid=None, want_out: bool = True,
             out_dtype=None, want_last: bool = True, segmented: bool = True, last_out: torch.Tensor | None = None):
    """m: (B, T, D) f32/bf16.  Returns (h_out or None, h_last f32 (B, D) or None)."""
    lib = _lib.load()
    if not (m.is_cuda and m.is_contiguous() and m.dim() == 3):
        raise RuntimeError("lsf_scan: expected a contiguous (B, T, D) CUDA tensor")
    B, T, D = m.shape
    if alpha_tensor is not None:
        if alpha_tensor.dtype != m.dtype or tuple(alpha_tensor.shape) != (B, T, D) or not alpha_tensor.is_contiguous():
            raise RuntimeError("lsf_scan: alpha tensor must match m in shape, dtype and layout")
    for name, t in (("alpha_scalar", alpha_scalar), ("act_var", act_var), ("var_scale", var_scale), ("h0", h0),
                    ("resid", resid)):
        if t is not None:
            _need(t, torch.float32, "lsf_scan." + name)
    out = torch.empty((B, T, D), dtype=out_dtype or m.dtype, device=m.device) if want_out else None
    if last_out is not None:
        h_last = _need(last_out, torch.float32, "lsf_scan.last_out")   # may alias h0 in unsegmented calls
        if h0 is not None and _overlap(last_out, h0):
            segmented = False
    else:
        h_last = torch.empty((B, D), dtype=torch.float32, device=m.device) if want_last else None
    scratch = None
    if segmented:
        nbytes = lib.jb200_lsf_scan_scratch_bytes(B, T, D)
        if nbytes:
            scratch = torch.empty((nbytes // 4,), dtype=torch.float32, device=m.device)
    _lib.check(
        lib.jb200_lsf_scan(_ptr(m), _dt(m), _ptr(alpha_tensor), _ptr(alpha_scalar), _ptr(act_var), _ptr(var_scale),
                           alpha_min, alpha_max, _ptr(h0), _ptr(resid), _ptr(out), _dt(out) if out is not None else 0,
                           _ptr(h_last), _ptr(scratch), B, T, D, _stream()),
        "jb200_lsf_scan",
    )
    return out, h_last


def lsf_step_norm(m: torch.Tensor, stats, probs_sum, top1_hist, E: int, n_tokens: int, n_elems: int,
                  balance_alpha: float, scalars: torch.Tensor, var_scale: torch.Tensor, alpha_min: float,
                  alpha_max: float, h_in, x: torch.Tensor, norm=None, h_out: torch.Tensor | None = None):
    """Single-token tail of a block in one launch: moe_finalize -> `scalars`, the LSF step h = a h_in + (1 - a) m
    with x += h in place, and (norm = (weight, eps)) the RMSNorm of the updated x.  m: bf16 (B, C); h_in f32 (B, C)
    or None; x: f32 (B, C).  Returns (xn bf16 (B, C) or None, h_out f32 (B, C)); h_out may be h_in."""
    lib = _lib.load()
    _need(m, torch.bfloat16, "lsf_step_norm.m")
    _need(x, torch.float32, "lsf_step_norm.x")
    B, C = m.shape
    if tuple(x.shape) != (B, C):
        raise RuntimeError("lsf_step_norm: x must have the shape of m")
    for name, t in (("h_in", h_in), ("h_out", h_out)):
        if t is not None and tuple(_need(t, torch.float32, "lsf_step_norm." + name).shape) != (B, C):
            raise RuntimeError(f"lsf_step_norm: {name} must be f32 (B, C)")
    _need(scalars, torch.float32, "lsf_step_norm.scalars")
    _need(var_scale, torch.float32, "lsf_step_norm.var_scale")
    if h_out is None:
        h_out = torch.empty((B, C), dtype=torch.float32, device=m.device)
    xn = w = None
    eps = 0.0
    if norm is not None:
        w, eps = _need(norm[0], torch.float32, "lsf_step_norm.norm weight"), float(norm[1])
        xn = torch.empty((B, C), dtype=torch.bfloat16, device=m.device)
    _lib.check(lib.jb200_lsf_step_norm(_ptr(m), _ptr(stats), _ptr(probs_sum), _ptr(top1_hist), E, n_tokens, n_elems,
                                       balance_alpha, _ptr(scalars), _ptr(var_scale), alpha_min, alpha_max, _ptr(h_in),
                                       _ptr(h_out), _ptr(x), _ptr(w), eps, _ptr(xn), B, C, _stream()),
               "jb200_lsf_step_norm")
    return xn, h_out


def sample(logits: torch.Tensor, u: torch.Tensor | None = None, *, temperature: float = 0.7, top_k: int = 50,
           top_p: float = 0.9, want_prob: bool = False):
    """One token per row of `logits` ((B, V) f32 or bf16, rows may be strided): temperature / top-k / top-p
    filtering of sample_next_token (jarvis_engine/evaluate_jarvis.py:158-185) and an inverse-CDF draw with
    the caller's uniform numbers u (B,) f32.  temperature <= 0: argmax.  -> int64 (B, 1) [, f32 (B,) prob]."""
    lib = _lib.load()
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise RuntimeError("sample: logits must be (B, V) with contiguous rows")
    if logits.dtype not in (torch.float32, torch.bfloat16) or not logits.is_cuda:
        raise RuntimeError("sample: logits must be a CUDA f32 or bf16 tensor")
    B, V = logits.shape
    greedy = temperature is None or temperature <= 0.0
    if u is None:
        if not greedy and top_k != 1:
            raise RuntimeError("sample: a uniform number per row (u) is needed to draw")
    else:
        _need(u, torch.float32, "sample.u")
        if u.numel() != B:
            raise RuntimeError("sample: u must hold one number per row")
    out = torch.empty((B, 1), dtype=torch.int64, device=logits.device)
    prob = torch.empty((B,), dtype=torch.float32, device=logits.device) if want_prob else None
    _lib.check(
        lib.jb200_sample(_ptr(logits), 0 if logits.dtype == torch.float32 else 1, logits.stride(0), B, V,
                         0.0 if greedy else float(temperature), int(top_k or 0), float(top_p if top_p is not None else 0.0),
                         _ptr(u) if u is not None else None, _ptr(out), _ptr(prob) if prob is not None else None, _stream()),
        "jb200_sample",
    )
    return (out, prob) if want_prob else out
