"""Thin tensor-level wrappers over the C ABI (one function per entry point).

Every function takes CUDA tensors, checks dtype/contiguity, passes raw device pointers and
the current CUDA stream, and raises RuntimeError with the library's message on failure.
Output tensors are allocated here with torch (device memory plumbing only).
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import EPI_BF16, EPI_F32, EPI_GELU_BF16, EPI_RESID_F32  # noqa: F401


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return None if t is None else t.data_ptr()


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


def ternary_linear(x: torch.Tensor, packed: torch.Tensor, alpha: torch.Tensor, *, epilogue: int = EPI_BF16,
                   out: torch.Tensor | None = None, alpha_rows: int | None = None, token_tile: int = 0):
    """epilogue(alpha * x @ unpack(packed)^T): x bf16 (M, K), packed uint8 (N, K/4)."""
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
                                 token_tile, _stream()),
        "jb200_ternary_linear",
    )
    return out


def ternary_linear_grouped(x: torch.Tensor, packed: torch.Tensor, alpha: torch.Tensor, seg_offsets: torch.Tensor, *,
                           epilogue: int = EPI_BF16, out: torch.Tensor | None = None, token_tile: int = 0):
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
        out = torch.zeros((M, N), dtype=odt, device=x.device)
    _lib.check(
        lib.jb200_ternary_linear_grouped(_ptr(x), M, K, _ptr(packed), _ptr(alpha), N, G, _ptr(seg_offsets), epilogue,
                                         _ptr(out), token_tile, _stream()),
        "jb200_ternary_linear_grouped",
    )
    return out


def selftest_bounded_wait(limit_ms: int = 50) -> int:
    """Runs the wait-that-must-give-up kernel and returns the device status it left."""
    lib = _lib.load()
    _lib.device_status(clear=True)
    _lib.check(lib.jb200_selftest_bounded_wait(limit_ms, _stream()), "jb200_selftest_bounded_wait")
    return _lib.device_status(clear=True)
