"""The allocation-free dispatch-metadata entry point (jb200_moe_metadata_static) must give exactly
what jb200_moe_metadata gives.  It serves callers that cannot allocate device memory at call time
(a host process whose device memory is fully owned by its own arena, or a loop that must never hit
cudaMalloc's device-wide stall), so the test drives it through the raw C ABI with caller-owned
outputs only, twice in a row on different inputs: the second call reuses the built-in work array
with the first call's leftovers still in it.  Collected last on purpose (file name)."""
import ctypes as C

import pytest
import torch

import jarvis_b200  # noqa: F401
from jarvis_b200 import _lib, ops

pytestmark = pytest.mark.gpu


def _static_metadata(idx: torch.Tensor, E: int):
    lib = _lib.load()
    N, K = idx.shape
    dev = idx.device
    outs = [torch.full(shape, -7, dtype=torch.int32, device=dev)
            for shape in ((E,), (E + 1,), (N, K), (N * K,), (N * K,))]
    rc = lib.jb200_moe_metadata_static(idx.data_ptr(), N, K, E, *[t.data_ptr() for t in outs],
                                       torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "jb200_moe_metadata_static")
    return outs


def test_static_metadata_matches_regular_entry_point_twice():
    g = torch.Generator().manual_seed(123)
    # first call: many chunks, skewed towards experts 0/1; second call: fewer tokens, other experts
    cases = [(torch.randint(0, 4, (50000, 2), generator=g).clamp(max=1), 4),
             (torch.randint(0, 8, (3333, 2), generator=g), 8)]
    for idx, E in cases:
        idx = idx.cuda()
        got = _static_metadata(idx, E)
        want = ops.moe_metadata(idx, E)
        torch.cuda.synchronize()
        for a, b in zip(got, want):
            assert torch.equal(a, b)      # index work: bit-exact
    assert _lib.device_status() == 0


def test_static_metadata_rejects_oversized_input():
    lib = _lib.load()
    limit = lib.jb200_moe_metadata_static_max_assignments()
    assert limit == 262144
    N = limit // 2 + 1
    idx = torch.zeros((N, 2), dtype=torch.int64, device="cuda")
    dummy = torch.zeros((N * 2,), dtype=torch.int32, device="cuda")
    rc = lib.jb200_moe_metadata_static(idx.data_ptr(), N, 2, 4, dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                       dummy.data_ptr(), dummy.data_ptr(), None)
    assert rc == _lib.ERR_ARG
    assert "exceeds the built-in scratch limit" in _lib.last_error()
