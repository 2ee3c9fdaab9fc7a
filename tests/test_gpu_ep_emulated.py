"""The peer-memory expert exchange for every world size, on ONE GPU: the gather and combine kernels take tables of
pointers to the other ranks' buffers, so W ranks are emulated as W sets of buffers in one process and every rank's
kernels are launched in turn (the phases are separated by barriers in the real thing, here by stream order).
world <= E (several experts per rank) and world > E (every expert served by world / E ranks, each taking one slice
of every source's rows) must both reproduce the single-GPU layer bit for bit: same rows in the same order through
the same GEMMs (dispatch order of sparse_model_cuda/sparse_model.cu:23-90)."""
import ctypes as C

import pytest
import torch

import jarvis_b200  # noqa: F401
from jarvis_b200 import _lib, modules as jm, ops, synthetic

pytestmark = pytest.mark.gpu


def _ptrs(tensors):
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device="cuda")


@pytest.mark.parametrize("world", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("skew", [False, True])
def test_emulated_ranks_reproduce_the_single_gpu_layer(world, skew):
    lib = _lib.load()
    E, K, Cm, N = 4, 2, 256, 4096
    torch.manual_seed(world)
    moe = synthetic.gaussian_ternary_(jm.SparseMoELayer(Cm), seed=world).cuda().eval()
    if skew:
        x, w_r, _ = synthetic.zipf_router_inputs(N, Cm, E, seed=world)
        with torch.no_grad():
            moe.router.weight.copy_(w_r.cuda())
        x = x.cuda()
    else:
        x = torch.randn(N, Cm, generator=torch.Generator().manual_seed(7)).bfloat16().cuda()
    want, _ = moe.run_rows(x)
    (p1, a1), (p2, a2) = moe.packed()
    w_route = moe.router.weight.detach().float().contiguous()

    n = N // world
    shards, per = max(1, world // E), max(1, E // world)
    max_rows = (n * K + shards - 1) // shards * world
    i32 = dict(dtype=torch.int32, device="cuda")
    xn = [x[r * n:(r + 1) * n].contiguous() for r in range(world)]
    routed = []
    gmap, offs, y, meta, disp, seg = [], [], [], [], [], []
    for r in range(world):
        idx, gates, _ = ops.router_top2(xn[r], w_route)
        counts, offsets, scatter, gather, _ = ops.moe_metadata(idx, E)
        routed.append((idx, gates, offsets, scatter))
        gmap.append(gather)
        offs.append(torch.cat([offsets, torch.tensor([n], **i32)]))
        y.append(torch.zeros(max_rows, Cm, dtype=torch.bfloat16, device="cuda"))
        meta.append(torch.zeros(per * (world + 1) + per + 1, **i32))
        disp.append(torch.zeros(max_rows, Cm, dtype=torch.bfloat16, device="cuda"))
        seg.append(torch.zeros(per + 1, **i32))
    t_offs, t_gmap, t_xn, t_y, t_meta = _ptrs(offs), _ptrs(gmap), _ptrs(xn), _ptrs(y), _ptrs(meta)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    total_rows = 0
    for r in range(world):       # phase 1: every owner pulls its rows and runs its experts
        _lib.check(lib.jb200_ep_pull_gather(t_offs.data_ptr(), t_gmap.data_ptr(), t_xn.data_ptr(), world, r, E, Cm, K, n,
                                            max_rows, disp[r].data_ptr(), seg[r].data_ptr(), meta[r].data_ptr(), stream),
                   "jb200_ep_pull_gather")
        owned = [r // shards] if shards > 1 else list(range(r * per, (r + 1) * per))
        sel = torch.tensor(owned, device="cuda")
        hid = ops.ternary_linear_grouped(disp[r], p1[sel].contiguous(), a1[sel].contiguous(), seg[r],
                                         epilogue=ops.EPI_GELU_BF16, prepared=True)
        ops.ternary_linear_grouped(hid, p2[sel].contiguous(), a2[sel].contiguous(), seg[r], epilogue=ops.EPI_BF16,
                                   out=y[r], prepared=True)
        total_rows += int(seg[r][-1])
    assert total_rows == N * K                       # every (token, slot) has exactly one owner
    outs = []
    stats = torch.zeros(2, dtype=torch.float64, device="cuda")
    for r in range(world):       # phase 2: every home rank pulls its tokens' expert outputs back
        idx, gates, offsets, scatter = routed[r]
        out = torch.empty(n, Cm, dtype=torch.bfloat16, device="cuda")
        _lib.check(lib.jb200_ep_pull_combine(t_y.data_ptr(), t_meta.data_ptr(), offsets.data_ptr(), idx.data_ptr(),
                                             gates.data_ptr(), scatter.data_ptr(), world, r, E, Cm, K, n, max_rows,
                                             out.data_ptr(), 1, stats.data_ptr(), stream), "jb200_ep_pull_combine")
        outs.append(out)
    got = torch.cat(outs)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert torch.equal(got, want)
    assert abs(float(stats[0]) - float(want.float().sum())) <= 1e-3 * float(want.float().abs().sum())


def test_world_sizes_that_do_not_fit_are_refused():
    lib = _lib.load()
    z = torch.zeros(8, dtype=torch.int64, device="cuda")
    buf = torch.zeros(1024, dtype=torch.int32, device="cuda")
    rc = lib.jb200_ep_pull_gather(z.data_ptr(), z.data_ptr(), z.data_ptr(), 3, 0, 4, 256, 2, 16, 64, buf.data_ptr(),
                                  buf.data_ptr(), buf.data_ptr(), C.c_void_p(0))
    assert rc == _lib.ERR_ARG and "unsupported shape" in _lib.last_error()
    rc = lib.jb200_ep_pull_gather(z.data_ptr(), z.data_ptr(), z.data_ptr(), 6, 0, 4, 256, 2, 16, 64, buf.data_ptr(),
                                  buf.data_ptr(), buf.data_ptr(), C.c_void_p(0))
    assert rc == _lib.ERR_ARG
