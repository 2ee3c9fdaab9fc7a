"""GPU parity of the ternary weight path: absmean quantisation + 2-bit packing (bit-exact)
and the tcgen05 ternary GEMM (rel-L2 <= 1e-2 against fp32, the tolerance the path states for
bf16 compute)."""
import pytest
import torch

import jarvis_b200  # noqa: F401
from jarvis_b200 import _lib, ops
from oracle import jarvis_oracle as orc

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-2


def rel_l2(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def test_bounded_wait_reports_status():
    assert ops.selftest_bounded_wait(50) == 0x7F
    assert _lib.device_status() == 0


@pytest.mark.parametrize("shape", [(128, 64), (1024, 1024), (2048, 1024), (1024, 2048), (3, 20)])
def test_pack_matches_oracle_bit_exact(shape):
    g = torch.Generator().manual_seed(shape[0] * 7 + shape[1])
    w = torch.randn(shape, generator=g) * 0.02
    w[0, :4] = torch.tensor([0.0, 1e-9, -1.0, 1.0])
    alpha_ref, q_ref = orc.absmean_quantize(w)
    packed_ref = orc.pack_ternary(q_ref)
    # with the oracle's alpha: codes must be bit-exact
    packed, alpha = ops.pack_ternary(w.cuda(), alpha=torch.tensor([alpha_ref]).cuda())
    assert torch.equal(packed.cpu(), packed_ref)
    # with the kernel's own alpha: alpha within 1e-6 relative and at most a handful of boundary codes differ
    packed2, alpha2 = ops.pack_ternary(w.cuda())
    assert abs(float(alpha2) - alpha_ref) <= 1e-6 * alpha_ref
    q2 = ops.unpack_ternary(packed2, shape, torch.float32).cpu()
    assert (q2 != q_ref).sum().item() <= 2
    # unpack(pack(q)) == q
    assert torch.equal(ops.unpack_ternary(packed, shape, torch.float32).cpu(), q_ref)
    assert torch.equal(ops.unpack_ternary(packed, shape, torch.bfloat16).float().cpu(), q_ref)


def test_pack_codes_patterns():
    for pat in (torch.zeros(8, 16), torch.ones(8, 16), -torch.ones(8, 16),
                torch.tensor([-1.0, 0.0, 1.0, 0.0]).repeat(8, 4)):
        packed = ops.pack_codes(pat.cuda())
        assert torch.equal(packed.cpu(), orc.pack_ternary(pat))
        assert torch.equal(ops.unpack_ternary(packed, pat.shape, torch.float32).cpu(), pat)


def _gemm_case(M, K, N, seed, epilogue=ops.EPI_BF16, token_tile=0, prepared=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = torch.randn(N, K, generator=g) * 0.02
    alpha, q = orc.absmean_quantize(w)
    packed = orc.pack_ternary(q)
    ref = orc.ternary_linear(x.float(), q, alpha)
    if epilogue == ops.EPI_GELU_BF16:
        ref = torch.nn.functional.gelu(ref)
    pk = ops.prepare_weights(packed.cuda()) if prepared else packed.cuda()
    y = ops.ternary_linear(x.cuda(), pk, torch.tensor([alpha]).cuda(), epilogue=epilogue,
                           token_tile=token_tile, prepared=prepared)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    return rel_l2(y.float().cpu(), ref)


@pytest.mark.parametrize("M,K,N", [(256, 64, 128), (256, 1024, 1024), (100, 1024, 256), (1, 128, 128),
                                   (777, 2048, 1024), (1024, 1024, 3072), (33, 64, 128)])
def test_ternary_linear_matches_fp32(M, K, N):
    assert _gemm_case(M, K, N, seed=M + K + N) <= REL_L2_TOL
    assert _gemm_case(M, K, N, seed=M + K + N, prepared=True) <= REL_L2_TOL


@pytest.mark.parametrize("tile", [32, 64, 128, 256])
def test_ternary_linear_token_tiles(tile):
    assert _gemm_case(600, 512, 256, seed=tile, token_tile=tile) <= REL_L2_TOL


def test_ternary_linear_epilogues():
    assert _gemm_case(300, 1024, 2048, seed=5, epilogue=ops.EPI_GELU_BF16) <= REL_L2_TOL
    assert _gemm_case(301, 1024, 2048, seed=5, epilogue=ops.EPI_GELU_BF16, prepared=True) <= REL_L2_TOL
    assert _gemm_case(299, 512, 256, seed=8, epilogue=ops.EPI_BF16, prepared=True) <= REL_L2_TOL
    assert _gemm_case(300, 1024, 1024, seed=6, epilogue=ops.EPI_F32) <= 5e-3
    # residual epilogue: out += alpha * acc
    g = torch.Generator().manual_seed(7)
    x = torch.randn(300, 1024, generator=g).bfloat16()
    w = torch.randn(1024, 1024, generator=g) * 0.02
    resid = torch.randn(300, 1024, generator=g)
    alpha, q = orc.absmean_quantize(w)
    out = resid.clone().cuda()
    ops.ternary_linear(x.cuda(), orc.pack_ternary(q).cuda(), torch.tensor([alpha]).cuda(), epilogue=ops.EPI_RESID_F32,
                       out=out)
    ref = resid + orc.ternary_linear(x.float(), q, alpha)
    assert rel_l2(out.cpu(), ref) <= 5e-3


def test_ternary_linear_exact_on_integers():
    """Small-integer activations make every product and partial sum exact in fp32, so the
    tensor-core result must equal the integer GEMM exactly (checks tiling / swizzle / decode)."""
    g = torch.Generator().manual_seed(11)
    M, K, N = 300, 512, 384
    x = torch.randint(-4, 5, (M, K), generator=g).float()
    q = torch.randint(-1, 2, (N, K), generator=g).float()
    y = ops.ternary_linear(x.bfloat16().cuda(), orc.pack_ternary(q).cuda(), torch.ones(1).cuda(), epilogue=ops.EPI_F32)
    assert torch.equal(y.cpu(), x @ q.t())
    # prepared layout: same result bit for bit (values decode to +-2, alpha is halved: both exact)
    prep = ops.prepare_weights(orc.pack_ternary(q).cuda())
    y2 = ops.ternary_linear(x.bfloat16().cuda(), prep, torch.ones(1).cuda(), epilogue=ops.EPI_F32, prepared=True)
    assert torch.equal(y2.cpu(), x @ q.t())
    # bf16 outputs through the paired-store epilogue (integers up to 256 are exact in bf16 for |y| small)
    xs = torch.randint(-1, 2, (M, 64), generator=g).float()
    qs = torch.randint(-1, 2, (N, 64), generator=g).float()
    for prepared in (False, True):
        pk = orc.pack_ternary(qs).cuda()
        pk = ops.prepare_weights(pk) if prepared else pk
        yb = ops.ternary_linear(xs.bfloat16().cuda(), pk, torch.ones(1).cuda(), prepared=prepared)
        assert torch.equal(yb.float().cpu(), xs @ qs.t())


def test_prepare_weights_is_a_bit_permutation():
    g = torch.Generator().manual_seed(13)
    q = torch.randint(-1, 2, (64, 256), generator=g).float()
    packed = orc.pack_ternary(q)
    prep = ops.prepare_weights(packed.cuda()).cpu()
    assert prep.shape == packed.shape
    w = packed.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    pw = prep.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    for k in range(16):
        c = (w >> (2 * k)) & 3
        f = (pw >> ((k & 1) * 16 + (k >> 1) * 2)) & 3
        assert torch.equal(f, torch.where(c == 1, 1, torch.where(c == 2, 3, 0)))


def test_stacked_alphas():
    """q/k/v stacked along N keep one alpha each."""
    g = torch.Generator().manual_seed(12)
    M, K = 200, 256
    x = torch.randint(-3, 4, (M, K), generator=g).float()
    qs = [torch.randint(-1, 2, (128, K), generator=g).float() for _ in range(3)]
    alphas = torch.tensor([0.5, 2.0, -1.0])
    y = ops.ternary_linear(x.bfloat16().cuda(), orc.pack_ternary(torch.cat(qs)).cuda(), alphas.cuda(),
                           epilogue=ops.EPI_F32, alpha_rows=128)
    ref = torch.cat([a * (x @ q.t()) for a, q in zip(alphas, qs)], dim=1)
    assert torch.equal(y.cpu(), ref)


@pytest.mark.parametrize("counts", [[100, 0, 37, 263], [0, 0, 0, 512], [1, 1, 1, 1], [300, 300, 300, 300]])
def test_grouped_ternary_linear(counts):
    g = torch.Generator().manual_seed(sum(counts))
    K, N, G = 256, 256, len(counts)
    M = sum(counts)
    offs = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32)
    x = torch.randint(-3, 4, (M, K), generator=g).float()
    q = torch.randint(-1, 2, (G, N, K), generator=g).float()
    alphas = torch.tensor([1.0, 0.5, 2.0, 4.0])[:G]
    y = ops.ternary_linear_grouped(x.bfloat16().cuda(), orc.pack_ternary(q).cuda(), alphas.cuda(), offs.cuda(),
                                   epilogue=ops.EPI_F32)
    ref = torch.cat([alphas[e] * (x[offs[e]:offs[e + 1]] @ q[e].t()) for e in range(G)])
    assert torch.equal(y.cpu(), ref)
    yp = ops.ternary_linear_grouped(x.bfloat16().cuda(), ops.prepare_weights(orc.pack_ternary(q).cuda()), alphas.cuda(),
                                    offs.cuda(), epilogue=ops.EPI_BF16, prepared=True)
    assert torch.equal(yp.float().cpu(), ref.bfloat16().float())
    assert _lib.device_status() == 0


@pytest.mark.parametrize("M,K,N", [(1, 64, 128), (300, 256, 384), (2048, 1024, 1152)])
def test_dense_linear_exact_on_integers(M, K, N):
    """Dense bf16 weights through the same pipeline (weight tiles by TMA): exact on small integers, for both
    output types, and equal to an fp32 matmul of the same bf16 operands on random data."""
    g = torch.Generator().manual_seed(M + K + N)
    x = torch.randint(-4, 5, (M, K), generator=g).float()
    w = torch.randint(-3, 4, (N, K), generator=g).float()
    ref = x @ w.t()
    y = ops.dense_linear(x.bfloat16().cuda(), w.bfloat16().cuda(), out_dtype=torch.float32)
    assert torch.equal(y.cpu(), ref)
    yb = ops.dense_linear(x.bfloat16().cuda(), w.bfloat16().cuda())
    assert torch.equal(yb.float().cpu(), ref.bfloat16().float())
    xr = torch.randn(M, K, generator=g).bfloat16()
    wr = (torch.randn(N, K, generator=g) * 0.02).bfloat16()
    yr = ops.dense_linear(xr.cuda(), wr.cuda(), out_dtype=torch.float32)
    want = xr.float() @ wr.float().t()
    assert float((yr.cpu() - want).norm() / want.norm()) < 1e-5
    assert _lib.device_status() == 0


def test_dense_linear_lm_head_shape():
    """The lm_head of the 606M model: 1024 -> 50257 (padded to 50304 rows of zeros), a slice of token rows
    against fp32 on the CPU."""
    g = torch.Generator().manual_seed(3)
    V, Vp, K, M = 50257, 50304, 1024, 512
    w = torch.zeros(Vp, K)
    w[:V] = torch.randn(V, K, generator=g) * 0.02
    x = torch.randn(M, K, generator=g).bfloat16()
    y = ops.dense_linear(x.cuda(), w.bfloat16().cuda())
    want = x.float() @ w.bfloat16().float().t()
    assert float((y.float().cpu() - want).norm() / want.norm()) < 3e-3      # bf16 rounding of the stored logits
    assert float(y[:, V:].abs().max()) == 0.0
    with pytest.raises(RuntimeError, match="multiple of 128"):
        ops.dense_linear(x.cuda(), w[:V].bfloat16().cuda())


def test_argument_errors_are_reported():
    x = torch.zeros(4, 100, dtype=torch.bfloat16, device="cuda")
    packed = torch.zeros(128, 25, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError, match="multiple of 64"):
        ops.ternary_linear(x, packed, torch.ones(1, device="cuda"))
