"""CPU-only checks: the C-ABI library loads and exports every declared symbol, argument errors are
reported without a GPU, host-side bit manipulation matches the oracle, modules keep the reference's
state-dict contract, and install() leaves keys untouched."""
import ctypes as C
import os
import struct
import sys

import pytest
import torch

import jarvis_b200
from jarvis_b200 import _lib, modules as jm
from oracle import jarvis_oracle as orc


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    declared = _lib.declared_symbols()
    assert len(declared) >= 25
    assert set(declared) == set(_lib.PROTOTYPES)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.jb200_abi_version() >= 7
    assert lib.jb200_moe_metadata_static_max_assignments() == 262144


def test_argument_errors_need_no_gpu():
    lib = _lib.load()
    rc = lib.jb200_ternary_linear(None, 16, 100, None, None, 128, 128, 0, None, 0, 0, None)
    assert rc == _lib.ERR_ARG and "multiple of 64" in _lib.last_error()
    rc = lib.jb200_pack_ternary(None, 4, 6, None, None, None, None, None)
    assert rc == _lib.ERR_ARG and "divisible by 4" in _lib.last_error()
    rc = lib.jb200_attn_scan(None, None, None, 64, None, None, None, 1, None, 0, None, None, 64, None, None, 1, 1, 1,
                             32, 0, None)
    assert rc == _lib.ERR_ARG and "head_dim" in _lib.last_error()
    rc = lib.jb200_lsf_scan(None, 0, None, None, None, None, 0.1, 0.99, None, None, None, 0, None, None, 1, 1, 3, None)
    assert rc == _lib.ERR_ARG and "even" in _lib.last_error()
    rc = lib.jb200_moe_metadata_static(None, 1 << 20, 2, 4, None, None, None, None, None, None)
    assert rc == _lib.ERR_ARG and "built-in scratch limit" in _lib.last_error()
    assert lib.jb200_pack_ternary_scratch_bytes(1024, 1024) > 0
    assert lib.jb200_moe_metadata_scratch_bytes(16384, 2, 4) == 2 * 128 * 4 * 4


def _bf16(h):
    return struct.unpack("<f", struct.pack("<I", h << 16))[0]


def test_host_decode_matches_oracle_unpack():
    lib = _lib.load()
    g = torch.Generator().manual_seed(0)
    q = torch.randint(-1, 2, (8, 64), generator=g).float()
    words = orc.pack_ternary(q).view(torch.int32).reshape(-1).tolist()
    flat = q.reshape(-1).tolist()
    for wi, w in enumerate(words):
        out = (C.c_uint32 * 8)()
        lib.jb200_host_decode16(w & 0xFFFFFFFF, out)
        outp = (C.c_uint32 * 8)()
        lib.jb200_host_decode16_prepared(w & 0xFFFFFFFF, outp)
        for j in range(16):
            want = flat[wi * 16 + j]
            assert _bf16((out[j // 2] >> (16 * (j % 2))) & 0xFFFF) == want
            assert _bf16((outp[j // 2] >> (16 * (j % 2))) & 0xFFFF) == 2.0 * want


def test_state_dict_contract():
    blk = jm.JarvisBlock(128, 2, 4, 2)
    assert len(blk.state_dict()) == 23
    model = jm.Jarvis(vocab_size=64, d_model=128, n_layers=3, n_heads=2, max_seq_len=64)
    assert len(model.state_dict()) == 3 * 23 + 3
    # the full-size model would have 24 * 23 + 3 = 555 keys
    st = model.get_backend_status()
    assert set(st) == {"has_cuda_attn_extension", "has_cuda_moe_extension", "attn_backend", "moe_backend",
                       "attn_cuda_blocks", "moe_cuda_blocks"}
    assert model.param_count()[0] == sum(p.numel() for p in model.parameters())


def test_no_cpu_fallback():
    with pytest.raises(RuntimeError):
        jm.TernaryLinear(64, 128)(torch.randn(2, 64))
    with pytest.raises(RuntimeError):
        jm.LiquidStateFusion(8)(torch.randn(1, 4, 8), torch.tensor(0.5))


# the reference checkout, when one is at hand: $JARVIS_REFERENCE, else a `reference` directory beside this repo
_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(os.environ.get("JARVIS_REFERENCE") or os.path.join(os.path.dirname(_REPO), "reference"), "jarvis_engine")


@pytest.mark.skipif(not os.path.isdir(REF), reason="reference tree not mounted")
def test_install_keeps_reference_state_dict_keys():
    sys.dont_write_bytecode = True
    sys.path.insert(0, REF)
    try:
        import jarvis_model as ref
    finally:
        sys.path.remove(REF)
    model = ref.Jarvis(vocab_size=64, d_model=128, n_layers=2, n_heads=2, max_seq_len=64, use_cuda_attn=False,
                       use_cuda_moe=False).eval()
    keys = list(model.state_dict().keys())
    weights = {k: v.clone() for k, v in model.state_dict().items()}
    params_before = dict(model.named_parameters())
    jarvis_b200.install(model)
    assert list(model.state_dict().keys()) == keys
    for k, v in model.state_dict().items():
        assert torch.equal(v, weights[k]), k
    # shared, not copied: the installed modules hold the very Parameter objects the model had
    for k, p in model.named_parameters():
        assert p is params_before[k], k
    assert isinstance(model.blocks[0].attn, jm.AssociativeLinearAttention)
    assert isinstance(model.blocks[1].moe, jm.SparseMoELayer)


def test_read_tbin_container_written_by_the_reference():
    """tests/golden/tiny.jarvis-tbin was produced by the reference's export_to_jarvis_tbin; the reader must
    recover exactly what the reference's own loader reconstructs (effective weights alpha * q, dense tensors
    through bf16)."""
    from jarvis_b200 import checkpoint as ck
    from tests.golden.loader import load
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tiny.jarvis-tbin")
    packed, meta = ck.read_tbin(path)
    g = load("tbin")
    assert meta["format"] == "jarvis-tbin" and meta["extra"] == {"note": "golden"}
    assert len(meta["tensors"]) == 26 and sum(e["is_ternary"] for e in meta["tensors"]) == 12
    for name in ("blocks.0.attn.q_proj.weight", "blocks.0.moe.w2.3.weight"):
        p, a = packed[name + ".packed_weight"], packed[name + ".alpha"]
        w_eff = orc.unpack_ternary(p, g["sd_" + name].shape) * a
        assert torch.equal(w_eff, g["sd_" + name]), name
    for name in ("tok_emb.weight", "blocks.0.moe.router.weight", "blocks.0.attn.gamma_raw"):
        assert torch.equal(packed[name].float(), g["sd_" + name]), name
    with pytest.raises(ValueError, match="magic"):
        bad = path + ".bad"
        try:
            with open(bad, "wb") as fh:
                fh.write(b"NOTATBIN" + b"\0" * 64)
            ck.read_tbin(bad)
        finally:
            os.remove(bad)


def test_cached_parameter_views_follow_in_place_updates_and_new_storage():
    """modules._f32 keeps `p.detach().float()` on the parameter until the parameter changes."""
    import torch
    from jarvis_b200 import modules as jm
    p = torch.nn.Parameter(torch.arange(6, dtype=torch.float32).reshape(2, 3))
    a = jm._f32(p)
    assert a is jm._f32(p) and a.data_ptr() == p.data_ptr() and not a.requires_grad
    with torch.no_grad():
        p.mul_(2.0)
    b = jm._f32(p)
    assert torch.equal(b, p.detach())
    p.data = torch.ones(2, 3)
    c = jm._f32(p)
    assert c is not b and torch.equal(c, torch.ones(2, 3))
    h = torch.nn.Parameter(torch.tensor([1.5, 2.5], dtype=torch.bfloat16))       # a host model kept in bf16
    f = jm._f32(h)
    assert f.dtype == torch.float32 and torch.equal(f, torch.tensor([1.5, 2.5]))
    with torch.no_grad():
        h.add_(1.0)
    assert torch.equal(jm._f32(h), torch.tensor([2.5, 3.5]))
    s = torch.nn.Parameter(torch.tensor(0.75))
    assert tuple(jm._f32(s, scalar=True).shape) == (1,)

