"""The reference-side binding on a GPU: `jarvis_b200.install(model)` swaps the attention / MoE / LSF / norm modules of
a HOST model that this package did not build, and the host's own forward then runs on the sm_100a kernels.

Two hosts:
  * a stand-in written here that follows the reference's block protocol call for call
    (JarvisBlock.forward / Jarvis.forward, jarvis_engine/jarvis_model.py:416-441, 488-536): it only composes
    modules through their public forward signatures, which is exactly what install() must keep working;
  * the reference's own `Jarvis`, when its tree is at hand ($JARVIS_REFERENCE or a `reference` directory beside
    the repository), also through the two import shims named `associative_attention` / `sparse_model`.
Results are compared with the CPU oracle on the same weights (rel-L2 <= 1.5e-2 on logits: bf16 compute + bf16 head).
"""
import os
import sys

import pytest
import torch
import torch.nn as nn

import jarvis_b200
from jarvis_b200 import _lib, modules as jm, synthetic
from oracle import jarvis_oracle as orc

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


class _W(nn.Module):
    """A bias-free linear layer's parameter holder (the host's TernaryLinear / nn.Linear stand-in)."""

    def __init__(self, out_f, in_f):
        super().__init__()
        self.weight = nn.Parameter(torch.randn(out_f, in_f) * 0.05)


class _PlainAttn(nn.Module):
    """Parameter / buffer names and attributes of the reference's AssociativeLinearAttention
    (jarvis_engine/jarvis_model.py:92-113); no forward: install() must replace it before it is ever called."""

    def __init__(self, d, h):
        super().__init__()
        self.n_heads = h
        self.q_proj, self.k_proj, self.v_proj, self.out_proj = _W(d, d), _W(d, d), _W(d, d), _W(d, d)
        self.gamma_raw = nn.Parameter(torch.full((h,), 2.94))
        i = torch.arange(64, dtype=torch.float32)
        diff = i[:, None] - i[None, :]
        for name, t in (("_diff_clamp", diff.clamp(min=0)), ("_causal", (diff >= 0).float()), ("_i_idx", i),
                        ("_i_idx_p1", i + 1), ("_c_m1_m_i", 63 - i)):
            self.register_buffer(name, t)
        self.rotary = nn.Module()
        self.rotary.max_seq_len_cached = 512


class _PlainMoE(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.num_experts, self.top_k, self.noise_std, self.balance_alpha = 4, 2, 0.1, 0.01
        self.router = nn.Linear(d, 4, bias=False)
        self.w1 = nn.ModuleList([_W(2 * d, d) for _ in range(4)])
        self.w2 = nn.ModuleList([_W(d, 2 * d) for _ in range(4)])


class _PlainLSF(nn.Module):
    def __init__(self):
        super().__init__()
        self.alpha_min, self.alpha_max = 0.1, 0.99
        self.var_scale = nn.Parameter(torch.tensor(1.0))


class _PlainNorm(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.eps = 1e-6
        self.weight = nn.Parameter(torch.ones(d))


class _HostBlock(nn.Module):
    """The reference block's composition over whatever modules sit in its attributes: plain parameter holders
    until install() swaps them."""

    def __init__(self, d, h):
        super().__init__()
        self.norm1, self.attn, self.norm2 = _PlainNorm(d), _PlainAttn(d, h), _PlainNorm(d)
        self.moe, self.liquid, self.reflect = _PlainMoE(d), _PlainLSF(), jm.ReflectivePenalty()

    def forward(self, x, h_prev=None, start_pos=0):
        x = x + self.attn(self.norm1(x), start_pos=start_pos)
        moe_out, l_balance, act_mean, act_var = self.moe(self.norm2(x))
        h_out, h_last = self.liquid(moe_out, act_var, h_prev)
        x = x + h_out
        return x, h_last, l_balance, self.reflect(act_mean, act_var)


class _HostModel(nn.Module):
    def __init__(self, vocab, d_model, n_layers, n_heads):
        super().__init__()
        self.tok_emb = nn.Embedding(vocab, d_model)
        self.blocks = nn.ModuleList([_HostBlock(d_model, n_heads) for _ in range(n_layers)])
        self.final_norm = _PlainNorm(d_model)
        self.lm_head = nn.Linear(d_model, vocab, bias=False)

    def forward(self, idx):
        x = self.tok_emb(idx)
        for blk in self.blocks:
            x, _, _, _ = blk(x)
        x = orc.rmsnorm(x, self.final_norm.weight)           # the host's own final norm and head stay its own
        return self.lm_head(x)


def test_install_on_a_foreign_host_model_runs_its_forward_on_the_kernels():
    torch.manual_seed(21)
    host = synthetic.gaussian_ternary_(_HostModel(512, 256, 2, 4), seed=21).eval()
    sd = {k: v.clone() for k, v in host.state_dict().items()}
    idx = torch.randint(0, 512, (2, 200), generator=torch.Generator().manual_seed(22))
    ref, _ = orc.model_forward(idx, sd, 2, 4)
    host = host.cuda()
    params_before = dict(host.named_parameters())
    keys_before = list(host.state_dict().keys())
    jarvis_b200.install(host)
    assert list(host.state_dict().keys()) == keys_before
    for name, prm in host.named_parameters():
        assert prm is params_before[name], name                      # shared, not copied
    _lib.kernel_launches(reset=True)
    with torch.no_grad():
        logits = host(idx.cuda())
    torch.cuda.synchronize()
    assert _lib.kernel_launches() > 0 and _lib.device_status() == 0
    assert rel_l2(logits, ref) <= 1.5e-2
    # a later in-place change of the host's weights reaches the installed modules (the packed copy is rebuilt)
    with torch.no_grad():
        host.blocks[0].attn.q_proj.weight.mul_(-1.0)
        sd["blocks.0.attn.q_proj.weight"] = -sd["blocks.0.attn.q_proj.weight"]
        logits2 = host(idx.cuda())
    ref2, _ = orc.model_forward(idx, sd, 2, 4)
    assert rel_l2(logits2, ref2) <= 1.5e-2 and rel_l2(logits2, ref) > 3 * rel_l2(logits2, ref2)


_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_REF_ROOT = os.environ.get("JARVIS_REFERENCE") or os.path.join(os.path.dirname(_REPO), "reference")
_REF = os.path.join(_REF_ROOT, "jarvis_engine")


@pytest.mark.skipif(not os.path.isdir(_REF), reason="reference tree not at hand")
def test_reference_jarvis_forward_over_installed_modules_and_import_shims(tmp_path):
    sys.dont_write_bytecode = True
    # (b) of the integration notes: two shims with the names the reference imports, ahead of its own directories
    (tmp_path / "associative_attention.py").write_text("from jarvis_b200.modules import CUDAAssociativeLinearAttention\n")
    (tmp_path / "sparse_model.py").write_text("from jarvis_b200.modules import CUDASparseMoELayer\n")
    sys.path.insert(0, _REF)
    sys.path.insert(0, str(tmp_path))
    try:
        for name in ("jarvis_model", "associative_attention", "sparse_model"):
            sys.modules.pop(name, None)
        import jarvis_model as ref
    finally:
        sys.path.remove(str(tmp_path))
        sys.path.remove(_REF)
    torch.manual_seed(31)
    kw = dict(vocab_size=512, d_model=256, n_layers=2, n_heads=4, max_seq_len=256)
    idx = torch.randint(0, 512, (2, 128), generator=torch.Generator().manual_seed(32))
    # (a) install() on the reference's own pure-PyTorch model
    model = synthetic.gaussian_ternary_(ref.Jarvis(use_cuda_attn=False, use_cuda_moe=False, **kw), seed=31).eval()
    with torch.no_grad():
        want, _ = model(idx)
    model = model.cuda()
    jarvis_b200.install(model)
    with torch.no_grad():
        got, _ = model(idx.cuda())
    assert rel_l2(got, want) <= 1.5e-2
    # (b) the reference constructs the shimmed classes itself
    shimmed = ref.Jarvis(use_cuda_attn=True, use_cuda_moe=True, **kw)
    assert isinstance(shimmed.blocks[0].attn, jm.AssociativeLinearAttention)
    assert isinstance(shimmed.blocks[0].moe, jm.SparseMoELayer)
    assert shimmed.get_backend_status()["attn_backend"] == "cuda"
