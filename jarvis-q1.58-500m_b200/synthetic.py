"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configurations
(they stand in for trained checkpoints and tokenised corpora, which a fresh machine does not have).

Used by bench.py, kernel_bench.py and the parity tests, so that the measured and the tested inputs are
the same recipe.  Plain torch; nothing here is on the hot path.
"""
from __future__ import annotations

import torch

ZIPF_S = 1.2


def zipf_shares(num_experts: int = 4, s: float = ZIPF_S) -> torch.Tensor:
    """Target top-1 load of expert e: (e + 1)^-s, normalised (s = 1.2, E = 4: 52.8 / 23.0 / 14.1 / 10.0 %)."""
    w = torch.tensor([1.0 / (e + 1) ** s for e in range(num_experts)], dtype=torch.float64)
    return (w / w.sum()).float()


def zipf_router_inputs(n_tokens: int, d_model: int = 1024, num_experts: int = 4, s: float = ZIPF_S, seed: int = 0,
                       device="cpu", rounds: int = 300):
    """Inputs of the MoE-alone configuration: x ~ N(0, 1) bf16 (n_tokens, d_model) and a router weight
    (E, d_model) whose TOP-1 histogram on x follows Zipf(s).

    The reference router has no bias (nn.Linear(d_model, E, bias=False), jarvis_engine/jarvis_model.py:206),
    so the skew is injected without touching the module API: input channel 0 is the constant 1 and router
    column 0 holds one offset per expert, calibrated on these very inputs (damped updates by
    log target - log share, deterministic for a seed) until the top-1 shares meet the target to 1e-3.
    Returns (x bf16, w_router f32, shares f32 (E,) achieved on x)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(n_tokens, d_model, generator=g)
    x[:, 0] = 1.0
    x = x.to(torch.bfloat16)
    bound = 1.0 / d_model ** 0.5                     # nn.Linear's default init range
    w = (torch.rand(num_experts, d_model, generator=g) * 2 - 1) * bound
    w[:, 0] = 0.0
    target = zipf_shares(num_experts, s)
    xd = x.to(device)
    base = xd.float() @ w.to(device).t()            # logits without the offsets
    off = torch.log(target).to(device)
    shares = None
    for _ in range(rounds):
        top1 = (base + off).argmax(dim=-1)
        shares = torch.bincount(top1, minlength=num_experts).float() / n_tokens
        if float((shares.cpu() - target).abs().max()) < 1e-3:
            break
        off = off + 0.25 * (torch.log(target.to(device)) - torch.log(shares.clamp_min(1e-6)))
        off = off - off.max()
    w[:, 0] = off.cpu()
    top1 = (base + off).argmax(dim=-1)
    shares = (torch.bincount(top1, minlength=num_experts).float() / n_tokens).cpu()
    return x, w, shares


def gaussian_ternary_(module: torch.nn.Module, seed: int = 0, std: float = 0.02, gamma_range=(0.90, 0.999)):
    """The benchmark's weight recipe applied in place to a block or model built from modules.py (or the
    reference's own classes: only names are used): every ternary matrix ~ N(0, std^2) (absmean quantisation
    then gives ~31 % zeros), per-head decay sigmoid(gamma_raw) ~ U[gamma_range].  Other tensors keep the
    constructor's initialisation, which the caller seeds with torch.manual_seed."""
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in module.named_parameters():
            leaf = name.rsplit(".", 1)[0]
            if name.endswith("_proj.weight") or ".w1." in "." + leaf + "." or ".w2." in "." + leaf + ".":
                p.copy_((torch.randn(p.shape, generator=g) * std).to(p.device))
            elif name.endswith("gamma_raw"):
                lo, hi = gamma_range
                p.copy_(torch.logit(torch.rand(p.shape, generator=g) * (hi - lo) + lo).to(p.device))
    return module


def ragged_prior_lengths(n_seq: int, max_len: int = 4096, seed: int = 0) -> torch.Tensor:
    """Prior lengths ~ U[1, max_len] of the ragged-decode configuration."""
    g = torch.Generator().manual_seed(seed)
    return torch.randint(1, max_len + 1, (n_seq,), generator=g)
