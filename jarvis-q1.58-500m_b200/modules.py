"""Drop-in modules: the reference's PyTorch module API over the sm_100a kernels.

Constructors, parameter / buffer names (so state dicts interchange: 23 tensors per block, 555 for
the 24-layer model), forward signatures and return tuples follow jarvis_engine/jarvis_model.py and
the CUDA drop-ins in associative_attention_cuda/associative_attention.py and
sparse_model_cuda/sparse_model.py.  Inference only (no autograd through the kernels), CUDA only:
a CPU tensor or a missing library raises, nothing falls back.

Numerics: the residual stream is carried in fp32, GEMM inputs and scan inputs are bf16, every
accumulation is fp32 -- the reference's autocast regime, checked against its fp32 CPU results.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops

# ----------------------------------------------------------------------------------------------
# small pieces
# ----------------------------------------------------------------------------------------------


def _f32(p: torch.Tensor, scalar: bool = False) -> torch.Tensor:
    """`p.detach().float().contiguous()` (reshaped to (1,) for scalars), cached on the parameter until it changes
    (in-place update or new storage): the views cost a few microseconds each, several times per layer."""
    key = (p.data_ptr(), p._version, scalar)
    c = getattr(p, "_jb_f32", None)
    if c is None or c[0] != key:
        t = p.detach().float().contiguous()
        c = (key, t.reshape(1) if scalar else t)
        p._jb_f32 = c
    return c[1]


class RMSNorm(nn.Module):
    """jarvis_engine/jarvis_model.py:19-26."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        return ops.rmsnorm(x.contiguous(), self.weight.detach().float(), self.eps, out_dtype=x.dtype)


class _PackCache:
    """Packed form of one or more fp32 weight matrices, rebuilt when any of them changes.  `packed` is
    kept in the GEMM's prepared layout (ops.prepare_weights of the canonical weight_packing.py bytes);
    `canonical` keeps the interchange layout."""

    def __init__(self):
        self.key = None
        self.packed = None
        self.canonical = None
        self.alpha = None

    def get(self, weights, stack: bool):
        key = tuple((w.data_ptr(), w._version, w.device) for w in weights)
        if key != self.key:
            pa = [ops.pack_ternary(w.detach().float().contiguous()) for w in weights]
            self.canonical = torch.stack([p for p, _ in pa]) if stack else torch.cat([p for p, _ in pa])
            self.packed = ops.prepare_weights(self.canonical)
            self.alpha = torch.cat([a for _, a in pa])
            self.key = key
        return self.packed, self.alpha


class TernaryLinear(nn.Module):
    """jarvis_engine/utils/ternary_ops.py:42-53.  The fp32 master weight is quantised and packed
    to 2 bits once (and again whenever it is modified), not on every forward."""

    def __init__(self, in_features, out_features, bias=False):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        self._cache = _PackCache()

    def packed(self):
        return self._cache.get([self.weight], stack=False)

    def forward(self, x):
        packed, alpha = self.packed()
        x2 = x.reshape(-1, x.shape[-1]).to(torch.bfloat16).contiguous()
        if x.dtype == torch.float32:
            y = ops.ternary_linear(x2, packed, alpha, epilogue=ops.EPI_F32, prepared=True)
        else:
            y = ops.ternary_linear(x2, packed, alpha, epilogue=ops.EPI_BF16, prepared=True).to(x.dtype)
        y = y.view(*x.shape[:-1], -1)
        return y if self.bias is None else y + self.bias


class RotaryEmbedding(nn.Module):
    """Same caches as jarvis_engine/jarvis_model.py:35-57 (fp32 cos/sin of shape (n, dim), grown by
    doubling); the kernels read the first half of the last axis (the two halves are equal)."""

    def __init__(self, dim: int, max_seq_len: int = 2048, base: float = 10000.0):
        super().__init__()
        self.dim = dim
        self.base = base
        inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2).float() / dim))
        self.register_buffer("inv_freq", inv_freq, persistent=False)
        self.max_seq_len_cached = 0
        self._half = None
        self._build_cache(max_seq_len, device=inv_freq.device)

    def _build_cache(self, seq_len: int, device):
        self.max_seq_len_cached = max(seq_len, 256)
        t = torch.arange(self.max_seq_len_cached, dtype=torch.float32, device=device)
        freqs = torch.outer(t, self.inv_freq.to(device))
        emb = torch.cat((freqs, freqs), dim=-1)
        self.register_buffer("cos_cached", emb.cos(), persistent=False)
        self.register_buffer("sin_cached", emb.sin(), persistent=False)
        self._half = None

    def half_tables(self, end_pos: int, device):
        if end_pos > self.max_seq_len_cached or self.cos_cached.device != device:
            self._build_cache(max(end_pos, self.max_seq_len_cached * 2), device=device)
        if self._half is None:
            h = self.dim // 2
            self._half = (self.cos_cached[:, :h].contiguous(), self.sin_cached[:, :h].contiguous())
        return self._half


def _as_rows_bf16(x):
    return x.reshape(-1, x.shape[-1]).to(torch.bfloat16).contiguous()


# ----------------------------------------------------------------------------------------------
# attention
# ----------------------------------------------------------------------------------------------
class AssociativeLinearAttention(nn.Module):
    """jarvis_engine/jarvis_model.py:89-191; `h_prev` as in CUDAAssociativeLinearAttention.forward
    (associative_attention_cuda/associative_attention.py:212).  `forward_with_state` additionally
    returns the final state (B, H, D, D) for decode hand-off, which the reference computes and drops."""

    CHUNK_SIZE = 64

    def __init__(self, d_model, n_heads, max_seq_len=2048):
        super().__init__()
        self.n_heads = n_heads
        self.head_dim = d_model // n_heads
        if self.head_dim != 64:
            raise ValueError("the sm_100a attention scan is built for head_dim == 64")
        self.q_proj = TernaryLinear(d_model, d_model)
        self.k_proj = TernaryLinear(d_model, d_model)
        self.v_proj = TernaryLinear(d_model, d_model)
        self.out_proj = TernaryLinear(d_model, d_model)
        self.gamma_raw = nn.Parameter(torch.full((n_heads,), 2.94))
        self.rotary = RotaryEmbedding(self.head_dim, max_seq_len=max_seq_len)
        cs = self.CHUNK_SIZE
        i = torch.arange(cs, dtype=torch.float32)
        diff = i.unsqueeze(1) - i.unsqueeze(0)
        # state-dict compatibility: the kernel derives its decay tables itself
        self.register_buffer("_diff_clamp", diff.clamp(min=0))
        self.register_buffer("_causal", (diff >= 0).float())
        self.register_buffer("_i_idx", i)
        self.register_buffer("_i_idx_p1", i + 1)
        self.register_buffer("_c_m1_m_i", (cs - 1) - i)
        self._qkv = _PackCache()
        self._qkv_rope = None      # (key, prepared packed q|k|v with the q/k head rows interleaved) for the fused prologue
        # T > 1: run the feature map + RoPE in the q/k/v GEMM's epilogue instead of the scan.  Off by default: at
        # B=8 x T=2048 the scan gets 32 us faster but the GEMM 43 us slower (its 8 epilogue warps have fewer
        # issue slots for that arithmetic than the scan's 16 warps per SM); the fused form rounds q', k' once
        # instead of twice, so it is the more accurate of the two.
        self.fuse_prologue = False
        self._gamma = None
        self.max_position = None   # optional upper bound of per-sequence start positions (avoids a sync)

    def qkv_packed(self):
        return self._qkv.get([self.q_proj.weight, self.k_proj.weight, self.v_proj.weight], stack=False)

    def qkv_packed_interleaved(self):
        """q|k|v in the prepared layout with the rows of every q and k head interleaved (feature i next to
        feature i + 32), the order ops.qkv_linear_rope works on."""
        self.qkv_packed()
        if self._qkv_rope is None or self._qkv_rope[0] is not self._qkv.canonical:
            canon, C = self._qkv.canonical, self.q_proj.weight.shape[0]
            rows = torch.cat([ops.interleave_head_rows(canon[:C], self.n_heads),
                              ops.interleave_head_rows(canon[C:2 * C], self.n_heads), canon[2 * C:]])
            self._qkv_rope = (canon, ops.prepare_weights(rows))
        return self._qkv_rope[1], self._qkv.alpha

    def scan_rows(self, xn_rows, B, T, start_pos=0, h_prev=None, want_state=False, inplace_state=False, cp=None):
        """xn_rows: bf16 (B*T, C) normalised input -> (o bf16 (B*T, C), state or None).
        cp: a parallel.ContextParallel when this rank holds one T-token slice of longer sequences
        (start_pos is then the position of the SEQUENCE's first token; the returned state is the one after
        the whole sequence)."""
        C = xn_rows.shape[1]
        if cp is not None:
            start_pos = start_pos + cp.rank * T
        fused = self.fuse_prologue and T > 1
        if not fused:
            packed, alpha = self.qkv_packed()
            qkv = ops.ternary_linear(xn_rows, packed, alpha, alpha_rows=C, prepared=True)
        if torch.is_tensor(start_pos):
            # per-sequence positions: size the table from the caller's bound when given (no host sync)
            end = (self.max_position if self.max_position is not None else int(start_pos.max())) + T
        else:
            end = int(start_pos) + T
        cos, sin = self.rotary.half_tables(end, xn_rows.device)
        if fused:
            packed, alpha = self.qkv_packed_interleaved()
            qkv = ops.qkv_linear_rope(xn_rows, packed, alpha, cos, sin, T, 2 * C, start_pos=start_pos, alpha_rows=C,
                                      prepared=True)
        gkey = (self.gamma_raw.data_ptr(), self.gamma_raw._version)
        if self._gamma is None or self._gamma[0] != gkey:
            self._gamma = (gkey, torch.sigmoid(self.gamma_raw.detach().float()))
        gamma = self._gamma[1]
        if h_prev is not None:
            h_prev = h_prev.to(torch.float32).contiguous()
        if cp is not None:
            def scan(state_in):
                return ops.attn_scan(qkv[:, :C], qkv[:, C:2 * C], qkv[:, 2 * C:], gamma, cos, sin, B, T, self.n_heads,
                                     start_pos=start_pos, state_in=state_in, want_state=True, qk_prepared=fused)
            def state_only():
                return ops.attn_scan(qkv[:, :C], qkv[:, C:2 * C], qkv[:, 2 * C:], gamma, cos, sin, B, T, self.n_heads,
                                     start_pos=start_pos, qk_prepared=fused, want_out=False)[1]
            return cp.attention(scan, gamma, T, h_prev, state_only=state_only if T > 1 else None)
        return ops.attn_scan(qkv[:, :C], qkv[:, C:2 * C], qkv[:, 2 * C:], gamma, cos, sin, B, T, self.n_heads,
                             start_pos=start_pos, state_in=h_prev, want_state=want_state,
                             state_out=h_prev if (inplace_state and h_prev is not None) else None, qk_prepared=fused)

    def forward_with_state(self, x, start_pos=0, h_prev=None):
        B, T, C = x.shape
        o, state = self.scan_rows(_as_rows_bf16(x), B, T, start_pos, h_prev, want_state=True)
        return self.out_proj(o).view(B, T, C).to(x.dtype), state

    def forward(self, x, start_pos: int = 0, h_prev=None):
        B, T, C = x.shape
        o, _ = self.scan_rows(_as_rows_bf16(x), B, T, start_pos, h_prev)
        packed, alpha = self.out_proj.packed()
        if x.dtype == torch.float32:
            return ops.ternary_linear(o, packed, alpha, epilogue=ops.EPI_F32, prepared=True).view(B, T, C)
        return ops.ternary_linear(o, packed, alpha, prepared=True).view(B, T, C).to(x.dtype)


CUDAAssociativeLinearAttention = AssociativeLinearAttention


# ----------------------------------------------------------------------------------------------
# MoE
# ----------------------------------------------------------------------------------------------
class SparseMoELayer(nn.Module):
    """jarvis_engine/jarvis_model.py:198-251 / sparse_model_cuda/sparse_model.py:87-178 (eval mode:
    no routing noise).  Router -> dispatch metadata -> gather -> grouped ternary GEMMs -> combine,
    all on the device: expert offsets never visit the host."""

    def __init__(self, d_model, num_experts=4, top_k=2, hidden_mult=2, noise_std=0.1, balance_alpha=0.01):
        super().__init__()
        if top_k != 2:
            raise ValueError("the router kernel implements top-2")
        self.num_experts = num_experts
        self.top_k = top_k
        self.noise_std = noise_std
        self.balance_alpha = balance_alpha
        self.router = nn.Linear(d_model, num_experts, bias=False)
        hidden = d_model * hidden_mult
        self.w1 = nn.ModuleList([TernaryLinear(d_model, hidden) for _ in range(num_experts)])
        self.w2 = nn.ModuleList([TernaryLinear(hidden, d_model) for _ in range(num_experts)])
        self._p1 = _PackCache()
        self._p2 = _PackCache()
        # When one batch is split over data-parallel ranks, the batch-global quantities of the layer
        # (act_mean / act_var, which set the LSF decay, and the f / P of the balance loss) need the
        # other ranks' partial sums: set to a torch.distributed group to all-reduce them (6 doubles and
        # 4 ints per layer).  None: the ranks' batches are independent calls.
        self.stats_group = None
        self._n_total_hint = None   # global token count when known (avoids a host read per layer)
        self._ep = None             # parallel.PeerExpertParallelMoE: experts spread over the ranks of a group
        self.last_routing = None  # (topk_idx, gates, metadata) of the most recent call, for inspection

    def packed(self):
        return (self._p1.get([m.weight for m in self.w1], stack=True),
                self._p2.get([m.weight for m in self.w2], stack=True))

    def run_rows(self, xn_rows, out_dtype=torch.bfloat16, acc=None, hist=None, scalars=None, norm=None,
                 finalize=True):
        """xn_rows: bf16 (N, C) -> (out (N, C), scalars f32 [l_balance, act_mean, act_var]).
        acc (f64 (2+E,)), hist (i32 (E,)) and scalars (f32 (3,)) may be passed in pre-zeroed (a model
        zeroes one block of them per forward instead of three small fills per layer).
        finalize=False (acc and hist passed in): the scalars are left to the caller's fused tail kernel and the
        second return value is the token count they are to be derived with."""
        if self.training:
            raise RuntimeError("SparseMoELayer (sm_100a): inference only; call .eval() first")
        N, C = xn_rows.shape
        E = self.num_experts
        dev = xn_rows.device
        if acc is None:
            acc = torch.zeros(2 + E, dtype=torch.float64, device=dev)   # [sum, sum^2, P_0..P_{E-1}]
        if hist is None:
            hist = torch.zeros(E, dtype=torch.int32, device=dev)
        # norm=(weight, eps): `xn_rows` is the un-normalised f32 residual stream and RMSNorm is fused into
        # the router kernel (one pass over the row, routing bit-identical to the separate kernels)
        w_r = _f32(self.router.weight)
        ep = self._ep
        in_slab = False
        if norm is not None and C <= 1024:
            # expert parallel: the normalised rows go straight into the buffer the other ranks read
            in_slab = ep is not None and N <= ep.ex.n_max
            xn_rows, idx, gates = ops.rmsnorm_router(xn_rows, norm[0], norm[1], w_r, probs_sum=acc[2:], top1_hist=hist,
                                                     xn_out=ep.ex.xn[:N] if in_slab else None)
        else:
            if norm is not None:
                xn_rows = ops.rmsnorm(xn_rows, norm[0], norm[1])
            idx, gates, _ = ops.router_top2(xn_rows, w_r, probs_sum=acc[2:], top1_hist=hist)
        # expert parallel: the gather map and the expert offsets are written where the other ranks read them
        meta_in_slab = ep is not None and N <= ep.ex.n_max
        if meta_in_slab:
            meta = ops.moe_metadata(idx, E, gather_out=ep.ex.gmap[:N * self.top_k], offsets_out=ep.ex.offs[:E + 1])
        else:
            meta = ops.moe_metadata(idx, E)
        counts, offsets, scatter, gather, gate_idx = meta
        if ep is not None:
            # the owners of the experts pull their rows from every rank, the home ranks pull the results back
            out = ep.run_routed(xn_rows, idx, gates, offsets, scatter, gather, x_in_slab=in_slab,
                                meta_in_slab=meta_in_slab, out_dtype=out_dtype, stats=acc[:2])
        else:
            (p1, a1), (p2, a2) = self.packed()
            disp = ops.dispatch_gather(xn_rows, gather)
            hid = ops.ternary_linear_grouped(disp, p1, a1, offsets, epilogue=ops.EPI_GELU_BF16, prepared=True)
            y = ops.ternary_linear_grouped(hid, p2, a2, offsets, epilogue=ops.EPI_BF16, prepared=True)
            out = ops.scatter_combine(y, gates, scatter, out_dtype=out_dtype, stats=acc[:2])
        n_total = N
        if self.stats_group is not None:
            import torch.distributed as dist
            # one all-reduce for everything: sums, P_e, the top-1 histogram and the token count travel as f64
            # (integers up to 2^53 are exact)
            both = torch.cat([acc, hist.to(torch.float64), torch.full((1,), float(N), dtype=torch.float64, device=dev)])
            dist.all_reduce(both, group=self.stats_group)
            acc.copy_(both[:2 + E])
            hist.copy_(both[2 + E:2 + 2 * E].to(torch.int32))
            n_total = int(both[-1].item()) if self._n_total_hint is None else self._n_total_hint
        self.last_routing = (idx, gates, meta)
        if not finalize:
            return out, n_total
        scalars = ops.moe_finalize(acc[:2], acc[2:], hist, E, n_total, n_total * C, self.balance_alpha, scalars=scalars)
        return out, scalars

    def forward(self, x):
        B, T, C = x.shape
        out, sc = self.run_rows(_as_rows_bf16(x), out_dtype=torch.float32 if x.dtype == torch.float32 else torch.bfloat16)
        return out.view(B, T, C).to(x.dtype), sc[0], sc[1], sc[2]


CUDASparseMoELayer = SparseMoELayer


# ----------------------------------------------------------------------------------------------
# LSF
# ----------------------------------------------------------------------------------------------
class LiquidStateFusion(nn.Module):
    """jarvis_engine/jarvis_model.py:261-314: one scalar decay per call derived from act_var."""

    def __init__(self, d_model, alpha_min=0.1, alpha_max=0.99):
        super().__init__()
        self.alpha_min = alpha_min
        self.alpha_max = alpha_max
        self.var_scale = nn.Parameter(torch.tensor(1.0))

    def forward(self, x, act_var, h_prev=None):
        act_var = torch.as_tensor(act_var, dtype=torch.float32, device=x.device).reshape(1)
        h0 = None if h_prev is None else h_prev.to(torch.float32).contiguous()
        m = x.contiguous()
        if m.dtype not in (torch.float32, torch.bfloat16):
            m = m.float()
        out, last = ops.lsf_scan(m, act_var=act_var, var_scale=_f32(self.var_scale, scalar=True),
                                 alpha_min=self.alpha_min, alpha_max=self.alpha_max, h0=h0)
        return out.to(x.dtype), last.to(x.dtype)


class LiquidStateFusionExt(nn.Module):
    """The extension flavour, liquid_fusion_cuda/liquid_state_fusion.py:269-294:
    forward(alpha (B,T,D), M (B,T,D), h0=None) -> H, with optional persistence of the last state."""

    def __init__(self, persistent=False):
        super().__init__()
        self.persistent = persistent
        self.h = None

    def reset_state(self):
        self.h = None

    def forward(self, alpha, M, h0=None):
        B, T, D = alpha.shape
        if alpha.dtype == torch.float64:
            raise TypeError("Double precision (float64) is not supported on CUDA for LiquidStateFusion.")
        if h0 is not None:
            init = h0
        elif self.persistent and self.h is not None and self.h.shape == (B, D) and self.h.device == alpha.device:
            init = self.h
        else:
            init = None
        H, last = ops.lsf_scan(M.contiguous(), alpha_tensor=alpha.contiguous(),
                               h0=None if init is None else init.float().contiguous())
        self.h = last.to(alpha.dtype) if self.persistent else None
        return H


class ReflectivePenalty(nn.Module):
    """jarvis_engine/jarvis_model.py:329-351 (scalar arithmetic; the EMA only moves in training)."""

    def __init__(self, lam=0.01, tau_max=1.0, ema_decay=0.99):
        super().__init__()
        self.lam = lam
        self.tau_max = tau_max
        self.ema_decay = ema_decay
        self.register_buffer("mu_t", torch.tensor(0.0))

    def forward(self, act_mean, act_var):
        l_reflect = self.lam * ((self.mu_t.detach() - act_mean) ** 2 + F.relu(act_var - self.tau_max))
        if self.training:
            self.mu_t = self.ema_decay * self.mu_t + (1.0 - self.ema_decay) * act_mean.detach()
        return l_reflect


# ----------------------------------------------------------------------------------------------
# block and model
# ----------------------------------------------------------------------------------------------
class JarvisBlock(nn.Module):
    """jarvis_engine/jarvis_model.py:399-441.  `forward` keeps the reference signature; the fused
    path `forward_rows` works on the fp32 residual stream in place and is what `Jarvis` calls."""

    def __init__(self, d_model, n_heads, num_experts=4, top_k=2, max_seq_len=2048, use_cuda_attn: bool = True,
                 use_cuda_moe: bool = True):
        super().__init__()
        self.norm1 = RMSNorm(d_model)
        self.attn = AssociativeLinearAttention(d_model, n_heads, max_seq_len=max_seq_len)
        self.norm2 = RMSNorm(d_model)
        self.moe = SparseMoELayer(d_model, num_experts=num_experts, top_k=top_k)
        self.liquid = LiquidStateFusion(d_model)
        self.reflect = ReflectivePenalty()

    def forward_rows(self, x, B, T, h_prev=None, start_pos=0, attn_state=None, want_attn_state=False,
                     inplace_state=False, scratch=None, cp=None):
        """x: f32 (B*T, C) residual stream, UPDATED IN PLACE.  Returns (h_last f32 (B, C), scalars f32
        [l_balance, act_mean, act_var], attention state or None).  cp (parallel.ContextParallel): this rank
        holds one T-token slice of every sequence; states returned are those after the whole sequence."""
        C = x.shape[1]
        xn = ops.rmsnorm(x, _f32(self.norm1.weight), self.norm1.eps)
        o, state = self.attn.scan_rows(xn, B, T, start_pos, attn_state, want_attn_state, inplace_state, cp=cp)
        po, ao = self.attn.out_proj.packed()
        ops.ternary_linear(o, po, ao, epilogue=ops.EPI_RESID_F32, out=x, prepared=True)          # x += attn(norm1(x))
        norm2 = (_f32(self.norm2.weight), self.norm2.eps)
        if scratch is None:
            moe_out, scalars = self.moe.run_rows(x, norm=norm2)
        else:
            moe_out, scalars = self.moe.run_rows(x, acc=scratch[0], hist=scratch[1], scalars=scratch[2], norm=norm2)
        if cp is not None:
            # the decay of the call (one scalar, from the statistics of the WHOLE batch: moe.stats_group) in
            # torch, for the weights of the slice-end sum; the scan kernel derives the same value itself
            lq = self.liquid
            alpha = lq.alpha_min + (lq.alpha_max - lq.alpha_min) * torch.sigmoid(-lq.var_scale.detach().float() * scalars[2])

            def scan(h_in):
                ops.lsf_scan(moe_out.view(B, T, C), act_var=scalars[2:3], var_scale=_f32(lq.var_scale, scalar=True),
                             alpha_min=lq.alpha_min, alpha_max=lq.alpha_max, h0=h_in.contiguous(),
                             resid=x.view(B, T, C), want_out=False)
            # the slice's end value from a zero carry: the scan kernel asked for its last value only (reads m once)
            _, end = ops.lsf_scan(moe_out.view(B, T, C), act_var=scalars[2:3], var_scale=_f32(lq.var_scale, scalar=True),
                                  alpha_min=lq.alpha_min, alpha_max=lq.alpha_max, want_out=False)
            _, h_last = cp.lsf(scan, end, alpha, T, None if h_prev is None else h_prev.float())
            return h_last, scalars, state
        _, h_last = ops.lsf_scan(moe_out.view(B, T, C), act_var=scalars[2:3],
                                 var_scale=_f32(self.liquid.var_scale, scalar=True),
                                 alpha_min=self.liquid.alpha_min, alpha_max=self.liquid.alpha_max,
                                 h0=None if h_prev is None else h_prev.float().contiguous(),
                                 resid=x.view(B, T, C), want_out=False,
                                 last_out=h_prev if (inplace_state and h_prev is not None) else None)
        # x += lsf(moe(norm2(x)))
        return h_last, scalars, state

    def step_rows(self, x, xn, B, h_prev, positions, attn_state, inplace_state, scratch, next_norm):
        """One token per sequence (decode): x f32 (B, C) residual stream, UPDATED IN PLACE; xn bf16 (B, C) =
        norm1(x), from the caller (the tail kernel of the block before this one made it).  The tail of the block
        is ONE launch: the MoE scalars, the LSF step with the residual add, and the RMSNorm `next_norm` =
        (weight, eps) of whatever follows (the next block's norm1 or the model's final norm).
        Returns (h_last, scalars, attention state, normalised rows for the next consumer)."""
        C = x.shape[1]
        o, state = self.attn.scan_rows(xn, B, 1, positions, attn_state, True, inplace_state)
        po, ao = self.attn.out_proj.packed()
        ops.ternary_linear(o, po, ao, epilogue=ops.EPI_RESID_F32, out=x, prepared=True)
        acc, hist, scalars = scratch
        moe, lq = self.moe, self.liquid
        moe_out, n_total = moe.run_rows(x, acc=acc, hist=hist, norm=(_f32(self.norm2.weight), self.norm2.eps),
                                        finalize=False)
        xn_next, h_last = ops.lsf_step_norm(
            moe_out, acc[:2], acc[2:], hist, moe.num_experts, n_total, n_total * C, moe.balance_alpha, scalars,
            _f32(lq.var_scale, scalar=True), lq.alpha_min, lq.alpha_max,
            None if h_prev is None else h_prev.float().contiguous(), x, norm=next_norm,
            h_out=h_prev if (inplace_state and h_prev is not None and h_prev.dtype == torch.float32) else None)
        return h_last, scalars, state, xn_next

    def forward(self, x, h_prev=None, start_pos: int = 0):
        B, T, C = x.shape
        rows = x.reshape(B * T, C).float().clone()
        h_last, sc, _ = self.forward_rows(rows, B, T, h_prev, start_pos)
        l_reflect = self.reflect(sc[1], sc[2])
        return rows.view(B, T, C).to(x.dtype), h_last.to(x.dtype), sc[0], l_reflect


class Jarvis(nn.Module):
    """jarvis_engine/jarvis_model.py:444-546.  forward(idx, targets=None, persist_state=False) ->
    (logits, loss); reset_state(); get_backend_status(); param_count().  Logits are bf16
    (`logits_dtype`).  Beyond the reference: `carry_attention_state=True` also hands the attention
    state S across persist_state calls (the reference carries only the LSF membrane and the RoPE
    offset, so it is off by default)."""

    def __init__(self, vocab_size=50257, d_model=1024, n_layers=24, n_heads=16, num_experts=4, top_k=2,
                 max_seq_len=1024, use_cuda_attn: bool = True, use_cuda_moe: bool = True):
        super().__init__()
        self.d_model = d_model
        self.use_cuda_attn = True
        self.use_cuda_moe = True
        self.tok_emb = nn.Embedding(vocab_size, d_model)
        self.blocks = nn.ModuleList([
            JarvisBlock(d_model, n_heads, num_experts, top_k, max_seq_len=max_seq_len) for _ in range(n_layers)
        ])
        self.final_norm = RMSNorm(d_model)
        self.lm_head = nn.Linear(d_model, vocab_size, bias=False)
        self._h_states: list = [None] * n_layers
        self._attn_states: list = [None] * n_layers
        self._token_pos: int = 0
        self.carry_attention_state = False
        self._cp = None
        self.logits_dtype = torch.bfloat16
        self._lm_head_bf16 = None
        self.last_aux = None

    def get_backend_status(self):
        n = len(self.blocks)
        return {
            "has_cuda_attn_extension": True,
            "has_cuda_moe_extension": True,
            "attn_backend": "cuda",
            "moe_backend": "cuda",
            "attn_cuda_blocks": f"{n}/{n}",
            "moe_cuda_blocks": f"{n}/{n}",
        }

    def reset_state(self):
        self._h_states = [None] * len(self.blocks)
        self._attn_states = [None] * len(self.blocks)
        self._token_pos = 0

    def _layer_scratch(self, device):
        """Per-forward accumulators of all layers, zeroed with three fills: (sum, sum^2, P) f64,
        top-1 histogram i32, and the [l_balance, act_mean, act_var] outputs f32."""
        n, E = len(self.blocks), self.blocks[0].moe.num_experts
        acc = torch.zeros((n, 2 + E), dtype=torch.float64, device=device)
        hist = torch.zeros((n, E), dtype=torch.int32, device=device)
        scal = torch.zeros((n, 3), dtype=torch.float32, device=device)
        return [(acc[i], hist[i], scal[i]) for i in range(n)]

    def _lm_head_weight(self):
        w = self.lm_head.weight
        key = (w.data_ptr(), w._version)
        if self._lm_head_bf16 is None or self._lm_head_bf16[0] != key:
            # rows padded with zeros to a multiple of 128, the out-feature tile of the GEMM kernel
            v = w.shape[0]
            wp = torch.zeros(((v + 127) // 128 * 128, w.shape[1]), dtype=torch.bfloat16, device=w.device)
            wp[:v] = w.detach().to(torch.bfloat16)
            self._lm_head_bf16 = (key, wp)
        return self._lm_head_bf16[1]

    def hidden_rows(self, idx, persist_state=False):
        """Embedding + all blocks + final norm -> bf16 (B*T, C) hidden rows."""
        if self.training:
            raise RuntimeError("Jarvis (sm_100a): inference only; call .eval() first")
        B, T = idx.shape
        x = ops.embedding(idx.contiguous(), _f32(self.tok_emb.weight)).view(B * T, self.d_model)
        start_pos = self._token_pos if persist_state else 0
        if persist_state:
            self._token_pos += T * (self._cp.world if self._cp is not None else 1)
        h_prevs = self._h_states if persist_state else [None] * len(self.blocks)
        s_prevs = self._attn_states if (persist_state and self.carry_attention_state) else [None] * len(self.blocks)
        new_h, new_s, aux = [], [], []
        scratch = self._layer_scratch(x.device)
        if self._cp is not None:
            for block in self.blocks:       # every rank holds B*T tokens: no host read of the all-reduced count
                block.moe._n_total_hint = B * T * self._cp.world
        for i, block in enumerate(self.blocks):
            h_prev = h_prevs[i]
            if h_prev is not None and h_prev.shape[0] != B:
                h_prev = None
            s_prev = s_prevs[i]
            if s_prev is not None and s_prev.shape[0] != B:
                s_prev = None
            h_last, sc, state = block.forward_rows(x, B, T, h_prev, start_pos, s_prev,
                                                   want_attn_state=self.carry_attention_state, scratch=scratch[i],
                                                   cp=self._cp)
            new_h.append(h_last)
            new_s.append(state)
            aux.append(sc)
        self._h_states = new_h
        self._attn_states = new_s
        self.last_aux = aux
        return ops.rmsnorm(x, _f32(self.final_norm.weight), self.final_norm.eps)

    @torch.no_grad()
    def step(self, idx, positions=None, state=None, max_position=None, inplace=False):
        """Explicit-state step for decode / chunked prefill, beyond the reference API: `state` is None
        (fresh sequences) or the dict returned by the previous call ({"h": LSF membranes, "S": attention
        states (B, H, 64, 64) f32, per layer}); `positions` is an int or an int32 (B,) tensor holding each
        sequence's first position (ragged batches).  With inplace=True (short steps only: one segment per
        sequence) the tensors of `state` are updated in place.  Returns (logits (B, T, vocab), new state)."""
        if self.training:
            raise RuntimeError("Jarvis (sm_100a): inference only; call .eval() first")
        B, T = idx.shape
        n = len(self.blocks)
        x = ops.embedding(idx.contiguous(), _f32(self.tok_emb.weight)).view(B * T, self.d_model)
        pos = 0 if positions is None else positions
        hs = state["h"] if state is not None else [None] * n
        Ss = state["S"] if state is not None else [None] * n
        new_h, new_s = [], []
        scratch = self._layer_scratch(x.device)
        if T == 1 and self.d_model <= 1024 and self.d_model % 8 == 0:
            # decode: every block's tail (MoE scalars + LSF step + the norm that follows) is one launch
            norms = [b.norm1 for b in self.blocks[1:]] + [self.final_norm]
            xn = ops.rmsnorm(x, _f32(self.blocks[0].norm1.weight), self.blocks[0].norm1.eps)
            for i, block in enumerate(self.blocks):
                block.attn.max_position = max_position
                h_last, _, S, xn = block.step_rows(x, xn, B, hs[i], pos, Ss[i], inplace and state is not None, scratch[i],
                                                   (_f32(norms[i].weight), norms[i].eps))
                new_h.append(h_last)
                new_s.append(S)
            hidden = xn
        else:
            for i, block in enumerate(self.blocks):
                block.attn.max_position = max_position
                h_last, _, S = block.forward_rows(x, B, T, hs[i], pos, Ss[i], want_attn_state=True,
                                                  inplace_state=inplace and state is not None, scratch=scratch[i])
                new_h.append(h_last)
                new_s.append(S)
            hidden = ops.rmsnorm(x, _f32(self.final_norm.weight), self.final_norm.eps)
        vocab = self.lm_head.weight.shape[0]
        logits = ops.dense_linear(hidden, self._lm_head_weight()).view(B, T, -1)[..., :vocab]
        return logits, {"h": new_h, "S": new_s}

    @torch.no_grad()
    def forward(self, idx, targets=None, persist_state=False):
        B, T = idx.shape
        hidden = self.hidden_rows(idx, persist_state)
        vocab = self.lm_head.weight.shape[0]
        # dense bf16 lm_head on the same tcgen05 pipeline as the ternary layers (weight tiles by TMA); the padded
        # vocabulary columns are sliced off as a view
        logits = ops.dense_linear(hidden, self._lm_head_weight()).view(B, T, -1)[..., :vocab]
        if self.logits_dtype != torch.bfloat16:
            logits = logits.to(self.logits_dtype)
        loss = None
        if targets is not None:
            ce = F.cross_entropy(logits.float().view(-1, logits.size(-1)), targets.view(-1))
            aux = torch.stack(self.last_aux)
            l_reflect = sum(b.reflect(sc[1], sc[2]) for b, sc in zip(self.blocks, self.last_aux))
            loss = ce + aux[:, 0].sum() + l_reflect
        return logits, loss

    def set_batch_split(self, group, global_tokens=None):
        """Treat the ranks of `group` as holding slices of ONE batch: every layer all-reduces its MoE
        statistics so that the LSF decay and the auxiliary scalars equal those of the unsplit batch
        (the reference derives one decay per call from the variance of the whole batch,
        jarvis_model.py:249-250, 297-298).  group=None restores independent per-rank batches."""
        for blk in self.blocks:
            blk.moe.stats_group = group
            blk.moe._n_total_hint = global_tokens

    def set_expert_parallel(self, group, max_tokens: int | None = None, global_tokens: int | None = None):
        """Spread the experts of every MoE layer over the ranks of `group` (one process per GPU on one node): the
        ranks hold slices of ONE batch (as with set_batch_split: the per-layer statistics are all-reduced, so the
        LSF decay and the auxiliary scalars are those of the whole batch), every rank routes its own tokens and
        the expert rows travel by peer-memory loads (parallel.PeerExpertParallelMoE; the reference has no
        multi-GPU code, jarvis_model.py:198-251 is the layer being split).  max_tokens: most tokens a rank
        passes per call.  group=None: back to local experts (frees the exchange buffers)."""
        from . import parallel
        ex = getattr(self, "_ep_exchange", None)
        for blk in self.blocks:
            blk.moe._ep = None
        if ex is not None:
            ex.close()
            self._ep_exchange = None
        self.set_batch_split(group, global_tokens)
        if group is None:
            return
        moe = self.blocks[0].moe
        if max_tokens is None:
            raise ValueError("set_expert_parallel: max_tokens (tokens per rank and call) is needed")
        ex = parallel.PeerExchange(moe.num_experts, moe.top_k, self.d_model, moe.w1[0].weight.shape[0], max_tokens,
                                   self.tok_emb.weight.device, group)
        self._ep_exchange = ex
        for blk in self.blocks:
            blk.moe._ep = parallel.PeerExpertParallelMoE(blk.moe, exchange=ex)

    def set_context_parallel(self, group):
        """Sequence parallelism of `forward` / `hidden_rows`: the ranks of `group` hold consecutive T-token slices
        of the same sequences (rank r: tokens [r*T, (r+1)*T)).  Every layer all-gathers the slices' attention
        and LSF end states (parallel.ContextParallel) and all-reduces its MoE statistics, so each rank's logits
        are those of its slice in a single-GPU run over the whole sequence.  group=None switches it off."""
        from . import parallel
        self._cp = None if group is None else parallel.ContextParallel(group)
        self.set_batch_split(group)

    def param_count(self):
        n = sum(p.numel() for p in self.parameters())
        return n, f"{n/1e6:.1f}M parameters"


class DecodeSession:
    """One-token-per-step decode of B concurrent sequences with the whole step captured in a CUDA
    graph (the pattern of the reference's runtime/cuda_graph_runner.py:47-70, applied to the real
    model).  The carried state lives in buffers owned by the session and is updated in place, so a
    replay costs one launch; per-sequence positions advance on the device."""

    def __init__(self, model: "Jarvis", state: dict, positions: torch.Tensor, max_position: int):
        self.model = model
        self.state = {"h": [t.float().contiguous() for t in state["h"]], "S": [t.float().contiguous() for t in state["S"]]}
        self.positions = positions.to(torch.int32).clone()
        self.max_position = max_position
        B = self.positions.shape[0]
        self.idx = torch.zeros((B, 1), dtype=torch.int64, device=self.positions.device)
        self.graph = None
        self.logits = None

    def _one(self):
        logits, _ = self.model.step(self.idx, self.positions, self.state, max_position=self.max_position, inplace=True)
        self.positions.add_(1)
        return logits

    def capture(self):
        """Two eager warm-up steps on a side stream, then capture.  The warm-up steps advance the state:
        call before feeding real tokens, or re-load the state afterwards with load_state()."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self._one()
        torch.cuda.current_stream().wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.logits = self._one()
        return self

    def load_state(self, state: dict, positions: torch.Tensor):
        for dst, src in zip(self.state["h"], state["h"]):
            dst.copy_(src)
        for dst, src in zip(self.state["S"], state["S"]):
            dst.copy_(src)
        self.positions.copy_(positions)

    def step(self, idx: torch.Tensor) -> torch.Tensor:
        """idx: int64 (B, 1) -> logits (B, 1, vocab) (a buffer reused by the next step)."""
        self.idx.copy_(idx)
        if self.graph is None:
            return self._one()
        self.graph.replay()
        return self.logits


class PrefillSession:
    """A fixed-shape stateless forward (B x T token ids -> logits) captured in a CUDA graph, the pattern of the
    reference's runtime/cuda_graph_runner.py:47-70 applied to the whole model.  The forward is ~340 launches; from
    Python each costs tens of microseconds of host time, which is hidden behind a 14 ms step at B=8 x T=2048 but
    not when the step is short (a small batch, or one batch split over several GPUs: the per-layer statistics
    all-reduce of set_batch_split is captured with it).  A replay is one launch; programmatic dependent launch
    edges are kept inside the graph."""

    def __init__(self, model: "Jarvis", batch: int, seq_len: int, device=None):
        self.model = model
        device = device or model.tok_emb.weight.device
        self.idx = torch.zeros((batch, seq_len), dtype=torch.int64, device=device)
        self.graph = None
        self.logits = None

    def capture(self):
        """Two eager warm-up passes on a side stream (weight packing, buffer set-up), then the capture."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(2):
                self.model(self.idx)
        torch.cuda.current_stream().wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.logits = self.model(self.idx)[0]
        return self

    def __call__(self, idx: torch.Tensor) -> torch.Tensor:
        """idx: int64 (B, T) -> logits (B, T, vocab) (a buffer reused by the next call)."""
        self.idx.copy_(idx)
        if self.graph is None:
            with torch.no_grad():
                return self.model(self.idx)[0]
        self.graph.replay()
        return self.logits


def install(model: nn.Module) -> nn.Module:
    """Swap the attention / MoE / LSF / norm modules of an existing reference `Jarvis` (or anything
    with the same `.blocks[i].{norm1,attn,norm2,moe,liquid}` layout) for the sm_100a ones, keeping the
    parameters (shared, not copied) and therefore the state-dict keys.  Mirrors the reference's own
    attribute-replacement mechanism (experiments/architecture_matrix/modular_memory.py:353-368)."""

    def adopt(dst: nn.Module, src: nn.Module):
        # the SAME Parameter / buffer objects are attached to the new module: no second copy of the weights,
        # and later in-place updates of the model's tensors (or `.to(device)` on the model) reach it
        src_params, src_bufs = dict(src.named_parameters()), dict(src.named_buffers())
        missing = [k for k in dst.state_dict() if k not in src_params and k not in src_bufs]
        if missing:
            raise RuntimeError(f"install: source module lacks {missing}")
        for name in [n for n, _ in dst.named_parameters()]:
            owner, leaf = dst, name
            while "." in leaf:
                head, leaf = leaf.split(".", 1)
                owner = getattr(owner, head)
            owner._parameters[leaf] = src_params[name]
        for name in [n for n, _ in dst.named_buffers()]:
            if name not in src_bufs:
                continue                 # non-persistent caches of the new module (RoPE tables)
            owner, leaf = dst, name
            while "." in leaf:
                head, leaf = leaf.split(".", 1)
                owner = getattr(owner, head)
            owner._buffers[leaf] = src_bufs[name]
        return dst.to(next(src.parameters()).device).eval()

    for blk in model.blocks:
        d_model = blk.norm1.weight.numel()
        blk.attn = adopt(AssociativeLinearAttention(d_model, blk.attn.n_heads,
                                                    max_seq_len=blk.attn.rotary.max_seq_len_cached), blk.attn)
        blk.moe = adopt(SparseMoELayer(d_model, blk.moe.num_experts, blk.moe.top_k, noise_std=blk.moe.noise_std,
                                       balance_alpha=blk.moe.balance_alpha), blk.moe)
        blk.liquid = adopt(LiquidStateFusion(d_model, blk.liquid.alpha_min, blk.liquid.alpha_max), blk.liquid)
        blk.norm1 = adopt(RMSNorm(d_model, blk.norm1.eps), blk.norm1)
        blk.norm2 = adopt(RMSNorm(d_model, blk.norm2.eps), blk.norm2)
    return model


def ternary_init_(module: nn.Module, std: float = 0.02, generator=None) -> nn.Module:
    """Gaussian (std 0.02) re-initialisation of every ternary layer: the synthetic-weight recipe the
    benchmarks and tests use in place of a trained checkpoint."""
    with torch.no_grad():
        for m in module.modules():
            if isinstance(m, TernaryLinear):
                m.weight.copy_(torch.randn(m.weight.shape, generator=generator) * std)
    return module


__all__ = [
    "RMSNorm", "TernaryLinear", "RotaryEmbedding", "AssociativeLinearAttention", "CUDAAssociativeLinearAttention",
    "SparseMoELayer", "CUDASparseMoELayer", "LiquidStateFusion", "LiquidStateFusionExt", "ReflectivePenalty",
    "JarvisBlock", "Jarvis", "DecodeSession", "install", "ternary_init_",
]
