"""CPU oracle for the Jarvis block-forward path.  TEST INFRASTRUCTURE ONLY.

A plain torch-on-CPU (fp32 unless stated) restatement of what the reference computes on the
block-forward path, written as free functions over explicit weight tensors.  It exists to
check the CUDA kernels: only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs
may import it; the product package never does.

Parity status: PINNED.  tests/golden/*.npz hold inputs and outputs produced by importing the
reference's own modules (tests/golden/make_golden.py, run where the reference tree is mounted),
and tests/test_oracle_golden.py checks every function below against them.

Each function cites the reference code it restates (paths relative to the reference root).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

CHUNK = 64  # AssociativeLinearAttention.CHUNK_SIZE, jarvis_engine/jarvis_model.py:90


# --------------------------------------------------------------------------------------
# ternary weights
# --------------------------------------------------------------------------------------
def absmean_quantize(w: torch.Tensor):
    """TernaryQuantizeSTE.forward, jarvis_engine/utils/ternary_ops.py:24-31.

    Returns (alpha as a python float holding the fp32 value, q in {-1, 0, +1} fp32)."""
    w = w.float()
    alpha = w.abs().mean().clamp(min=1e-8)
    q = torch.round(torch.clamp(w / alpha, -1.0, 1.0))
    return float(alpha), q


def pack_ternary(q: torch.Tensor) -> torch.Tensor:
    """pack_ternary_tensor, runtime/weight_packing.py:22-51: code 0/1/2 for 0/+1/-1, four
    codes per byte along the last axis, first element in the lowest two bits."""
    if q.shape[-1] % 4 != 0:
        raise AssertionError("Last dimension must be divisible by 4")
    codes = torch.where(q == 1, 1, torch.where(q == -1, 2, 0)).to(torch.uint8)
    c = codes.reshape(*q.shape[:-1], q.shape[-1] // 4, 4)
    return (c[..., 0] | (c[..., 1] << 2) | (c[..., 2] << 4) | (c[..., 3] << 6)).contiguous()


def unpack_ternary(packed: torch.Tensor, shape, dtype=torch.float32) -> torch.Tensor:
    """unpack_ternary_tensor, runtime/weight_packing.py:53-70."""
    p = packed.reshape(-1, 1).to(torch.int32)
    codes = (p >> torch.tensor([0, 2, 4, 6], dtype=torch.int32)) & 3
    vals = (codes == 1).to(dtype) - (codes == 2).to(dtype)
    return vals.reshape(tuple(shape))


def ternary_linear(x: torch.Tensor, q: torch.Tensor, alpha: float) -> torch.Tensor:
    """TernaryLinear.forward, jarvis_engine/utils/ternary_ops.py:51-53 (no bias)."""
    return F.linear(x, q * alpha)


def ternary_linear_from_weight(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    alpha, q = absmean_quantize(w)
    return ternary_linear(x, q, alpha)


# --------------------------------------------------------------------------------------
# norm, feature map, RoPE
# --------------------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """RMSNorm.forward, jarvis_engine/jarvis_model.py:25-26."""
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight


def rope_tables(n_pos: int, head_dim: int = 64, base: float = 10000.0):
    """cos/sin caches of RotaryEmbedding, jarvis_engine/jarvis_model.py:42-57 (fp32).
    Returns (cos, sin) of shape (n_pos, head_dim); the two halves of the last axis are equal."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2).float() / head_dim))
    freqs = torch.outer(torch.arange(n_pos, dtype=torch.float32), inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def feature_map_rope(q: torch.Tensor, k: torch.Tensor, start_pos: int = 0):
    """ELU+1 feature map (q additionally / sqrt(D)) followed by half-split RoPE:
    jarvis_engine/jarvis_model.py:124-128 with RotaryEmbedding.forward :59-71 and rotate_half
    :29-32.  q, k: (B, H, T, D)."""
    D = q.shape[-1]
    T = q.shape[-2]
    q = (F.elu(q) + 1.0) / math.sqrt(D)
    k = F.elu(k) + 1.0
    if torch.is_tensor(start_pos):
        # per-sequence first positions (ragged decode): the reference takes one int for the whole batch
        # (RotaryEmbedding.forward, jarvis_model.py:59-68); this is the same table, gathered per sequence
        cos_t, sin_t = rope_tables(int(start_pos.max()) + T, D)
        pos = start_pos.long()[:, None] + torch.arange(T)[None, :]
        cos = cos_t[pos].to(q.dtype)[:, None]          # (B, 1, T, D)
        sin = sin_t[pos].to(q.dtype)[:, None]
    else:
        cos, sin = rope_tables(start_pos + T, D)
        cos = cos[start_pos:].to(q.dtype)
        sin = sin[start_pos:].to(q.dtype)

    def rot(x):
        x1, x2 = x[..., : D // 2], x[..., D // 2:]
        return torch.cat((-x2, x1), dim=-1)

    return q * cos + rot(q) * sin, k * cos + rot(k) * sin


# --------------------------------------------------------------------------------------
# associative linear-attention scan
# --------------------------------------------------------------------------------------
def attn_scan_chunked(q, k, v, gamma, state0=None, chunk: int = CHUNK):
    """Chunkwise evaluation of S_t = gamma*S_{t-1} + v_t (x) k_t, o_t = S_t q_t with the state
    laid out (B, H, D_v, D_k): jarvis_engine/jarvis_model.py:131-190 (a ragged last chunk is
    handled like a full one with its own length, :164-172).  The carried-state arguments follow
    CUDAAssociativeLinearAttention's h_prev path
    (associative_attention_cuda/associative_attention.py:273-308).

    q, k (already feature-mapped + rotated), v: (B, H, T, D); gamma: (H,) in (0, 1).
    Returns (o (B, H, T, D), final state (B, H, D, D))."""
    B, H, T, D = q.shape
    log_g = torch.log(gamma.to(torch.float32))
    S = torch.zeros(B, H, D, D, dtype=q.dtype) if state0 is None else state0.clone()
    outs = []
    for s in range(0, T, chunk):
        c = min(chunk, T - s)
        qc, kc, vc = q[:, :, s:s + c], k[:, :, s:s + c], v[:, :, s:s + c]
        i = torch.arange(c, dtype=torch.float32)
        lag = i[:, None] - i[None, :]
        decay = (torch.exp(log_g[:, None, None] * lag.clamp(min=0)) * (lag >= 0)).to(q.dtype)   # (H, c, c)
        into = torch.exp(log_g[:, None] * (i + 1)).to(q.dtype)                                  # (H, c)
        tail = torch.exp(log_g[:, None] * (c - 1 - i)).to(q.dtype)                              # (H, c)
        whole = torch.exp(log_g * c).to(q.dtype)                                                # (H,)
        scores = torch.einsum("bhid,bhjd->bhij", qc, kc) * decay
        intra = torch.einsum("bhij,bhjd->bhid", scores, vc)
        cross = torch.einsum("bhde,bhie->bhid", S, qc) * into[None, :, :, None]
        outs.append(intra + cross)
        S = whole[None, :, None, None] * S + torch.einsum("bhid,bhie->bhde", vc * tail[None, :, :, None], kc)
    return torch.cat(outs, dim=2), S


def attn_scan_recurrent(q, k, v, gamma, state0=None):
    """Token-by-token fp64 evaluation of the same recurrence (the paper form quoted at
    jarvis_engine/jarvis_model.py:77-80); an independent check of the chunked algebra."""
    B, H, T, D = q.shape
    q, k, v = q.double(), k.double(), v.double()
    g = gamma.double()[None, :, None, None]
    S = torch.zeros(B, H, D, D, dtype=torch.float64) if state0 is None else state0.double().clone()
    o = torch.empty(B, H, T, D, dtype=torch.float64)
    for t in range(T):
        S = g * S + v[:, :, t, :, None] * k[:, :, t, None, :]
        o[:, :, t] = torch.einsum("bhde,bhe->bhd", S, q[:, :, t])
    return o, S


def attention_forward(x, wq, wk, wv, wo, gamma_raw, n_heads: int, start_pos: int = 0, state0=None,
                      return_state: bool = False):
    """AssociativeLinearAttention.forward, jarvis_engine/jarvis_model.py:115-191.  x: (B, T, C)."""
    B, T, C = x.shape
    D = C // n_heads

    def heads(t):
        return t.view(B, T, n_heads, D).transpose(1, 2)

    q = heads(ternary_linear_from_weight(x, wq))
    k = heads(ternary_linear_from_weight(x, wk))
    v = heads(ternary_linear_from_weight(x, wv))
    q, k = feature_map_rope(q, k, start_pos)
    o, S = attn_scan_chunked(q, k, v, torch.sigmoid(gamma_raw), state0)
    y = ternary_linear_from_weight(o.transpose(1, 2).reshape(B, T, C), wo)
    return (y, S) if return_state else y


# --------------------------------------------------------------------------------------
# MoE: router, dispatch order, experts, side outputs
# --------------------------------------------------------------------------------------
def top2_lowest_index_first(probs: torch.Tensor):
    """Top-2 of each row with ties resolved towards the lower expert id (torch.topk leaves the
    order of equal values unspecified; the kernels and this oracle fix it)."""
    E = probs.shape[-1]
    ar = torch.arange(E)
    p0, i0 = probs.max(dim=-1)
    i0 = torch.where(probs == p0[:, None], ar, E).min(dim=-1).values
    masked = probs.clone()
    masked[torch.arange(probs.shape[0]), i0] = -1.0
    p1 = masked.max(dim=-1).values
    i1 = torch.where(masked == p1[:, None], ar, E).min(dim=-1).values
    return torch.stack((p0, p1), dim=-1), torch.stack((i0, i1), dim=-1)


def router_top2(x_flat: torch.Tensor, w_router: torch.Tensor):
    """Eval-mode router of SparseMoELayer.forward, jarvis_engine/jarvis_model.py:218-224:
    logits -> softmax -> top-2 -> gates renormalised with +1e-8.  Returns (idx int64 (N, 2),
    gates (N, 2), probs (N, E))."""
    probs = F.softmax(F.linear(x_flat, w_router), dim=-1)
    top_p, top_i = top2_lowest_index_first(probs)
    gates = top_p / (top_p.sum(dim=-1, keepdim=True) + 1e-8)
    return top_i, gates, probs


def moe_metadata(topk_idx: torch.Tensor, num_experts: int):
    """Dispatch order of moe_compute_metadata_kernel, sparse_model_cuda/sparse_model.cu:23-90:
    assignments m = token*K + k are stably partitioned by expert id.  Returns int32 tensors
    (counts (E,), offsets (E+1,), scatter_map (N, K): slot of m, gather_map (M,): token of slot,
    gate_idx_map (M,): k of slot)."""
    N, K = topk_idx.shape
    flat = topk_idx.reshape(-1)
    order = torch.sort(flat, stable=True).indices              # slot -> m
    counts = torch.bincount(flat, minlength=num_experts)[:num_experts]
    offsets = torch.zeros(num_experts + 1, dtype=torch.int64)
    offsets[1:] = counts.cumsum(0)
    scatter = torch.empty(N * K, dtype=torch.int64)
    scatter[order] = torch.arange(N * K)
    i32 = torch.int32
    return (counts.to(i32), offsets.to(i32), scatter.view(N, K).to(i32), (order // K).to(i32), (order % K).to(i32))


def moe_forward(x, w_router, w1, w2, balance_alpha: float = 0.01):
    """Eval-mode SparseMoELayer.forward, jarvis_engine/jarvis_model.py:213-251.
    w1: list of (hidden, C) weights, w2: list of (C, hidden).  Returns (out (B, T, C), l_balance,
    act_mean, act_var, aux dict with idx / gates / probs)."""
    B, T, C = x.shape
    E = len(w1)
    xf = x.reshape(B * T, C)
    idx, gates, probs = router_top2(xf, w_router)
    out = torch.zeros_like(xf)
    for e in range(E):
        alpha1, q1 = absmean_quantize(w1[e])
        alpha2, q2 = absmean_quantize(w2[e])
        for kslot in range(idx.shape[1]):
            rows = (idx[:, kslot] == e).nonzero(as_tuple=True)[0]
            if rows.numel() == 0:
                continue
            h = F.gelu(ternary_linear(xf[rows], q1, alpha1))
            out[rows] += gates[rows, kslot, None] * ternary_linear(h, q2, alpha2)
    f = F.one_hot(idx[:, 0], num_classes=E).float().mean(dim=0)
    l_balance = balance_alpha * E * (f * probs.mean(dim=0)).sum()
    out = out.view(B, T, C)
    return out, l_balance, out.mean(), out.var(), {"idx": idx, "gates": gates, "probs": probs}


# --------------------------------------------------------------------------------------
# Liquid State Fusion
# --------------------------------------------------------------------------------------
def lsf_alpha(act_var, var_scale, alpha_min: float = 0.1, alpha_max: float = 0.99):
    """jarvis_engine/jarvis_model.py:297-298: one scalar decay per call."""
    return alpha_min + (alpha_max - alpha_min) * torch.sigmoid(-var_scale * act_var)


def lsf_scan(m: torch.Tensor, alpha, h0=None):
    """h_t = a_t*h_{t-1} + (1-a_t)*m_t, sequentially (the loop the reference validates its
    extension against, liquid_fusion_cuda/validate_liquid_state_fusion.py:11-19).  `alpha` is a
    scalar (model semantics) or a (B, T, D) tensor (extension API).  m: (B, T, D)."""
    B, T, D = m.shape
    h = torch.zeros(B, D, dtype=m.dtype) if h0 is None else h0.clone()
    out = torch.empty_like(m)
    per_elem = torch.is_tensor(alpha) and alpha.dim() == 3
    for t in range(T):
        a = alpha[:, t] if per_elem else alpha
        h = a * h + (1.0 - a) * m[:, t]
        out[:, t] = h
    return out


def lsf_model(m: torch.Tensor, act_var, var_scale, h_prev=None):
    """LiquidStateFusion.forward, jarvis_engine/jarvis_model.py:281-314, in its closed form
    (decay-matrix product + carry term).  Returns (h_out (B, T, C), h_last (B, C))."""
    B, T, C = m.shape
    if h_prev is None:
        h_prev = m.new_zeros(B, C)
    alpha = lsf_alpha(act_var, var_scale)
    t = torch.arange(T, dtype=torch.float32)
    lag = t[:, None] - t[None, :]
    log_a = torch.log(alpha)
    kernel = (torch.exp(log_a * lag.clamp(min=0)) * (lag >= 0)).to(m.dtype)
    h_out = (1.0 - alpha) * torch.matmul(kernel, m) + torch.exp(log_a * (t + 1)).view(1, T, 1).to(m.dtype) * h_prev[:, None]
    return h_out, h_out[:, -1, :]


# --------------------------------------------------------------------------------------
# block and model
# --------------------------------------------------------------------------------------
def block_forward(x, p: dict, n_heads: int, h_prev=None, start_pos: int = 0, attn_state0=None):
    """JarvisBlock.forward, jarvis_engine/jarvis_model.py:416-441 (eval mode).  `p` maps the
    block's state-dict names (norm1.weight, attn.q_proj.weight, ..., moe.w1.0.weight, ...,
    liquid.var_scale) to tensors.  Returns a dict with x, h_last, l_balance, l_reflect and the
    intermediate values the stage tests compare."""
    E = sum(1 for name in p if name.startswith("moe.w1."))
    a, S = attention_forward(rmsnorm(x, p["norm1.weight"]), p["attn.q_proj.weight"], p["attn.k_proj.weight"],
                             p["attn.v_proj.weight"], p["attn.out_proj.weight"], p["attn.gamma_raw"], n_heads,
                             start_pos, attn_state0, return_state=True)
    x = x + a
    moe_out, l_bal, act_mean, act_var, aux = moe_forward(
        rmsnorm(x, p["norm2.weight"]), p["moe.router.weight"],
        [p[f"moe.w1.{e}.weight"] for e in range(E)], [p[f"moe.w2.{e}.weight"] for e in range(E)])
    h_out, h_last = lsf_model(moe_out, act_var, p["liquid.var_scale"], h_prev)
    x = x + h_out
    # ReflectivePenalty.forward, jarvis_engine/jarvis_model.py:340-351, eval mode (mu_t fixed)
    mu_t = p.get("reflect.mu_t", torch.tensor(0.0))
    l_reflect = 0.01 * ((mu_t - act_mean) ** 2 + F.relu(act_var - 1.0))
    return {"x": x, "h_last": h_last, "l_balance": l_bal, "l_reflect": l_reflect, "attn_state": S,
            "moe_out": moe_out, "act_mean": act_mean, "act_var": act_var, **aux}


def model_forward(idx, sd: dict, n_layers: int, n_heads: int, h_prevs=None, start_pos: int = 0,
                  return_hidden: bool = False):
    """Jarvis.forward without targets, jarvis_engine/jarvis_model.py:488-536.  `sd` is a model
    state dict (tok_emb.weight, blocks.{i}.*, final_norm.weight, lm_head.weight)."""
    x = F.embedding(idx, sd["tok_emb.weight"])
    h_last = []
    for i in range(n_layers):
        pre = f"blocks.{i}."
        p = {name[len(pre):]: t for name, t in sd.items() if name.startswith(pre)}
        r = block_forward(x, p, n_heads, None if h_prevs is None else h_prevs[i], start_pos)
        x = r["x"]
        h_last.append(r["h_last"])
    hidden = rmsnorm(x, sd["final_norm.weight"])
    if return_hidden:
        return hidden, h_last
    return F.linear(hidden, sd["lm_head.weight"]), h_last


def model_step(idx, sd: dict, n_layers: int, n_heads: int, h_prevs=None, attn_states=None, positions=0):
    """State-carrying step: like model_forward, but every block also receives and returns its attention
    state S (the h_prev path of associative_attention.py:273-308, which the reference model never
    feeds) and `positions` may be a per-sequence tensor.  The LSF decay is computed from the step's own
    batch, as in every reference call.  Returns (logits, h_last list, attention-state list)."""
    x = F.embedding(idx, sd["tok_emb.weight"])
    h_last, states = [], []
    for i in range(n_layers):
        pre = f"blocks.{i}."
        p = {name[len(pre):]: t for name, t in sd.items() if name.startswith(pre)}
        r = block_forward(x, p, n_heads, None if h_prevs is None else h_prevs[i], positions,
                          None if attn_states is None else attn_states[i])
        x = r["x"]
        h_last.append(r["h_last"])
        states.append(r["attn_state"])
    return F.linear(rmsnorm(x, sd["final_norm.weight"]), sd["lm_head.weight"]), h_last, states


# ---- decode driver: sampling filter ----------------------------------------------------------------
def sample_filtered_probs(logits: torch.Tensor, temperature: float = 0.7, top_k: int = 50, top_p: float = 0.9):
    """The distribution sample_next_token draws from (jarvis_engine/evaluate_jarvis.py:158-185), for
    temperature > 0: logits / max(T, 1e-5); everything below the top_k-th value -> -inf (ties with it
    stay); sort descending, softmax, cumulative sum, drop sorted position i >= 1 when the cumulative
    probability before it exceeds top_p (only for 0 < top_p < 1); softmax of what is left.  (B, V) -> (B, V)."""
    x = logits.float() / max(temperature, 1e-5)
    if top_k is not None and top_k > 0:
        kth = torch.topk(x, min(top_k, x.size(-1))).values[:, [-1]]
        x = x.masked_fill(x < kth, float("-inf"))
    if top_p is not None and 0.0 < top_p < 1.0:
        sx, si = torch.sort(x, descending=True, stable=True)
        cum = torch.cumsum(F.softmax(sx, dim=-1), dim=-1)
        remove = cum > top_p
        remove[..., 1:] = remove[..., :-1].clone()
        remove[..., 0] = False
        x = x.masked_fill(remove.scatter(1, si, remove), float("-inf"))
    return F.softmax(x, dim=-1)


def sample_inverse_cdf(logits: torch.Tensor, u: torch.Tensor, temperature: float = 0.7, top_k: int = 50,
                       top_p: float = 0.9):
    """One draw per row from sample_filtered_probs with the caller's uniform numbers: the kept tokens are
    walked in descending order of probability (equal probability: lower id first) and the first one whose
    running sum exceeds u is taken.  temperature <= 0: argmax with the lowest id among equals (the
    reference's torch.argmax branch).  The reference itself draws with torch.multinomial, whose random
    stream cannot be reproduced elsewhere; the filtered distribution is what is pinned to it.
    -> (tokens int64 (B, 1), probability of each drawn token (B,))."""
    B, V = logits.shape
    if temperature is None or temperature <= 0.0:
        x = logits.float()
        best = x.max(dim=-1, keepdim=True).values
        tok = torch.where(x == best, torch.arange(V).expand(B, V), torch.full((B, V), V)).min(dim=-1, keepdim=True).values
        return tok, torch.ones(B)
    p = sample_filtered_probs(logits, temperature, top_k, top_p)
    sp, si = torch.sort(p, descending=True, stable=True)      # stable: equal values keep ascending ids
    toks, probs = [], []
    for b in range(B):
        c, pick = 0.0, None
        n_kept = int((sp[b] > 0).sum())
        for i in range(n_kept):
            c += float(sp[b, i])
            if c > float(u[b]):
                pick = i
                break
        if pick is None:
            pick = n_kept - 1
        toks.append(int(si[b, pick]))
        probs.append(float(sp[b, pick]))
    return torch.tensor(toks).view(B, 1), torch.tensor(probs)
