"""Multi-GPU forms of the path: expert parallelism of the top-2 MoE layer and context (sequence) parallelism of
the two scans, over the ranks of one node.

Expert parallelism:

The reference has no distributed code; this adds the one exchange the path has when the 4 experts
live on different GPUs: an all-to-all of dispatched token rows before the expert FFN and its inverse
after it (NCCL over NVLink on GPUs; any torch.distributed backend works, which is how the logic is
tested with gloo on CPU).  Tokens stay data-parallel: every rank routes its own tokens with the
replicated router, so routing and gates are those of the single-GPU layer.

Ownership: with `world <= E` rank r owns the `E / world` consecutive experts starting at
`r * E / world`; with `world > E` each expert is served by `world / E` consecutive ranks and every
source rank cuts its rows for that expert into that many contiguous parts (the packed weights are
1 MiB per expert, so replicas are free).  Inside an expert the rows arrive ordered by (source rank,
local stable order): when ranks hold contiguous token ranges this is exactly the single-GPU dispatch
order (moe_compute_metadata_kernel, sparse_model_cuda/sparse_model.cu:23-90).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def ops_stream() -> int:
    from . import ops
    return ops._stream()


def owner_plan(world: int, num_experts: int):
    """-> (rounds, plan) with plan[round][dst_rank] = (expert, part, nparts): which slice of which
    expert's rows a source sends to `dst_rank` in that all-to-all round."""
    if world <= num_experts:
        if num_experts % world:
            raise ValueError(f"num_experts ({num_experts}) must be divisible by the world size ({world})")
        per = num_experts // world
        return per, [[(d * per + j, 0, 1) for d in range(world)] for j in range(per)]
    if world % num_experts:
        raise ValueError(f"world size ({world}) must be a multiple of num_experts ({num_experts})")
    shards = world // num_experts
    return 1, [[(d // shards, d % shards, shards) for d in range(world)]]


def part_bounds(count: int, part: int, nparts: int):
    return count * part // nparts, count * (part + 1) // nparts


def send_layout(counts, plan_round):
    """Row ranges (begin, end) inside the expert-sorted dispatched rows for every destination."""
    offsets = [0]
    for c in counts:
        offsets.append(offsets[-1] + int(c))
    out = []
    for expert, part, nparts in plan_round:
        lo, hi = part_bounds(int(counts[expert]), part, nparts)
        out.append((offsets[expert] + lo, offsets[expert] + hi))
    return out


class ExpertParallelMoE:
    """Runs a `SparseMoELayer`'s experts across a process group.

    `compute(rows, owned_experts, seg_offsets) -> rows` applies w2(GELU(w1(.))) of the listed experts
    to the contiguous row segments; the default uses the layer's packed weights and the grouped
    tcgen05 GEMM.  `route`, `gather`, `combine` default to the CUDA kernels as well; tests on CPU pass
    oracle implementations."""

    def __init__(self, moe, group=None, route=None, gather=None, combine=None, compute=None):
        self.moe = moe
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.rounds, self.plan = owner_plan(self.world, moe.num_experts)
        self.owned = [self.plan[j][self.rank][0] for j in range(self.rounds)]
        self._route = route or self._route_cuda
        self._gather = gather or self._gather_cuda
        self._combine = combine or self._combine_cuda
        self._compute = compute or self._compute_cuda
        self._owned_weights = None
        self.last_recv_counts = None

    # ---- default CUDA stages ------------------------------------------------------------------
    def _route_cuda(self, x):
        from . import ops
        idx, gates, _ = ops.router_top2(x, self.moe.router.weight.detach().float().contiguous())
        counts, offsets, scatter, gather, _ = ops.moe_metadata(idx, self.moe.num_experts)
        return idx, gates, counts, scatter, gather

    def _gather_cuda(self, x, gather_map):
        from . import ops
        return ops.dispatch_gather(x, gather_map)

    def _combine_cuda(self, y, gates, scatter_map, out_dtype):
        from . import ops
        return ops.scatter_combine(y, gates, scatter_map, out_dtype=out_dtype)

    def _compute_cuda(self, rows, owned, seg_offsets):
        from . import ops
        (p1, a1), (p2, a2) = self.moe.packed()
        key = (p1.data_ptr(), p2.data_ptr(), tuple(owned))
        if self._owned_weights is None or self._owned_weights[0] != key:
            sel = torch.tensor(owned, device=p1.device)
            self._owned_weights = (key, p1[sel].contiguous(), a1[sel].contiguous(), p2[sel].contiguous(),
                                   a2[sel].contiguous())
        _, q1, b1, q2, b2 = self._owned_weights
        hid = ops.ternary_linear_grouped(rows, q1, b1, seg_offsets, epilogue=ops.EPI_GELU_BF16, prepared=True)
        return ops.ternary_linear_grouped(hid, q2, b2, seg_offsets, epilogue=ops.EPI_BF16, prepared=True)

    # ---- the exchange -------------------------------------------------------------------------
    def run_rows(self, x, out_dtype=None):
        """x: (N_local, C) rows of this rank -> (N_local, C) MoE output (same values as the single-GPU layer)."""
        out_dtype = out_dtype or x.dtype
        idx, gates, counts, scatter_map, gather_map = self._route(x)
        dispatched = self._gather(x, gather_map)                         # expert-sorted rows
        counts_h = [int(c) for c in counts.cpu().tolist()]               # host sync: NCCL needs split sizes
        C = x.shape[1]
        recv_bufs, send_sizes_all, recv_sizes_all, layouts = [], [], [], []
        for j in range(self.rounds):
            layout = send_layout(counts_h, self.plan[j])
            send_sizes = [hi - lo for lo, hi in layout]
            t_send = torch.tensor(send_sizes, dtype=torch.int64, device=x.device)
            t_recv = torch.empty_like(t_send)
            dist.all_to_all_single(t_recv, t_send, group=self.group)
            recv_sizes = [int(v) for v in t_recv.cpu().tolist()]
            contiguous = all(layout[d][1] == layout[d + 1][0] for d in range(self.world - 1))
            send = dispatched[layout[0][0]:layout[-1][1]] if contiguous else torch.cat(
                [dispatched[lo:hi] for lo, hi in layout])
            recv = torch.empty((sum(recv_sizes), C), dtype=x.dtype, device=x.device)
            dist.all_to_all_single(recv, send.contiguous(), recv_sizes, send_sizes, group=self.group)
            recv_bufs.append(recv)
            send_sizes_all.append(send_sizes)
            recv_sizes_all.append(recv_sizes)
            layouts.append(layout)
        self.last_recv_counts = recv_sizes_all
        rows = recv_bufs[0] if self.rounds == 1 else torch.cat(recv_bufs)
        seg = [0]
        for r in recv_bufs:
            seg.append(seg[-1] + r.shape[0])
        seg_offsets = torch.tensor(seg, dtype=torch.int32, device=x.device)
        y_rows = self._compute(rows, self.owned, seg_offsets) if rows.shape[0] else rows
        y_disp = torch.empty_like(dispatched)
        for j in range(self.rounds):
            back = torch.empty((sum(send_sizes_all[j]), C), dtype=x.dtype, device=x.device)
            dist.all_to_all_single(back, y_rows[seg[j]:seg[j + 1]].contiguous(), send_sizes_all[j], recv_sizes_all[j],
                                   group=self.group)
            pos = 0
            for lo, hi in layouts[j]:
                y_disp[lo:hi] = back[pos:pos + hi - lo]
                pos += hi - lo
        return self._combine(y_disp, gates, scatter_map, out_dtype), (idx, gates)


class ContextParallel:
    """Sequence (context) parallelism for the two recurrences of the block: rank r of the group holds tokens
    [r * T_local, (r + 1) * T_local) of EVERY sequence of the batch.

    Both scans are linear in their carried state, so a rank's slice can be scanned from a zero state, the
    slices' end states combined across ranks, and the true incoming state fed to a second, final pass:

      attention  S_out = gamma^T_local * S_in + D_r      (D_r: end state of slice r scanned from zero)
      LSF        h_out = alpha^T_local * h_in + e_r      (e_r: end value of slice r scanned from zero)

    One all-gather of D_r (B, H, 64, 64 f32) and one of e_r (B, C f32) per layer; every rank folds the
    contributions of the ranks before it (the reference has no multi-GPU code; the combine is the one its
    chunk-parallel attention path applies between chunks, jarvis_engine/jarvis_model.py:131-190).
    The scans themselves are passed in, so the class runs with the CUDA kernels or with the CPU oracle."""

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)

    def _gather(self, t: torch.Tensor) -> torch.Tensor:
        """-> (world, *t.shape): every rank's tensor, in rank order."""
        if t.is_cuda:   # NCCL: one output tensor, no per-rank copies
            out = torch.empty((self.world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
            dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
            return out
        parts = [torch.empty_like(t) for _ in range(self.world)]
        dist.all_gather(parts, t.contiguous(), group=self.group)
        return torch.stack(parts)

    def _fold(self, parts: torch.Tensor, decay: torch.Tensor, init):
        """parts: (W, ...) end states of the slices from zero; decay: per-slice decay, broadcastable to parts[0]
        (gamma^T_local per head, or alpha^T_local).  State entering slice r: sum_{r' < r} decay^(r-1-r') parts[r']
        + decay^r init; state after the last slice: the same with r = W.  Two weighted sums instead of a loop
        of W small updates."""
        W = self.world
        out = []
        for upto in (self.rank, W):
            acc = torch.zeros_like(parts[0]) if init is None else decay.pow(float(upto)) * init
            if upto > 0:
                expo = torch.arange(upto - 1, -1, -1, device=parts.device, dtype=torch.float32)
                w = decay.unsqueeze(0).pow(expo.view((-1,) + (1,) * decay.dim()))       # (upto, *decay.shape)
                acc = acc + (w * parts[:upto]).sum(dim=0)
            out.append(acc)
        return out[0], out[1]

    def attention_states(self, delta: torch.Tensor, gamma: torch.Tensor, t_local: int, state0=None):
        """delta: this rank's D_r (B, H, Dv, Dk); gamma: (H,) decays.  -> (state entering this rank's slice,
        state after the last rank's slice); `state0` is the state before the first token of the sequence."""
        parts = self._gather(delta.float())
        g = gamma.float().to(delta.device).pow(float(t_local)).view(1, -1, 1, 1)
        return self._fold(parts, g, None if state0 is None else state0.float())

    def lsf_states(self, end: torch.Tensor, alpha, t_local: int, h0=None):
        """end: this rank's e_r (B, C); alpha: scalar decay of the call.  -> (carry into this rank's slice,
        membrane after the last rank's slice)."""
        parts = self._gather(end.float())
        a = torch.as_tensor(alpha, dtype=torch.float32, device=end.device).reshape(1, 1).pow(float(t_local))
        return self._fold(parts, a, None if h0 is None else h0.float())

    @staticmethod
    def lsf_slice_end(m: torch.Tensor, alpha) -> torch.Tensor:
        """End value of h_t = alpha h_{t-1} + (1 - alpha) m_t over a slice (B, T, C) started from zero: a
        weighted sum over t, so it needs no scan: sum_t (1 - alpha) alpha^(T-1-t) m_t  ->  (B, C) f32."""
        T = m.shape[1]
        a = torch.as_tensor(alpha, dtype=torch.float32, device=m.device).reshape(())
        w = (1.0 - a) * a.pow(torch.arange(T - 1, -1, -1, device=m.device, dtype=torch.float32))
        return torch.einsum("btc,t->bc", m.float(), w)

    # ---- the two scans of one layer ----------------------------------------------------------------
    def attention(self, scan, gamma, t_local: int, state0=None, state_only=None):
        """scan(state_in) -> (o, state_out) runs this rank's slice; state_only() -> D_r, when given, is a cheaper
        way to get the slice's end state from a zero state (k/v only).  Rank 0 without an initial state needs one
        full pass (its output is final and its end state is D_0); the others get D_r first and scan once more
        from the true incoming state.  -> (o of this rank's slice, state after the whole sequence)."""
        second = self.rank > 0 or state0 is not None
        o = None
        if second and state_only is not None:
            delta = state_only()
        else:
            o, delta = scan(None)
        s_in, s_last = self.attention_states(delta, gamma, t_local, state0)
        if second:
            o, _ = scan(s_in)
        return o, s_last

    def lsf(self, scan, slice_end: torch.Tensor, alpha, t_local: int, h0=None):
        """scan(h_in) applies the LSF scan to this rank's slice from the carry h_in and returns its result;
        slice_end is the slice's end value from a zero carry (B, C) (lsf_slice_end, or the scan kernel asked
        for its last value only).  -> (scan's result, membrane after the whole sequence)."""
        h_in, h_last = self.lsf_states(slice_end, alpha, t_local, h0)
        return scan(h_in), h_last


class PeerExchange:
    """The buffers of the peer-memory expert exchange: one slab per rank (rows, gather map, offsets, expert outputs,
    row bookkeeping) allocated once and mapped into every other rank through its CUDA IPC handle
    (jb200_peer_buffer_*), plus the stream-ordered barrier that separates the phases.  One exchange serves any
    number of layers (every call ends with a barrier, so the buffers are free again)."""

    def __init__(self, num_experts: int, top_k: int, d_model: int, hidden: int, max_tokens: int, device, group=None):
        import ctypes as C_
        from . import _lib
        self._lib = _lib
        lib = _lib.load()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        E, K, C = num_experts, top_k, d_model
        if not ((self.world <= E and E % self.world == 0) or (self.world > E and self.world % E == 0)):
            raise ValueError(f"peer expert parallelism: world ({self.world}) must divide or be a multiple of num_experts ({E})")
        self.shards = max(1, self.world // E)           # ranks serving one expert
        self.per = max(1, E // self.world)              # experts (expert parts) owned by a rank
        self.C, self.E, self.K, self.n_max, self.hidden = C, E, K, max_tokens, hidden
        # every slot of every rank on one expert, cut into `shards` parts (rounded up): the worst case
        self.max_rows = (max_tokens * K + self.shards - 1) // self.shards * self.world
        layout, off = {}, 0
        for name, nbytes in (("xn", max_tokens * C * 2), ("y", self.max_rows * C * 2), ("gmap", max_tokens * K * 4),
                             ("offs", (E + 2) * 4), ("meta", (self.per * (self.world + 1) + self.per + 1) * 4),
                             ("flags", 32 * 4)):
            layout[name] = off
            off = (off + nbytes + 255) // 256 * 256
        self._slab_bytes = off
        with torch.cuda.device(device):
            ptr, handle = C_.c_void_p(), (C_.c_ubyte * 64)()
            _lib.check(lib.jb200_peer_buffer_alloc(off, C_.byref(ptr), handle), "jb200_peer_buffer_alloc")
            self._slab = ptr.value
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=group)
            self._opened, bases = [], []
            for r, h in enumerate(handles):
                if r == self.rank:
                    bases.append(self._slab)
                    continue
                p = C_.c_void_p()
                _lib.check(lib.jb200_peer_buffer_open((C_.c_ubyte * 64).from_buffer_copy(h), C_.byref(p)), "jb200_peer_buffer_open")
                self._opened.append(p.value)
                bases.append(p.value)

        class _Raw:      # zero-copy torch view of the slab
            def __init__(self, address, nbytes):
                self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (address, False), "version": 2}

        slab = torch.as_tensor(_Raw(self._slab, off), device=device)
        slab.zero_()

        def view(name, dtype, shape):
            n = 1
            for d in shape:
                n *= d
            nbytes = n * torch.empty((), dtype=dtype).element_size()
            return slab[layout[name]:layout[name] + nbytes].view(dtype).view(shape)

        self.xn = view("xn", torch.bfloat16, (max_tokens, C))
        self.y = view("y", torch.bfloat16, (self.max_rows, C))
        self.gmap = view("gmap", torch.int32, (max_tokens * K,))
        self.offs = view("offs", torch.int32, (E + 2,))
        self.n_published = -1          # the token count last written behind the offsets
        self.meta = view("meta", torch.int32, (self.per * (self.world + 1) + self.per + 1,))
        self.ptrs = {name: torch.tensor([b + layout[name] for b in bases], dtype=torch.int64, device=device) for name in layout}
        self.disp = torch.empty((self.max_rows, C), dtype=torch.bfloat16, device=device)
        self.hid = torch.empty((self.max_rows, hidden), dtype=torch.bfloat16, device=device)
        self.seg = torch.zeros((self.per + 1,), dtype=torch.int32, device=device)
        self._flag = torch.zeros((1,), dtype=torch.float32, device=device)
        self.owned = ([self.rank // self.shards] if self.shards > 1
                      else list(range(self.rank * self.per, (self.rank + 1) * self.per)))
        torch.cuda.synchronize(device)
        dist.all_reduce(self._flag, group=self.group)      # every slab (and its zeroed flag block) exists and is mapped
        torch.cuda.synchronize(device)

    def barrier(self):
        """Stream-ordered barrier over the ranks: every rank's earlier kernels have finished (and their writes are
        visible to the peers) before any rank's later kernels start.  Flags in the peer-mapped slabs
        (jb200_peer_barrier), not a collective of the communication library: a few microseconds."""
        self._lib.check(self._lib.load().jb200_peer_barrier(self.ptrs["flags"].data_ptr(), self.world, self.rank,
                                                           ops_stream()), "jb200_peer_barrier")

    def close(self):
        """Unmap the peers' slabs and free this rank's (call on every rank before the process group goes away)."""
        if self._slab is None:
            return
        torch.cuda.synchronize()
        dist.all_reduce(self._flag, group=self.group)      # every rank is done with the peers' slabs
        torch.cuda.synchronize()
        lib = self._lib.load()
        for p in self._opened:
            self._lib.check(lib.jb200_peer_buffer_close(p), "jb200_peer_buffer_close")
        self._opened = []
        dist.barrier(group=self.group)              # nobody still maps this rank's slab
        self.xn = self.y = self.gmap = self.offs = self.meta = None
        self._lib.check(lib.jb200_peer_buffer_free(self._slab), "jb200_peer_buffer_free")
        self._slab = None


class PeerExpertParallelMoE:
    """Expert parallelism with the two exchanges done by kernels that read the other GPUs' memory directly
    (csrc/ep_peer.cu) instead of NCCL all-to-alls: the owner of an expert pulls its input rows from every rank's
    routing result, the home rank of a token pulls its expert outputs back.  One process per GPU on one node;
    world <= num_experts (E / world experts per rank) or a multiple of it (every expert served by world / E ranks,
    each taking one contiguous slice of every source's rows); at most `max_tokens` tokens per rank and call.

    No count is ever read back to the host; the phases are separated by stream-ordered barriers (a one-element
    all-reduce).  Results equal the single-GPU layer bit for bit when ranks hold contiguous token ranges (same rows
    in the same order through the same GEMMs).  Several layers may share one `PeerExchange`."""

    def __init__(self, moe, max_tokens: int = 0, group=None, out_dtype=torch.bfloat16, exchange: PeerExchange | None = None):
        from . import _lib
        self._lib = _lib
        self.moe = moe
        self._own_exchange = exchange is None
        if exchange is None:
            dev = moe.router.weight.device
            exchange = PeerExchange(moe.num_experts, moe.top_k, moe.router.weight.shape[1], moe.w1[0].weight.shape[0],
                                    max_tokens, dev, group)
        self.ex = exchange
        self.group, self.world, self.rank = exchange.group, exchange.world, exchange.rank
        self.out_dtype = out_dtype
        self._w = None
        self.seg = exchange.seg

    def _owned_weights(self):
        (p1, a1), (p2, a2) = self.moe.packed()
        key = (p1.data_ptr(), p2.data_ptr())
        if self._w is None or self._w[0] != key:
            sel = torch.tensor(self.ex.owned, device=p1.device)
            self._w = (key, p1[sel].contiguous(), a1[sel].contiguous(), p2[sel].contiguous(), a2[sel].contiguous())
        return self._w[1:]

    def barrier(self):
        self.ex.barrier()

    def close(self):
        if self._own_exchange:
            self.ex.close()

    def run_routed(self, x, idx, gates, offsets, scatter, gather, *, x_in_slab=False, meta_in_slab=False, out_dtype=None,
                   stats=None):
        """The exchange for rows that are already routed: x bf16 (N, C) (or already sitting in the exchange's row
        buffer), idx / gates / offsets / scatter / gather = this rank's router and dispatch-metadata results
        (meta_in_slab: gather and offsets ARE the exchange's own buffers, written there by the metadata kernels)."""
        from . import ops
        ex = self.ex
        lib, C, E, K = self._lib.load(), ex.C, ex.E, ex.K
        N = idx.shape[0]
        if N > ex.n_max:
            raise RuntimeError(f"PeerExpertParallelMoE: {N} tokens exceed max_tokens={ex.n_max}")
        stream = ops_stream()
        if not x_in_slab:
            ex.xn[:N].copy_(x)
        if not meta_in_slab:
            ex.gmap[:N * K].copy_(gather)
            ex.offs[:E + 1].copy_(offsets)
        if ex.n_published != N:                         # the row count of this rank, read by the peers' gathers
            ex.offs[E + 1:].fill_(N)
            ex.n_published = N
        ex.barrier()                                    # every rank's rows and routing are in place
        self._lib.check(lib.jb200_ep_pull_gather(ex.ptrs["offs"].data_ptr(), ex.ptrs["gmap"].data_ptr(),
                                                 ex.ptrs["xn"].data_ptr(), ex.world, ex.rank, E, C, K, ex.n_max,
                                                 ex.max_rows, ex.disp.data_ptr(), ex.seg.data_ptr(),
                                                 ex.meta.data_ptr(), stream), "jb200_ep_pull_gather")
        p1, a1, p2, a2 = self._owned_weights()
        ops.ternary_linear_grouped(ex.disp, p1, a1, ex.seg, epilogue=ops.EPI_GELU_BF16, out=ex.hid, prepared=True)
        ops.ternary_linear_grouped(ex.hid, p2, a2, ex.seg, epilogue=ops.EPI_BF16, out=ex.y, prepared=True)
        ex.barrier()                                    # every owner's outputs (and row bookkeeping) are in place
        odt = out_dtype or self.out_dtype
        out = torch.empty((N, C), dtype=odt, device=idx.device)
        self._lib.check(lib.jb200_ep_pull_combine(ex.ptrs["y"].data_ptr(), ex.ptrs["meta"].data_ptr(),
                                                  offsets.data_ptr(), idx.data_ptr(), gates.data_ptr(), scatter.data_ptr(),
                                                  ex.world, ex.rank, E, C, K, N, ex.max_rows, out.data_ptr(),
                                                  1 if odt == torch.bfloat16 else 0,
                                                  None if stats is None else stats.data_ptr(), stream),
                        "jb200_ep_pull_combine")
        # No barrier at the end: what the next call writes before ITS first barrier (rows, gather map, offsets)
        # was last read by the peers' gathers, which finished before the second barrier above; everything else
        # (dispatched rows, expert outputs, bookkeeping) is written after that first barrier, which no rank passes
        # before every rank's combine of this call has finished.
        return out

    def run_rows(self, x, stats=None):
        """x: bf16 (N_local, C) rows of this rank -> ((N_local, C) MoE output, (topk_idx, gates))."""
        from . import ops
        ex = self.ex
        idx, gates, _ = ops.router_top2(x, self.moe.router.weight.detach().float().contiguous())
        N = idx.shape[0]
        if N > ex.n_max:
            raise RuntimeError(f"PeerExpertParallelMoE: {N} tokens exceed max_tokens={ex.n_max}")
        # the gather map and the offsets go straight into the buffers the other ranks read; rows that the caller
        # already keeps in the exchange's row buffer (x is ex.xn[:N]) are not copied either
        counts, offsets, scatter, gather, _ = ops.moe_metadata(idx, ex.E, gather_out=ex.gmap[:N * ex.K],
                                                               offsets_out=ex.offs[:ex.E + 1])
        return self.run_routed(x, idx, gates, offsets, scatter, gather, x_in_slab=x.data_ptr() == ex.xn.data_ptr(),
                               meta_in_slab=True, stats=stats), (idx, gates)
