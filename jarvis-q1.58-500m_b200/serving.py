"""Decode driver: continuous batching over real slots, a CUDA-graphed step and next-token sampling.

The reference has the three pieces as separate prototypes: a slot policy that only appends a dummy token
(`ContinuousBatchingScheduler`, experiments/exp_batching_continuous.py:131-177), a CUDA-graph replay wrapper
(runtime/cuda_graph_runner.py:47-70) and the sampling filter of its REPL (`sample_next_token`,
jarvis_engine/evaluate_jarvis.py:158-185).  Here they drive the real model:

* `ContinuousBatchingScheduler` keeps the reference's names and policy (`add_request`, `waiting_queue`,
  `active_slots`, `step()`: fill empty slots in slot order from the queue, advance every active request by
  one token, retire the finished ones) and delegates the token generation to an engine.
* `CudaDecodeEngine` owns the per-slot recurrent state of every layer (attention S (64x64 per head) and the
  LSF membrane), admits a request by prefilling all but the last prompt token into its slot, and runs one
  batched, CUDA-graphed single-token step per iteration followed by the sampling kernel.  Every active slot
  therefore produces exactly one token per iteration, newly admitted ones included (their step consumes the
  last prompt token), which is the reference policy's accounting.

As in the reference model, the LSF decay of a step is a function of the MoE output variance of ALL rows of
the step's batch (jarvis_model.py:249-250, 297-298), so idle slots (fed `pad_token` from a zero state)
take part in it; their state is reset on release so that it stays finite.
"""
from __future__ import annotations

import collections
import time
from typing import Dict, List, Optional

import torch


class Request:
    """Same fields as the reference's Request (exp_batching_continuous.py:131-139)."""

    def __init__(self, req_id: int, prompt_tokens: List[int], max_new_tokens: int):
        if len(prompt_tokens) == 0:
            raise ValueError("Request: the prompt must hold at least one token")
        self.req_id = req_id
        self.prompt_tokens = list(prompt_tokens)
        self.max_new_tokens = max_new_tokens
        self.generated_tokens: List[int] = []
        self.is_finished = False
        self.arrival_time = time.time()
        self.finish_time: Optional[float] = None
        self.error: Optional[str] = None


class ContinuousBatchingScheduler:
    """Slot policy of exp_batching_continuous.py:141-177 over an engine with
    `admit(slot, prompt_tokens, max_new_tokens)`, `release(slot)` and `step(active_slots) -> {slot: token}`.
    A request the engine refuses (ValueError from `admit`: its positions would run past the engine's limit)
    is retired at once, unfinished, with the message in `req.error`; the slot goes to the next request."""

    def __init__(self, engine, max_batch_size: int = 8, eos_token: Optional[int] = None):
        self.engine = engine
        self.max_batch_size = max_batch_size
        self.eos_token = eos_token
        self.waiting_queue = collections.deque()
        self.active_slots: Dict[int, Request] = {}  # slot_idx -> Request
        self.completed: List[Request] = []

    def add_request(self, req: Request):
        self.waiting_queue.append(req)

    def step(self) -> int:
        """One iteration: fill empty slots, advance every active request by one token, retire the finished.
        Returns the number of requests advanced (0 when idle)."""
        for slot in range(self.max_batch_size):
            while slot not in self.active_slots and self.waiting_queue:
                req = self.waiting_queue.popleft()
                try:
                    self.engine.admit(slot, req.prompt_tokens, req.max_new_tokens)
                except ValueError as exc:
                    req.error = str(exc)
                    req.finish_time = time.time()
                    self.completed.append(req)
                    continue
                self.active_slots[slot] = req
        if not self.active_slots:
            return 0
        tokens = self.engine.step(sorted(self.active_slots))
        finished = []
        for slot, req in self.active_slots.items():
            tok = int(tokens[slot])
            req.generated_tokens.append(tok)
            if len(req.generated_tokens) >= req.max_new_tokens or (self.eos_token is not None and tok == self.eos_token):
                req.is_finished = True
                req.finish_time = time.time()
                finished.append(slot)
        for slot in finished:
            self.engine.release(slot)
            self.completed.append(self.active_slots.pop(slot))
        return len(self.active_slots) + len(finished)

    def run(self, max_iterations: Optional[int] = None) -> int:
        """Iterate until no request is active or waiting; returns the number of iterations."""
        it = 0
        while (self.active_slots or self.waiting_queue) and (max_iterations is None or it < max_iterations):
            self.step()
            it += 1
        return it


class CudaDecodeEngine:
    """Per-slot recurrent state + one CUDA-graphed batched step + the sampling kernel.

    temperature <= 0 selects argmax.  `seed` fixes the uniform numbers fed to the sampling kernel.
    `record=True` keeps, per iteration, the step's inputs and logits (for tests and debugging)."""

    def __init__(self, model, max_batch_size: int = 8, max_position: int = 4096, temperature: float = 0.7,
                 top_k: int = 50, top_p: float = 0.9, seed: int = 0, pad_token: int = 0, use_cuda_graph: bool = True,
                 record: bool = False):
        from . import ops
        from .modules import DecodeSession
        self._ops = ops
        self.model = model
        self.B = max_batch_size
        self.max_position = max_position
        self.temperature, self.top_k, self.top_p = temperature, top_k, top_p
        self.pad_token = pad_token
        dev = model.tok_emb.weight.device
        self.device = dev
        blk = model.blocks[0]
        n, C, H = len(model.blocks), model.d_model, blk.attn.n_heads
        state = {"h": [torch.zeros((self.B, C), dtype=torch.float32, device=dev) for _ in range(n)],
                 "S": [torch.zeros((self.B, H, 64, 64), dtype=torch.float32, device=dev) for _ in range(n)]}
        positions = torch.zeros((self.B,), dtype=torch.int32, device=dev)
        self.session = DecodeSession(model, state, positions, max_position)
        self.next_token = torch.full((self.B, 1), pad_token, dtype=torch.int64, device=dev)
        self.active = torch.zeros((self.B,), dtype=torch.int32, device=dev)
        self.gen = torch.Generator(device=dev)
        self.gen.manual_seed(seed)
        self.record = [] if record else None
        if use_cuda_graph:
            self.session.capture()          # its warm-up steps advance the (all idle) slots: start again from zero
            self._zero_all()

    def _zero_all(self):
        for t in self.session.state["h"] + self.session.state["S"]:
            t.zero_()
        self.session.positions.zero_()

    def _zero_slot(self, slot: int):
        for t in self.session.state["h"] + self.session.state["S"]:
            t[slot].zero_()
        self.session.positions[slot] = 0
        self.next_token[slot, 0] = self.pad_token

    def admit(self, slot: int, prompt_tokens: List[int], max_new_tokens: int = 0):
        """Prefill prompt[:-1] into the slot's state; the step of this iteration consumes prompt[-1].
        The RoPE table captured in the step's graph has `max_position` rows and the kernels clamp positions
        to it silently, so a request whose last generated token would sit beyond the table is refused here."""
        if len(prompt_tokens) + max(int(max_new_tokens), 0) > self.max_position:
            raise ValueError(f"prompt of {len(prompt_tokens)} tokens + {max_new_tokens} new tokens exceeds "
                             f"max_position={self.max_position}")
        if len(prompt_tokens) == 1:
            self._zero_slot(slot)           # longer prompts overwrite every tensor of the slot below
        if len(prompt_tokens) > 1:
            ctx = torch.tensor([prompt_tokens[:-1]], dtype=torch.int64, device=self.device)
            for blk in self.model.blocks:
                blk.attn.max_position = self.max_position
            _, st = self.model.step(ctx, positions=0, state=None, max_position=self.max_position)
            for dst, src in zip(self.session.state["h"], st["h"]):
                dst[slot].copy_(src[0])
            for dst, src in zip(self.session.state["S"], st["S"]):
                dst[slot].copy_(src[0])
            self.session.positions[slot] = len(prompt_tokens) - 1
        self.next_token[slot, 0] = int(prompt_tokens[-1])
        self.active[slot] = 1

    def release(self, slot: int):
        self._zero_slot(slot)
        self.active[slot] = 0

    def step(self, active_slots: List[int]) -> Dict[int, int]:
        """One token for every slot (idle ones run the pad token); returns {slot: token} for the active ones."""
        ops = self._ops
        if self.record is not None:
            self.record.append({"idx": self.next_token.clone(), "positions": self.session.positions.clone(),
                                "h": [t.clone() for t in self.session.state["h"]],
                                "S": [t.clone() for t in self.session.state["S"]]})
        logits = self.session.step(self.next_token)            # (B, 1, vocab) bf16, rows strided by the padded vocab
        rows = logits[:, 0, :]
        greedy = self.temperature is None or self.temperature <= 0.0
        u = None if greedy else torch.rand((self.B,), dtype=torch.float32, device=self.device, generator=self.gen)
        tok = ops.sample(rows, u, temperature=0.0 if greedy else self.temperature, top_k=self.top_k, top_p=self.top_p)
        if self.record is not None:
            self.record[-1]["logits"] = rows.float().clone()
            self.record[-1]["tokens"] = tok.clone()
        # active slots feed their own token back; idle ones go back to the pad token at position 0 from a zero
        # state (their step just ran, which moved their state: clear it again so that it stays the same, finite
        # contribution to the batch statistics every iteration)
        act = self.active.to(torch.int64).view(-1, 1)
        self.next_token.copy_(tok * act + self.pad_token * (1 - act))
        if len(active_slots) != self.B:
            idle = torch.tensor([s for s in range(self.B) if s not in set(active_slots)], dtype=torch.int64,
                                device=self.device)
            for t in self.session.state["h"] + self.session.state["S"]:
                t.index_fill_(0, idle, 0.0)
            self.session.positions.index_fill_(0, idle, 0)
        host = tok.view(-1).tolist()                          # one small device-to-host read per iteration
        return {s: host[s] for s in active_slots}


def build_scheduler(model, max_batch_size: int = 8, eos_token: Optional[int] = None, **engine_kwargs):
    """ContinuousBatchingScheduler over a CudaDecodeEngine for `model` (a jarvis_b200 `Jarvis` in eval mode)."""
    engine = CudaDecodeEngine(model, max_batch_size=max_batch_size, **engine_kwargs)
    return ContinuousBatchingScheduler(engine, max_batch_size=max_batch_size, eos_token=eos_token)
