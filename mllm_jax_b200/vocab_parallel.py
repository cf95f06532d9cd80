"""Vocabulary-parallel GRPO loss: each rank holds V/k columns of every logits row.

This is the tp-sharded case of the reference (lm_head kernel partitioned over "tp",
MLLM_JAX/utils.py:245), where XLA inserts an all-reduce(max) and an all-reduce(sum) around
log_softmax (MLLM_JAX/train_modules/__init__.py:125).  Here each rank computes per-token
partials (max, sumexp, sum e*y, chosen-or-0) with one streaming kernel, the ranks exchange
16 bytes per token (one NCCL all-gather over NVLink), every rank merges all partials and runs
the per-token epilogue, and the backward needs no further communication.  One process per GPU.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .ops import LossConfig, TokenLossProblem


def shard_bounds(vocab_total: int, rank: int, world: int) -> tuple[int, int]:
    """[start, stop) of the columns rank `rank` holds; the vocabulary must split evenly."""
    if vocab_total % world:
        raise ValueError(f"vocabulary of {vocab_total} does not split evenly over {world} ranks")
    per = vocab_total // world
    return rank * per, (rank + 1) * per


def exchange_partials(partials: torch.Tensor, group=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gather the per-rank partials [N, 4] (or [N, 6]: entropy at temperature != 1) into [world, N, width]
    (rank-major), on any backend."""
    if partials.dim() != 2 or partials.shape[1] not in (4, 6):
        raise ValueError(f"partials must be [N, 4] or [N, 6], got {tuple(partials.shape)}")
    world = dist.get_world_size(group)
    if out is None:
        out = torch.empty(world, *partials.shape, dtype=partials.dtype, device=partials.device)
    elif out.shape != (world, *partials.shape):
        raise ValueError("gather buffer has the wrong shape")
    dist.all_gather_into_tensor(out.view(-1), partials.contiguous().view(-1), group=group)
    return out


class PeerExchange:
    """Exchange buffers of the fused sharded kernel: one zeroed symmetric-memory buffer per rank,
    mapped into every rank's address space by torch.distributed's symmetric memory (cuMem handles
    with access granted to the local device).  One process per GPU on one node.  The kernels only
    ever STORE into a peer's buffer and poll their own."""

    def __init__(self, n_tokens: int, device: torch.device, group=None):
        import os

        # The kernels use plain peer stores only; keep the buffers off NVLink multicast objects.
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        from . import _lib

        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("the fused sharded kernel supports at most 8 vocabulary shards")
        self.n_tokens = int(n_tokens)
        nbytes = int(_lib.load().mllm_grpo_exchange_bytes(self.n_tokens, self.world))
        if self.world == 1:
            self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
            self.ptrs = [self.buf.data_ptr()]
            self.handle = None
        else:
            self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
            self.buf.zero_()
            torch.cuda.synchronize(device)
            self.handle = symm_mem.rendezvous(self.buf, self.group)
            self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
            if len(self.ptrs) != self.world or self.ptrs[self.rank] != self.buf.data_ptr():
                raise RuntimeError("symmetric memory rendezvous returned unexpected buffer pointers")
        self.epoch = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=group)  # every buffer is zeroed and mapped before anyone stores into it

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch


class VocabParallelLoss:
    """fwd+bwd of the loss on this rank's column shard.  Buffers are allocated once and reused."""

    def __init__(self, vocab_total: int, cfg: Optional[LossConfig] = None, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.vocab_total = int(vocab_total)
        self.start, self.stop = shard_bounds(self.vocab_total, self.rank, self.world)
        self.cfg = cfg or LossConfig()
        self._gathered = None
        self._partials = None
        self._peer = None

    def problem(self, shard_logits, token_ids, mask, advantages, total_valid, old_logps=None, ref_logps=None,
                scored_rows=None) -> TokenLossProblem:
        T = shard_logits.shape[1] if scored_rows is None else scored_rows
        p = TokenLossProblem(shard_logits, token_ids, mask, advantages, total_valid, old_logps, ref_logps, self.cfg,
                             scored_rows=T, vocab=self.stop - self.start, vocab_start=self.start,
                             vocab_total=self.vocab_total)
        # 4 floats per token, 6 when the entropy is wanted at temperature != 1 (two more sums on y/temperature)
        width = 6 if (self.cfg.compute_entropy and self.cfg.temperature != 1.0) else 4
        if self._partials is None or self._partials.shape != (p.N, width):
            self._partials = torch.empty(p.N, width, dtype=torch.float32, device=shard_logits.device)
            self._gathered = torch.empty(self.world, p.N, width, dtype=torch.float32, device=shard_logits.device)
        p.partials, p.gathered, p.n_shards = self._partials, self._gathered, self.world
        return p

    def forward(self, p: TokenLossProblem) -> None:
        p.run("mllm_grpo_fwd_partials")
        exchange_partials(p.partials, self.group, out=p.gathered)
        p.run("mllm_grpo_combine")

    def backward(self, p: TokenLossProblem, dlogits: Optional[torch.Tensor] = None, grad_scale: float = 1.0) -> torch.Tensor:
        p.grad_scale = float(grad_scale)
        if dlogits is not None:
            p.dlogits = dlogits
        elif p.dlogits is None:
            p.alloc_dlogits()
        p.run("mllm_grpo_bwd")
        return p.dlogits

    def value_and_grad(self, shard_logits, token_ids, mask, advantages, total_valid, old_logps=None, ref_logps=None,
                       dlogits=None) -> dict:
        p = self.problem(shard_logits, token_ids, mask, advantages, total_valid, old_logps, ref_logps)
        self.forward(p)
        d = self.backward(p, dlogits)
        return {"loss": p.loss.reshape(()), "per_token_logps": p.per_token_logps, "token_entropy": p.token_entropy,
                "dlogits": d, "problem": p}

    def plan_fused(self, shard_logits, token_ids, mask, advantages, total_valid, old_logps=None, ref_logps=None,
                   dlogits=None, grad_scale: float = 1.0, scored_rows: Optional[int] = None,
                   peer_wait_ms: int = 0) -> TokenLossProblem:
        """Bind buffers once for repeated fused steps on the same addresses (static shapes, new
        contents each step): `step_fused(plan)` then only bumps the epoch and launches.
        scored_rows = L - 1 takes the reference layout (row i scored against token i + 1, side arrays [B, L-1])."""
        p = self.problem(shard_logits, token_ids, mask, advantages, total_valid, old_logps, ref_logps, scored_rows)
        if self._peer is None or self._peer.n_tokens != p.N:
            self._peer = PeerExchange(p.N, shard_logits.device, self.group)
        p.peer_ptrs, p.shard_rank, p.n_shards = self._peer.ptrs, self.rank, self.world
        p.grad_scale = float(grad_scale)
        p.peer_wait_ms = int(peer_wait_ms)  # tolerated skew between ranks; 0 = the library's 2000 ms
        if dlogits is not None:
            p.dlogits = dlogits
        else:
            p.alloc_dlogits()
        return p

    def step_fused(self, p: TokenLossProblem) -> dict:
        """One fused step on a plan.  The returned "device_status" is the int32 word the kernel ORs
        MLLM_GRPO_DEV_* bits into: after a synchronisation, `raise_on_timeout(out)` (or a NaN loss) tells
        that a peer did not show up within the wait limit and the step must be thrown away."""
        p.exchange_epoch = self._peer.next_epoch()
        p.run("mllm_grpo_fwd_bwd_sharded", reuse_args=p.exchange_epoch > 1 and getattr(p, "_planned", False))
        p._planned = True
        return {"loss": p.loss.reshape(()), "per_token_logps": p.per_token_logps, "token_entropy": p.token_entropy,
                "dlogits": p.dlogits, "problem": p, "device_status": p.device_status}

    @staticmethod
    def raise_on_timeout(out: dict) -> None:
        """Synchronising check of a fused step's status word; clears it so that the next step waits again."""
        from . import _lib

        status = int(out["device_status"].item())
        if status & _lib.DEV_WAIT_TIMEOUT:
            out["device_status"].zero_()
            raise RuntimeError("vocabulary-parallel loss: a rank's partials did not arrive within the wait limit; "
                               "the step's loss is NaN and its gradient must not be used")

    def value_and_grad_fused(self, shard_logits, token_ids, mask, advantages, total_valid, old_logps=None,
                             ref_logps=None, dlogits=None, grad_scale: float = 1.0,
                             scored_rows: Optional[int] = None) -> dict:
        """Same result as value_and_grad through ONE kernel per GPU (mllm_grpo_fwd_bwd_sharded): the
        per-token partials cross NVLink as peer stores issued by the kernel itself, and the row shard
        is re-read from L2 for the backward.  All ranks must call it the same number of times.
        The entropy at temperature != 1 needs two more sums per shard than the kernel's exchange record carries:
        that combination takes the all-gather path (value_and_grad) instead."""
        if self.cfg.compute_entropy and self.cfg.temperature != 1.0:
            return self.value_and_grad(shard_logits, token_ids, mask, advantages, total_valid, old_logps, ref_logps,
                                       dlogits)
        return self.step_fused(self.plan_fused(shard_logits, token_ids, mask, advantages, total_valid, old_logps,
                                               ref_logps, dlogits, grad_scale, scored_rows))


class TokenParallelLoss:
    """Rows split across ranks (the reference's real runs: batch over ("dp", "fsdp"), tp = 1,
    plugins/training/runner/grpo_gsm8k.py:282).  `total_valid_token_count` is already global by contract
    (:770), so each rank's loss is its share of the global loss and the only exchange is a scalar sum.
    The gradient of a rank's rows needs no communication at all."""

    def __init__(self, cfg: Optional[LossConfig] = None, group=None):
        self.group = group
        self.cfg = cfg or LossConfig()

    def value_and_grad(self, local_logits, token_ids, mask, advantages, total_valid_global, old_logps=None,
                       ref_logps=None, dlogits=None, reduce_loss: bool = True, shifted: bool = False) -> dict:
        """This rank's rows through mllm_grpo_fwd_bwd.  total_valid_global must be the count over ALL ranks'
        rows; out["loss"] is then the global loss (sum of the ranks' shares) and out["local_loss"] this rank's
        share.  shifted=True takes the reference layout (input_ids / labels [B, L])."""
        from .ops import grpo_value_and_grad

        if total_valid_global is None:
            raise ValueError("token-parallel ranks need the global total_valid_token_count")
        out = grpo_value_and_grad(local_logits, token_ids, mask, advantages, total_valid_global, old_logps, ref_logps,
                                  cfg=self.cfg, dlogits=dlogits, shifted=shifted)
        out["local_loss"] = out["loss"]
        if reduce_loss:
            out["loss"] = self.reduce_loss(out["loss"])
        return out

    def reduce_loss(self, local_loss: torch.Tensor) -> torch.Tensor:
        total = local_loss.detach().clone()
        dist.all_reduce(total, op=dist.ReduceOp.SUM, group=self.group)
        return total

    def reduce_loss_async(self, local_loss: torch.Tensor):
        """The same sum without making the compute stream wait for it: returns (total, work).  Nothing after the
        loss kernel depends on the global loss (the gradient is complete per rank), so the next step's kernel can
        run while the scalar crosses NVLink; call work.wait() before reading `total`."""
        total = local_loss.detach().clone()
        work = dist.all_reduce(total, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        return total, work
