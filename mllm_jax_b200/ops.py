"""Python operators over the C ABI: the fused GRPO / PPO-clip token loss.

These functions keep the argument names and semantics of the region they
replace in demon2036/MLLM-JAX, `TrainGRPOModule.__call__`
(MLLM_JAX/train_modules/__init__.py:118-180), and of its gradient with respect
to the logits (plugins/training/update/train_step.py:24).  Tensors are torch
CUDA tensors used only as device buffers: every computation happens inside
`libmllm_grpo.so`, reached through raw pointers and the current CUDA stream.
Nothing here falls back to torch math or to the CPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from ._lib import GrpoArgs


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


@dataclass
class LossConfig:
    """Operator attributes; defaults are TrainGRPOModule's (train_modules/__init__.py:89-93),
    except beta, which is 0 wherever the reference is actually configured
    (plugins/training/config.py:40) and only acts when ref log-probs are given."""

    temperature: float = 1.0
    epsilon_low: float = 0.2
    epsilon_high: float = 0.3
    beta: float = 0.0
    softcap: Optional[float] = None
    compute_entropy: bool = True
    cross_entropy: bool = False  # masked cross-entropy (SFT) instead of the clipped surrogate


class TokenLossProblem:
    """Device buffers of one call, laid out as the C ABI wants them.

    logits: bf16 [B, L, V] (or a [B, L, ld] view with V leading columns used).
    The first `scored_rows` rows of each sequence are scored; side arrays are
    [B, scored_rows].  Keeps references so the buffers outlive the launch.
    """

    def __init__(self, logits: torch.Tensor, chosen_ids: torch.Tensor, mask: Optional[torch.Tensor],
                 advantages: Optional[torch.Tensor], total_valid_token_count, old_logps: Optional[torch.Tensor],
                 ref_logps: Optional[torch.Tensor], cfg: LossConfig, *, scored_rows: int,
                 vocab: Optional[int] = None, vocab_start: int = 0, vocab_total: Optional[int] = None):
        if not logits.is_cuda:
            raise RuntimeError("the GRPO loss kernels run on a CUDA device only (no CPU path)")
        if logits.dtype != torch.bfloat16:
            raise TypeError(f"logits must be bfloat16, got {logits.dtype}")
        if logits.dim() != 3:
            raise ValueError(f"logits must be [B, L, V], got shape {tuple(logits.shape)}")
        B, L, Vfull = logits.shape
        if logits.stride(2) != 1 or (B > 1 and logits.stride(0) != L * logits.stride(1)):
            raise ValueError("logits must have unit stride on the vocabulary and rows evenly spaced")
        self.logits = logits
        self.row_stride = logits.stride(1)
        self._init_side(B, L, int(scored_rows), int(vocab) if vocab is not None else Vfull, logits.device, chosen_ids,
                        mask, advantages, total_valid_token_count, old_logps, ref_logps, cfg, vocab_start=vocab_start,
                        vocab_total=vocab_total)

    def _init_side(self, B, L, T, V, dev, chosen_ids, mask, advantages, total_valid_token_count, old_logps, ref_logps,
                   cfg: LossConfig, vocab_start: int = 0, vocab_total: Optional[int] = None):
        """Everything but the logits: geometry, per-token side arrays, outputs and residuals.  Also used on its
        own by callers that have no logits tensor (the folded lm_head forward)."""
        if not hasattr(self, "logits"):
            self.logits = None
            self.row_stride = V
        self.cfg = cfg
        self.B, self.L, self.T = B, L, T
        self.V = V
        self.vocab_start = int(vocab_start)
        self.vocab_total = int(vocab_total) if vocab_total is not None else self.vocab_start + self.V
        N = B * self.T
        self.N = N

        def side(t, name, dtype):
            if t is None:
                return None
            t = t.to(device=dev, dtype=dtype).contiguous()
            if t.numel() != N:
                raise ValueError(f"{name} must have {B}x{self.T} elements, got shape {tuple(t.shape)}")
            return t

        self.chosen_ids = side(chosen_ids, "chosen ids", torch.int32)
        self.mask = side(mask, "mask", torch.float32)
        self.old_logps = side(old_logps, "old_per_token_logps", torch.float32)
        self.ref_logps = side(ref_logps, "ref_per_token_logps", torch.float32)
        self.adv_per_token = 0
        self.advantages = None
        if advantages is not None:
            adv = advantages.to(device=dev, dtype=torch.float32)
            if adv.dim() == 2 and adv.shape[1] == 1:
                adv = adv[:, 0]
            if adv.numel() == B and adv.dim() == 1:
                self.adv_per_token = 0
            elif adv.numel() == N:
                self.adv_per_token = 1
            else:
                # same complaint as plugins/training/ppo/module.py:94
                raise ValueError(f"advantages shape {tuple(advantages.shape)} does not match per_token_logps {(B, self.T)}")
            self.advantages = adv.contiguous()

        self.total_valid_dev = None
        self.total_valid = 1.0
        tv = total_valid_token_count
        if tv is None:
            # inputs.get("total_valid_token_count", mask_loss.sum()), train_modules/__init__.py:179
            tv = self.mask.sum() if self.mask is not None else float(N)
        if isinstance(tv, torch.Tensor):
            self.total_valid_dev = tv.to(device=dev, dtype=torch.float32).reshape(1)
        else:
            self.total_valid = float(tv)

        # outputs and residuals
        self.per_token_logps = torch.empty(B, self.T, dtype=torch.float32, device=dev)
        self.token_entropy = torch.empty(B, self.T, dtype=torch.float32, device=dev) if cfg.compute_entropy else None
        self.lse = torch.empty(N, dtype=torch.float32, device=dev)
        self.grad_coef = torch.empty(N, dtype=torch.float32, device=dev)
        self.loss = torch.empty(1, dtype=torch.float32, device=dev)
        self.loss_terms = torch.empty(N, dtype=torch.float32, device=dev)
        self.device_status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.dlogits: Optional[torch.Tensor] = None
        self.grad_scale_dev: Optional[torch.Tensor] = None
        self.grad_scale = 1.0
        self.partials: Optional[torch.Tensor] = None
        self.gathered: Optional[torch.Tensor] = None
        self.n_shards = 0
        self.shard_rank = 0
        self.peer_ptrs = None      # device addresses of every rank's exchange buffer (fused sharded path)
        self.exchange_epoch = 0
        self.peer_wait_ms = 0      # 0 = the library's default (2000 ms)
        self.lse_scaled: Optional[torch.Tensor] = None         # residual of the entropy gradient (temperature != 1)
        self.entropy_cotangent: Optional[torch.Tensor] = None  # [B, T] cotangent of token_entropy for mllm_grpo_bwd

    def args(self) -> GrpoArgs:
        a = GrpoArgs()
        a.n_seqs, a.seq_rows, a.scored_rows = self.B, self.L, self.T
        a.vocab, a.row_stride = self.V, self.row_stride
        a.vocab_start, a.vocab_total = self.vocab_start, self.vocab_total
        c = self.cfg
        a.temperature, a.epsilon_low, a.epsilon_high, a.beta = c.temperature, c.epsilon_low, c.epsilon_high, c.beta
        a.softcap = float(c.softcap) if c.softcap else 0.0
        a.adv_per_token = self.adv_per_token
        a.flags = (0 if c.compute_entropy else _lib.FLAG_SKIP_ENTROPY) | (_lib.FLAG_CE_LOSS if c.cross_entropy else 0)
        a.grad_scale, a.total_valid = self.grad_scale, self.total_valid
        a.logits = _ptr(self.logits)
        a.chosen_ids, a.mask, a.advantages = _ptr(self.chosen_ids), _ptr(self.mask), _ptr(self.advantages)
        a.old_logps, a.ref_logps = _ptr(self.old_logps), _ptr(self.ref_logps)
        a.total_valid_dev, a.grad_scale_dev = _ptr(self.total_valid_dev), _ptr(self.grad_scale_dev)
        a.per_token_logps, a.token_entropy = _ptr(self.per_token_logps), _ptr(self.token_entropy)
        a.lse, a.grad_coef, a.loss, a.loss_terms = _ptr(self.lse), _ptr(self.grad_coef), _ptr(self.loss), _ptr(self.loss_terms)
        if self.dlogits is not None and (self.dlogits.shape != self.logits.shape or
                                         self.dlogits.stride() != self.logits.stride() or
                                         self.dlogits.dtype != torch.bfloat16 or
                                         self.dlogits.device != self.logits.device):
            # one row stride serves both buffers in the kernels: a differently laid out gradient buffer
            # would be written out of bounds
            raise ValueError("dlogits must match logits in shape, strides, dtype and device "
                             f"(logits {tuple(self.logits.shape)}/{self.logits.stride()}, "
                             f"dlogits {tuple(self.dlogits.shape)}/{self.dlogits.stride()})")
        a.dlogits = _ptr(self.dlogits)
        a.partials, a.gathered_partials, a.n_shards = _ptr(self.partials), _ptr(self.gathered), self.n_shards
        a.device_status = _ptr(self.device_status)
        a.shard_rank, a.exchange_epoch, a.peer_wait_ms = self.shard_rank, self.exchange_epoch, int(self.peer_wait_ms)
        a.lse_scaled, a.entropy_cotangent = _ptr(self.lse_scaled), _ptr(self.entropy_cotangent)
        if self.peer_ptrs is not None:
            for q, ptr in enumerate(self.peer_ptrs):
                a.peer_exchange[q] = ptr
        return a

    def alloc_dlogits(self, inplace: bool = False) -> torch.Tensor:
        """Gradient buffer with exactly the strides of the logits (also for strided views)."""
        if inplace:
            self.dlogits = self.logits
        else:
            self.dlogits = torch.empty_strided(self.logits.shape, self.logits.stride(), dtype=self.logits.dtype,
                                               device=self.logits.device)
        return self.dlogits

    def run(self, entry: str, reuse_args: bool = False) -> None:
        """Launch one entry point on the current stream.  reuse_args=True reuses the argument struct of
        the previous launch (same buffers and attributes; only exchange_epoch is refreshed)."""
        if reuse_args and getattr(self, "_args", None) is not None:
            a = self._args
            a.exchange_epoch = self.exchange_epoch
        else:
            a = self._args = self.args()
        with torch.cuda.device(self.per_token_logps.device):
            _lib.call(entry, a, _stream())


class _GrpoLoss(torch.autograd.Function):
    """torch counterpart of a jax.custom_vjp around the loss: forward saves (lse, grad_coef),
    backward receives the scalar cotangent of the loss and streams the logits once more."""

    @staticmethod
    def forward(ctx, logits, prob: TokenLossProblem, inplace_backward: bool, eager_grad: bool = False,
                entropy_grad: bool = False):
        ctx.eager = bool(eager_grad) and logits.requires_grad
        ctx.entropy_grad = bool(entropy_grad) and prob.token_entropy is not None
        if ctx.entropy_grad:
            if ctx.eager:
                raise ValueError("the entropy's cotangent is only known in backward(): eager_grad cannot serve it")
            if prob.cfg.temperature != 1.0:
                prob.lse_scaled = torch.empty_like(prob.lse)
        if ctx.eager:
            # forward and gradient in one kernel (cotangent 1); backward applies a late cotangent, if any
            prob.grad_scale = 1.0
            prob.alloc_dlogits(inplace_backward)
            prob.run("mllm_grpo_fwd_bwd")
        else:
            prob.run("mllm_grpo_fwd")
        ctx.prob = prob
        ctx.inplace = inplace_backward
        ctx.mark_non_differentiable(prob.per_token_logps)
        ent = prob.token_entropy if prob.token_entropy is not None else prob.per_token_logps.new_empty(0)
        if not ctx.entropy_grad:
            ctx.mark_non_differentiable(ent)
        return prob.loss.reshape(()), prob.per_token_logps, ent

    @staticmethod
    def backward(ctx, grad_loss, _g_lp, g_ent):
        prob: TokenLossProblem = ctx.prob
        if grad_loss is None:  # only the entropy output was used
            grad_loss = prob.loss.new_zeros(())
        prob.grad_scale_dev = grad_loss.to(torch.float32).reshape(1).contiguous()
        if ctx.eager:
            prob.run("mllm_grpo_scale_grad")  # returns at once on the device when the cotangent is 1
            return prob.dlogits, None, None, None, None
        prob.alloc_dlogits(ctx.inplace)
        if ctx.entropy_grad and g_ent is not None:
            # dlogits = grad_loss * grad_coef/Nv * (softmax - onehot) + g_ent * dH/dlogits in one sweep
            prob.entropy_cotangent = g_ent.to(torch.float32).contiguous()
            prob.run("mllm_grpo_bwd")
            prob.entropy_cotangent = None
        else:
            prob.run("mllm_grpo_bwd")
        return prob.dlogits, None, None, None, None


def _shifted_side(input_ids: torch.Tensor, labels: torch.Tensor):
    # chosen_ids = input_ids[:, 1:]; mask_loss = labels[:, 1:]   (train_modules/__init__.py:118-120)
    return input_ids[:, 1:], labels[:, 1:]


def grpo_token_loss(logits: torch.Tensor, input_ids: torch.Tensor, labels: torch.Tensor, advantages: torch.Tensor,
                    total_valid_token_count=None, old_per_token_logps: Optional[torch.Tensor] = None,
                    ref_per_token_logps: Optional[torch.Tensor] = None, *, temperature: float = 1.0,
                    epsilon_low: float = 0.2, epsilon_high: float = 0.3, beta: float = 0.0,
                    softcap: Optional[float] = None, compute_entropy: bool = True,
                    inplace_backward: bool = False, eager_grad: bool = False, entropy_grad: bool = False) -> dict:
    """GRPO token loss on the reference layout.

    entropy_grad=True makes the returned token_entropy differentiable with respect to the logits as well
    (the -entropy_coef * entropy term of plugins/training/ppo/module.py:140): backward() then adds
    cotangent * dH/dlogits inside the same streaming sweep.

    eager_grad=True computes dlogits together with the loss in one kernel (logits cross HBM once)
    and lets backward() merely hand them over; a cotangent other than 1 is applied by one extra
    in-place pass.  With inplace_backward=True that gradient overwrites the logits right away.

    logits [B, L, V] bf16, input_ids / labels [B, L], advantages [B] or [B, L-1],
    old/ref log-probs [B, L-1] or None.  Row i of a sequence is scored against
    token i+1; row L-1 is not scored and gets a zero gradient.
    Returns {"loss": f32[] (differentiable w.r.t. logits), "per_token_logps":
    f32[B, L-1], "token_entropy": f32[B, L-1]}.
    """
    cfg = LossConfig(temperature, epsilon_low, epsilon_high, beta, softcap, compute_entropy)
    ids, mask = _shifted_side(input_ids, labels)
    prob = TokenLossProblem(logits, ids, mask, advantages, total_valid_token_count, old_per_token_logps,
                            ref_per_token_logps, cfg, scored_rows=logits.shape[1] - 1)
    loss, lp, ent = _GrpoLoss.apply(logits, prob, inplace_backward, eager_grad, entropy_grad)
    return {"loss": loss, "per_token_logps": lp, "token_entropy": ent if compute_entropy else None}


def grpo_token_loss_flat(logits: torch.Tensor, token_ids: torch.Tensor, mask: torch.Tensor,
                         advantages: torch.Tensor, total_valid_token_count=None,
                         old_per_token_logps: Optional[torch.Tensor] = None,
                         ref_per_token_logps: Optional[torch.Tensor] = None, *, temperature: float = 1.0,
                         epsilon_low: float = 0.2, epsilon_high: float = 0.3, beta: float = 0.0,
                         softcap: Optional[float] = None, compute_entropy: bool = True,
                         inplace_backward: bool = False) -> dict:
    """Same loss with token ids already aligned to the rows: logits [B, T, V] (or [N, V]),
    token_ids / mask [B, T], advantages [B] or [B, T]; every row is scored."""
    if logits.dim() == 2:
        logits = logits.unsqueeze(0)
        token_ids, mask = token_ids.reshape(1, -1), mask.reshape(1, -1)
        if advantages.numel() == logits.shape[1]:
            advantages = advantages.reshape(1, -1)
    cfg = LossConfig(temperature, epsilon_low, epsilon_high, beta, softcap, compute_entropy)
    prob = TokenLossProblem(logits, token_ids, mask, advantages, total_valid_token_count, old_per_token_logps,
                            ref_per_token_logps, cfg, scored_rows=logits.shape[1])
    loss, lp, ent = _GrpoLoss.apply(logits, prob, inplace_backward)
    return {"loss": loss, "per_token_logps": lp, "token_entropy": ent if compute_entropy else None}


def grpo_value_and_grad(logits: torch.Tensor, token_ids: torch.Tensor, mask: torch.Tensor, advantages: torch.Tensor,
                        total_valid_token_count=None, old_per_token_logps: Optional[torch.Tensor] = None,
                        ref_per_token_logps: Optional[torch.Tensor] = None, *, shifted: bool = False,
                        cfg: Optional[LossConfig] = None, grad_scale: float = 1.0, inplace: bool = False,
                        dlogits: Optional[torch.Tensor] = None) -> dict:
    """Loss and dlogits in one call (the shape of jax.value_and_grad in training_step,
    plugins/training/update/train_step.py:24), through mllm_grpo_fwd_bwd.

    shifted=True takes the reference layout (token_ids = input_ids [B, L], mask = labels [B, L]);
    shifted=False takes aligned [B, T] arrays.  Returns loss, per_token_logps, token_entropy, dlogits.
    """
    cfg = cfg or LossConfig()
    if logits.dim() == 2:
        logits = logits.unsqueeze(0)
        token_ids, mask = token_ids.reshape(1, -1), mask.reshape(1, -1)
    if shifted:
        token_ids, mask = _shifted_side(token_ids, mask)
    T = logits.shape[1] - 1 if shifted else logits.shape[1]
    prob = TokenLossProblem(logits, token_ids, mask, advantages, total_valid_token_count, old_per_token_logps,
                            ref_per_token_logps, cfg, scored_rows=T)
    prob.grad_scale = float(grad_scale)
    if dlogits is not None:
        if dlogits.shape != logits.shape or dlogits.stride() != logits.stride() or dlogits.dtype != torch.bfloat16:
            raise ValueError("dlogits must match logits in shape, strides and dtype")
        prob.dlogits = dlogits
    else:
        prob.alloc_dlogits(inplace)
    prob.run("mllm_grpo_fwd_bwd")
    return {"loss": prob.loss.reshape(()), "per_token_logps": prob.per_token_logps,
            "token_entropy": prob.token_entropy, "dlogits": prob.dlogits, "problem": prob}


def token_logprobs(logits: torch.Tensor, token_ids: torch.Tensor, *, shifted: bool = False, temperature: float = 1.0,
                   softcap: Optional[float] = None, compute_entropy: bool = False) -> dict:
    """Forward-only log-probs of the chosen tokens (one read of the logits): the reference-model
    pass (train_modules/__init__.py:129-132) and the first PPO epoch's collection of
    old_per_token_logps (plugins/training/update/ppo.py:39-43)."""
    if logits.dim() == 2:
        logits = logits.unsqueeze(0)
        token_ids = token_ids.reshape(1, -1)
    if shifted:
        token_ids = token_ids[:, 1:]
    T = logits.shape[1] - 1 if shifted else logits.shape[1]
    cfg = LossConfig(temperature=temperature, softcap=softcap, compute_entropy=compute_entropy)
    prob = TokenLossProblem(logits, token_ids, None, None, 1.0, None, None, cfg, scored_rows=T)
    prob.run("mllm_grpo_logprobs")
    return {"per_token_logps": prob.per_token_logps, "token_entropy": prob.token_entropy, "lse": prob.lse.view(-1, T)}


def check_device_status(prob: TokenLossProblem) -> int:
    """Synchronises and returns the MLLM_GRPO_DEV_* bits the kernels raised (0 = clean)."""
    return int(prob.device_status.item())


def sft_cross_entropy(logits: torch.Tensor, input_ids: torch.Tensor, labels: torch.Tensor,
                      attention_mask: Optional[torch.Tensor] = None, *, label_ignore_id: int = -100,
                      inplace_backward: bool = False) -> dict:
    """Causal-LM cross-entropy of TrainSftModule (plugins/sft/jax/sft_module.py:29-45) on the same
    streaming kernels: logits [B, L, V] bf16, labels [B, L] with `label_ignore_id` on unsupervised
    positions.  valid = (labels[:, 1:] != ignore) & attention_mask[:, 1:]; loss = sum(-lp * valid) /
    max(valid.sum(), 1).  Returns {"loss" (differentiable w.r.t. logits), "token_count"}."""
    shift_labels = labels[:, 1:]
    valid = shift_labels != int(label_ignore_id)
    if attention_mask is not None:
        valid = valid & attention_mask[:, 1:].bool()
    safe = torch.where(valid, shift_labels, torch.zeros_like(shift_labels))
    count = valid.sum()
    cfg = LossConfig(compute_entropy=False, cross_entropy=True)
    prob = TokenLossProblem(logits, safe, valid.to(torch.float32), None, torch.clamp(count.to(torch.float32), min=1.0),
                            None, None, cfg, scored_rows=logits.shape[1] - 1)
    loss, _lp, _ent = _GrpoLoss.apply(logits, prob, inplace_backward)
    return {"loss": loss, "token_count": count.to(torch.int32)}
