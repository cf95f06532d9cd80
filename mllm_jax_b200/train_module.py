"""Host-side mirror of the reference's loss modules, backed by the CUDA kernels.

`TrainGRPOModule` keeps the fields, the `inputs` dict and the returned dict of
MLLM_JAX/train_modules/__init__.py:84-192; `ppo_policy_terms` covers the policy
part of PPOActorCriticModule.__call__ (plugins/training/ppo/module.py:66-102) and
`ppo_value_loss` its value-loss tail (:104-140).
The model is any callable `model(input_ids=..., attention_mask=...) ->
(logits, cache)` producing bf16 CUDA logits; gradients flow into it through
torch autograd exactly where jax.value_and_grad differentiates the reference.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional

import torch

from .ops import grpo_token_loss


def per_sample_entropy_cuda(token_entropy: torch.Tensor, mask_loss: torch.Tensor):
    """`entropy` and `entropy_loss` [B] through the library's kernel (mllm_grpo_entropy_stats)."""
    import ctypes as C

    from . import _lib

    B, T = token_entropy.shape
    dev = token_entropy.device
    H = token_entropy.to(torch.float32).contiguous()
    m = mask_loss.to(device=dev, dtype=torch.float32).contiguous()
    out = torch.empty(2, B, dtype=torch.float32, device=dev)
    a = _lib.GrpoArgs()
    a.n_seqs, a.seq_rows, a.scored_rows, a.vocab, a.row_stride = B, T, T, 1, 1
    a.temperature = 1.0
    a.token_entropy, a.mask = H.data_ptr(), m.data_ptr()
    a.sample_entropy, a.sample_entropy_window = out[0].data_ptr(), out[1].data_ptr()
    with torch.cuda.device(dev):
        _lib.call("mllm_grpo_entropy_stats", a, torch.cuda.current_stream().cuda_stream)
    return out[0], out[1]


def per_sample_entropy(token_entropy: torch.Tensor, mask_loss: torch.Tensor):
    """`entropy` and `entropy_loss` of the reference's return dict.

    entropy[b]      = sum_t H_t m_t / sum_t m_t                       (train_modules/__init__.py:141-143)
    entropy_loss[b] = the same over tokens whose running count of valid tokens is in [4, 100]  (:148-157)
    A sample with no valid token divides 0 by 0, as the reference does.
    """
    m = mask_loss.to(token_entropy.dtype)
    avg = (token_entropy * m).sum(-1) / m.sum(-1)
    valid = mask_loss == 1
    cum = torch.cumsum(valid.to(torch.int32), dim=-1)
    window = valid & (cum >= 4) & (cum <= 100)
    w = window.to(token_entropy.dtype)
    avg_trunc = (token_entropy * w).sum(-1) / w.sum(-1)
    return avg, avg_trunc


@dataclass
class TrainGRPOModule:
    """Drop-in for the reference module: same fields (train_modules/__init__.py:85-94).

    `pad_token_id`, `num_pre_Q`, `max_lengths`, `entropy_threshold` are carried and unused, as in
    the reference.  With the default `use_kl=False` the loss is the reference's: the clipped surrogate
    alone, whatever `beta` and `ref_model` are (the reference computes the reference-policy log-probs but
    drops the KL term, :129-132, :176-180, :191, so they are not computed here at all).
    `use_kl=True` is an extension: beta * k3 KL against the reference policy is added to the loss and its
    gradient, with the log-probs taken from `inputs["ref_per_token_logps"]` or from `ref_model`.
    """

    model: Any
    pad_token_id: float = 0
    num_pre_Q: int = 8
    ref_model: Any = None
    beta: float = 0.04
    temperature: float = 1.0
    max_lengths: float = 2048
    epsilon_low: float = 0.2
    epsilon_high: float = 0.3
    entropy_threshold: float = 0.3
    softcap: Optional[float] = None
    eager_grad: bool = True  # loss and dlogits from one kernel; backward() applies a late cotangent if any
    use_kl: bool = False     # extension, off by default: add beta * k3 KL to the reference policy

    def __call__(self, inputs: Mapping[str, Any]) -> dict:
        from .ops import token_logprobs

        input_ids = inputs["input_ids"]
        attention_mask = inputs["attention_mask"]
        labels = inputs["labels"]
        logits, _ = self.model(input_ids=input_ids, attention_mask=attention_mask)

        ref_lp = inputs.get("ref_per_token_logps") if self.use_kl else None
        if self.use_kl and ref_lp is None and self.beta != 0 and self.ref_model is not None:
            with torch.no_grad():
                ref_logits, _ = self.ref_model(input_ids=input_ids, attention_mask=attention_mask)
            # reference-policy log-probs are not divided by the temperature (:130-132)
            ref_lp = token_logprobs(ref_logits, input_ids, shifted=True, softcap=self.softcap)["per_token_logps"]

        out = grpo_token_loss(
            logits, input_ids, labels, inputs["advantages"],
            total_valid_token_count=inputs.get("total_valid_token_count"),
            old_per_token_logps=inputs.get("old_per_token_logps"),
            ref_per_token_logps=ref_lp,
            temperature=self.temperature, epsilon_low=self.epsilon_low, epsilon_high=self.epsilon_high,
            beta=self.beta if ref_lp is not None else 0.0, softcap=self.softcap, eager_grad=self.eager_grad,
        )
        entropy, entropy_loss = per_sample_entropy_cuda(out["token_entropy"], labels[:, 1:])
        return {
            "loss": out["loss"],
            "per_token_logps": out["per_token_logps"].detach(),
            "entropy": entropy,
            "entropy_loss": entropy_loss,
        }


def ppo_policy_terms(logits: torch.Tensor, inputs: Mapping[str, Any], *, temperature: float = 1.0,
                     epsilon_low: float = 0.2, epsilon_high: float = 0.2, entropy_grad: bool = False) -> dict:
    """Policy loss, global entropy and log-probs as PPOActorCriticModule computes them
    (plugins/training/ppo/module.py:66-102): advantages [B], [B, 1] or [B, L-1]; entropy is one
    masked mean over the batch with a 1e-8 guard (:77).  The value-loss tail (:104-140) is
    `ppo_value_loss`."""
    labels = inputs["labels"]
    out = grpo_token_loss(
        logits, inputs["input_ids"], labels, inputs["advantages"],
        total_valid_token_count=inputs.get("total_valid_token_count"),
        old_per_token_logps=inputs.get("old_per_token_logps"),
        temperature=temperature, epsilon_low=epsilon_low, epsilon_high=epsilon_high, entropy_grad=entropy_grad,
    )
    m = labels[:, 1:].to(torch.float32)
    entropy = (out["token_entropy"] * m).sum() / (m.sum() + 1e-8)
    return {"policy_loss": out["loss"], "entropy": entropy, "per_token_logps": out["per_token_logps"].detach()}


def _to_positions(x: torch.Tensor, name: str, shape: tuple, dev) -> torch.Tensor:
    """[B], [B, 1] or [B, T] -> contiguous f32 [B, T] (the broadcasting of ppo/module.py:108-125)."""
    x = x.to(device=dev, dtype=torch.float32)
    if x.dim() == 1:
        x = x[:, None]
    if tuple(x.shape) != shape:
        if x.shape[1] == 1:
            x = x.expand(shape)
        else:
            raise ValueError(f"{name} shape {tuple(x.shape)} does not match value_pred {shape}")
    return x.contiguous()


def ppo_value_loss(values: torch.Tensor, inputs: Mapping[str, Any], *, value_clip_range: Optional[float] = 0.2,
                   value_coef: float = 0.5, grad_scale: float = 1.0) -> dict:
    """Value-loss tail of PPOActorCriticModule.__call__ (plugins/training/ppo/module.py:104-140)
    through mllm_ppo_value_loss.

    values [B, L] is the value head's output for every position; `inputs` holds labels [B, L],
    advantages, and optionally returns, old_values (or values), total_valid_token_count, with the
    reference's meanings and broadcasting.  Returns value_loss, value_pred_mean, return_mean
    (scalars) and dvalues [B, L] = grad_scale x value_coef x d value_loss / d values, which is the
    value head's share of the gradient of loss = policy_loss + value_coef x value_loss (:140)."""
    from . import _lib

    if values.dim() != 2 or values.shape[1] < 2:
        raise ValueError(f"values must be [B, L] with L >= 2, got {tuple(values.shape)}")
    if not values.is_cuda:
        raise RuntimeError("ppo_value_loss needs CUDA tensors: the kernels have no CPU path")
    dev = values.device
    B, L = values.shape
    T = L - 1
    shape = (B, T)
    v = values.detach().to(torch.float32).contiguous()
    mask = inputs["labels"][:, 1:].to(device=dev, dtype=torch.float32).contiguous()      # :67
    returns = inputs.get("returns")
    adv = None
    if returns is None:
        adv = _to_positions(inputs["advantages"], "advantages", shape, dev)              # :87-94, :107
    else:
        returns = _to_positions(returns, "returns", shape, dev)                          # :108-114
    old = inputs.get("old_values", inputs.get("values"))                                 # :116
    if old is not None:
        old = _to_positions(old, "old_values", shape, dev)                               # :119-125
    tv = inputs.get("total_valid_token_count")
    tv_dev = None
    if tv is None:
        tv_dev = mask.sum().reshape(1)                                                   # :101
    elif isinstance(tv, torch.Tensor):
        tv_dev = tv.to(device=dev, dtype=torch.float32).reshape(1)
    out = torch.empty(3, dtype=torch.float32, device=dev)
    dvalues = torch.empty(B, L, dtype=torch.float32, device=dev)
    lib = _lib.load()
    work = torch.empty(int(lib.mllm_ppo_value_workspace_bytes(B, L)) // 8, dtype=torch.float64, device=dev)
    a = _lib.PpoValueArgs()
    a.n_seqs, a.seq_rows, a.scored_rows = B, L, T
    a.clip_range = -1.0 if value_clip_range is None else float(value_clip_range)
    a.grad_scale = float(grad_scale) * float(value_coef)
    a.total_valid = float("nan") if tv_dev is not None else float(tv)
    a.adv_per_token = 1
    a.total_valid_dev = None if tv_dev is None else tv_dev.data_ptr()
    a.values = v.data_ptr()
    a.returns = None if returns is None else returns.data_ptr()
    a.advantages = None if adv is None else adv.data_ptr()
    a.old_values = None if old is None else old.data_ptr()
    a.mask = mask.data_ptr()
    a.dvalues, a.out, a.workspace = dvalues.data_ptr(), out.data_ptr(), work.data_ptr()
    with torch.cuda.device(dev):
        _lib.call("mllm_ppo_value_loss", a, torch.cuda.current_stream().cuda_stream)
    return {"value_loss": out[0], "value_pred_mean": out[1], "return_mean": out[2], "dvalues": dvalues}


class _ValueLoss(torch.autograd.Function):
    """value_loss as a differentiable function of the value head's output (the kernel has already
    produced d value_loss / d values in the forward, as in the eager form of the token loss)."""

    @staticmethod
    def forward(ctx, values, inputs, value_clip_range):
        out = ppo_value_loss(values, inputs, value_clip_range=value_clip_range, value_coef=1.0)
        ctx.save_for_backward(out["dvalues"])
        ctx.values_dtype = values.dtype
        ctx.mark_non_differentiable(out["value_pred_mean"], out["return_mean"])
        return out["value_loss"], out["value_pred_mean"], out["return_mean"]

    @staticmethod
    def backward(ctx, grad_loss, _grad_mean, _grad_return):
        (dvalues,) = ctx.saved_tensors
        return (grad_loss * dvalues).to(ctx.values_dtype), None, None


def ppo_actor_critic_terms(logits: torch.Tensor, values: torch.Tensor, inputs: Mapping[str, Any], *,
                           temperature: float = 1.0, epsilon_low: float = 0.2, epsilon_high: float = 0.2,
                           value_coef: float = 0.5, value_clip_range: Optional[float] = 0.2,
                           entropy_coef: float = 0.0) -> dict:
    """The return dict of PPOActorCriticModule.__call__ (plugins/training/ppo/module.py:142-150) from
    the lm_head's logits [B, L, V] and the value head's values [B, L]; `loss` is differentiable with
    respect to both.  A non-zero entropy_coef (:140; 0.0 in every configuration the reference ships) makes
    the entropy differentiable too: its cotangent per token rides along in the backward sweep of the logits."""
    want_entropy_grad = float(entropy_coef) != 0.0
    pol = ppo_policy_terms(logits, inputs, temperature=temperature, epsilon_low=epsilon_low,
                           epsilon_high=epsilon_high, entropy_grad=want_entropy_grad)
    value_loss, value_pred_mean, return_mean = _ValueLoss.apply(values, inputs, value_clip_range)
    loss = pol["policy_loss"] + float(value_coef) * value_loss                                     # :140
    if want_entropy_grad:
        loss = loss - float(entropy_coef) * pol["entropy"]
    return {"loss": loss, "policy_loss": pol["policy_loss"], "value_loss": value_loss, "entropy": pol["entropy"],
            "value_pred_mean": value_pred_mean, "return_mean": return_mean,
            "per_token_logps": pol["per_token_logps"]}
