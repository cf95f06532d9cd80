"""CPU oracle of the GRPO token loss -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may
import this module, and only as the checker or as the timed CPU baseline.  Nothing in
the mllm_jax_b200 package imports it.

PARITY UNPINNED: the reference's loss is jax.numpy code inside a Flax module; JAX is
not installable where this was written, the reference's tests never exercise the loss
and it ships no golden vectors for it.  The functions below restate the reference's
expressions one for one in torch-CPU (`reference_call`, `ppo_policy_call`) and,
independently, as closed-form NumPy float64 (`analytic_rows`); the two derivations are
checked against each other and against hand-derivable known answers in tests/.

Reference lines restated (paths inside demon2036/MLLM-JAX):
  MLLM_JAX/train_modules/__init__.py:118-126   shift, log_softmax, gather, / temperature
  MLLM_JAX/train_modules/__init__.py:136-157   token entropy, per-sample means, 4..100 window
  MLLM_JAX/train_modules/__init__.py:161-180   old log-probs, ratio, clip, surrogate, masked sum / Nv
  MLLM_JAX/train_modules/__init__.py:185-192   returned dict
  plugins/training/ppo/module.py:66-102        same policy math, [B, L-1] advantages, global entropy
  plugins/training/update/train_step.py:24     value_and_grad (torch autograd stands in for it)
  plugins/sft/jax/sft_module.py:36             the f32 upcast before log_softmax ("bf16 in, fp32 accumulate")
  deprecated/MLLM_JAX/language/gemma/transformer.py:337-339   final-logit soft-cap
Extension not present in the reference: beta * k3 KL against given reference log-probs,
k3 = e^(ref - lp) - (ref - lp) - 1, added to the per-token loss (identical to the
reference when beta == 0).
"""
from __future__ import annotations

from typing import Any, Mapping, Optional

import numpy as np
import torch


def _softcap(logits: torch.Tensor, cap: Optional[float]) -> torch.Tensor:
    # logits = tanh(logits / cap) * cap      (gemma/transformer.py:337-339)
    if cap is None or cap == 0:
        return logits
    return torch.tanh(logits / cap) * cap


def reference_call(logits: torch.Tensor, inputs: Mapping[str, Any], *, beta: float = 0.0, temperature: float = 1.0,
                   epsilon_low: float = 0.2, epsilon_high: float = 0.3, upcast: bool = True,
                   softcap: Optional[float] = None, dtype: torch.dtype = torch.float32) -> dict:
    """TrainGRPOModule.__call__ from the logits on (train_modules/__init__.py:118-192).

    `logits` [B, L, V] plays the role of `self.model(...)`'s output (:105).  upcast=True casts
    them to `dtype` first (the gate: bf16 in, fp32 accumulate); upcast=False keeps the
    reference's as-written bf16 arithmetic (reported, not gated).
    inputs: input_ids [B, L], labels [B, L], advantages [B]; optional old_per_token_logps
    [B, L-1], total_valid_token_count, ref_per_token_logps [B, L-1] (KL extension).
    """
    input_ids = inputs["input_ids"].long()
    labels = inputs["labels"]
    if upcast:
        logits = logits.to(dtype)
    work = logits.dtype
    logits = _softcap(logits, softcap)

    chosen_ids = input_ids[:, 1:]                                             # :118
    mask_loss = labels[:, 1:].to(work)                                        # :120
    per_token_logps = torch.gather(                                           # :124-126
        torch.log_softmax(logits[..., :-1, :], dim=-1), -1, chosen_ids[..., None]
    )[..., 0] / temperature

    probs = torch.softmax(logits[..., :-1, :] / temperature, dim=-1)          # :136
    token_entropy = -torch.sum(probs * torch.log(probs + 1e-9), dim=-1)       # :138

    masked_token_entropy = token_entropy * mask_loss                          # :141
    sum_entropy_per_sample = masked_token_entropy.sum(dim=-1)                 # :142
    avg_entropy_per_sample = sum_entropy_per_sample / mask_loss.sum(dim=-1)   # :143

    valid_mask_for_metric = labels[:, 1:] == 1                                # :148
    cum_valid = torch.cumsum(valid_mask_for_metric.to(torch.int64), dim=-1)   # :149
    entropy_calc_mask = valid_mask_for_metric & (cum_valid >= 4) & (cum_valid <= 100)  # :150-153
    masked_trunc = token_entropy * entropy_calc_mask.to(work)                 # :155
    avg_entropy_per_sample_truncated = masked_trunc.sum(dim=-1) / entropy_calc_mask.sum(dim=-1)  # :156-157

    if "old_per_token_logps" in inputs and inputs["old_per_token_logps"] is not None:   # :161-165
        old_per_token_logps = inputs["old_per_token_logps"].to(work)
    else:
        old_per_token_logps = per_token_logps.detach()

    ratio = torch.exp(per_token_logps - old_per_token_logps)                  # :169
    clipped_ratio = torch.clamp(ratio, 1.0 - epsilon_low, 1.0 + epsilon_high)  # :170

    adv = inputs["advantages"].to(work)
    adv_broadcast = adv[..., None] if adv.dim() == 1 else adv                 # :173 (and ppo/module.py:87-94)
    per_token_loss1 = ratio * adv_broadcast                                   # :174
    per_token_loss2 = clipped_ratio * adv_broadcast                           # :175
    per_token_ppo_loss = torch.minimum(per_token_loss1, per_token_loss2)      # :176
    per_token_loss = -per_token_ppo_loss                                      # :178

    ref = inputs.get("ref_per_token_logps")
    per_token_kl = None
    if ref is not None and beta != 0:
        d = ref.to(work) - per_token_logps
        per_token_kl = torch.exp(d) - d - 1.0                                 # k3 estimator (extension)
        per_token_loss = per_token_loss + beta * per_token_kl

    tv = inputs.get("total_valid_token_count")
    total_valid_token_count = mask_loss.sum() if tv is None else tv           # :179
    loss = (per_token_loss * mask_loss).sum() / total_valid_token_count       # :180

    return {                                                                  # :185-192
        "loss": loss,
        "per_token_logps": per_token_logps.detach(),
        "entropy": avg_entropy_per_sample.detach(),
        "entropy_loss": avg_entropy_per_sample_truncated.detach(),
        "token_entropy": token_entropy.detach(),
        "per_token_kl": None if per_token_kl is None else per_token_kl.detach(),
    }


def reference_value_and_grad(logits_bf16: torch.Tensor, inputs: Mapping[str, Any], *, dtype=torch.float32,
                             **attrs) -> dict:
    """jax.value_and_grad of the loss w.r.t. the logits (update/train_step.py:24), by torch autograd.
    Returns the dict of reference_call plus "dlogits" [B, L, V] in `dtype` (row L-1 is zero)."""
    x = logits_bf16.detach().to(dtype).requires_grad_(True)
    out = reference_call(x, inputs, upcast=True, dtype=dtype, **attrs)
    out["loss"].backward()
    out["dlogits"] = x.grad
    out["loss"] = out["loss"].detach()
    return out


def ppo_policy_call(logits: torch.Tensor, inputs: Mapping[str, Any], *, temperature: float = 1.0,
                    epsilon_low: float = 0.2, epsilon_high: float = 0.2, dtype=torch.float32,
                    detach_entropy: bool = True) -> dict:
    """Policy part of PPOActorCriticModule.__call__ (plugins/training/ppo/module.py:66-102).
    detach_entropy=False keeps the entropy attached to the logits, for the -entropy_coef * entropy term of :140."""
    logits = logits.to(dtype)
    input_ids = inputs["input_ids"].long()
    chosen_ids = input_ids[:, 1:]                                             # :66
    mask_loss = inputs["labels"][:, 1:].to(dtype)                             # :67
    per_token_logps = torch.gather(torch.log_softmax(logits[..., :-1, :], dim=-1), -1,
                                   chosen_ids[..., None])[..., 0] / float(temperature)          # :69-73
    probs = torch.softmax(logits[..., :-1, :] / float(temperature), dim=-1)   # :75
    token_entropy = -torch.sum(probs * torch.log(probs + 1e-9), dim=-1)       # :76
    entropy = (token_entropy * mask_loss).sum() / (mask_loss.sum() + 1e-8)    # :77
    old = inputs.get("old_per_token_logps")
    old = per_token_logps.detach() if old is None else old.to(dtype)          # :79-82
    ratio = torch.exp(per_token_logps - old)                                  # :84
    clipped_ratio = torch.clamp(ratio, 1.0 - float(epsilon_low), 1.0 + float(epsilon_high))     # :85
    advantages = inputs["advantages"].to(dtype)                               # :87-94
    if advantages.dim() == 1:
        advantages = advantages[:, None]
    if advantages.shape != per_token_logps.shape:
        if advantages.shape[1] == 1:
            advantages = advantages.expand(per_token_logps.shape)
        else:
            raise ValueError(f"advantages shape {tuple(advantages.shape)} does not match per_token_logps "
                             f"{tuple(per_token_logps.shape)}")
    per_token_ppo_loss = torch.minimum(ratio * advantages, clipped_ratio * advantages)          # :96-98
    per_token_loss = -per_token_ppo_loss                                      # :99
    tv = inputs.get("total_valid_token_count")
    total_valid_token_count = mask_loss.sum() if tv is None else tv           # :101
    policy_loss = (per_token_loss * mask_loss).sum() / total_valid_token_count  # :102
    return {"policy_loss": policy_loss, "entropy": entropy.detach() if detach_entropy else entropy,
            "per_token_logps": per_token_logps.detach()}


def ppo_value_call(values: torch.Tensor, inputs: Mapping[str, Any], *, value_clip_range: Optional[float] = 0.2,
                   dtype=torch.float32) -> dict:
    """Value-loss tail of PPOActorCriticModule.__call__ (plugins/training/ppo/module.py:104-148).
    `values` [B, L] may require grad; autograd then gives d value_loss / d values."""
    mask_loss = inputs["labels"][:, 1:].to(dtype)                             # :67
    value_pred = values[:, :-1]                                               # :104
    shape = value_pred.shape

    def positions(x, name):
        if x.dim() == 1:
            x = x[:, None]
        if x.shape != shape:
            if x.shape[1] == 1:
                x = x.expand(shape)
            else:
                raise ValueError(f"{name} shape {tuple(x.shape)} does not match value_pred {tuple(shape)}")
        return x

    returns = inputs.get("returns")                                           # :105
    if returns is None:
        returns = positions(inputs["advantages"].to(dtype), "advantages") + value_pred          # :106-107
    returns = positions(returns, "returns")                                   # :108-114
    old_values = inputs.get("old_values", inputs.get("values"))               # :116
    if old_values is None:
        old_values = value_pred.detach()                                      # :117-118
    old_values = positions(old_values, "old_values")                          # :119-125
    value_pred, returns, old_values = value_pred.to(dtype), returns.to(dtype), old_values.to(dtype)  # :127-129
    if value_clip_range is not None:
        c = float(value_clip_range)
        value_clipped = old_values + torch.clamp(value_pred - old_values, -c, c)                # :133
        value_loss = torch.maximum((value_pred - returns) ** 2, (value_clipped - returns) ** 2)  # :134
    else:
        value_loss = (value_pred - returns) ** 2                              # :136
    tv = inputs.get("total_valid_token_count")
    total_valid_token_count = mask_loss.sum() if tv is None else tv           # :101
    value_loss = (value_loss * mask_loss).sum() / total_valid_token_count     # :138
    return {"value_loss": value_loss, "value_pred_mean": value_pred.mean().detach(),            # :147
            "return_mean": returns.mean().detach()}                           # :148


def sft_call(logits: torch.Tensor, inputs: Mapping[str, Any], *, label_ignore_id: int = -100,
             dtype=torch.float32) -> dict:
    """TrainSftModule.__call__ from the logits on (plugins/sft/jax/sft_module.py:29-45)."""
    labels = inputs["labels"].long()
    attention_mask = inputs["attention_mask"]
    shift_logits = logits[:, :-1, :]                                          # :29
    shift_labels = labels[:, 1:]                                              # :30
    shift_attention = attention_mask[:, 1:]                                   # :31
    valid = (shift_labels != int(label_ignore_id)) & shift_attention.bool()   # :33
    safe_labels = torch.where(valid, shift_labels, torch.zeros_like(shift_labels))  # :34
    log_probs = torch.log_softmax(shift_logits.to(dtype), dim=-1)             # :36
    chosen = torch.gather(log_probs, -1, safe_labels[..., None])[..., 0]      # :37
    per_token_loss = -chosen                                                  # :38
    mask_f = valid.to(dtype)
    loss = (per_token_loss * mask_f).sum() / torch.clamp(mask_f.sum(), min=1.0)  # _masked_mean, :10-13
    return {"loss": loss, "token_count": valid.to(torch.int32).sum()}         # :41-45


def lm_head_logits(hidden: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """logits = self.lm_head(hidden_states) (MLLM_JAX/language/qwen2/modular_qwen2.py:182; a bias-free Dense) in
    float64 from the exact bf16 operands: hidden [..., H] x weight [V, H]^T.  The checker of the folded
    lm_head + loss kernels, whose logits are f32 accumulators that are never rounded to bf16."""
    return hidden.double() @ weight.double().t()


def analytic_rows(x: np.ndarray, chosen: np.ndarray, mask: np.ndarray, adv: np.ndarray,
                  old: Optional[np.ndarray], ref: Optional[np.ndarray], total_valid: float, *, beta: float = 0.0,
                  temperature: float = 1.0, epsilon_low: float = 0.2, epsilon_high: float = 0.3,
                  softcap: Optional[float] = None, grad_scale: float = 1.0, want_grad: bool = True) -> dict:
    """Closed-form float64 statement of the same operator on a set of rows, derived by hand
    (no autograd): x [n, V] logits (already exact bf16 values), chosen/mask/adv/old/ref [n].

      y = x or cap*tanh(x/cap);  lse = logsumexp(y);  lp = (y_c - lse)/temp
      ratio = e^(lp-old); ppo = min(ratio*A, clip(ratio)*A); kl = e^(ref-lp) - (ref-lp) - 1
      term = mask*(-ppo + beta*kl);   loss contribution = term/total_valid
      w = A*ratio*sel - beta*(1 - e^(ref-lp)), sel = 1 iff the unclipped branch is the active min
      dx_j = grad_scale*mask*w/(total_valid*temp) * (softmax(y)_j - [j == c]) * dy/dx
    """
    x = np.asarray(x, dtype=np.float64)
    n, V = x.shape
    if softcap:
        th = np.tanh(x / softcap)
        y = softcap * th
        dydx = 1.0 - th * th
    else:
        y, dydx = x, None
    M = y.max(axis=1, keepdims=True)
    e = np.exp(y - M)
    S = e.sum(axis=1, keepdims=True)
    lse = (M + np.log(S))[:, 0]
    rows = np.arange(n)
    yc = y[rows, chosen]
    lp = (yc - lse) / temperature
    # entropy of softmax(y/temp): exact, and with the reference's +1e-9 guard
    yt = y / temperature
    Mt = yt.max(axis=1, keepdims=True)
    et = np.exp(yt - Mt)
    pt = et / et.sum(axis=1, keepdims=True)
    with np.errstate(divide="ignore", invalid="ignore"):
        H_exact = -np.where(pt > 0, pt * np.log(pt), 0.0).sum(axis=1)
    H_guard = -(pt * np.log(pt + 1e-9)).sum(axis=1)
    oldv = lp if old is None else np.asarray(old, dtype=np.float64)
    ratio = np.exp(lp - oldv)
    lo, hi = 1.0 - epsilon_low, 1.0 + epsilon_high
    clipped = np.clip(ratio, lo, hi)
    A = np.asarray(adv, dtype=np.float64)
    m = np.asarray(mask, dtype=np.float64)
    ppo = np.minimum(ratio * A, clipped * A)
    sel = np.where(ratio > hi, A < 0, np.where(ratio < lo, A > 0, True)).astype(np.float64)
    term = -ppo
    w = A * ratio * sel
    if ref is not None and beta != 0:
        d = np.asarray(ref, dtype=np.float64) - lp
        term = term + beta * (np.exp(d) - d - 1.0)
        w = w - beta * (1.0 - np.exp(d))
    out = {"lp": lp, "lse": lse, "entropy_exact": H_exact, "entropy_guard": H_guard, "loss_terms": m * term,
           "loss_part": float((m * term).sum() / total_valid), "grad_coef": m * w / temperature}
    if want_grad:
        g = grad_scale * m * w / (total_valid * temperature)
        p = e / S
        p[rows, chosen] -= 1.0
        dx = g[:, None] * p
        if dydx is not None:
            dx = dx * dydx
        out["dlogits"] = dx
    return out


def shard_partials(x: np.ndarray, chosen: np.ndarray, vocab_start: int, softcap: Optional[float] = None,
                   temperature: Optional[float] = None) -> np.ndarray:
    """(max, sumexp, sum e*y, chosen-or-0) of a column shard x [n, Vs] in float64: what one
    vocabulary shard contributes before the cross-shard max / sum (the collectives XLA inserts
    for log_softmax over tp-sharded logits, MLLM_JAX/utils.py:245).  With a temperature other than 1 the record
    has six entries: (max, sumexp, 0, chosen-or-0, sum e2, sum e2*y) with e2 = e^((y - max)/temperature), the sums
    the entropy of softmax(y / temperature) needs (train_modules/__init__.py:136-138)."""
    x = np.asarray(x, dtype=np.float64)
    y = softcap * np.tanh(x / softcap) if softcap else x
    M = y.max(axis=1)
    e = np.exp(y - M[:, None])
    loc = np.asarray(chosen) - vocab_start
    inside = (loc >= 0) & (loc < x.shape[1])
    yc = np.where(inside, y[np.arange(x.shape[0]), np.clip(loc, 0, x.shape[1] - 1)], 0.0)
    if temperature is not None and temperature != 1.0:
        e2 = np.exp((y - M[:, None]) / temperature)
        return np.stack([M, e.sum(axis=1), np.zeros_like(M), yc, e2.sum(axis=1), (e2 * y).sum(axis=1)], axis=1)
    return np.stack([M, e.sum(axis=1), (e * y).sum(axis=1), yc], axis=1)


def time_reference_value_and_grad(logits_bf16: torch.Tensor, inputs: Mapping[str, Any], *, repeats: int = 1,
                                  threads: Optional[int] = None, **attrs) -> float:
    """Seconds per fwd+bwd of the torch-CPU restatement (the CPU baseline); best of `repeats`."""
    import time

    if threads:
        torch.set_num_threads(int(threads))
    best = float("inf")
    for _ in range(max(1, repeats)):
        t0 = time.perf_counter()
        reference_value_and_grad(logits_bf16, inputs, **attrs)
        best = min(best, time.perf_counter() - t0)
    return best
