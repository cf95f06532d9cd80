"""lm_head projection and GRPO loss chunk by chunk, without ever holding the [N, V] logits.

The reference materialises logits = lm_head(hidden) for the whole batch
(MLLM_JAX/language/qwen2/modular_qwen2.py:182) and keeps them for the backward sweep; at
32768 x 151936 that is 10 GB of logits plus 10 GB of dlogits.  Here whole sequences are processed
in chunks: one library GEMM produces the chunk's bf16 logits, the fused loss kernel overwrites them
in place with dlogits (mllm_grpo_fwd_bwd, logits read from HBM once), and two more library GEMMs
fold the chunk into dhidden and dweight.  Peak extra memory is one chunk of logits.

The GEMMs are library calls (cuBLAS through torch: bf16 operands, f32 accumulation, the weight
gradient summed over chunks in f32); the loss and its gradient are this package's kernels.  On one
B200 at 32768 x 3584 -> 151936 with 8192-row chunks a step takes 81.6 ms with the weight gradient
(three GEMMs at 1.31 PFLOP/s, the loss kernels hidden behind them) and 55 ms without.
A single kernel that keeps the logits tile in tensor memory and never writes it at all is the next
step beyond this file.
"""
from __future__ import annotations

from typing import Optional

import torch

from .ops import LossConfig, TokenLossProblem


def linear_grpo_value_and_grad(hidden: torch.Tensor, weight: torch.Tensor, token_ids: torch.Tensor,
                               mask: torch.Tensor, advantages: torch.Tensor, total_valid_token_count,
                               old_per_token_logps: Optional[torch.Tensor] = None,
                               ref_per_token_logps: Optional[torch.Tensor] = None, *,
                               cfg: Optional[LossConfig] = None, chunk_rows: int = 8192,
                               want_weight_grad: bool = True) -> dict:
    """hidden [B, T, H] bf16, weight [V, H] bf16 (logits = hidden @ weight.T), token_ids / mask /
    old / ref [B, T] aligned with the rows, advantages [B] or [B, T], total_valid_token_count the
    GLOBAL normaliser (number or scalar tensor; required, because a chunk cannot know it).

    Returns loss, per_token_logps [B, T], token_entropy [B, T], dhidden [B, T, H] bf16 and
    dweight [V, H] f32 (None if want_weight_grad is False)."""
    if hidden.dim() != 3 or weight.dim() != 2 or hidden.shape[2] != weight.shape[1]:
        raise ValueError(f"hidden {tuple(hidden.shape)} and weight {tuple(weight.shape)} do not match")
    if hidden.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise TypeError("hidden and weight must be bfloat16")
    if total_valid_token_count is None:
        raise ValueError("total_valid_token_count is required: it is global over all chunks")
    cfg = cfg or LossConfig()
    B, T, H = hidden.shape
    V = weight.shape[0]
    dev = hidden.device
    seqs = max(1, min(B, int(chunk_rows) // max(T, 1)))
    lp = torch.empty(B, T, dtype=torch.float32, device=dev)
    ent = torch.empty(B, T, dtype=torch.float32, device=dev) if cfg.compute_entropy else None
    dhidden = torch.empty_like(hidden)
    dweight = torch.zeros(V, H, dtype=torch.float32, device=dev) if want_weight_grad else None
    loss = torch.zeros((), dtype=torch.float32, device=dev)
    logits_buf = torch.empty(seqs, T, V, dtype=torch.bfloat16, device=dev)
    wt = weight.t()
    status = 0
    for s in range(0, B, seqs):
        e = min(B, s + seqs)
        n = e - s
        logits = logits_buf[:n]
        torch.matmul(hidden[s:e], wt, out=logits)  # library GEMM: the chunk's bf16 logits
        sl = slice(s, e)
        prob = TokenLossProblem(logits, token_ids[sl], mask[sl], advantages[sl], total_valid_token_count,
                                None if old_per_token_logps is None else old_per_token_logps[sl],
                                None if ref_per_token_logps is None else ref_per_token_logps[sl], cfg, scored_rows=T)
        prob.alloc_dlogits(inplace=True)  # dlogits overwrite the chunk's logits
        prob.run("mllm_grpo_fwd_bwd")
        loss += prob.loss[0]  # chunks are added in order: deterministic
        lp[sl] = prob.per_token_logps
        if ent is not None:
            ent[sl] = prob.token_entropy
        d = prob.dlogits.view(n * T, V)
        torch.matmul(d, weight, out=dhidden[sl].view(n * T, H))
        if dweight is not None:
            # bf16 operands on the tensor cores, f32 accumulation straight into the f32 sum over chunks
            torch.addmm(dweight, d.t(), hidden[sl].reshape(n * T, H), out_dtype=torch.float32, out=dweight)
        status = prob.device_status if status == 0 else status | prob.device_status
    return {"loss": loss, "per_token_logps": lp, "token_entropy": ent, "dhidden": dhidden, "dweight": dweight,
            "device_status": status}
