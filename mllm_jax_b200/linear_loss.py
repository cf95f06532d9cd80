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
`lm_head_forward` goes one step further for the forward: the logits tile lives in tensor memory only
(hand-written tcgen05 / TMA kernel, mllm_lm_head_partials) and is reduced there to the per-row softmax
statistics, so forward-only passes (reference-model log-probs, the first PPO epoch's old log-probs, the
loss value itself) never write or read a logits tensor at all.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .ops import LossConfig, TokenLossProblem


def lm_head_forward(hidden: torch.Tensor, weight: torch.Tensor, token_ids: torch.Tensor,
                    mask: Optional[torch.Tensor] = None, advantages: Optional[torch.Tensor] = None,
                    total_valid_token_count=None, old_per_token_logps: Optional[torch.Tensor] = None,
                    ref_per_token_logps: Optional[torch.Tensor] = None, *, cfg: Optional[LossConfig] = None,
                    workspace: Optional[torch.Tensor] = None, vocab_start: int = 0,
                    vocab_total: Optional[int] = None, group=None, weight_layout: str = "vh") -> dict:
    """Forward of lm_head + loss without logits in HBM.

    tp-sharded head (lm_head kernel partitioned over "tp", MLLM_JAX/utils.py:245): pass this rank's weight rows
    [vocab_start, vocab_start + V) with vocab_total and the process group; token_ids stay GLOBAL ids.  The ranks'
    per-row partials (16 bytes per row and vocabulary range) are all-gathered and merged on every rank, so all
    outputs are replicated.

    hidden [B, T, H] (or [N, H]) bf16, weight [V, H] bf16 (logits = hidden @ weight.T, never stored) or, with
    weight_layout="hv", [H, V] (logits = hidden @ weight: a flax Dense kernel as stored, no transpose needed),
    token_ids [B, T] aligned with the rows.  With `advantages` given the whole forward runs (loss, residuals
    lse / grad_coef for a later backward); without, only per_token_logps, token_entropy and lse are meaningful
    (the reference-model pass, train_modules/__init__.py:129-132, and plugins/training/update/ppo.py:39-43).
    Two launches: the tensor-core kernel writes per-row partials for each vocabulary range, and
    mllm_grpo_combine merges them and runs the per-token epilogue.  H must be a multiple of 64.
    The logits are the f32 accumulators (not rounded to bf16 on the way)."""
    cfg = cfg or LossConfig()
    if hidden.dim() == 2:
        hidden = hidden.unsqueeze(0)
        token_ids = token_ids.reshape(1, -1)
    if not hidden.is_cuda:
        raise RuntimeError("lm_head_forward needs CUDA tensors: the kernels have no CPU path")
    if hidden.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise TypeError("hidden and weight must be bfloat16")
    B, T, H = hidden.shape
    if weight_layout not in ("vh", "hv"):
        raise ValueError("weight_layout must be 'vh' ([V, H]) or 'hv' ([H, V])")
    hv = weight_layout == "hv"
    V = weight.shape[1] if hv else weight.shape[0]
    if weight.shape[0 if hv else 1] != H or hidden.stride(2) != 1 or weight.stride(1) != 1 or \
            hidden.stride(0) != T * hidden.stride(1):
        raise ValueError(f"hidden {tuple(hidden.shape)} / weight {tuple(weight.shape)}: need [B, T, H] rows evenly "
                         "spaced and a [V, H] (or [H, V]) weight with unit stride along its last dimension")
    if cfg.temperature != 1.0 and cfg.compute_entropy:
        raise ValueError("the entropy of the folded forward needs temperature 1 (pass compute_entropy=False)")
    dev = hidden.device
    N = B * T
    lib = _lib.load()
    splits = int(lib.mllm_lm_head_splits(N, V))
    nbytes = int(lib.mllm_lm_head_partials_bytes(N, V))
    if workspace is None:
        workspace = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    elif workspace.numel() * workspace.element_size() < nbytes or workspace.data_ptr() % 16:
        raise ValueError(f"workspace must hold {nbytes} bytes at a 16-byte aligned address")
    forward_only = advantages is None
    if forward_only:
        advantages = torch.zeros(B, dtype=torch.float32, device=dev)
    # side arrays, outputs and residuals exactly as for materialised logits; no logits tensor is bound
    prob = TokenLossProblem.__new__(TokenLossProblem)
    v_all = int(vocab_total) if vocab_total is not None else int(vocab_start) + V
    TokenLossProblem._init_side(prob, B, T, T, v_all, dev, token_ids, mask, advantages, total_valid_token_count,
                                old_per_token_logps, ref_per_token_logps, cfg)
    a = _lib.LmHeadArgs()
    a.n_rows, a.vocab, a.hidden_dim = N, V, H
    a.hidden_stride, a.weight_stride = hidden.stride(1), weight.stride(0)
    a.vocab_start, a.vocab_total = int(vocab_start), int(vocab_total) if vocab_total is not None else int(vocab_start) + V
    a.softcap = float(cfg.softcap) if cfg.softcap else 0.0
    a.flags = (0 if cfg.compute_entropy else _lib.FLAG_SKIP_ENTROPY) | (_lib.LM_HEAD_FLAG_WEIGHT_HV if hv else 0)
    a.hidden, a.weight = hidden.data_ptr(), weight.data_ptr()
    a.chosen_ids, a.partials = prob.chosen_ids.data_ptr(), workspace.data_ptr()
    a.device_status = prob.device_status.data_ptr()
    with torch.cuda.device(dev):
        _lib.call("mllm_lm_head_partials", a, torch.cuda.current_stream().cuda_stream)
        parts, n_parts = workspace, splits
        if group is not None:
            import torch.distributed as dist

            k = dist.get_world_size(group)
            mine = workspace[:nbytes]
            parts = torch.empty(k * nbytes, dtype=torch.uint8, device=dev)
            dist.all_gather_into_tensor(parts, mine, group=group)  # [k, splits, N, 4] f32: rank-major vocabulary ranges
            n_parts = k * splits
        g = prob.args()
        g.gathered_partials, g.n_shards = parts.data_ptr(), n_parts
        _lib.call("mllm_grpo_combine", g, torch.cuda.current_stream().cuda_stream)
    prob._keepalive = (hidden, weight, workspace, parts)
    out = {"per_token_logps": prob.per_token_logps, "token_entropy": prob.token_entropy, "lse": prob.lse.view(B, T),
           "problem": prob, "splits": splits}
    if not forward_only:
        out["loss"] = prob.loss.reshape(())
    return out


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
