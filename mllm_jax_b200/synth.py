"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configs.

They stand in for the reference's real workload (GSM8K rollouts of Qwen2.5 models, fetched at
plugins/training/runner/grpo_gsm8k.py:453): logits ~ N(0, sigma^2) rounded to bf16, token ids
uniform over the vocabulary, old / reference log-probs = exact log-probs + Gaussian noise,
group-normalised Bernoulli rewards as advantages, right-padded completion masks.  Only input
generation happens here (torch RNG and a chunked log-softmax); no loss math.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    n_seqs: int           # B
    seq_len: int          # T scored rows per sequence (token ids already aligned to rows)
    vocab: int            # V
    sigma: float = 2.0    # logits ~ N(0, sigma^2)
    reward_p: float = 0.5
    len_lo: int = 64
    len_hi: int = 256
    group: int = 8
    softcap: Optional[float] = None
    epsilon_low: float = 0.2
    epsilon_high: float = 0.2
    beta: float = 0.04
    old_noise: float = 0.05
    ref_noise: float = 0.1
    half_valid_runs: bool = False  # token sweep: 50% of tokens valid, in contiguous runs

    @property
    def n_tokens(self) -> int:
        return self.n_seqs * self.seq_len


CONFIGS = {
    # Qwen2.5-0.5B-shaped; small enough for the CPU restatement
    "cfg0": Workload("cfg0-qwen2.5-0.5b", 8, 256, 151936, 2.0, 0.5, 64, 256),
    # Qwen2.5-7B-shaped on one B200: 4 prompts x group 8
    "cfg1": Workload("cfg1-qwen2.5-7b", 32, 1024, 151936, 2.0, 0.5, 256, 1024),
    # Llama-3-8B-shaped, vocab-parallel
    "cfg2": Workload("cfg2-llama3-8b", 64, 2048, 128256, 2.0, 0.3, 512, 2048),
    # Gemma-2-shaped with final-logit soft-cap 30
    "cfg3": Workload("cfg3-gemma2-softcap", 16, 4096, 256000, 4.0, 0.5, 1024, 4096, softcap=30.0),
}


def sweep_workload(n_tokens: int) -> Workload:
    """Token-count sweep at V=151936: one 'sequence' per 1024 tokens, half the tokens valid."""
    seq = 1024 if n_tokens % 1024 == 0 else n_tokens
    return Workload(f"cfg4-sweep-{n_tokens}", n_tokens // seq, seq, 151936, half_valid_runs=True)


def scaled(w: Workload, **kw) -> Workload:
    return replace(w, **kw)


def group_advantages(rewards: torch.Tensor, group: int, eps: float = 1e-6) -> torch.Tensor:
    """(r - mean) / (std + eps) inside each group of `group` consecutive samples (population std)."""
    r = rewards.reshape(-1, group)
    mean = r.mean(dim=1, keepdim=True)
    std = r.std(dim=1, unbiased=False, keepdim=True)
    return ((r - mean) / (std + eps)).reshape(-1)


def exact_logprobs(logits: torch.Tensor, ids: torch.Tensor, softcap: Optional[float] = None,
                   chunk_rows: int = 512) -> torch.Tensor:
    """Chosen-token log-probs in f32 by a chunked log-softmax (input generation only)."""
    flat = logits.reshape(-1, logits.shape[-1])
    idf = ids.reshape(-1).long()
    out = torch.empty(flat.shape[0], dtype=torch.float32, device=logits.device)
    for s in range(0, flat.shape[0], chunk_rows):
        x = flat[s:s + chunk_rows].float()
        if softcap:
            x = torch.tanh(x / softcap) * softcap
        lsm = torch.log_softmax(x, dim=-1)
        out[s:s + chunk_rows] = lsm.gather(1, idf[s:s + chunk_rows, None])[:, 0]
    return out.reshape(ids.shape)


def make_inputs(w: Workload, seed: int = 0, device: str = "cpu", vocab_shard: Optional[tuple] = None,
                logits_chunk_rows: int = 2048) -> dict:
    """Build one batch.  Returns logits [B, T, V] bf16, token_ids / mask / old / ref [B, T],
    advantages [B], total_valid (float).  With vocab_shard=(rank, k) only columns
    [rank*V/k, (rank+1)*V/k) of the logits are materialised (same values as the full tensor
    would hold is NOT guaranteed; old/ref then derive from noise alone and are still seeded)."""
    dev = torch.device(device)
    g = torch.Generator(device=dev)
    g.manual_seed(1000003 * seed + 17)
    B, T, V = w.n_seqs, w.seq_len, w.vocab
    cols = V
    if vocab_shard is not None:
        rank, k = vocab_shard
        if V % k:
            raise ValueError(f"vocab {V} does not split over {k} shards")
        cols = V // k
        g.manual_seed(1000003 * seed + 17 + 7919 * (rank + 1))
    logits = torch.empty(B, T, cols, dtype=torch.bfloat16, device=dev)
    flat = logits.view(B * T, cols)
    for s in range(0, B * T, logits_chunk_rows):
        n = min(logits_chunk_rows, B * T - s)
        flat[s:s + n] = (torch.randn(n, cols, generator=g, device=dev, dtype=torch.float32) * w.sigma).to(torch.bfloat16)

    gs = torch.Generator(device="cpu")
    gs.manual_seed(7 * seed + 3)
    ids = torch.randint(0, V, (B, T), generator=gs, dtype=torch.int64).to(torch.int32)
    # advantages: groups of `group` completions, Bernoulli rewards; an all-equal group is re-drawn
    adv = torch.empty(B, dtype=torch.float32)
    for s in range(0, B, w.group):
        n = min(w.group, B - s)
        for _ in range(64):
            r = (torch.rand(n, generator=gs) < w.reward_p).float()
            if n == 1 or r.min() != r.max():
                break
        adv[s:s + n] = group_advantages(r, n) if n > 1 else r
    if w.half_valid_runs:
        # contiguous runs: the first half of every sequence-sized block is valid
        mask = (torch.arange(T)[None, :] < T // 2).expand(B, T).float().contiguous()
    else:
        lens = torch.randint(w.len_lo, w.len_hi + 1, (B,), generator=gs)
        mask = (torch.arange(T)[None, :] < lens[:, None]).float()
    noise_old = torch.randn(B, T, generator=gs) * w.old_noise
    noise_ref = torch.randn(B, T, generator=gs) * w.ref_noise
    ids, adv, mask = ids.to(dev), adv.to(dev), mask.to(dev)
    if vocab_shard is None:
        lp = exact_logprobs(logits, ids, w.softcap)
    else:
        lp = torch.full((B, T), -12.0, device=dev)  # placeholder centre; the shards never see full rows
    return {
        "logits": logits, "token_ids": ids, "mask": mask, "advantages": adv,
        "old_logps": lp + noise_old.to(dev), "ref_logps": lp + noise_ref.to(dev),
        "total_valid": float(mask.sum().item()), "exact_logps": lp,
    }
