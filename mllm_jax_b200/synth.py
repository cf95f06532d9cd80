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
    return Workload(f"cfg4-sweep-{n_tokens}", n_tokens // seq, seq, 151936, half_valid_runs=True,
                    group=min(8, n_tokens // seq))


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


BLOCK_ROWS = 1024  # logits are generated in blocks of this many rows, each block from its own seed


def parse_workload(name: str) -> Workload:
    """cfg0..cfg3, or cfg4-<tokens> for one point of the token-count sweep (e.g. cfg4-65536, cfg4-1048576)."""
    if name in CONFIGS:
        return CONFIGS[name]
    if name.startswith("cfg4-"):
        return sweep_workload(int(name[5:]))
    raise ValueError(f"unknown workload {name!r}: expected one of {sorted(CONFIGS)} or cfg4-<tokens>")


def side_arrays(w: Workload, seed: int = 0):
    """Per-token side inputs of the whole batch (small, CPU, one generator): token ids [B, T] i32, advantages [B]
    (groups of `group` completions, Bernoulli rewards, group-normalised; an all-equal group is re-drawn), mask
    [B, T], and the noise added to the exact log-probs for old / ref."""
    B, T, V = w.n_seqs, w.seq_len, w.vocab
    gs = torch.Generator(device="cpu")
    gs.manual_seed(7 * seed + 3)
    ids = torch.randint(0, V, (B, T), generator=gs, dtype=torch.int64).to(torch.int32)
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
    return ids, adv, mask, noise_old, noise_ref


def make_inputs(w: Workload, seed: int = 0, device: str = "cpu", vocab_shard: Optional[tuple] = None,
                row_shard: Optional[tuple] = None, want_logits: bool = True) -> dict:
    """Build one batch.  Returns logits [B, T, V] bf16, token_ids / mask / old / ref [B, T],
    advantages [B], total_valid (float, over the WHOLE batch).

    The logits are generated block by block (BLOCK_ROWS rows of the flattened [B*T, V] tensor), block i
    from a generator seeded by (seed, i), always at full width.  So every shard is a slice of one and the
    same tensor, whatever the number of ranks:
      vocab_shard=(rank, k): only columns [rank*V/k, (rank+1)*V/k) are kept (side arrays whole);
      row_shard=(rank, k):   only sequences [rank*B/k, (rank+1)*B/k) are generated and returned
                             (side arrays sliced to them; total_valid stays global).
    old / ref log-probs are the exact log-probs of the full rows plus seeded noise in either case.
    (Blocks are bit-identical across shardings on one kind of device; CPU and CUDA generators differ.)"""
    dev = torch.device(device)
    B, T, V = w.n_seqs, w.seq_len, w.vocab
    c0, c1 = 0, V
    if vocab_shard is not None:
        rank, k = vocab_shard
        if V % k:
            raise ValueError(f"vocab {V} does not split over {k} shards")
        c0, c1 = rank * (V // k), (rank + 1) * (V // k)
    b0, b1 = 0, B
    if row_shard is not None:
        rank, k = row_shard
        if B % k:
            raise ValueError(f"{B} sequences do not split over {k} ranks")
        b0, b1 = rank * (B // k), (rank + 1) * (B // k)

    ids, adv, mask, noise_old, noise_ref = side_arrays(w, seed)
    total_valid = float(mask.sum().item())

    r0, r1 = b0 * T, b1 * T  # rows of the flattened tensor this call materialises
    logits = torch.empty(b1 - b0, T, c1 - c0, dtype=torch.bfloat16, device=dev) if want_logits else None
    flat = logits.view(r1 - r0, c1 - c0) if want_logits else None
    lp = torch.empty(r1 - r0, dtype=torch.float32, device=dev)
    ids_dev = ids.to(dev).reshape(-1)
    g = torch.Generator(device=dev)
    for blk in range(r0 // BLOCK_ROWS, (r1 + BLOCK_ROWS - 1) // BLOCK_ROWS):
        s, e = blk * BLOCK_ROWS, min((blk + 1) * BLOCK_ROWS, B * T)
        g.manual_seed(1000003 * seed + 17 + 7919 * blk)
        x = (torch.randn(e - s, V, generator=g, device=dev, dtype=torch.float32) * w.sigma).to(torch.bfloat16)
        lo, hi = max(s, r0), min(e, r1)
        x = x[lo - s:hi - s]
        lp[lo - r0:hi - r0] = exact_logprobs(x, ids_dev[lo:hi], w.softcap)
        if want_logits:
            flat[lo - r0:hi - r0] = x[:, c0:c1]
        del x

    sl = slice(b0, b1)
    lp = lp.view(b1 - b0, T)
    return {
        "logits": logits, "token_ids": ids[sl].to(dev), "mask": mask[sl].to(dev), "advantages": adv[sl].to(dev),
        "old_logps": lp + noise_old[sl].to(dev), "ref_logps": lp + noise_ref[sl].to(dev),
        "total_valid": total_valid, "exact_logps": lp,
    }
