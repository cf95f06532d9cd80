"""PPO-epoch driver around the loss: the host loop of plugins/training/update/ppo.py:6-46.

Epoch 0 runs every micro-batch with `old_per_token_logps` absent (ratio == 1, gradient still
flows) and keeps the `per_token_logps` each step returns; their concatenation becomes
`old_per_token_logps` for the later epochs.  `train_step(state, batch) -> (state, metrics)` is the
caller's step (model forward, `TrainGRPOModule`, backward, optimizer); `slice_data(x, n, i)` cuts
micro-batch i of n out of one array of the global batch.
"""
from __future__ import annotations

from typing import Any, Callable, Mapping, Optional

import torch


def slice_micro_batch(x: Any, n_micro: int, index: int) -> Any:
    """Default `slice_data`: rows [index*B/n, (index+1)*B/n) of a tensor; scalars pass through
    (the jitted dynamic_slice at plugins/training/runner/grpo_gsm8k.py:185-190)."""
    if not isinstance(x, torch.Tensor) or x.dim() == 0:
        return x
    per = x.shape[0] // int(n_micro)
    return x[index * per:(index + 1) * per]


def ppo_update(*, state: Any, datas: Mapping[str, Any], total_valid_token_count: Any,
               train_step: Callable[[Any, Any], tuple], slice_data: Callable[[Any, int, int], Any] = slice_micro_batch,
               grad_accum_steps: int, ppo_steps: int) -> tuple:
    """Returns (state, datas with old_per_token_logps filled in, metrics of the last step, entropy of
    the last step of epoch 0), like the reference."""
    batch = dict(datas)
    last: Mapping[str, Any] = {}
    entropy: Optional[Any] = None
    collected = []
    for epoch in range(int(ppo_steps)):
        for micro in range(int(grad_accum_steps)):
            local = {k: slice_data(v, int(grad_accum_steps), micro) for k, v in batch.items()}
            local["total_valid_token_count"] = total_valid_token_count
            state, last = train_step(state, local)
            if epoch == 0:
                collected.append(last["per_token_logps"])
        if epoch == 0:
            batch["old_per_token_logps"] = torch.cat(collected, dim=0)
            entropy = last.get("entropy")
    return state, batch, last, entropy
