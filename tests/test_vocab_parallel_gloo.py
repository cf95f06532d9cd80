"""Host logic of the vocabulary-parallel path on CPU: two gloo ranks exchange per-token partials
(produced here by the oracle, since the kernels need a GPU) and every rank merges them to the
unsharded answer.  Also the shard arithmetic and its error cases."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mllm_jax_b200.vocab_parallel import exchange_partials, shard_bounds
from oracle import grpo_oracle as O
from tests.util import make_case


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, L, V = 2, 7, 64 * world
        logits, inputs = make_case(B, L, V, seed=77, old="noisy")
        N = B * (L - 1)
        x = logits[:, :-1].double().numpy().reshape(N, V)
        c = inputs["input_ids"][:, 1:].long().numpy().reshape(-1)
        lo, hi = shard_bounds(V, rank, world)
        mine = torch.from_numpy(O.shard_partials(x[:, lo:hi], c, lo)).float()
        gathered = exchange_partials(mine)
        assert gathered.shape == (world, N, 4)
        assert torch.equal(gathered[rank], mine)
        P = gathered.double().numpy()
        M = P[:, :, 0].max(axis=0)
        S = (P[:, :, 1] * np.exp(P[:, :, 0] - M)).sum(axis=0)
        lp = P[:, :, 3].sum(axis=0) - (M + np.log(S))
        ref = O.reference_call(logits, inputs)["per_token_logps"].numpy().reshape(-1)
        ret[rank] = float(np.abs(lp - ref).max())
        # token-parallel: the global loss is the plain sum of the ranks' losses
        from mllm_jax_b200.vocab_parallel import TokenParallelLoss
        total = TokenParallelLoss().reduce_loss(torch.tensor(float(rank + 1)))
        assert total.item() == sum(range(1, world + 1))
        # the form that does not make the caller wait: the local value is left alone, the sum is ready after wait()
        local = torch.tensor(float(10 * (rank + 1)))
        total2, work = TokenParallelLoss().reduce_loss_async(local)
        work.wait()
        assert total2.item() == 10 * sum(range(1, world + 1)) and local.item() == 10 * (rank + 1)
        # a mismatched buffer is refused before any communication
        try:
            exchange_partials(mine, out=torch.empty(world, N + 1, 4))
            ret[rank] = 1e9
        except ValueError:
            pass
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_rank_exchange_and_merge():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert sorted(ret.keys()) == [0, 1]
    assert max(ret.values()) < 1e-5


def test_shard_bounds():
    assert shard_bounds(151936, 3, 8) == (3 * 18992, 4 * 18992)
    assert shard_bounds(128256, 0, 2) == (0, 64128)
    with pytest.raises(ValueError):
        shard_bounds(1001, 0, 8)
    with pytest.raises(ValueError):
        exchange_partials(torch.zeros(5, 3))  # never reaches the process group
