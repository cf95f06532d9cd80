"""Vocabulary-parallel paths on real GPUs.

World size 1 always runs (the fused sharded kernel then exchanges with itself, which exercises the
publish / wait / merge protocol and both epoch parities on one GPU).  With more GPUs, jobs of 2, 4
and 8 ranks are spawned (as many as the box has): every rank checks the NCCL path and the fused
peer-store path against the CPU oracle, including several back-to-back calls without any barrier in
between, and a token-parallel job checks the row-sharded mode the reference's own runs use."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.util import ENT_ATOL, LP_ATOL, assert_dlogits_close, assert_loss_close, make_case, to_device

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run_rank(rank, world, port, ret):
    import mllm_jax_b200 as G
    from mllm_jax_b200.vocab_parallel import VocabParallelLoss
    from oracle import grpo_oracle as O

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl" if world > 1 else "gloo", rank=rank, world_size=world,
                            device_id=dev if world > 1 else None)
    try:
        B, L, V = 3, 41, 4096 * world
        logits, inputs = make_case(B, L, V, seed=91, old="wide", ref=True)
        attrs = dict(beta=0.04, epsilon_low=0.2, epsilon_high=0.3)
        ref = O.reference_value_and_grad(logits, inputs, **attrs)
        vp = VocabParallelLoss(V, G.LossConfig(**attrs))
        din = to_device(inputs, dev)
        # the shard as its own contiguous tensor, aligned ids (flat layout: score rows 0..L-2 against ids 1..L-1)
        shard = logits[:, :-1, vp.start:vp.stop].contiguous().to(dev)
        args = (shard, din["input_ids"][:, 1:], din["labels"][:, 1:], din["advantages"],
                din["total_valid_token_count"], din["old_per_token_logps"], din["ref_per_token_logps"])
        want_d = ref["dlogits"][:, :-1, vp.start:vp.stop]
        outs = {"nccl": vp.value_and_grad(*args) if world > 1 else None}
        for i in range(3):  # three fused calls in a row: both epoch parities, no barrier between them
            outs[f"fused{i}"] = vp.value_and_grad_fused(*args, dlogits=torch.empty_like(shard))
        # the reference layout on a strided shard view: L rows per sequence, L-1 scored, last row zero
        full = logits.to(dev)[:, :, vp.start:vp.stop]
        shifted = vp.value_and_grad_fused(full, *args[1:], scored_rows=L - 1)  # gradient buffer with the view's strides
        torch.cuda.synchronize()
        assert_dlogits_close(shifted["dlogits"], ref["dlogits"][:, :, vp.start:vp.stop], what="shifted shard view")
        assert (shifted["per_token_logps"].cpu() - ref["per_token_logps"]).abs().max() <= LP_ATOL
        for name, out in outs.items():
            if out is None:
                continue
            assert G.ops.check_device_status(out["problem"]) == 0, name
            assert (out["per_token_logps"].cpu() - ref["per_token_logps"]).abs().max() <= LP_ATOL, name
            assert (out["token_entropy"].cpu() - ref["token_entropy"]).abs().max() <= ENT_ATOL, name
            assert_loss_close(out["loss"].item(), ref["loss"].item(), what=name)
            assert_dlogits_close(out["dlogits"], want_d, what=name)
        # every sharded kernel family behind the fused entry: register-fed unsplit rows in load batches of 4, 6 and 8
        # (warp-level exchange), shards split over clusters of 2, 4 and 8 CTAs, and the staged form again
        from mllm_jax_b200._lib import plan_override

        for cluster, threads, batch, staged in [(1, 256, 4, 0), (1, 256, 6, 0), (1, 256, 8, 0), (1, 128, 8, 0),
                                                (2, 128, 10, -1), (4, 128, 8, -1), (8, 128, 6, -1), (1, 256, 0, 1)]:
            name = f"plan cl={cluster} th={threads} batch={batch} staged={staged}"
            with plan_override(cluster=cluster, threads=threads, load_batch=batch, staged=staged):
                out = vp.value_and_grad_fused(*args, dlogits=torch.empty_like(shard))
                torch.cuda.synchronize()
            assert G.ops.check_device_status(out["problem"]) == 0, name
            assert (out["per_token_logps"].cpu() - ref["per_token_logps"]).abs().max() <= LP_ATOL, name
            assert (out["token_entropy"].cpu() - ref["token_entropy"]).abs().max() <= ENT_ATOL, name
            assert_loss_close(out["loss"].item(), ref["loss"].item(), what=name)
            assert_dlogits_close(out["dlogits"], want_d, what=name)
        # soft-capped logits through the fused path
        big, big_in = make_case(B, L, V, seed=96, old="wide", ref=True, sigma=6.0)
        cap_attrs = dict(beta=0.04, epsilon_low=0.2, epsilon_high=0.3, softcap=30.0)
        ref_c = O.reference_value_and_grad(big, big_in, **cap_attrs)
        vpc = VocabParallelLoss(V, G.LossConfig(**cap_attrs))
        dc = to_device(big_in, dev)
        sh = big[:, :-1, vp.start:vp.stop].contiguous().to(dev)
        oc = vpc.value_and_grad_fused(sh, dc["input_ids"][:, 1:], dc["labels"][:, 1:], dc["advantages"],
                                      dc["total_valid_token_count"], dc["old_per_token_logps"],
                                      dc["ref_per_token_logps"], dlogits=torch.empty_like(sh))
        torch.cuda.synchronize()
        assert (oc["per_token_logps"].cpu() - ref_c["per_token_logps"]).abs().max() <= LP_ATOL
        assert_loss_close(oc["loss"].item(), ref_c["loss"].item(), what="fused soft-cap")
        assert_dlogits_close(oc["dlogits"], ref_c["dlogits"][:, :-1, vp.start:vp.stop], what="fused soft-cap")
        if world > 1:
            # tp-sharded lm_head folded into the forward: every rank multiplies by its own weight rows, the
            # per-row partials are all-gathered (16 bytes per row and vocabulary range) and merged on every rank
            from mllm_jax_b200.linear_loss import lm_head_forward

            g = torch.Generator().manual_seed(95)
            H = 128
            hidden = torch.randn(B, L - 1, H, generator=g).to(torch.bfloat16)
            weight = (torch.randn(V, H, generator=g) * 0.3).to(torch.bfloat16)
            x64 = O.lm_head_logits(hidden, weight)
            ids = inputs["input_ids"][:, 1:]
            want = torch.log_softmax(x64, -1).gather(-1, ids.long()[..., None])[..., 0]
            out = lm_head_forward(hidden.to(dev), weight[vp.start:vp.stop].contiguous().to(dev), ids.to(dev),
                                  vocab_start=vp.start, vocab_total=V, group=dist.group.WORLD)
            torch.cuda.synchronize()
            assert (out["per_token_logps"].cpu().double() - want).abs().max() <= LP_ATOL, "sharded lm_head forward"
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


def _spawn(world):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_run_rank, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert dict(ret) == {r: "ok" for r in range(world)}


@pytest.mark.timeout(300)
def test_fused_sharded_kernel_world_size_one(cuda):
    _spawn(1)


@pytest.mark.timeout(600)
@pytest.mark.parametrize("world", [2, 4, 8])
def test_ranks_nccl_and_fused(cuda, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _spawn(world)


def _run_token_parallel_rank(rank, world, port, ret):
    import mllm_jax_b200 as G
    from mllm_jax_b200.vocab_parallel import TokenParallelLoss
    from oracle import grpo_oracle as O

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        per, L, V = 3, 33, 5000
        B = per * world
        logits, inputs = make_case(B, L, V, seed=93, old="wide", ref=True)
        attrs = dict(beta=0.04, epsilon_low=0.2, epsilon_high=0.3)
        ref = O.reference_value_and_grad(logits, inputs, **attrs)  # the whole batch, global normaliser
        sl = slice(rank * per, (rank + 1) * per)
        din = to_device({k: (v[sl] if isinstance(v, torch.Tensor) else v) for k, v in inputs.items()}, dev)
        tp = TokenParallelLoss(G.LossConfig(**attrs))
        out = tp.value_and_grad(logits[sl].to(dev), din["input_ids"], din["labels"], din["advantages"],
                                din["total_valid_token_count"], din["old_per_token_logps"],
                                din["ref_per_token_logps"], shifted=True)
        torch.cuda.synchronize()
        assert_loss_close(out["loss"].item(), ref["loss"].item(), what="sum of the ranks' losses")
        assert (out["per_token_logps"].cpu() - ref["per_token_logps"][sl]).abs().max() <= LP_ATOL
        assert_dlogits_close(out["dlogits"], ref["dlogits"][sl], what=f"token-parallel rank {rank}")
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_token_parallel_two_ranks(cuda):
    """Rows split over ranks (the reference's dp/fsdp batch sharding, plugins/training/runner/grpo_gsm8k.py:282)
    with the global total_valid_token_count (:770): the ranks' losses add up to the oracle's loss of the whole
    batch and every rank's dlogits are its rows of the oracle's gradient."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_run_token_parallel_rank, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert dict(ret) == {0: "ok", 1: "ok"}


@pytest.mark.timeout(120)
@pytest.mark.parametrize("rows", [3, 6000])
def test_missing_peer_times_out_with_status(cuda, rows):
    """Failure detection without a GPU fault: rank 0 of a pretended 2-rank job runs alone, so the
    words of rank 1 never arrive.  The first waits give up after their wall-clock limit and every
    later row sees the raised bit and does not wait, so the whole call costs about one limit however
    many rows it has; the kernel ends normally, the loss is NaN, no gradient is written for the rows
    that gave up, MLLM_GRPO_DEV_WAIT_TIMEOUT is raised for the host and the context stays usable."""
    import time

    import mllm_jax_b200 as G
    from mllm_jax_b200 import _lib

    B, L, V = 1, rows + 1, 512
    logits, inputs = make_case(B, L, V, seed=92, old="none", mask_kind="ones")
    din = to_device(inputs, cuda)
    x = logits[:, :-1].contiguous().to(cuda)
    p = G.TokenLossProblem(x, din["input_ids"][:, 1:], din["labels"][:, 1:], din["advantages"], float(rows), None,
                           None, G.LossConfig(), scored_rows=L - 1, vocab=V, vocab_start=0, vocab_total=2 * V)
    nbytes = int(_lib.load().mllm_grpo_exchange_bytes(p.N, 2))
    mine = torch.zeros(nbytes, dtype=torch.uint8, device=cuda)
    absent_peer = torch.zeros(nbytes, dtype=torch.uint8, device=cuda)  # stands in for rank 1's buffer
    p.peer_ptrs, p.shard_rank, p.n_shards, p.exchange_epoch = [mine.data_ptr(), absent_peer.data_ptr()], 0, 2, 1
    p.peer_wait_ms = 500
    p.alloc_dlogits()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    p.run("mllm_grpo_fwd_bwd_sharded")
    torch.cuda.synchronize()
    took = time.perf_counter() - t0
    assert 0.4 <= took <= 5.0, took  # one limit (plus scheduling), not one per row or per wave
    assert G.ops.check_device_status(p) & _lib.DEV_WAIT_TIMEOUT
    assert torch.isnan(p.loss).all() and torch.isnan(p.per_token_logps).all()
    assert (p.dlogits == 0).all()
    # the bit is sticky: a call that starts with it set does not wait at all
    p.exchange_epoch = 2
    t0 = time.perf_counter()
    p.run("mllm_grpo_fwd_bwd_sharded")
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 0.4 and torch.isnan(p.loss).all()
    # the context is still healthy: an ordinary call works afterwards
    q = G.TokenLossProblem(x, din["input_ids"][:, 1:], din["labels"][:, 1:], din["advantages"], float(rows), None,
                           None, G.LossConfig(), scored_rows=L - 1)
    q.run("mllm_grpo_fwd")
    torch.cuda.synchronize()
    assert torch.isfinite(q.loss).all() and G.ops.check_device_status(q) == 0


def test_sharded_entry_needs_a_status_word(cuda):
    import mllm_jax_b200 as G
    from mllm_jax_b200 import _lib

    logits, inputs = make_case(1, 4, 512, seed=94, old="none", mask_kind="ones")
    din = to_device(inputs, cuda)
    x = logits[:, :-1].contiguous().to(cuda)
    p = G.TokenLossProblem(x, din["input_ids"][:, 1:], din["labels"][:, 1:], din["advantages"], 3.0, None, None,
                           G.LossConfig(), scored_rows=3, vocab=512, vocab_start=0, vocab_total=512)
    buf = torch.zeros(int(_lib.load().mllm_grpo_exchange_bytes(p.N, 1)), dtype=torch.uint8, device=cuda)
    p.peer_ptrs, p.shard_rank, p.n_shards, p.exchange_epoch = [buf.data_ptr()], 0, 1, 1
    p.alloc_dlogits()
    p.device_status = None
    with pytest.raises(_lib.GrpoError) as e:
        p.run("mllm_grpo_fwd_bwd_sharded")
    assert e.value.status == 1
