"""lm_head projection folded into the forward of the loss (tcgen05 / TMA kernel).

The oracle computes logits = hidden x weight^T in float64 from the same bf16 operands
(MLLM_JAX/language/qwen2/modular_qwen2.py:182) and runs the loss restatement on them; the kernel's
logits are f32 tensor-core accumulators that never leave the chip, so log-probs are held to the usual
2e-3 abs, entropy to 5e-4 and the loss to 1e-4 rel."""
import pytest
import torch

import mllm_jax_b200 as G
from mllm_jax_b200.linear_loss import lm_head_forward
from oracle import grpo_oracle as O
from tests.util import ENT_ATOL, LP_ATOL, assert_loss_close, make_case

pytestmark = pytest.mark.gpu


def _case(B, T, H, V, seed, scale=0.5, **kw):
    g = torch.Generator().manual_seed(seed)
    hidden = torch.randn(B, T, H, generator=g).to(torch.bfloat16)
    weight = (torch.randn(V, H, generator=g) * scale / H ** 0.5 * 4).to(torch.bfloat16)
    logits64 = O.lm_head_logits(hidden, weight)                      # [B, T, V] float64
    _, inputs = make_case(B, T + 1, V, seed=seed + 1, old="none", **kw)
    ids, mask = inputs["input_ids"][:, 1:], inputs["labels"][:, 1:]
    lp0 = torch.log_softmax(logits64, -1).gather(-1, ids.long()[..., None])[..., 0].float()
    old = lp0 + 0.3 * torch.randn(B, T, generator=g)
    ref_lp = lp0 + 0.1 * torch.randn(B, T, generator=g)
    nv = float(mask.sum()) or 1.0
    z = torch.zeros(B, 1, dtype=ids.dtype)
    oin = {"input_ids": torch.cat([z, ids], 1), "labels": torch.cat([z, mask], 1), "advantages": inputs["advantages"],
           "total_valid_token_count": nv, "old_per_token_logps": old, "ref_per_token_logps": ref_lp}
    shifted = torch.cat([logits64, logits64[:, :1]], 1)              # the unscored last position
    return hidden, weight, ids, mask, inputs["advantages"], nv, old, ref_lp, oin, shifted


@pytest.mark.parametrize("B,T,H,V", [
    (1, 128, 64, 256),       # exactly one tile, one k-block
    (2, 150, 192, 1000),     # ragged rows (300 = 2 tiles + 44) and a ragged last vocabulary tile
    (1, 130, 128, 10240),    # 40 vocabulary tiles: three splits, accumulator ping-pong inside a CTA
    (3, 50, 896, 4099),      # vocabulary not a multiple of 8, Qwen2.5-0.5B's hidden size
])
@pytest.mark.parametrize("layout", ["vh", "hv"])
def test_folded_forward_matches_oracle(cuda, B, T, H, V, layout):
    """layout "vh": weight [V, H] (K-major operand); "hv": weight [H, V] as a flax Dense kernel stores it
    (MN-major operand, needs a vocabulary that is a multiple of 8 for TMA's 16-byte row pitch)."""
    if layout == "hv" and V % 8:
        pytest.skip("[H, V] weights need V % 8 == 0")
    hidden, weight, ids, mask, adv, nv, old, ref_lp, oin, shifted = _case(B, T, H, V, seed=300 + H)
    ref = O.reference_call(shifted, oin, beta=0.04, dtype=torch.float64)
    w_dev = weight.to(cuda) if layout == "vh" else weight.t().contiguous().to(cuda)
    out = lm_head_forward(hidden.to(cuda), w_dev, ids.to(cuda), mask.to(cuda), adv.to(cuda), nv,
                          old.to(cuda), ref_lp.to(cuda), cfg=G.LossConfig(beta=0.04), weight_layout=layout)
    torch.cuda.synchronize()
    assert G.ops.check_device_status(out["problem"]) == 0
    assert (out["per_token_logps"].cpu().double() - ref["per_token_logps"]).abs().max() <= LP_ATOL
    assert (out["token_entropy"].cpu().double() - ref["token_entropy"]).abs().max() <= ENT_ATOL
    assert_loss_close(out["loss"].item(), ref["loss"].item())
    # the residuals feed the ordinary backward: lse against the oracle's logsumexp
    lse = torch.logsumexp(shifted[:, :-1], -1)
    assert (out["lse"].cpu().double() - lse).abs().max() <= LP_ATOL


def test_folded_forward_softcap_and_tile_edges(cuda):
    """Soft-capped logits, and chosen tokens on the first / last column of vocabulary tiles and splits."""
    B, T, H, V = 1, 64, 128, 256 * 17 + 8
    hidden, weight, ids, mask, adv, nv, old, ref_lp, oin, shifted = _case(B, T, H, V, seed=77, scale=6.0)
    edges = torch.tensor([0, 255, 256, 511, 256 * 9 - 1, 256 * 9, V - 1, V - 8])
    ids[0, :edges.numel()] = edges.to(ids.dtype)
    oin["input_ids"][0, 1:1 + edges.numel()] = edges.to(ids.dtype)
    ref = O.reference_call(shifted, oin, softcap=30.0, dtype=torch.float64)
    out = lm_head_forward(hidden.to(cuda), weight.to(cuda), ids.to(cuda), mask.to(cuda), adv.to(cuda), nv,
                          old.to(cuda), None, cfg=G.LossConfig(softcap=30.0))
    torch.cuda.synchronize()
    assert G.ops.check_device_status(out["problem"]) == 0
    assert (out["per_token_logps"].cpu().double() - ref["per_token_logps"]).abs().max() <= LP_ATOL
    assert (out["token_entropy"].cpu().double() - ref["token_entropy"]).abs().max() <= ENT_ATOL
    assert_loss_close(out["loss"].item(), ref["loss"].item())


def test_folded_forward_only_logprobs(cuda):
    """No advantages: the reference-model pass (log-probs and entropy only)."""
    hidden, weight, ids, *_rest, oin, shifted = _case(2, 70, 256, 3000, seed=78)
    lp = torch.log_softmax(shifted[:, :-1], -1).gather(-1, ids.long()[..., None])[..., 0]
    out = lm_head_forward(hidden.to(cuda), weight.to(cuda), ids.to(cuda))
    torch.cuda.synchronize()
    assert (out["per_token_logps"].cpu().double() - lp).abs().max() <= LP_ATOL


def test_folded_forward_hv_weight_shard(cuda):
    """A vocabulary shard of an [H, V] weight is a column range of it (no copy): strided rows, global ids."""
    B, T, H, V = 1, 140, 128, 2048
    hidden, weight, ids, mask, adv, nv, old, ref_lp, oin, shifted = _case(B, T, H, V, seed=92)
    lp_ref = torch.log_softmax(shifted[:, :-1], -1).gather(-1, ids.long()[..., None])[..., 0]
    w_hv = weight.t().contiguous().to(cuda)  # [H, V]
    full = lm_head_forward(hidden.to(cuda), w_hv, ids.to(cuda), weight_layout="hv")
    assert (full["per_token_logps"].cpu().double() - lp_ref).abs().max() <= LP_ATOL
    # the upper half of the vocabulary alone: every chosen id below 1024 belongs to "another shard"
    upper = lm_head_forward(hidden.to(cuda), w_hv[:, 1024:], ids.to(cuda), weight_layout="hv", vocab_start=1024,
                            vocab_total=V)
    torch.cuda.synchronize()
    lse_upper = torch.logsumexp(shifted[:, :-1, 1024:], -1)
    assert (upper["lse"].cpu().double() - lse_upper).abs().max() <= LP_ATOL


def test_folded_forward_rejects_what_it_cannot_run(cuda):
    hidden = torch.zeros(1, 4, 72, dtype=torch.bfloat16, device=cuda)  # hidden size not a multiple of 64
    weight = torch.zeros(16, 72, dtype=torch.bfloat16, device=cuda)
    ids = torch.zeros(1, 4, dtype=torch.int32, device=cuda)
    with pytest.raises(G.GrpoError) as e:
        lm_head_forward(hidden, weight, ids)
    assert e.value.status == 7


@pytest.mark.timeout(600)
def test_folded_forward_full_vocabulary_and_hidden_size(cuda):
    """The benchmark's shape per row (H = 3584, V = 151936: 594 vocabulary tiles in 38 splits, 56 k-blocks) on
    300 rows; 24 sampled rows against float64 logits of the same operands."""
    import numpy as np

    B, T, H, V = 1, 300, 3584, 151936
    g = torch.Generator(device=cuda).manual_seed(5)
    hidden = torch.randn(B, T, H, generator=g, device=cuda).to(torch.bfloat16)
    weight = (torch.randn(V, H, generator=g, device=cuda) * (2.0 / H ** 0.5)).to(torch.bfloat16)
    gc = torch.Generator().manual_seed(6)
    ids = torch.randint(0, V, (B, T), generator=gc, dtype=torch.int64).to(torch.int32)
    ids[0, :4] = torch.tensor([0, V - 1, 255, 256], dtype=torch.int32)
    mask = (torch.rand(B, T, generator=gc) < 0.7).float()
    adv = torch.randn(B, generator=gc)
    nv = float(mask.sum())
    lp_dev = lm_head_forward(hidden, weight, ids.to(cuda))["per_token_logps"].cpu()
    old = lp_dev + 0.3 * torch.randn(B, T, generator=gc)
    out = lm_head_forward(hidden, weight, ids.to(cuda), mask.to(cuda), adv.to(cuda), nv, old.to(cuda), None,
                          cfg=G.LossConfig(epsilon_low=0.2, epsilon_high=0.2))
    torch.cuda.synchronize()
    assert G.ops.check_device_status(out["problem"]) == 0
    rows = torch.cat([torch.arange(4), torch.randint(4, T, (20,), generator=gc)]).unique()
    x64 = O.lm_head_logits(hidden[0, rows.to(cuda)].cpu(), weight.cpu()).numpy()
    pick = lambda t: t.reshape(-1)[rows].double().cpu().numpy()  # noqa: E731
    an = O.analytic_rows(x64, ids.reshape(-1)[rows].long().numpy(), pick(mask), np.full(rows.numel(), adv.item()),
                         pick(old), None, nv, epsilon_low=0.2, epsilon_high=0.2, want_grad=False)
    assert np.abs(pick(out["per_token_logps"]) - an["lp"]).max() <= LP_ATOL
    assert np.abs(pick(out["token_entropy"]) - an["entropy_guard"]).max() <= ENT_ATOL
    assert np.abs(pick(out["lse"]) - an["lse"]).max() <= LP_ATOL
    assert np.allclose(pick(out["problem"].loss_terms), an["loss_terms"], atol=2e-3)
    # the loss is the fixed-order sum of the per-token terms
    assert_loss_close(out["loss"].item(), out["problem"].loss_terms.double().sum().item() / nv)


def test_folded_forward_on_a_vocabulary_shard(cuda):
    """One vocabulary shard of a tp-sharded head (global ids, vocab_start): the partials of two shards, merged
    by one combine over both shards' vocabulary ranges, reproduce the unsharded result."""
    from mllm_jax_b200 import _lib

    B, T, H, V = 2, 90, 128, 2 * 1000
    hidden, weight, ids, mask, adv, nv, old, ref_lp, oin, shifted = _case(B, T, H, V, seed=91)
    ref = O.reference_call(shifted, oin, dtype=torch.float64)
    full = lm_head_forward(hidden.to(cuda), weight.to(cuda), ids.to(cuda), mask.to(cuda), adv.to(cuda), nv,
                           old.to(cuda), None)
    lib = _lib.load()
    N, half = B * T, V // 2
    splits = int(lib.mllm_lm_head_splits(N, half))
    nbytes = int(lib.mllm_lm_head_partials_bytes(N, half))
    both = torch.empty(2 * nbytes, dtype=torch.uint8, device=cuda)
    hid, wt, idd = hidden.to(cuda), weight.to(cuda), ids.to(cuda).contiguous()
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    for r in range(2):  # what rank r of a 2-rank job computes; the all-gather is the concatenation
        a = _lib.LmHeadArgs()
        a.n_rows, a.vocab, a.hidden_dim, a.hidden_stride, a.weight_stride = N, half, H, H, H
        a.vocab_start, a.vocab_total = r * half, V
        a.hidden, a.weight = hid.data_ptr(), wt[r * half:(r + 1) * half].data_ptr()
        a.chosen_ids, a.partials = idd.data_ptr(), both[r * nbytes:].data_ptr()
        a.device_status = status.data_ptr()
        _lib.call("mllm_lm_head_partials", a, torch.cuda.current_stream().cuda_stream)
    prob = full["problem"]
    g = prob.args()
    g.gathered_partials, g.n_shards = both.data_ptr(), 2 * splits
    prob.per_token_logps.fill_(float("nan"))
    _lib.call("mllm_grpo_combine", g, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert (prob.per_token_logps.cpu().double() - ref["per_token_logps"]).abs().max() <= LP_ATOL
    assert (prob.token_entropy.cpu().double() - ref["token_entropy"]).abs().max() <= ENT_ATOL
    assert_loss_close(prob.loss.item(), ref["loss"].item())
