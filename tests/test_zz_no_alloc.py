"""mllm_grpo_fwd_static_scratch: the forward for callers that cannot allocate.

Some users of this library run inside a memory plan they do not own: an XLA custom-call handler
gets exactly the operand and result buffers the compiler planned, and a serving loop may have
promised never to touch the allocator once it is warm.  Neither can cudaMalloc the per-token
scratch the ordinary forward wants, so this entry point keeps that scratch in a fixed 4 MiB array
inside the library.  The test drives it through the C ABI with `loss_terms` left NULL and compares
every output with the ordinary forward and with the CPU oracle, on two calls in a row (the second
smaller, so it runs over whatever the first left in the array), and checks that an over-sized
problem is refused.

The file name sorts last on purpose: a run that stops at the first failure has by then run all
other tests.
"""
import ctypes as C

import pytest
import torch

import mllm_jax_b200 as G
from mllm_jax_b200 import _lib
from oracle import grpo_oracle as O
from tests.util import ENT_ATOL, LOSS_RTOL, LP_ATOL, assert_loss_close, make_case, to_device

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_TOKENS = 1 << 20


def _problem(cuda, B, L, V, seed, want_oracle=False):
    logits, inputs = make_case(B, L, V, seed=seed, old="wide", ref=True)
    din = to_device(inputs, cuda)
    if want_oracle:
        return O.reference_call(logits, inputs, beta=0.04)
    return G.TokenLossProblem(logits.to(cuda), din["input_ids"][:, 1:], din["labels"][:, 1:], din["advantages"],
                              din["total_valid_token_count"], din["old_per_token_logps"], din["ref_per_token_logps"],
                              G.LossConfig(beta=0.04), scored_rows=L - 1)


def test_static_scratch_forward_matches_ordinary_forward(cuda):
    for (B, L, V, seed) in ((6, 41, 5003, 901), (2, 9, 1000, 902)):  # two calls in a row, second smaller
        ref = _problem(cuda, B, L, V, seed)
        ref.run("mllm_grpo_fwd")
        new = _problem(cuda, B, L, V, seed)
        new.loss_terms = None  # the entry point must not need it
        new.loss.fill_(float("nan"))
        args = new.args()
        assert args.loss_terms is None
        _lib.call("mllm_grpo_fwd_static_scratch", args, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert abs(new.loss.item() - ref.loss.item()) <= LOSS_RTOL * abs(ref.loss.item())
        assert (new.per_token_logps - ref.per_token_logps).abs().max().item() <= LP_ATOL
        assert (new.token_entropy - ref.token_entropy).abs().max().item() <= 5e-4
        assert torch.allclose(new.lse, ref.lse, atol=LP_ATOL)
        assert torch.allclose(new.grad_coef, ref.grad_coef, rtol=1e-4, atol=1e-6)
        # and against the CPU oracle, not only against the library itself
        want = _problem(cuda, B, L, V, seed, want_oracle=True)
        assert_loss_close(new.loss.item(), want["loss"].item(), what="static scratch vs oracle")
        assert (new.per_token_logps.cpu() - want["per_token_logps"]).abs().max().item() <= LP_ATOL
        assert (new.token_entropy.cpu() - want["token_entropy"]).abs().max().item() <= ENT_ATOL
        # the backward consumes the residuals of the new forward just like the ordinary ones
        new.alloc_dlogits()
        new.run("mllm_grpo_bwd")
        ref.alloc_dlogits()
        ref.run("mllm_grpo_bwd")
        assert torch.equal(new.dlogits, ref.dlogits)


def test_static_scratch_rejects_oversized_problem(cuda):
    a = _lib.GrpoArgs()
    a.struct_size = C.sizeof(_lib.GrpoArgs)
    a.n_seqs, a.seq_rows, a.scored_rows, a.vocab, a.row_stride = STATIC_SCRATCH_TOKENS + 1, 1, 1, 8, 8
    a.temperature = 1.0
    status = _lib.load().mllm_grpo_fwd_static_scratch(C.byref(a), None)
    assert status == 8  # MLLM_GRPO_ERR_TOO_LARGE
    assert b"too large" in _lib.load().mllm_grpo_status_string(status)
