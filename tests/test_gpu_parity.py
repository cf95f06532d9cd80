"""Parity of the CUDA path (through the C ABI) against the CPU oracle on the same seeded inputs.

Gates: per-token log-prob 2e-3 abs, loss 1e-4 rel, dlogits 1e-2 rel (see tests/util.py);
entropy 5e-4 abs.  Covers ragged sizes and alignments, every optional input, the reference
(shifted) and flat layouts, in-place backward, the fused entry point, vocabulary shards,
the golden fixtures, and the full-size workload through row samples and row-sum properties.
"""
import os

import numpy as np
import pytest
import torch

import mllm_jax_b200 as G
from mllm_jax_b200 import synth
from oracle import grpo_oracle as O
from tests.util import (ENT_ATOL, LP_ATOL, assert_dlogits_close, assert_loss_close, make_case, to_device)

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def run_both(logits, inputs, cuda, *, fused=False, **attrs):
    """Oracle on CPU and kernels on the GPU for one reference-layout case."""
    o_attrs = {k: v for k, v in attrs.items() if k != "inplace_backward"}
    ref = O.reference_value_and_grad(logits, inputs, **o_attrs)
    x = logits.to(cuda)
    din = to_device(inputs, cuda)
    if fused:
        cfg = G.LossConfig(temperature=attrs.get("temperature", 1.0), epsilon_low=attrs.get("epsilon_low", 0.2),
                           epsilon_high=attrs.get("epsilon_high", 0.3), beta=attrs.get("beta", 0.0),
                           softcap=attrs.get("softcap"))
        out = G.grpo_value_and_grad(x, din["input_ids"], din["labels"], din["advantages"],
                                    din.get("total_valid_token_count"), din.get("old_per_token_logps"),
                                    din.get("ref_per_token_logps"), shifted=True, cfg=cfg)
        got = {"loss": out["loss"], "per_token_logps": out["per_token_logps"],
               "token_entropy": out["token_entropy"], "dlogits": out["dlogits"]}
    else:
        xg = x.clone().requires_grad_(True)
        out = G.grpo_token_loss(xg, din["input_ids"], din["labels"], din["advantages"],
                                din.get("total_valid_token_count"), din.get("old_per_token_logps"),
                                din.get("ref_per_token_logps"), **attrs)
        out["loss"].backward()
        got = {"loss": out["loss"].detach(), "per_token_logps": out["per_token_logps"],
               "token_entropy": out["token_entropy"], "dlogits": xg.grad}
    torch.cuda.synchronize()
    return ref, got


def check(ref, got, what=""):
    lp_err = (got["per_token_logps"].cpu() - ref["per_token_logps"]).abs().max().item()
    assert lp_err <= LP_ATOL, f"{what}: log-prob error {lp_err:.3e}"
    assert_loss_close(got["loss"].item(), ref["loss"].item(), what=what)
    if got["token_entropy"] is not None:
        e_err = (got["token_entropy"].cpu() - ref["token_entropy"]).abs().max().item()
        assert e_err <= ENT_ATOL, f"{what}: entropy error {e_err:.3e}"
    assert got["dlogits"].dtype == torch.bfloat16
    assert_dlogits_close(got["dlogits"], ref["dlogits"], what=what)
    return lp_err


@pytest.mark.parametrize("V", [8, 129, 1000, 4099, 32000])
@pytest.mark.parametrize("B,L", [(1, 2), (3, 2), (2, 130)])
def test_ragged_sizes(cuda, V, B, L):
    if V == 32000 and L == 130:
        L = 40
    logits, inputs = make_case(B, L, V, seed=V + B, old="noisy", ref=True)
    ref, got = run_both(logits, inputs, cuda, beta=0.04)
    check(ref, got, f"V={V} B={B} L={L}")


def test_full_vocab_rows(cuda):
    logits, inputs = make_case(2, 9, 151936, seed=5, old="noisy", ref=True)
    ref, got = run_both(logits, inputs, cuda, beta=0.04, epsilon_low=0.2, epsilon_high=0.2)
    err = check(ref, got, "V=151936")
    assert err < 2e-4  # far inside the gate on ordinary rows


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("kind", ["no_old", "wide_clip", "kl", "token_adv", "random_mask", "temp", "softcap"])
def test_options(cuda, kind, fused):
    kw, attrs = dict(old="noisy"), {}
    if kind == "no_old":
        kw = dict(old="none")
    elif kind == "wide_clip":
        kw = dict(old="wide")
        attrs = dict(epsilon_low=0.1, epsilon_high=0.15)
    elif kind == "kl":
        kw = dict(old="wide", ref=True)
        attrs = dict(beta=0.5)
    elif kind == "token_adv":
        kw = dict(old="wide", per_token_adv=True)
    elif kind == "random_mask":
        kw = dict(old="noisy", mask_kind="random")
    elif kind == "temp":
        attrs = dict(temperature=0.7)
    elif kind == "softcap":
        kw = dict(old="noisy", ref=True, sigma=4.0)
        attrs = dict(softcap=30.0, beta=0.04)
    logits, inputs = make_case(3, 11, 5003, seed=31, **kw)
    ref, got = run_both(logits, inputs, cuda, fused=fused, **attrs)
    check(ref, got, f"{kind} fused={fused}")


def test_softcap_full_gemma_vocab(cuda):
    logits, inputs = make_case(1, 4, 256000, seed=32, old="noisy", ref=True, sigma=4.0)
    ref, got = run_both(logits, inputs, cuda, softcap=30.0, beta=0.04, epsilon_low=0.2, epsilon_high=0.2)
    check(ref, got, "gemma softcap")


def test_unaligned_and_strided_views(cuda):
    """Rows that start off a 16-byte boundary and a padded row stride."""
    B, L, V = 2, 6, 1003
    logits, inputs = make_case(B, L, V, seed=33, old="noisy")
    ref = O.reference_value_and_grad(logits, inputs)
    din = to_device(inputs, cuda)
    for offset, ld in ((1, V), (3, V + 5), (0, V + 13), (7, V + 8)):
        buf = torch.zeros(B * L * ld + 16, dtype=torch.bfloat16, device=cuda)
        view = buf[offset:offset + B * L * ld].view(B, L, ld)[:, :, :V]
        view.copy_(logits.to(cuda))
        prob = G.TokenLossProblem(view, din["input_ids"][:, 1:], din["labels"][:, 1:], din["advantages"],
                                  din["total_valid_token_count"], din["old_per_token_logps"], None,
                                  G.LossConfig(), scored_rows=L - 1, vocab=V)
        dbuf = torch.full_like(buf, 7.0)
        prob.dlogits = dbuf[offset:offset + B * L * ld].view(B, L, ld)[:, :, :V]
        prob.run("mllm_grpo_fwd_bwd")
        torch.cuda.synchronize()
        got = {"loss": prob.loss[0], "per_token_logps": prob.per_token_logps, "token_entropy": prob.token_entropy,
               "dlogits": prob.dlogits}
        check(ref, got, f"offset={offset} ld={ld}")
        # padding columns and guard elements around the output are untouched
        full = dbuf[offset:offset + B * L * ld].view(B, L, ld)
        assert (full[:, :, V:] == 7.0).all()
        assert (dbuf[:offset] == 7.0).all() and (dbuf[offset + B * L * ld:] == 7.0).all()


def test_mismatched_phase_uses_scalar_path(cuda):
    """logits and dlogits rows at different offsets from a 16-byte boundary."""
    B, L, V = 1, 3, 515
    logits, inputs = make_case(B, L, V, seed=34, old="noisy")
    ref = O.reference_value_and_grad(logits, inputs)
    din = to_device(inputs, cuda)
    x = logits.to(cuda)
    prob = G.TokenLossProblem(x, din["input_ids"][:, 1:], din["labels"][:, 1:], din["advantages"],
                              din["total_valid_token_count"], din["old_per_token_logps"], None, G.LossConfig(),
                              scored_rows=L - 1)
    dbuf = torch.zeros(B * L * V + 8, dtype=torch.bfloat16, device=cuda)
    prob.dlogits = dbuf[3:3 + B * L * V].view(B, L, V)
    prob.run("mllm_grpo_fwd_bwd")
    assert_dlogits_close(prob.dlogits, ref["dlogits"], what="phase mismatch")


def test_inplace_backward(cuda):
    logits, inputs = make_case(2, 7, 4096, seed=35, old="wide")
    ref = O.reference_value_and_grad(logits, inputs)
    din = to_device(inputs, cuda)
    x = logits.to(cuda)
    out = G.grpo_value_and_grad(x, din["input_ids"], din["labels"], din["advantages"],
                                din["total_valid_token_count"], din["old_per_token_logps"], shifted=True, inplace=True)
    assert out["dlogits"].data_ptr() == x.data_ptr()
    assert_dlogits_close(out["dlogits"], ref["dlogits"], what="in place")


def test_flat_layout_and_upstream_cotangent(cuda):
    """Aligned [B, T] ids; the loss is scaled before backward so grad_scale != 1 reaches the kernel."""
    B, T, V = 4, 16, 2000
    logits, inputs = make_case(B, T + 1, V, seed=36, old="noisy")
    ref = O.reference_value_and_grad(logits, inputs)
    x = logits[:, :T].contiguous().to(cuda).requires_grad_(True)
    din = to_device(inputs, cuda)
    out = G.grpo_token_loss_flat(x, din["input_ids"][:, 1:], din["labels"][:, 1:], din["advantages"],
                                 din["total_valid_token_count"], din["old_per_token_logps"])
    (out["loss"] * 3.0).backward()
    assert_loss_close(out["loss"].item(), ref["loss"].item())
    assert_dlogits_close(x.grad, 3.0 * ref["dlogits"][:, :T], what="flat")


def test_default_total_valid_is_mask_sum(cuda):
    logits, inputs = make_case(2, 9, 300, seed=37, old="noisy")
    inputs.pop("total_valid_token_count")
    ref, got = run_both(logits, inputs, cuda)
    check(ref, got, "default Nv")


def test_logprobs_only(cuda):
    logits, inputs = make_case(2, 9, 7001, seed=38, old="none")
    ref = O.reference_call(logits, inputs, temperature=1.0)
    out = G.token_logprobs(logits.to(cuda), inputs["input_ids"].to(cuda), shifted=True, compute_entropy=True)
    assert (out["per_token_logps"].cpu() - ref["per_token_logps"]).abs().max() <= LP_ATOL
    assert (out["token_entropy"].cpu() - ref["token_entropy"]).abs().max() <= ENT_ATOL


@pytest.mark.parametrize("k", [2, 4, 8])
@pytest.mark.parametrize("softcap", [None, 30.0])
def test_vocab_shards_on_one_gpu(cuda, k, softcap):
    """k column shards run one after the other on one GPU, then combined: equals the oracle."""
    B, L, V = 2, 6, 1024 * k
    logits, inputs = make_case(B, L, V, seed=39 + k, old="wide", ref=True, sigma=4.0 if softcap else 2.0)
    attrs = dict(beta=0.04, softcap=softcap)
    ref = O.reference_value_and_grad(logits, inputs, **attrs)
    din = to_device(inputs, cuda)
    x = logits.to(cuda)
    cfg = G.LossConfig(beta=0.04, softcap=softcap)
    N, Vs = B * (L - 1), V // k
    gathered = torch.empty(k, N, 4, device=cuda)
    probs = []
    for r in range(k):
        shard = x[:, :, r * Vs:(r + 1) * Vs]  # a view: row stride V, columns of shard r
        p = G.TokenLossProblem(shard, din["input_ids"][:, 1:], din["labels"][:, 1:], din["advantages"],
                               din["total_valid_token_count"], din["old_per_token_logps"],
                               din["ref_per_token_logps"], cfg, scored_rows=L - 1, vocab=Vs, vocab_start=r * Vs,
                               vocab_total=V)
        p.partials = gathered[r]
        p.run("mllm_grpo_fwd_partials")
        probs.append(p)
    want = np.stack([O.shard_partials(logits[:, :-1, r * Vs:(r + 1) * Vs].double().numpy().reshape(N, Vs),
                                      inputs["input_ids"][:, 1:].numpy().reshape(-1), r * Vs, softcap)
                     for r in range(k)])
    assert np.allclose(gathered.cpu().numpy(), want, rtol=2e-4, atol=1e-5)
    dfull = torch.empty_like(x)
    for r, p in enumerate(probs):
        p.gathered, p.n_shards = gathered, k
        p.run("mllm_grpo_combine")
        p.dlogits = dfull[:, :, r * Vs:(r + 1) * Vs]
        p.run("mllm_grpo_bwd")
    torch.cuda.synchronize()
    got = {"loss": probs[0].loss[0], "per_token_logps": probs[0].per_token_logps,
           "token_entropy": probs[0].token_entropy, "dlogits": dfull}
    check(ref, got, f"k={k}")
    for p in probs[1:]:  # every shard reaches the same replicated outputs
        assert torch.equal(p.per_token_logps, probs[0].per_token_logps)
        assert torch.equal(p.loss, probs[0].loss)


def test_vocab_shards_entropy_at_other_temperatures(cuda):
    """Entropy of softmax(y / temperature) from vocabulary shards: the partial record grows to six floats (two
    more sums on y/temperature), merged like the others (MLLM_JAX/train_modules/__init__.py:136-138 under the
    tp sharding of MLLM_JAX/utils.py:245)."""
    from mllm_jax_b200 import _lib

    B, L, V, k, temp = 2, 9, 4 * 1000, 4, 0.7
    logits, inputs = make_case(B, L, V, seed=45, old="wide", ref=True)
    logits[0, 2, 100:900] = float("-inf")
    attrs = dict(beta=0.04, temperature=temp)
    ref = O.reference_value_and_grad(logits, inputs, **attrs)
    din = to_device(inputs, cuda)
    x = logits.to(cuda)
    cfg = G.LossConfig(beta=0.04, temperature=temp)
    N, Vs = B * (L - 1), V // k
    probs = []
    for r in range(k):
        p = G.TokenLossProblem(x[:, :, r * Vs:(r + 1) * Vs], din["input_ids"][:, 1:], din["labels"][:, 1:],
                               din["advantages"], din["total_valid_token_count"], din["old_per_token_logps"],
                               din["ref_per_token_logps"], cfg, scored_rows=L - 1, vocab=Vs, vocab_start=r * Vs,
                               vocab_total=V)
        probs.append(p)
    width = int(_lib.load().mllm_grpo_partial_width(probs[0].args()))
    assert width == 6
    gathered = torch.empty(k, N, width, device=cuda)
    for r, p in enumerate(probs):
        p.partials = gathered[r]
        p.run("mllm_grpo_fwd_partials")
    want = np.stack([O.shard_partials(logits[:, :-1, r * Vs:(r + 1) * Vs].double().numpy().reshape(N, Vs),
                                      inputs["input_ids"][:, 1:].numpy().reshape(-1), r * Vs, None, temp)
                     for r in range(k)])
    finite = np.isfinite(want)
    assert np.allclose(gathered.cpu().numpy()[finite], want[finite], rtol=3e-4, atol=1e-5)
    dfull = torch.empty_like(x)
    for r, p in enumerate(probs):
        p.gathered, p.n_shards = gathered, k
        p.run("mllm_grpo_combine")
        p.dlogits = dfull[:, :, r * Vs:(r + 1) * Vs]
        p.run("mllm_grpo_bwd")
    torch.cuda.synchronize()
    got = {"loss": probs[0].loss[0], "per_token_logps": probs[0].per_token_logps,
           "token_entropy": probs[0].token_entropy, "dlogits": dfull}
    check(ref, got, "entropy from shards at temperature 0.7")


@pytest.mark.parametrize("eager", [False, True])
def test_golden_fixtures(cuda, eager):
    """Committed fixtures through both autograd forms: separate forward / backward kernels, and the
    eager form the module mirror uses (loss and gradient from one kernel)."""
    for f in sorted(os.listdir(GOLDEN)):
        if not f.endswith(".npz"):
            continue
        z = np.load(os.path.join(GOLDEN, f))
        logits = torch.from_numpy(z["logits_bf16_bits"].astype(np.int16)).view(torch.bfloat16).to(cuda)
        kw = dict(temperature=float(z["temperature"]), epsilon_low=float(z["epsilon_low"]),
                  epsilon_high=float(z["epsilon_high"]), beta=float(z["beta"]), softcap=float(z["softcap"]) or None)
        old = torch.from_numpy(z["old_per_token_logps"]).to(cuda) if "old_per_token_logps" in z.files else None
        rf = torch.from_numpy(z["ref_per_token_logps"]).to(cuda) if "ref_per_token_logps" in z.files else None
        x = logits.clone().requires_grad_(True)
        out = G.grpo_token_loss(x, torch.from_numpy(z["input_ids"]).to(cuda), torch.from_numpy(z["labels"]).to(cuda),
                                torch.from_numpy(z["advantages"]).to(cuda), float(z["total_valid_token_count"]),
                                old, rf, eager_grad=eager, **kw)
        out["loss"].backward()
        ref = {"loss": torch.tensor(float(z["loss"])), "per_token_logps": torch.from_numpy(z["per_token_logps"]),
               "token_entropy": torch.from_numpy(z["token_entropy"]), "dlogits": torch.from_numpy(z["dlogits"])}
        got = {"loss": out["loss"].detach(), "per_token_logps": out["per_token_logps"],
               "token_entropy": out["token_entropy"], "dlogits": x.grad}
        check(ref, got, f)


def test_module_mirror_matches_reference_dict(cuda):
    """TrainGRPOModule(inputs) returns the reference's dict; gradients reach the model's parameters."""
    B, L, V, H = 3, 120, 640, 32
    g = torch.Generator().manual_seed(40)
    hidden = torch.randn(B, L, H, generator=g)
    weight = torch.randn(H, V, generator=g) * 0.5
    _, inputs = make_case(B, L, V, seed=41, old="none")
    w_gpu = weight.to(cuda).requires_grad_(True)

    def model(input_ids, attention_mask):
        return (hidden.to(cuda) @ w_gpu).to(torch.bfloat16), None

    mod = G.TrainGRPOModule(model=model, pad_token_id=0, num_pre_Q=8, beta=0.0)
    out = mod(to_device(inputs, cuda))
    out["loss"].backward()
    # oracle on the same bf16 logits
    logits = (hidden.to(cuda) @ weight.to(cuda)).to(torch.bfloat16).cpu()
    ref = O.reference_value_and_grad(logits, inputs, beta=0.0)
    assert set(out) == {"loss", "per_token_logps", "entropy", "entropy_loss"}
    assert_loss_close(out["loss"].item(), ref["loss"].item())
    assert torch.allclose(out["entropy"].cpu(), ref["entropy"], atol=ENT_ATOL, equal_nan=True)
    assert torch.allclose(out["entropy_loss"].cpu(), ref["entropy_loss"], atol=ENT_ATOL, equal_nan=True)
    dW = hidden.reshape(-1, H).T @ ref["dlogits"].reshape(-1, V)
    rel = (w_gpu.grad.cpu() - dW).abs().max() / dW.abs().max()
    assert rel < 2e-2


def test_ppo_policy_terms(cuda):
    logits, inputs = make_case(2, 30, 900, seed=42, old="wide", per_token_adv=True)
    ref = O.ppo_policy_call(logits, inputs)
    out = G.ppo_policy_terms(logits.to(cuda), to_device(inputs, cuda))
    assert_loss_close(out["policy_loss"].item(), ref["policy_loss"].item())
    assert abs(out["entropy"].item() - ref["entropy"].item()) <= ENT_ATOL
    with pytest.raises(ValueError):
        G.ppo_policy_terms(logits.to(cuda), {**to_device(inputs, cuda), "advantages": torch.zeros(2, 4)})


def test_out_of_range_ids_are_clamped_and_flagged(cuda):
    logits, inputs = make_case(1, 4, 100, seed=43, old="none", mask_kind="ones")
    bad = {**inputs, "input_ids": inputs["input_ids"].clone()}
    bad["input_ids"][0, 2] = 100
    bad["input_ids"][0, 3] = -4
    fixed = {**inputs, "input_ids": bad["input_ids"].clamp(0, 99)}
    ref = O.reference_call(logits, fixed)
    din = to_device(bad, cuda)
    prob = G.TokenLossProblem(logits.to(cuda), din["input_ids"][:, 1:], din["labels"][:, 1:], din["advantages"],
                              3.0, None, None, G.LossConfig(), scored_rows=3)
    prob.run("mllm_grpo_fwd")
    assert (prob.per_token_logps.cpu() - ref["per_token_logps"]).abs().max() <= LP_ATOL
    assert G.ops.check_device_status(prob) & 1


def test_deterministic_repeat(cuda):
    logits, inputs = make_case(4, 33, 3001, seed=44, old="wide", ref=True)
    x, din = logits.to(cuda), to_device(inputs, cuda)
    outs = []
    for _ in range(3):
        o = G.grpo_value_and_grad(x, din["input_ids"], din["labels"], din["advantages"],
                                  din["total_valid_token_count"], din["old_per_token_logps"],
                                  din["ref_per_token_logps"], shifted=True, cfg=G.LossConfig(beta=0.04))
        outs.append((o["loss"].clone(), o["dlogits"].clone()))
    assert all(torch.equal(outs[0][0], o[0]) and torch.equal(outs[0][1], o[1]) for o in outs[1:])


def test_full_size_workload_properties(cuda):
    """The benchmark workload (32768 x 151936) is too big for the oracle: check sampled rows against
    it, and size-independent properties on everything (row sums ~ 0, zero rows exactly zero,
    loss equals the sum over sampled + unsampled rows recomputed from per-token outputs)."""
    w = synth.CONFIGS["cfg1"]
    data = synth.make_inputs(w, seed=0, device="cuda")
    cfg = G.LossConfig(epsilon_low=w.epsilon_low, epsilon_high=w.epsilon_high, beta=w.beta)
    out = G.grpo_value_and_grad(data["logits"], data["token_ids"], data["mask"], data["advantages"],
                                data["total_valid"], data["old_logps"], data["ref_logps"], cfg=cfg)
    torch.cuda.synchronize()
    N, V = w.n_tokens, w.vocab
    d = out["dlogits"].view(N, V)
    mask = data["mask"].view(N)
    # zero rows are exactly zero; every row sums to ~0 (bf16 rounding of V terms)
    rs = torch.empty(N, device=cuda)
    absmax = torch.empty(N, device=cuda)
    for s in range(0, N, 2048):
        blk = d[s:s + 2048].float()
        rs[s:s + 2048] = blk.sum(1)
        absmax[s:s + 2048] = blk.abs().amax(1)
    assert (absmax[mask == 0] == 0).all()
    assert (absmax[mask == 1] > 0).float().mean() > 0.99
    assert (rs.abs() <= 0.02 * absmax + 1e-12).all()
    # sampled rows against the closed-form oracle
    gen = torch.Generator().manual_seed(7)
    rows = torch.cat([torch.tensor([0, N - 1]), torch.randint(0, N, (510,), generator=gen)]).unique()
    x = data["logits"].view(N, V)[rows.to(cuda)].double().cpu().numpy()
    advN = data["advantages"][:, None].expand(w.n_seqs, w.seq_len).reshape(N)
    pick = lambda t: t.reshape(N)[rows.to(cuda)].double().cpu().numpy()  # noqa: E731
    an = O.analytic_rows(x, data["token_ids"].reshape(N)[rows.to(cuda)].long().cpu().numpy(), pick(mask), pick(advN),
                         pick(data["old_logps"]), pick(data["ref_logps"]), data["total_valid"], beta=w.beta,
                         epsilon_low=w.epsilon_low, epsilon_high=w.epsilon_high)
    assert np.abs(pick(out["per_token_logps"]) - an["lp"]).max() <= LP_ATOL
    assert np.abs(pick(out["token_entropy"]) - an["entropy_guard"]).max() <= ENT_ATOL
    assert_dlogits_close(d[rows.to(cuda)], torch.from_numpy(an["dlogits"]), what="cfg1 sampled rows")
    # the loss equals the fixed-order sum of the per-token terms the kernel wrote
    terms = out["problem"].loss_terms.double().sum().item() / data["total_valid"]
    assert_loss_close(out["loss"].item(), terms)
    # and the sampled terms match the oracle's
    assert np.allclose(out["problem"].loss_terms[rows.to(cuda)].cpu().numpy(), an["loss_terms"], atol=2e-3)


def test_sft_cross_entropy(cuda):
    """Masked causal-LM cross-entropy (the SFT plugin's loss) on the same kernels, against the oracle."""
    B, L, V = 3, 21, 5000
    logits, inputs = make_case(B, L, V, seed=45, old="none")
    labels = inputs["input_ids"].clone().long()
    labels[:, :5] = -100  # prompt positions are not supervised
    att = torch.ones(B, L, dtype=torch.int32)
    att[1, 15:] = 0  # padding
    x = logits.float().requires_grad_(True)
    ref = O.sft_call(x, {"labels": labels, "attention_mask": att})
    ref["loss"].backward()
    xg = logits.to(cuda).requires_grad_(True)
    out = G.sft_cross_entropy(xg, inputs["input_ids"].to(cuda), labels.to(cuda), att.to(cuda))
    out["loss"].backward()
    assert int(out["token_count"]) == int(ref["token_count"])
    assert_loss_close(out["loss"].item(), ref["loss"].item())
    assert_dlogits_close(xg.grad, x.grad, what="sft cross-entropy")
    # no supervised token at all: loss 0 and zero gradient (denominator clamps to 1)
    none = torch.full_like(labels, -100)
    xz = logits.to(cuda).requires_grad_(True)
    z = G.sft_cross_entropy(xz, inputs["input_ids"].to(cuda), none.to(cuda), att.to(cuda))
    z["loss"].backward()
    assert z["loss"].item() == 0.0 and int(z["token_count"]) == 0 and (xz.grad == 0).all()


@pytest.mark.parametrize("B,T", [(1, 1), (3, 7), (4, 130), (2, 5000)])
def test_entropy_stats_kernel(cuda, B, T):
    """Per-sample entropy monitors: the kernel against the host restatement of train_modules :141-157."""
    from mllm_jax_b200.train_module import per_sample_entropy, per_sample_entropy_cuda

    g = torch.Generator().manual_seed(46 + T)
    H = torch.rand(B, T, generator=g) * 5
    mask = (torch.rand(B, T, generator=g) < 0.7).to(torch.int32)
    if B > 1:
        mask[1] = 0  # a sample without valid tokens: 0/0
    want = per_sample_entropy(H, mask)
    got = per_sample_entropy_cuda(H.to(cuda), mask.to(cuda))
    for w, gt in zip(want, got):
        assert torch.allclose(gt.cpu(), w, atol=1e-5, rtol=1e-5, equal_nan=True)


@pytest.mark.parametrize("scale", [1.0, -2.5])
def test_eager_gradient_in_forward(cuda, scale):
    """eager_grad: dlogits come out of the forward kernel; a late cotangent is applied in place."""
    logits, inputs = make_case(3, 17, 4096, seed=47, old="wide", ref=True)
    ref = O.reference_value_and_grad(logits, inputs, beta=0.04)
    din = to_device(inputs, cuda)
    x = logits.to(cuda).requires_grad_(True)
    before = G.launch_count()
    out = G.grpo_token_loss(x, din["input_ids"], din["labels"], din["advantages"], din["total_valid_token_count"],
                            din["old_per_token_logps"], din["ref_per_token_logps"], beta=0.04, eager_grad=True)
    (out["loss"] * scale).backward()
    torch.cuda.synchronize()
    assert G.launch_count() - before == 3  # two-pass kernel, loss reduction, cotangent check
    assert_loss_close(out["loss"].item(), ref["loss"].item())
    assert_dlogits_close(x.grad, scale * ref["dlogits"], what="eager")


def test_minus_infinity_logits(cuda):
    """Vocabulary entries masked with -inf: log-probs, loss and dlogits stay exact, and the entropy
    monitor counts such entries as 0 like the reference's p * log(p + 1e-9) does
    (MLLM_JAX/train_modules/__init__.py:138)."""
    from mllm_jax_b200._lib import plan_override

    B, L, V = 2, 6, 4096
    logits, inputs = make_case(B, L, V, seed=48, old="none")
    logits[:, :, 1000:1500] = float("-inf")
    logits[0, 1, 3000:] = float("-inf")  # one row has more of them, the others keep the common path
    inputs["input_ids"] = inputs["input_ids"] % 1000  # chosen tokens are finite
    ref = O.reference_value_and_grad(logits, inputs)
    assert torch.isfinite(ref["token_entropy"]).all()
    x = logits.to(cuda)
    din = to_device(inputs, cuda)
    for kw in (dict(), dict(sweeps=True), dict(cluster=2, threads=128), dict(cluster=1, threads=256, staged=1)):
        with plan_override(**kw):
            out = G.grpo_value_and_grad(x, din["input_ids"], din["labels"], din["advantages"],
                                        din["total_valid_token_count"], None, None, shifted=True)
        assert (out["per_token_logps"].cpu() - ref["per_token_logps"]).abs().max() <= LP_ATOL
        assert (out["token_entropy"].cpu() - ref["token_entropy"]).abs().max() <= ENT_ATOL, kw
        assert_loss_close(out["loss"].item(), ref["loss"].item())
        assert_dlogits_close(out["dlogits"], ref["dlogits"], what=f"-inf logits {kw}")
        assert (out["dlogits"][:, :, 1000:1500] == 0).all()
    # temperature != 1: the entropy's own pair of sums is repaired the same way
    ref_t = O.reference_value_and_grad(logits, inputs, temperature=0.7)
    out = G.grpo_value_and_grad(x, din["input_ids"], din["labels"], din["advantages"],
                                din["total_valid_token_count"], None, None, shifted=True,
                                cfg=G.LossConfig(temperature=0.7))
    assert (out["token_entropy"].cpu() - ref_t["token_entropy"]).abs().max() <= ENT_ATOL


def test_extreme_logits_and_tiny_vocab(cuda):
    """bf16 extremes (+-3e38 entries, a 1e4 spike) and a one-column vocabulary."""
    B, L, V = 1, 5, 256
    logits, inputs = make_case(B, L, V, seed=49, old="none", mask_kind="ones")
    logits[0, 0, 3] = 1.0e4
    logits[0, 1, 7] = -3.0e38
    logits[0, 2, :] = -3.0e38
    logits[0, 2, 5] = 3.0e38
    ref = O.reference_value_and_grad(logits, inputs)
    out = G.grpo_value_and_grad(logits.to(cuda), inputs["input_ids"].to(cuda), inputs["labels"].to(cuda),
                                inputs["advantages"].to(cuda), inputs["total_valid_token_count"], shifted=True)
    finite = torch.isfinite(ref["per_token_logps"])
    assert torch.equal(torch.isfinite(out["per_token_logps"].cpu()), finite)
    assert (out["per_token_logps"].cpu()[finite] - ref["per_token_logps"][finite]).abs().max() <= LP_ATOL
    # one column: log-prob 0, entropy 0, zero gradient
    one = torch.randn(2, 4, 1, generator=torch.Generator().manual_seed(64)).to(torch.bfloat16)
    ids = torch.zeros(2, 4, dtype=torch.int32)
    o1 = G.grpo_value_and_grad(one.to(cuda), ids.to(cuda), torch.ones(2, 4, dtype=torch.int32).to(cuda),
                               torch.tensor([1.0, -1.0]).to(cuda), 6.0, shifted=True)
    assert o1["per_token_logps"].abs().max() == 0 and o1["token_entropy"].abs().max() == 0
    # g*(softmax - onehot) with softmax == 1: zero up to the f32 rounding of g*e^(x - lse) against g (|g| <= 1/6)
    assert o1["dlogits"].float().abs().max() <= 1e-6 and o1["loss"].item() == 0.0


@pytest.mark.parametrize("name,rows", [("cfg2", 4), ("cfg3", 2)])
def test_other_config_shapes_sampled_rows(cuda, name, rows):
    """Llama-3 (V=128256) and Gemma-2 (V=256000, soft-cap 30, logits ~ N(0, 4^2)) shapes at a few
    thousand rows: sampled rows against the closed-form oracle, zero rows exactly zero."""
    w = synth.scaled(synth.CONFIGS[name], n_seqs=rows)
    data = synth.make_inputs(w, seed=3, device="cuda")
    cfg = G.LossConfig(epsilon_low=w.epsilon_low, epsilon_high=w.epsilon_high, beta=w.beta, softcap=w.softcap)
    out = G.grpo_value_and_grad(data["logits"], data["token_ids"], data["mask"], data["advantages"],
                                data["total_valid"], data["old_logps"], data["ref_logps"], cfg=cfg)
    torch.cuda.synchronize()
    N, V = w.n_tokens, w.vocab
    d = out["dlogits"].view(N, V)
    mask = data["mask"].view(N)
    gen = torch.Generator().manual_seed(11)
    rows_idx = torch.cat([torch.tensor([0, N - 1]), torch.randint(0, N, (126,), generator=gen)]).unique().to(cuda)
    x = data["logits"].view(N, V)[rows_idx].double().cpu().numpy()
    advN = data["advantages"][:, None].expand(w.n_seqs, w.seq_len).reshape(N)
    pick = lambda t: t.reshape(N)[rows_idx].double().cpu().numpy()  # noqa: E731
    an = O.analytic_rows(x, data["token_ids"].reshape(N)[rows_idx].long().cpu().numpy(), pick(mask), pick(advN),
                         pick(data["old_logps"]), pick(data["ref_logps"]), data["total_valid"], beta=w.beta,
                         epsilon_low=w.epsilon_low, epsilon_high=w.epsilon_high, softcap=w.softcap)
    assert np.abs(pick(out["per_token_logps"]) - an["lp"]).max() <= LP_ATOL
    assert np.abs(pick(out["token_entropy"]) - an["entropy_guard"]).max() <= ENT_ATOL
    assert_dlogits_close(d[rows_idx], torch.from_numpy(an["dlogits"]), what=f"{name} sampled rows")
    zero = (mask == 0).nonzero()[:64, 0]
    assert (d[zero] == 0).all()


def test_chunked_lm_head_and_loss(cuda):
    """hidden @ W^T and the loss chunk by chunk: equals the oracle on the full logits, and the
    chunk size does not change the result."""
    from mllm_jax_b200.linear_loss import linear_grpo_value_and_grad

    B, T, H, V = 6, 17, 64, 4096
    g = torch.Generator().manual_seed(50)
    hidden = (torch.randn(B, T, H, generator=g) * 0.5).to(torch.bfloat16).to(cuda)
    weight = (torch.randn(V, H, generator=g) * 0.5).to(torch.bfloat16).to(cuda)
    logits = torch.matmul(hidden, weight.t())  # what the chunks will hold
    _, inputs = make_case(B, T + 1, V, seed=51, old="none")
    ids, mask = inputs["input_ids"][:, 1:], inputs["labels"][:, 1:]
    lg = logits.float().cpu()
    lp0 = torch.log_softmax(lg, -1).gather(-1, ids.long()[..., None])[..., 0]
    old = lp0 + 0.3 * torch.randn(B, T, generator=g)
    nv = float(mask.sum())
    # oracle on the shifted layout: append a dummy last row, prepend a dummy id / label
    z = torch.zeros(B, 1, dtype=ids.dtype)
    oin = {"input_ids": torch.cat([z, ids], 1), "labels": torch.cat([z, mask], 1), "advantages": inputs["advantages"],
           "total_valid_token_count": nv, "old_per_token_logps": old}
    ref = O.reference_value_and_grad(torch.cat([logits.cpu(), logits.cpu()[:, :1]], 1), oin)
    dl = ref["dlogits"][:, :T].reshape(B * T, V)
    dW_ref = dl.t() @ hidden.float().cpu().reshape(B * T, H)
    dH_ref = (dl @ weight.float().cpu()).reshape(B, T, H)
    outs = []
    for chunk in (T, 3 * T, 10 ** 6):
        out = linear_grpo_value_and_grad(hidden, weight, ids.to(cuda), mask.to(cuda), inputs["advantages"].to(cuda),
                                         nv, old.to(cuda), chunk_rows=chunk)
        torch.cuda.synchronize()
        assert (out["per_token_logps"].cpu() - ref["per_token_logps"]).abs().max() <= LP_ATOL
        assert_loss_close(out["loss"].item(), ref["loss"].item())
        assert (out["dweight"].cpu() - dW_ref).abs().max() <= 2e-2 * dW_ref.abs().max()
        assert (out["dhidden"].float().cpu() - dH_ref).abs().max() <= 2e-2 * dH_ref.abs().max()
        outs.append(out)
    assert torch.equal(outs[0]["per_token_logps"], outs[2]["per_token_logps"])
    assert torch.equal(outs[0]["dhidden"], outs[2]["dhidden"])


@pytest.mark.parametrize("clip", [0.2, None])
@pytest.mark.parametrize("returns", ["given", "per_sample", "absent"])
@pytest.mark.parametrize("old", ["given", "absent"])
def test_ppo_value_loss(cuda, clip, returns, old):
    """Value-loss tail of the PPO module: loss, monitors and the gradient with respect to the values."""
    B, L = 5, 301
    g = torch.Generator().manual_seed(61)
    values = torch.randn(B, L, generator=g)
    labels = (torch.rand(B, L, generator=g) < 0.6).float()
    inputs = {"labels": labels, "advantages": torch.randn(B, generator=g)}
    if returns == "given":
        inputs["returns"] = values[:, :-1] + torch.randn(B, L - 1, generator=g)
    elif returns == "per_sample":
        inputs["returns"] = torch.randn(B, 1, generator=g)
    if old == "given":
        inputs["old_values"] = values[:, :-1] + 0.3 * torch.randn(B, L - 1, generator=g)
    for tv in (None, 777.0):
        if tv is not None:
            inputs["total_valid_token_count"] = tv
        v = values.clone().requires_grad_(True)
        ref = O.ppo_value_call(v, inputs, value_clip_range=clip)
        (0.5 * ref["value_loss"]).backward()
        out = G.ppo_value_loss(values.to(cuda), to_device(inputs, cuda), value_clip_range=clip, value_coef=0.5)
        torch.cuda.synchronize()
        for key in ("value_loss", "value_pred_mean", "return_mean"):
            assert out[key].item() == pytest.approx(ref[key].item(), rel=1e-5, abs=1e-6), key
        dref = v.grad
        assert (out["dvalues"].cpu() - dref).abs().max() <= 1e-5 * dref.abs().max() + 1e-9
        assert (out["dvalues"][:, -1] == 0).all()
    with pytest.raises(ValueError):
        G.ppo_value_loss(values.to(cuda), {**to_device(inputs, cuda), "returns": torch.zeros(B, 4)})


def test_ppo_actor_critic_terms(cuda):
    """Return dict of the PPO module: total loss and its gradient into the value head and the logits."""
    logits, inputs = make_case(3, 40, 700, seed=62, old="wide", per_token_adv=True)
    g = torch.Generator().manual_seed(63)
    values = torch.randn(3, 40, generator=g)
    inputs = {**inputs, "returns": torch.randn(3, 39, generator=g), "old_values": values[:, :-1] + 0.25}
    v = values.clone().requires_grad_(True)
    ref_p = O.ppo_policy_call(logits, inputs)
    ref_v = O.ppo_value_call(v, inputs, value_clip_range=0.2)
    ref_loss = ref_p["policy_loss"] + 0.5 * ref_v["value_loss"]
    ref_loss.backward()
    x = logits.to(cuda).requires_grad_(True)
    vg = values.to(cuda).requires_grad_(True)
    out = G.ppo_actor_critic_terms(x, vg, to_device(inputs, cuda))
    out["loss"].backward()
    torch.cuda.synchronize()
    assert_loss_close(out["loss"].item(), ref_loss.item())
    assert_loss_close(out["value_loss"].item(), ref_v["value_loss"].item())
    assert (vg.grad.cpu() - v.grad).abs().max() <= 1e-5 * v.grad.abs().max()
    assert x.grad is not None and x.grad.abs().max() > 0
    assert sorted(out) == sorted(["loss", "policy_loss", "value_loss", "entropy", "value_pred_mean", "return_mean",
                                  "per_token_logps"])


@pytest.mark.parametrize("temperature", [1.0, 0.7])
@pytest.mark.parametrize("softcap", [None, 30.0])
def test_ppo_entropy_coef_reaches_the_logits(cuda, temperature, softcap):
    """loss = policy_loss + value_coef * value_loss - entropy_coef * entropy (plugins/training/ppo/module.py:140):
    with entropy_coef != 0 the entropy's gradient is added to dlogits inside the backward sweep."""
    logits, inputs = make_case(3, 21, 1544, seed=64, old="wide", per_token_adv=True, sigma=3.0 if softcap else 2.0)
    logits[0, 2, 100:300] = float("-inf")
    g = torch.Generator().manual_seed(65)
    values = torch.randn(3, 21, generator=g)
    inputs = {**inputs, "returns": torch.randn(3, 20, generator=g)}
    coef = 0.37
    xr = logits.float().requires_grad_(True)
    capped = xr if softcap is None else torch.tanh(xr / softcap) * softcap
    ref_p = O.ppo_policy_call(capped, inputs, temperature=temperature, detach_entropy=False)
    ref_v = O.ppo_value_call(values, inputs, value_clip_range=0.2)
    ref_loss = ref_p["policy_loss"] + 0.5 * ref_v["value_loss"] - coef * ref_p["entropy"]
    ref_loss.backward()
    x = logits.to(cuda).requires_grad_(True)
    if softcap is None:
        out = G.ppo_actor_critic_terms(x, values.to(cuda), to_device(inputs, cuda), temperature=temperature,
                                       entropy_coef=coef)
        loss = out["loss"]
    else:  # the PPO module has no soft-cap; drive the operator directly
        din = to_device(inputs, cuda)
        o = G.grpo_token_loss(x, din["input_ids"], din["labels"], din["advantages"], din["total_valid_token_count"],
                              din["old_per_token_logps"], temperature=temperature, epsilon_low=0.2, epsilon_high=0.2,
                              softcap=softcap, entropy_grad=True)
        m = din["labels"][:, 1:].float()
        loss = o["loss"] + 0.5 * ref_v["value_loss"].item() - coef * (o["token_entropy"] * m).sum() / (m.sum() + 1e-8)
    loss.backward()
    torch.cuda.synchronize()
    assert_loss_close(loss.item(), ref_loss.item())
    assert_dlogits_close(x.grad, xr.grad, what=f"entropy_coef temperature={temperature} softcap={softcap}")


@pytest.mark.parametrize("V", [18992, 50000, 151936])
def test_cuda_graph_capture_and_replay(cuda, V):
    """The entry points enqueue on the caller's stream, allocate nothing and never synchronise, so a
    step can be captured in a CUDA graph; replays reproduce the eager launch bit for bit (staged
    short rows, register-fed rows and the cluster split of long rows)."""
    logits, inputs = make_case(2, 9, V, seed=70, old="wide", ref=True)
    din = to_device(inputs, cuda)
    out = G.grpo_value_and_grad(logits.to(cuda), din["input_ids"], din["labels"], din["advantages"],
                                din["total_valid_token_count"], din["old_per_token_logps"],
                                din["ref_per_token_logps"], shifted=True, cfg=G.LossConfig(beta=0.04))
    prob = out["problem"]
    torch.cuda.synchronize()
    want = [t.clone() for t in (prob.dlogits, prob.loss, prob.per_token_logps, prob.token_entropy)]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        prob.run("mllm_grpo_fwd_bwd", reuse_args=True)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        prob.run("mllm_grpo_fwd_bwd", reuse_args=True)
    for _ in range(2):
        for t in (prob.dlogits, prob.loss, prob.per_token_logps, prob.token_entropy):
            t.fill_(7.0)
        graph.replay()
        torch.cuda.synchronize()
        for got, ref in zip((prob.dlogits, prob.loss, prob.per_token_logps, prob.token_entropy), want):
            assert torch.equal(got, ref)
