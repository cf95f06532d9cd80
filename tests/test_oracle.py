"""Pins the CPU oracle: known answers derivable by hand, two independent derivations
(torch autograd restatement vs closed-form NumPy float64) agreeing, finite differences,
and the committed golden fixtures.  No GPU."""
import math
import os

import numpy as np
import pytest
import torch

from oracle import grpo_oracle as O
from tests.util import make_case

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _rows(logits, inputs):
    """Flatten the reference layout into aligned rows for analytic_rows."""
    B, L, V = logits.shape
    x = logits[:, :-1].double().numpy().reshape(-1, V)
    c = inputs["input_ids"][:, 1:].long().numpy().reshape(-1)
    m = inputs["labels"][:, 1:].double().numpy().reshape(-1)
    adv = inputs["advantages"].double()
    adv = (adv[:, None].expand(B, L - 1) if adv.dim() == 1 else adv).numpy().reshape(-1)
    old = inputs.get("old_per_token_logps")
    ref = inputs.get("ref_per_token_logps")
    old = None if old is None else old.double().numpy().reshape(-1)
    ref = None if ref is None else ref.double().numpy().reshape(-1)
    return x, c, m, adv, old, ref


def test_constant_logits_give_uniform_logprob_and_entropy():
    B, L, V = 2, 5, 1000
    logits = torch.full((B, L, V), 0.75, dtype=torch.bfloat16)
    _, inputs = make_case(B, L, V, seed=1, old="none")
    out = O.reference_call(logits, inputs)
    assert torch.allclose(out["per_token_logps"], torch.full((B, L - 1), -math.log(V)), atol=1e-5)
    assert torch.allclose(out["token_entropy"], torch.full((B, L - 1), math.log(V)), atol=1e-4)


def test_ratio_one_loss_is_minus_masked_advantage_mean():
    logits, inputs = make_case(3, 7, 257, seed=2, old="none")
    out = O.reference_value_and_grad(logits, inputs)
    m = inputs["labels"][:, 1:].float()
    expect = -(inputs["advantages"][:, None] * m).sum() / inputs["total_valid_token_count"]
    assert abs(out["loss"].item() - expect.item()) < 1e-6
    # dlogits = -(A m / Nv) (onehot - softmax)
    p = torch.softmax(logits[:, :-1].float(), -1)
    onehot = torch.zeros_like(p).scatter_(-1, inputs["input_ids"][:, 1:].long()[..., None], 1.0)
    g = -(inputs["advantages"][:, None] * m / inputs["total_valid_token_count"])[..., None] * (onehot - p)
    assert torch.allclose(out["dlogits"][:, :-1], g, atol=1e-7)
    assert (out["dlogits"][:, -1] == 0).all()


def test_dominant_logit():
    B, L, V = 1, 4, 300
    logits = torch.zeros(B, L, V, dtype=torch.bfloat16)
    ids = torch.tensor([[5, 17, 42, 99]], dtype=torch.int32)
    for t in range(L - 1):
        logits[0, t, ids[0, t + 1]] = 50.0
    inputs = {"input_ids": ids, "labels": torch.ones(B, L, dtype=torch.int32), "advantages": torch.ones(B)}
    out = O.reference_call(logits, inputs)
    assert out["per_token_logps"].abs().max() < 1e-6
    assert out["token_entropy"].abs().max() < 1e-6


def test_rows_sum_to_zero_and_masked_rows_are_zero():
    logits, inputs = make_case(4, 9, 129, seed=3, old="wide", ref=True)
    out = O.reference_value_and_grad(logits, inputs, beta=0.04)
    d = out["dlogits"]
    assert d.sum(-1).abs().max() < 1e-6
    m = inputs["labels"][:, 1:]
    assert (d[:, :-1][m == 0] == 0).all()
    assert (d[:, -1] == 0).all()


@pytest.mark.parametrize("ratio,A,expect_grad", [(1.5, 1.0, False), (1.5, -1.0, True), (0.5, 1.0, True),
                                                 (0.5, -1.0, False), (1.1, 1.0, True), (0.9, -1.0, True)])
def test_clip_gating(ratio, A, expect_grad):
    """The four zero / non-zero gradient cases of PPO clipping, plus two inside the interval."""
    V = 17
    logits, inputs = make_case(1, 2, V, seed=4, old="none", mask_kind="ones")
    lp = torch.log_softmax(logits[:, :-1].float(), -1).gather(-1, inputs["input_ids"][:, 1:].long()[..., None])[..., 0]
    inputs["old_per_token_logps"] = lp - math.log(ratio)
    inputs["advantages"] = torch.tensor([A])
    inputs["total_valid_token_count"] = 1.0
    out = O.reference_value_and_grad(logits, inputs, epsilon_low=0.2, epsilon_high=0.3)
    has_grad = out["dlogits"].abs().max().item() > 0
    assert has_grad == expect_grad
    x, c, m, adv, old, ref = _rows(logits, inputs)
    an = O.analytic_rows(x, c, m, adv, old, ref, 1.0, epsilon_low=0.2, epsilon_high=0.3)
    assert (np.abs(an["dlogits"]).max() > 0) == expect_grad
    clipped = min(max(ratio, 0.8), 1.3)
    assert abs(out["loss"].item() - (-min(ratio * A, clipped * A))) < 1e-5


def test_kl_zero_when_ref_equals_lp():
    logits, inputs = make_case(2, 6, 64, seed=5, old="none", mask_kind="ones")
    base = O.reference_value_and_grad(logits, inputs, beta=0.0)
    inputs["ref_per_token_logps"] = base["per_token_logps"].clone()
    kl = O.reference_value_and_grad(logits, inputs, beta=0.5)
    assert abs(kl["loss"].item() - base["loss"].item()) < 1e-6
    assert torch.allclose(kl["dlogits"], base["dlogits"], atol=1e-6)
    assert kl["per_token_kl"].abs().max() < 1e-6


def test_k3_value_against_hand_computation():
    logits, inputs = make_case(1, 3, 32, seed=6, old="none", mask_kind="ones")
    lp = O.reference_call(logits, inputs)["per_token_logps"]
    inputs["ref_per_token_logps"] = lp + torch.tensor([[0.3, -0.2]])
    inputs["advantages"] = torch.zeros(1)
    inputs["total_valid_token_count"] = 2.0
    out = O.reference_call(logits, inputs, beta=0.04)
    k3 = [math.exp(0.3) - 0.3 - 1, math.exp(-0.2) + 0.2 - 1]
    assert abs(out["loss"].item() - 0.04 * sum(k3) / 2.0) < 1e-6


@pytest.mark.parametrize("softcap", [None, 30.0])
def test_autograd_matches_closed_form(softcap):
    """Two independent derivations of loss, log-probs, entropy and dlogits agree."""
    logits, inputs = make_case(3, 8, 1000, seed=7, old="wide", ref=True, sigma=4.0)
    attrs = dict(beta=0.04, temperature=1.0, epsilon_low=0.2, epsilon_high=0.3, softcap=softcap)
    ag = O.reference_value_and_grad(logits, inputs, dtype=torch.float64, **attrs)
    x, c, m, adv, old, ref = _rows(logits, inputs)
    an = O.analytic_rows(x, c, m, adv, old, ref, inputs["total_valid_token_count"], **attrs)
    B, L, V = logits.shape
    assert np.allclose(ag["per_token_logps"].numpy().reshape(-1), an["lp"], atol=1e-10)
    assert abs(ag["loss"].item() - an["loss_part"]) < 1e-12
    assert np.allclose(ag["token_entropy"].numpy().reshape(-1), an["entropy_guard"], atol=1e-10)
    assert np.abs(an["entropy_guard"] - an["entropy_exact"]).max() <= V * 1e-9
    assert np.allclose(ag["dlogits"][:, :-1].numpy().reshape(-1, V), an["dlogits"], atol=1e-12)


def test_temperature_semantics():
    """Temperature divides the log-prob (not the logits) but divides the logits for entropy."""
    logits, inputs = make_case(2, 5, 200, seed=8, old="none", mask_kind="ones")
    t1 = O.reference_call(logits, inputs, temperature=1.0)
    t2 = O.reference_call(logits, inputs, temperature=2.0)
    assert torch.allclose(t2["per_token_logps"], t1["per_token_logps"] / 2.0, atol=1e-6)
    p = torch.softmax(logits[:, :-1].float() / 2.0, -1)
    H = -(p * torch.log(p)).sum(-1)
    assert torch.allclose(t2["token_entropy"], H, atol=1e-4)
    x, c, m, adv, old, ref = _rows(logits, inputs)
    an = O.analytic_rows(x, c, m, adv, old, ref, inputs["total_valid_token_count"], temperature=2.0)
    ag = O.reference_value_and_grad(logits, inputs, temperature=2.0, dtype=torch.float64)
    assert np.allclose(ag["dlogits"][:, :-1].numpy().reshape(-1, 200), an["dlogits"], atol=1e-12)


def test_finite_differences_float64():
    """Central differences of the f64 loss on V=17, N=5 confirm the gradient."""
    B, L, V = 1, 6, 17
    logits, inputs = make_case(B, L, V, seed=9, old="wide", ref=True, mask_kind="ones")
    attrs = dict(beta=0.04, epsilon_low=0.2, epsilon_high=0.3)
    ag = O.reference_value_and_grad(logits, inputs, dtype=torch.float64, **attrs)
    x0 = logits.double()
    h = 1e-6
    fd = torch.zeros_like(x0)
    for t in range(L):
        for j in range(V):
            xp, xm = x0.clone(), x0.clone()
            xp[0, t, j] += h
            xm[0, t, j] -= h
            lp_ = O.reference_call(xp, inputs, dtype=torch.float64, **attrs)["loss"].item()
            lm_ = O.reference_call(xm, inputs, dtype=torch.float64, **attrs)["loss"].item()
            fd[0, t, j] = (lp_ - lm_) / (2 * h)
    assert torch.allclose(fd, ag["dlogits"], atol=1e-7)


@pytest.mark.parametrize("k", [2, 4, 8])
def test_sharded_combine_equals_unsharded(k):
    logits, inputs = make_case(2, 5, 64 * k, seed=10, old="none")
    x, c, m, adv, old, ref = _rows(logits, inputs)
    V = x.shape[1]
    parts = [O.shard_partials(x[:, r * V // k:(r + 1) * V // k], c, r * V // k) for r in range(k)]
    P = np.stack(parts)  # [k, n, 4]
    M = P[:, :, 0].max(axis=0)
    S = (P[:, :, 1] * np.exp(P[:, :, 0] - M)).sum(axis=0)
    U = (P[:, :, 2] * np.exp(P[:, :, 0] - M)).sum(axis=0)
    yc = P[:, :, 3].sum(axis=0)
    lse = M + np.log(S)
    an = O.analytic_rows(x, c, m, adv, old, ref, 1.0)
    assert np.allclose(yc - lse, an["lp"], atol=1e-12)
    assert np.allclose(lse - U / S, an["entropy_exact"], atol=1e-10)


def test_softcap_large_cap_reproduces_uncapped():
    logits, inputs = make_case(2, 5, 100, seed=11, old="noisy")
    a = O.reference_value_and_grad(logits, inputs, dtype=torch.float64)
    b = O.reference_value_and_grad(logits, inputs, dtype=torch.float64, softcap=1e7)
    assert torch.allclose(a["per_token_logps"], b["per_token_logps"], atol=1e-9)
    assert torch.allclose(a["dlogits"], b["dlogits"], atol=1e-12)


def test_ppo_policy_equals_grpo_with_broadcast_advantages():
    logits, inputs = make_case(3, 7, 150, seed=12, old="noisy")
    a = O.reference_call(logits, inputs, epsilon_low=0.2, epsilon_high=0.2)
    b = O.ppo_policy_call(logits, inputs, epsilon_low=0.2, epsilon_high=0.2)
    assert abs(a["loss"].item() - b["policy_loss"].item()) < 1e-7
    assert torch.equal(a["per_token_logps"], b["per_token_logps"])
    adv2 = inputs["advantages"][:, None].expand(3, 6).contiguous()
    c = O.ppo_policy_call(logits, {**inputs, "advantages": adv2}, epsilon_low=0.2, epsilon_high=0.2)
    assert abs(c["policy_loss"].item() - b["policy_loss"].item()) < 1e-7
    with pytest.raises(ValueError):
        O.ppo_policy_call(logits, {**inputs, "advantages": torch.zeros(3, 4)})


def test_entropy_window_and_zero_length_sample():
    """entropy_loss averages tokens whose running valid count is in [4, 100]; an all-masked sample is 0/0."""
    B, L, V = 2, 130, 50
    logits, inputs = make_case(B, L, V, seed=13, old="none", mask_kind="ones")
    inputs["labels"][1] = 0
    out = O.reference_call(logits, inputs)
    H = out["token_entropy"][0]
    assert abs(out["entropy_loss"][0].item() - H[3:100].mean().item()) < 1e-5
    assert abs(out["entropy"][0].item() - H.mean().item()) < 1e-5
    assert math.isnan(out["entropy"][1].item()) and math.isnan(out["entropy_loss"][1].item())


def test_bf16_as_written_deviation_is_reported_not_gated():
    """The reference as written keeps bf16 through log_softmax; its log-probs sit on a bf16 grid."""
    logits, inputs = make_case(2, 5, 2000, seed=14, old="none")
    f32 = O.reference_call(logits, inputs, upcast=True)
    asw = O.reference_call(logits, inputs, upcast=False)
    assert asw["per_token_logps"].dtype == torch.bfloat16
    dev = (asw["per_token_logps"].float() - f32["per_token_logps"]).abs().max().item()
    assert dev < 0.13  # two bf16 roundings near |lp| ~ 8..16 (spacing 0.0625)


def test_golden_fixtures_match_oracle():
    files = sorted(f for f in os.listdir(GOLDEN) if f.endswith(".npz"))
    assert files, "no golden fixtures committed"
    for f in files:
        z = np.load(os.path.join(GOLDEN, f), allow_pickle=False)
        logits = torch.from_numpy(z["logits_bf16_bits"].astype(np.int16)).view(torch.bfloat16)
        inputs = {"input_ids": torch.from_numpy(z["input_ids"]), "labels": torch.from_numpy(z["labels"]),
                  "advantages": torch.from_numpy(z["advantages"]),
                  "total_valid_token_count": float(z["total_valid_token_count"])}
        if "old_per_token_logps" in z.files:
            inputs["old_per_token_logps"] = torch.from_numpy(z["old_per_token_logps"])
        if "ref_per_token_logps" in z.files:
            inputs["ref_per_token_logps"] = torch.from_numpy(z["ref_per_token_logps"])
        attrs = dict(beta=float(z["beta"]), temperature=float(z["temperature"]), epsilon_low=float(z["epsilon_low"]),
                     epsilon_high=float(z["epsilon_high"]), softcap=float(z["softcap"]) or None)
        out = O.reference_value_and_grad(logits, inputs, **attrs)
        assert np.allclose(out["per_token_logps"].numpy(), z["per_token_logps"], atol=2e-5), f
        assert abs(out["loss"].item() - float(z["loss"])) <= 2e-6 * max(1.0, abs(float(z["loss"]))), f
        assert np.allclose(out["token_entropy"].numpy(), z["token_entropy"], atol=5e-5), f
        assert np.allclose(out["dlogits"].numpy(), z["dlogits"], atol=1e-7, rtol=1e-4), f


def test_sft_cross_entropy_known_answer():
    """Uniform logits: every supervised token costs log V; unsupervised ones are ignored."""
    B, L, V = 2, 6, 50
    logits = torch.zeros(B, L, V, dtype=torch.bfloat16)
    labels = torch.randint(0, V, (B, L), generator=torch.Generator().manual_seed(59))
    labels[:, :2] = -100
    att = torch.ones(B, L, dtype=torch.int32)
    out = O.sft_call(logits, {"labels": labels, "attention_mask": att})
    assert abs(out["loss"].item() - math.log(V)) < 1e-5 and int(out["token_count"]) == B * (L - 2)
    empty = O.sft_call(logits, {"labels": torch.full((B, L), -100), "attention_mask": att})
    assert empty["loss"].item() == 0.0


def test_value_loss_known_answers():
    """Hand-computed cases of the value-loss tail (plugins/training/ppo/module.py:104-138)."""
    labels = torch.ones(1, 4)
    values = torch.tensor([[1.0, 2.0, 3.0, 99.0]])
    base = {"labels": labels, "advantages": torch.zeros(1)}
    # no range: plain squared error over positions 0..L-2
    out = O.ppo_value_call(values, {**base, "returns": torch.tensor([[0.0, 0.0, 0.0]])}, value_clip_range=None)
    assert out["value_loss"].item() == pytest.approx((1 + 4 + 9) / 3)
    assert out["value_pred_mean"].item() == pytest.approx(2.0) and out["return_mean"].item() == 0.0
    # range 0.5 around old = 0: clipped prediction 0.5, (0.5 - r)^2 with r = 4 is the larger term at every position
    out = O.ppo_value_call(values, {**base, "returns": torch.full((1, 3), 4.0), "old_values": torch.zeros(1, 3)},
                           value_clip_range=0.5)
    assert out["value_loss"].item() == pytest.approx(3.5 ** 2)
    # returns absent: advantages + value_pred, so both terms are advantages^2 when old_values is absent as well
    out = O.ppo_value_call(values, {"labels": labels, "advantages": torch.tensor([3.0])})
    assert out["value_loss"].item() == pytest.approx(9.0)
    assert out["return_mean"].item() == pytest.approx(5.0)
    # mask and the global normaliser
    lab = torch.tensor([[1.0, 1.0, 0.0, 1.0]])
    out = O.ppo_value_call(values, {"labels": lab, "advantages": torch.zeros(1), "returns": torch.zeros(1, 3),
                                    "total_valid_token_count": 10.0}, value_clip_range=None)
    assert out["value_loss"].item() == pytest.approx((1 + 9) / 10.0)  # position t is weighted by labels[t + 1]


def test_value_loss_gradient_cases():
    """d value_loss / d values: 2(v - r) m / Nv where the unclipped term is active, 0 where the clipped one is."""
    values = torch.tensor([[1.0, 1.0, 1.0, 7.0]], requires_grad=True)
    inputs = {"labels": torch.ones(1, 4), "advantages": torch.zeros(1),
              "returns": torch.tensor([[3.0, 3.0, 0.0]]),
              # position 0: inside the range; 1: clipped to 0.5 and (0.5 - 3)^2 is larger -> zero gradient;
              # 2: clipped to 0.5 but (1 - 0)^2 > (0.5 - 0)^2 -> the unclipped term drives the gradient
              "old_values": torch.tensor([[1.0, 0.0, 0.0]])}
    O.ppo_value_call(values, inputs, value_clip_range=0.5)["value_loss"].backward()
    g = values.grad[0]
    assert g[0].item() == pytest.approx(2 * (1 - 3) / 3)
    assert g[1].item() == 0.0
    assert g[2].item() == pytest.approx(2 * (1 - 0) / 3)
    assert g[3].item() == 0.0  # the last position never enters (values[:, :-1])
