"""The implementations behind mllm_grpo_fwd_bwd.

The default is the two-pass kernel whose second read of a row is served on chip (L2, or shared memory
for short unsplit rows; long rows are split over a thread-block cluster); the separate forward and
backward kernels serve the rows it cannot take.  The tests force every cluster size, thread count,
load-batch size and the staged form through the library's tuning hook, check that the single-kernel
path really ran (2 launches instead of 3), and compare with the CPU oracle under the usual gates."""
import pytest
import torch

import mllm_jax_b200 as G
from mllm_jax_b200._lib import plan_override
from oracle import grpo_oracle as O
from tests.test_gpu_parity import check
from tests.util import make_case, to_device

pytestmark = pytest.mark.gpu


def run_fused(logits, inputs, cuda, expect_fused=True, inplace=False, compute_entropy=True, **attrs):
    ref = O.reference_value_and_grad(logits, inputs, **attrs)
    din = to_device(inputs, cuda)
    cfg = G.LossConfig(temperature=attrs.get("temperature", 1.0), epsilon_low=attrs.get("epsilon_low", 0.2),
                       epsilon_high=attrs.get("epsilon_high", 0.3), beta=attrs.get("beta", 0.0),
                       softcap=attrs.get("softcap"), compute_entropy=compute_entropy)
    x = logits.to(cuda)
    before = G.launch_count()
    out = G.grpo_value_and_grad(x, din["input_ids"], din["labels"], din["advantages"],
                                din.get("total_valid_token_count"), din.get("old_per_token_logps"),
                                din.get("ref_per_token_logps"), shifted=True, cfg=cfg, inplace=inplace)
    torch.cuda.synchronize()
    launched = G.launch_count() - before
    assert launched == (2 if expect_fused else 3), f"{launched} launches"
    assert G.ops.check_device_status(out["problem"]) == 0
    got = {"loss": out["loss"], "per_token_logps": out["per_token_logps"],
           "token_entropy": out["token_entropy"] if compute_entropy else None, "dlogits": out["dlogits"]}
    return ref, got


@pytest.mark.parametrize("V", [64, 1024, 4104, 128256, 151936, 256000])
def test_vocab_sizes_default_plan(cuda, V):
    B, L = (2, 5) if V > 100000 else (3, 70)
    logits, inputs = make_case(B, L, V, seed=60, old="noisy", ref=True)
    ref, got = run_fused(logits, inputs, cuda, beta=0.04, epsilon_low=0.2, epsilon_high=0.2)
    check(ref, got, f"V={V}")


@pytest.mark.parametrize("V", [22528, 24112, 24120, 24576])
def test_staged_rows_up_to_the_48k_boundary(cuda, V):
    """Unsplit rows of 44-48 KB are staged in shared memory; static + dynamic shared memory then exceeds
    the 48 KB a launch gets without opting in, so the launcher has to raise the limit itself."""
    logits, inputs = make_case(2, 7, V, seed=67, old="wide", ref=True)
    ref, got = run_fused(logits, inputs, cuda, beta=0.04)
    check(ref, got, f"V={V}")


@pytest.mark.parametrize("kind", ["no_old", "token_adv", "random_mask", "softcap", "no_entropy", "all_masked",
                                  "single_row"])
def test_options_fused(cuda, kind):
    kw, attrs, extra = dict(old="noisy"), {}, {}
    B, L, V = 3, 19, 8192
    if kind == "no_old":
        kw = dict(old="none")
    elif kind == "token_adv":
        kw = dict(old="wide", per_token_adv=True)
    elif kind == "random_mask":
        kw = dict(old="noisy", mask_kind="random")
    elif kind == "softcap":
        kw = dict(old="noisy", ref=True, sigma=4.0)
        attrs = dict(softcap=30.0, beta=0.04)
    elif kind == "no_entropy":
        extra = dict(compute_entropy=False)
    elif kind == "single_row":
        B, L = 1, 2
    logits, inputs = make_case(B, L, V, seed=62, **kw)
    if kind == "all_masked":
        inputs["labels"].zero_()
        inputs["total_valid_token_count"] = 1.0
    ref, got = run_fused(logits, inputs, cuda, **attrs, **extra)
    check(ref, got, kind)


def test_temperature_other_than_one(cuda):
    logits, inputs = make_case(2, 9, 4096, seed=63, old="noisy")
    ref, got = run_fused(logits, inputs, cuda, temperature=0.7)
    check(ref, got, "temperature")


def test_unaligned_vocab(cuda):
    logits, inputs = make_case(2, 9, 4099, seed=64, old="noisy")
    ref, got = run_fused(logits, inputs, cuda)
    check(ref, got, "V=4099")


def test_fused_inplace_and_padded_stride(cuda):
    logits, inputs = make_case(2, 12, 4096, seed=65, old="wide")
    ref, got = run_fused(logits, inputs, cuda, inplace=True)
    check(ref, got, "in place")
    # padded row stride (multiple of 8 elements), guard columns untouched
    B, L, V, ld = 2, 12, 4096, 4096 + 24
    din = to_device(inputs, cuda)
    buf = torch.zeros(B, L, ld, dtype=torch.bfloat16, device=cuda)
    buf[:, :, :V] = logits.to(cuda)
    dbuf = torch.full_like(buf, 3.0)
    prob = G.TokenLossProblem(buf[:, :, :V], din["input_ids"][:, 1:], din["labels"][:, 1:], din["advantages"],
                              din["total_valid_token_count"], din["old_per_token_logps"], None, G.LossConfig(),
                              scored_rows=L - 1, vocab=V)
    prob.dlogits = dbuf[:, :, :V]
    before = G.launch_count()
    prob.run("mllm_grpo_fwd_bwd")
    torch.cuda.synchronize()
    assert G.launch_count() - before == 2
    check(ref, {"loss": prob.loss[0], "per_token_logps": prob.per_token_logps, "token_entropy": prob.token_entropy,
                "dlogits": prob.dlogits}, "padded stride")
    assert (dbuf[:, :, V:] == 3.0).all()


def test_fused_equals_two_sweeps_closely(cuda):
    """Both paths see the same inputs; outputs other than dlogits agree to rounding, dlogits to bf16."""
    logits, inputs = make_case(4, 50, 16000, seed=66, old="wide", ref=True)
    din = to_device(inputs, cuda)
    x = logits.to(cuda)
    args = (x, din["input_ids"], din["labels"], din["advantages"], din["total_valid_token_count"],
            din["old_per_token_logps"], din["ref_per_token_logps"])
    a = G.grpo_value_and_grad(*args, shifted=True, cfg=G.LossConfig(beta=0.04))
    with plan_override(sweeps=True):
        b = G.grpo_value_and_grad(*args, shifted=True, cfg=G.LossConfig(beta=0.04))
    torch.cuda.synchronize()
    assert (a["per_token_logps"] - b["per_token_logps"]).abs().max() < 2e-5
    assert abs(a["loss"].item() - b["loss"].item()) < 1e-6
    da, db = a["dlogits"].float(), b["dlogits"].float()
    assert (da - db).abs().max() <= 0.01 * db.abs().max()


@pytest.mark.parametrize("sweeps,cluster,threads,batch,staged", [
    (0, 1, 512, 0, -1), (0, 1, 128, 0, 0), (0, 1, 64, 0, 0), (0, 1, 256, 0, 1), (0, 2, 256, 0, -1),
    (0, 4, 256, 0, -1), (0, 4, 128, 6, -1), (0, 8, 128, 10, -1), (0, 2, 128, 8, -1), (0, 6, 128, 6, -1),
    (0, 6, 128, 8, -1), (0, 1, 256, 6, 0), (0, 1, 256, 8, 0), (0, 0, 0, 0, -1),
    (1, 0, 0, 0, -1)])
@pytest.mark.parametrize("kind", ["kl", "softcap", "shifted_tail"])
def test_every_fwd_bwd_plan(cuda, sweeps, cluster, threads, batch, staged, kind):
    """Every plan behind mllm_grpo_fwd_bwd gives the oracle's answer."""
    kw, attrs = dict(old="wide", ref=True), dict(beta=0.04)
    V = 16384
    if kind == "softcap":
        kw, attrs = dict(old="noisy", ref=True, sigma=4.0), dict(beta=0.04, softcap=30.0)
    elif kind == "shifted_tail":
        V = 8 * 1013  # slices of unequal length
    logits, inputs = make_case(3, 23, V, seed=70, **kw)
    with plan_override(sweeps=bool(sweeps), cluster=cluster, threads=threads, load_batch=batch, staged=staged):
        ref, got = run_fused(logits, inputs, cuda, expect_fused=not sweeps, **attrs)
    check(ref, got, f"sweeps={sweeps} cl={cluster} th={threads} batch={batch} staged={staged} {kind}")
