"""The single-kernel implementations behind mllm_grpo_fwd_bwd.

"auto" picks the two-pass kernel whose second read is served by L2 (rows split over a cluster
when they are long); "cluster" is the row-resident kernel (distributed shared memory, TMA bulk
copies in and out), taken only for 16-byte-aligned full rows; "sweeps" is the separate forward
and backward kernels.  The tests force every mode, cluster size and thread count, check that a
single-kernel path really ran (2 launches instead of 3), and compare with the CPU oracle under
the usual gates."""
import os

import pytest
import torch

import mllm_jax_b200 as G
from oracle import grpo_oracle as O
from tests.test_gpu_parity import check
from tests.util import make_case, to_device

pytestmark = pytest.mark.gpu

ENV = ("MLLM_GRPO_FWD_BWD_MODE", "MLLM_GRPO_L2_CLUSTER", "MLLM_GRPO_L2_THREADS",
       "MLLM_GRPO_FUSED_CLUSTER", "MLLM_GRPO_FUSED_THREADS", "MLLM_GRPO_FUSED_STAGES", "MLLM_GRPO_FUSED_CLUSTERS",
       )


@pytest.fixture(autouse=True)
def clean_env():
    saved = {k: os.environ.pop(k, None) for k in ENV}
    yield
    for k, v in saved.items():
        os.environ.pop(k, None)
        if v is not None:
            os.environ[k] = v


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


@pytest.mark.parametrize("cluster", [1, 2, 4, 8])
@pytest.mark.parametrize("threads", [256, 512])
def test_cluster_sizes(cuda, cluster, threads):
    os.environ["MLLM_GRPO_FWD_BWD_MODE"] = "cluster"
    os.environ["MLLM_GRPO_FUSED_CLUSTER"] = str(cluster)
    os.environ["MLLM_GRPO_FUSED_THREADS"] = str(threads)
    logits, inputs = make_case(5, 41, 32000, seed=50 + cluster, old="wide", ref=True)
    ref, got = run_fused(logits, inputs, cuda, beta=0.04)
    check(ref, got, f"cluster={cluster} threads={threads}")


@pytest.mark.parametrize("mode", ["auto", "cluster"])
@pytest.mark.parametrize("V", [64, 1024, 4104, 128256, 151936, 256000])
def test_vocab_sizes_default_plan(cuda, V, mode):
    os.environ["MLLM_GRPO_FWD_BWD_MODE"] = mode
    B, L = (2, 5) if V > 100000 else (3, 70)
    logits, inputs = make_case(B, L, V, seed=60, old="noisy", ref=True)
    ref, got = run_fused(logits, inputs, cuda, beta=0.04, epsilon_low=0.2, epsilon_high=0.2)
    check(ref, got, f"V={V}")


@pytest.mark.parametrize("stages", [2, 3])
@pytest.mark.parametrize("clusters", [1, 3, 0])
def test_few_stages_and_few_clusters(cuda, stages, clusters):
    """Long per-cluster row sequences (pipeline wrap-around of stages and exchange slots)."""
    os.environ["MLLM_GRPO_FWD_BWD_MODE"] = "cluster"
    os.environ["MLLM_GRPO_FUSED_CLUSTER"] = "2"
    os.environ["MLLM_GRPO_FUSED_STAGES"] = str(stages)
    if clusters:
        os.environ["MLLM_GRPO_FUSED_CLUSTERS"] = str(clusters)
    logits, inputs = make_case(3, 30, 2048, seed=61, old="wide", ref=True)
    ref, got = run_fused(logits, inputs, cuda, beta=0.1)
    check(ref, got, f"stages={stages} clusters={clusters}")


@pytest.mark.parametrize("mode", ["auto", "cluster"])
@pytest.mark.parametrize("kind", ["no_old", "token_adv", "random_mask", "softcap", "no_entropy", "all_masked",
                                  "single_row"])
def test_options_fused(cuda, kind, mode):
    os.environ["MLLM_GRPO_FWD_BWD_MODE"] = mode
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


@pytest.mark.parametrize("mode", ["auto", "cluster"])
def test_temperature_other_than_one(cuda, mode):
    """The row-resident kernel does not do temperature != 1 (falls back to the sweeps); auto does."""
    os.environ["MLLM_GRPO_FWD_BWD_MODE"] = mode
    logits, inputs = make_case(2, 9, 4096, seed=63, old="noisy")
    ref, got = run_fused(logits, inputs, cuda, expect_fused=(mode == "auto"), temperature=0.7)
    check(ref, got, "temperature")


@pytest.mark.parametrize("mode", ["auto", "cluster"])
def test_unaligned_vocab(cuda, mode):
    os.environ["MLLM_GRPO_FWD_BWD_MODE"] = mode
    logits, inputs = make_case(2, 9, 4099, seed=64, old="noisy")
    ref, got = run_fused(logits, inputs, cuda, expect_fused=(mode == "auto"))
    check(ref, got, "V=4099")


@pytest.mark.parametrize("mode", ["auto", "cluster"])
def test_fused_inplace_and_padded_stride(cuda, mode):
    os.environ["MLLM_GRPO_FWD_BWD_MODE"] = mode
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
    os.environ["MLLM_GRPO_FWD_BWD_MODE"] = "sweeps"
    b = G.grpo_value_and_grad(*args, shifted=True, cfg=G.LossConfig(beta=0.04))
    torch.cuda.synchronize()
    assert (a["per_token_logps"] - b["per_token_logps"]).abs().max() < 2e-5
    assert abs(a["loss"].item() - b["loss"].item()) < 1e-6
    da, db = a["dlogits"].float(), b["dlogits"].float()
    assert (da - db).abs().max() <= 0.01 * db.abs().max()


@pytest.mark.parametrize("mode,cluster,threads", [("auto", 1, 512), ("auto", 1, 128), ("auto", 2, 256),
                                                  ("auto", 4, 256), ("auto", 4, 128), ("auto", 8, 128),
                                                  ("auto", 0, 0), ("cluster", 0, 0), ("sweeps", 0, 0)])
@pytest.mark.parametrize("kind", ["kl", "softcap", "shifted_tail"])
def test_every_fwd_bwd_mode(cuda, mode, cluster, threads, kind):
    """All implementations behind mllm_grpo_fwd_bwd give the oracle's answer."""
    os.environ["MLLM_GRPO_FWD_BWD_MODE"] = mode
    if cluster:
        os.environ["MLLM_GRPO_L2_CLUSTER"] = str(cluster)
    if threads:
        os.environ["MLLM_GRPO_L2_THREADS"] = str(threads)
    kw, attrs = dict(old="wide", ref=True), dict(beta=0.04)
    V = 16384
    if kind == "softcap":
        kw, attrs = dict(old="noisy", ref=True, sigma=4.0), dict(beta=0.04, softcap=30.0)
    elif kind == "shifted_tail":
        V = 8 * 1013  # slices of unequal length
    logits, inputs = make_case(3, 23, V, seed=70, **kw)
    ref, got = run_fused(logits, inputs, cuda, expect_fused=(mode != "sweeps"), **attrs)
    check(ref, got, f"{mode} cl={cluster} th={threads} {kind}")
