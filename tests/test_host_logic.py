"""Host-side pieces that need no GPU: the per-sample entropy reductions of the module mirror,
the synthetic workload generator, and the package surface."""
import math

import torch

from mllm_jax_b200 import per_sample_entropy, synth
from oracle import grpo_oracle as O
from tests.util import make_case


def test_per_sample_entropy_matches_reference_expressions():
    logits, inputs = make_case(3, 140, 40, seed=21, old="none", mask_kind="random")
    inputs["labels"][2] = 0
    out = O.reference_call(logits, inputs)
    ent, ent_loss = per_sample_entropy(out["token_entropy"], inputs["labels"][:, 1:])
    assert torch.allclose(ent[:2], out["entropy"][:2], atol=1e-6)
    assert torch.allclose(ent_loss[:2], out["entropy_loss"][:2], atol=1e-6)
    assert math.isnan(ent[2].item()) and math.isnan(ent_loss[2].item())


def test_synth_shapes_and_distributions():
    w = synth.scaled(synth.CONFIGS["cfg0"], vocab=512, n_seqs=8, seq_len=64, len_lo=16, len_hi=64)
    a = synth.make_inputs(w, seed=0)
    b = synth.make_inputs(w, seed=0)
    c = synth.make_inputs(w, seed=1)
    assert a["logits"].shape == (8, 64, 512) and a["logits"].dtype == torch.bfloat16
    assert torch.equal(a["logits"], b["logits"]) and not torch.equal(a["logits"], c["logits"])
    assert abs(a["logits"].float().std().item() - 2.0) < 0.05
    lens = a["mask"].sum(1)
    assert lens.min() >= 16 and lens.max() <= 64
    assert (a["mask"][:, :-1] >= a["mask"][:, 1:]).all()  # right-padded
    assert a["total_valid"] == float(a["mask"].sum())
    assert abs(a["advantages"].sum().item()) < 1e-4  # group-normalised
    assert (a["old_logps"] - a["exact_logps"]).std().item() < 0.07
    assert (a["token_ids"] >= 0).all() and (a["token_ids"] < 512).all()
    # exact log-probs agree with the oracle
    inputs = {"input_ids": torch.cat([a["token_ids"][:, :1], a["token_ids"]], 1),
              "labels": torch.ones(8, 65, dtype=torch.int32), "advantages": a["advantages"]}
    lg = torch.cat([a["logits"], a["logits"][:, :1]], 1)
    ref = O.reference_call(lg, inputs)
    assert torch.allclose(ref["per_token_logps"], a["exact_logps"], atol=1e-5)


def test_group_advantages_known_answer():
    r = torch.tensor([1.0, 0.0, 0.0, 1.0, 1.0, 1.0, 1.0, 0.0])
    adv = synth.group_advantages(r, 8)
    mean, std = 5 / 8, math.sqrt(5 / 8 * 3 / 8)
    assert torch.allclose(adv, (r - mean) / (std + 1e-6), atol=1e-6)


def test_sweep_workload_masks_half():
    w = synth.scaled(synth.sweep_workload(4096), vocab=64)
    a = synth.make_inputs(w)
    assert a["mask"].mean().item() == 0.5


def test_ppo_update_collects_old_logps_in_first_epoch():
    """Epoch 0 sees no old log-probs and its per_token_logps become the later epochs' old ones."""
    from mllm_jax_b200.update import ppo_update

    B, T = 8, 5
    data = {"input_ids": torch.arange(B * (T + 1)).reshape(B, T + 1), "advantages": torch.arange(B).float()}
    seen = []

    def train_step(state, batch):
        seen.append((state, "old_per_token_logps" in batch, batch["input_ids"][:, 0].tolist(),
                     batch["total_valid_token_count"]))
        lp = batch["input_ids"][:, 1:].float() * 0.5 + state
        return state + 1, {"per_token_logps": lp, "entropy": torch.tensor(float(state)), "loss": torch.tensor(0.0)}

    state, out, last, entropy = ppo_update(state=0, datas=data, total_valid_token_count=37, train_step=train_step,
                                           grad_accum_steps=4, ppo_steps=3)
    assert state == 12 and len(seen) == 12
    assert [s[1] for s in seen] == [False] * 4 + [True] * 8
    assert seen[1][2] == [12, 18] and all(s[3] == 37 for s in seen)
    assert out["old_per_token_logps"].shape == (B, T)
    expect = torch.cat([data["input_ids"][2 * i:2 * i + 2, 1:].float() * 0.5 + i for i in range(4)])
    assert torch.equal(out["old_per_token_logps"], expect)
    assert entropy.item() == 3.0 and last["entropy"].item() == 11.0
    assert "old_per_token_logps" not in data  # the caller's dict is not modified


def test_synthetic_shards_are_slices_of_one_tensor():
    """Vocabulary and row shards of a workload are slices of the tensor the unsharded call builds, and old / ref
    log-probs are the same in every mode (so runs at different GPU counts see the same problem)."""
    import torch

    from mllm_jax_b200 import synth

    w = synth.scaled(synth.CONFIGS["cfg0"], n_seqs=6, seq_len=700, vocab=512, group=3)  # blocks straddle sequences
    full = synth.make_inputs(w, seed=2)
    for r in range(4):
        sh = synth.make_inputs(w, seed=2, vocab_shard=(r, 4))
        assert torch.equal(sh["logits"], full["logits"][:, :, r * 128:(r + 1) * 128])
        assert torch.equal(sh["old_logps"], full["old_logps"]) and torch.equal(sh["ref_logps"], full["ref_logps"])
    for r in range(3):
        rs = synth.make_inputs(w, seed=2, row_shard=(r, 3))
        assert torch.equal(rs["logits"], full["logits"][2 * r:2 * r + 2])
        assert torch.equal(rs["old_logps"], full["old_logps"][2 * r:2 * r + 2])
        assert torch.equal(rs["advantages"], full["advantages"][2 * r:2 * r + 2])
        assert rs["total_valid"] == full["total_valid"]  # the normaliser stays global
    assert not torch.equal(synth.make_inputs(w, seed=3)["logits"], full["logits"])
    none = synth.make_inputs(w, seed=2, want_logits=False)
    assert none["logits"] is None and torch.equal(none["exact_logps"], full["exact_logps"])


def test_workload_names_and_chunking():
    import pytest

    import bench
    from mllm_jax_b200 import synth

    assert synth.parse_workload("cfg2").vocab == 128256
    w = synth.parse_workload("cfg4-1048576")
    assert w.n_tokens == 1048576 and w.vocab == 151936 and w.half_valid_runs
    with pytest.raises(ValueError):
        synth.parse_workload("cfg9")
    # one GPU: 1M rows x 151936 = 318.6 GB -> 8 launches of 131072 rows over one 39.8 GB buffer
    seqs, chunks = bench.chunking(w, w.n_seqs, w.vocab)
    assert chunks == 8 and seqs * w.seq_len == 131072
    # 8 GPUs vocabulary-sharded: 39.8 GB per GPU fits in one launch
    assert bench.chunking(w, w.n_seqs, w.vocab // 8) == (w.n_seqs, 1)
    # cfg1 never chunks
    c1 = synth.CONFIGS["cfg1"]
    assert bench.chunking(c1, c1.n_seqs, c1.vocab) == (c1.n_seqs, 1)


def test_pinned_buffer_placement_reads_sysfs(tmp_path):
    """The NUMA helpers parse sysfs as laid out by Linux and do nothing where it is silent."""
    from mllm_jax_b200 import host_io

    assert host_io.parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert host_io.parse_cpulist("") == set()
    dev = tmp_path / "bus/pci/devices/0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    node = tmp_path / "devices/system/node/node1"
    node.mkdir(parents=True)
    (node / "cpulist").write_text("4-7\n")
    assert host_io.numa_node_of("0000:1b:00.0", str(tmp_path)) == 1
    assert host_io.cpus_of_node(1, str(tmp_path)) == {4, 5, 6, 7}
    (dev / "numa_node").write_text("-1\n")
    assert host_io.numa_node_of("0000:1b:00.0", str(tmp_path)) is None
    assert host_io.numa_node_of("0000:ff:00.0", str(tmp_path)) is None
    assert host_io.cpus_of_node(3, str(tmp_path)) == set()
