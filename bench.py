#!/usr/bin/env python
"""Benchmark of the fused GRPO token loss (fwd+bwd) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg1] [--parallelism vocab|token]
                    [--impl ours|reference]

One step = one forward+backward pass of the loss over one batch of synthetic logits that is already
resident in HBM.  Workloads: cfg0..cfg3 (the benchmark configurations) and cfg4-<tokens> (one point of
the token-count sweep, e.g. cfg4-65536, cfg4-1048576).  N=1 runs the whole batch on one GPU.  N>1
(launched by torch.distributed.run, one rank per GPU) runs the same global batch sharded:
  --parallelism vocab (default): V/N columns per rank, ONE kernel per GPU with the exchange of the
      per-token partials inside it (peer stores over NVLink); `--vp-mode nccl` selects three kernels
      with an NCCL all-gather between them instead.
  --parallelism token: B/N sequences per rank, each through the single-GPU kernel, and one scalar
      all-reduce of the loss (the reference's dp/fsdp batch sharding).
Every shard is a slice of the same seeded tensor the 1-GPU run uses.  A batch whose logits exceed
45 GB per GPU is run as equal row chunks over one buffer (stated in `config`).
Prints ONE JSON line on rank 0; `extra` holds short runs of the other configurations.
`--impl reference` times the CPU restatement of the reference's jnp expressions (the reference itself
needs JAX, which exists neither where this was written nor on the GPU hosts).
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "fused GRPO loss fwd+bwd tokens/s"
UNIT = "tokens/s"
# DRAM bytes per logit element the one-kernel step moves (dram__bytes_read + dram__bytes_write of ncu
# captures on small cases of the same kernels, see profiles/): one bf16 read + one bf16 write.
NCU_TRAFFIC_PER_ELEMENT = {"two_pass_kernel": 4.003, "two_pass_kernel_softcap": 4.08, "two_pass_kernel_long_rows": 4.10}
CHUNK_BYTES = 45e9  # largest logits buffer per GPU; bigger batches run as row chunks over one buffer
DEFAULT_EXTRA = "cfg2,cfg3,cfg4-65536"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="cfg1")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--parallelism", default="vocab", choices=["vocab", "token"],
                    help="N>1: shard the vocabulary (default) or the sequences")
    ap.add_argument("--cpu-sample-tokens", type=int, default=512)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--extra", default=None,
                    help="comma-separated workloads measured briefly after the main one and reported under "
                         f"'extra' (default for the default workload: {DEFAULT_EXTRA}; 'none' to skip)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--vocab", type=int, default=0, help="override the workload's vocabulary size (tuning only)")
    ap.add_argument("--rows", type=int, default=0, help="override the number of sequences (tuning only)")
    ap.add_argument("--vp-mode", default="fused", choices=["fused", "nccl"],
                    help="vocab-parallel: exchange inside the kernel over peer stores, or three kernels + NCCL all-gather")
    ap.add_argument("--plan", default=None,
                    help="tuning only: sweeps,cluster,threads,load_batch,staged for mllm_grpo_set_plan_override "
                         "(0 / -1 = automatic), e.g. 0,2,128,6,-1")
    ap.add_argument("--self-exchange", action="store_true",
                    help="tuning only, 1 GPU: run the vocabulary-sharded kernel as a single shard that exchanges with itself")
    ap.add_argument("--hidden", type=int, default=3584, help="--fold-lm-head: hidden size (a multiple of 64)")
    ap.add_argument("--fold-lm-head", action="store_true",
                    help="time the lm_head projection folded into the loss (hidden x weight -> log-probs without "
                         "logits in HBM) instead of the loss on materialised logits; 1 GPU")
    return ap.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def oracle_inputs(data):
    """Aligned synthetic batch -> the reference's shifted inputs dict (one dummy leading position)."""
    ids, mask = data["token_ids"], data["mask"]
    B = ids.shape[0]
    z = torch.zeros(B, 1, dtype=ids.dtype)
    return {"input_ids": torch.cat([z, ids.cpu()], 1), "labels": torch.cat([z, mask.cpu().to(ids.dtype)], 1),
            "advantages": data["advantages"].cpu(), "total_valid_token_count": data["total_valid"],
            "old_per_token_logps": data["old_logps"].cpu(), "ref_per_token_logps": data["ref_logps"].cpu()}


def cpu_baseline(args, w, steps=None, warmup=1):
    """Times the CPU restatement on a bounded sample of the same workload (rank 0 only).
    steps=None: repeat for about 10 s (at least 3 passes); else exactly `steps` passes."""
    from mllm_jax_b200 import synth
    from oracle import grpo_oracle as O

    nseq = max(1, args.cpu_sample_tokens // 64)
    sample = synth.scaled(w, n_seqs=nseq, seq_len=64, len_lo=16, len_hi=64, group=min(w.group, nseq),
                          half_valid_runs=False)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    data = synth.make_inputs(sample, seed=1)
    inputs = oracle_inputs(data)
    logits = torch.cat([data["logits"], data["logits"][:, :1]], 1)  # the unscored last position
    attrs = dict(beta=w.beta, epsilon_low=w.epsilon_low, epsilon_high=w.epsilon_high, softcap=w.softcap)
    # shift: row i scores token i+1, so oracle_inputs prepends a dummy id/label and a dummy last row is appended
    for _ in range(max(1, warmup)):
        O.reference_value_and_grad(logits, inputs, **attrs)
    t0 = time.perf_counter()
    reps = 0
    while (reps < steps) if steps else (reps < 3 or (time.perf_counter() - t0 < 10.0 and reps < 50)):
        O.reference_value_and_grad(logits, inputs, **attrs)
        reps += 1
    sec = (time.perf_counter() - t0) / reps
    return {"value": sample.n_tokens / sec, "unit": UNIT, "cores": cores, "kind": "port", "ms_per_pass": sec * 1e3,
            "sample": f"{sample.n_tokens} tokens x V={w.vocab} per pass, {reps} passes, torch-CPU restatement + autograd"}


class Job:
    """Process-wide state of one bench run."""

    def __init__(self, args):
        self.args = args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the GRPO loss kernels have no CPU path")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.dist = None
        self.self_exchange = bool(getattr(args, "self_exchange", False)) and self.world == 1
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist
        elif self.self_exchange:
            import torch.distributed as dist

            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29533")
            dist.init_process_group("gloo", rank=0, world_size=1)
            self.dist = dist
        self.peaks, self.peak_kind = peaks()

    def barrier(self):
        if self.dist is not None and self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, x: float) -> float:
        if self.dist is None or self.world == 1:
            return x
        t = torch.tensor([x], device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())


def config_dict(w, world: int, mode: str, parallelism: str, seed: int) -> dict:
    """The `config` object of a line: the same for this package's arm and for the reference arm, which derives it
    from the workload alone (the mask comes from the seeded side arrays, no logits needed)."""
    from mllm_jax_b200 import synth

    v_local = w.vocab // world if mode == "vocab" else w.vocab
    seqs_local = w.n_seqs // world if mode == "token" else w.n_seqs
    chunk_seqs, n_chunks = chunking(w, seqs_local, v_local)
    rows_chunk = chunk_seqs * w.seq_len
    wc = w
    if n_chunks > 1:
        total = chunk_seqs * (world if mode == "token" else 1)
        wc = synth.scaled(w, n_seqs=total, group=min(w.group, total))
    mask = synth.side_arrays(wc, seed)[2]
    return {"workload": w.name, "rows": w.n_tokens, "vocab": w.vocab, "global_batch": w.n_seqs, "seq_len": w.seq_len,
            "parallelism": parallelism,
            "l2": "inputs (%.1f GB per GPU per launch) exceed the 126 MB L2" % (2.0 * v_local * rows_chunk / 1e9),
            "chunks": None if n_chunks == 1 else
            f"{n_chunks} launches per step over ONE buffer of {rows_chunk} rows ({2.0 * v_local * rows_chunk / 1e9:.1f} GB "
            f"of logits per GPU): the full batch does not fit beside its gradient",
            "mask_valid_fraction": float(mask.double().mean().item()),
            "epsilon": [w.epsilon_low, w.epsilon_high], "beta": w.beta, "softcap": w.softcap}


def default_parallelism(world: int, mode: str, seqs_local: int) -> str:
    if world == 1:
        return "single"
    if mode == "token":
        return f"token-parallel dp{world}: {seqs_local} sequences per rank, scalar loss all-reduce (NCCL)"
    return f"vocab-parallel tp{world}, exchange: peer stores inside the kernel"


def chunking(w, rows_local_seqs: int, v_local: int):
    """(sequences per chunk, chunks): the largest divisor of this rank's sequences whose logits fit CHUNK_BYTES."""
    per_seq = w.seq_len * v_local * 2.0
    best = 1
    for c in range(1, rows_local_seqs + 1):
        if rows_local_seqs % c == 0 and c * per_seq <= CHUNK_BYTES:
            best = c
    return best, rows_local_seqs // best


def sample_rows(n_rows: int, count: int = 64, seed: int = 7) -> torch.Tensor:
    gen = torch.Generator().manual_seed(seed)
    rows = torch.cat([torch.tensor([0, n_rows - 1]), torch.randint(0, n_rows, (max(count - 2, 0),), generator=gen)])
    return rows.unique()


def parity_check(job: Job, w, data, out, mode: str, v_local: int) -> dict:
    """Sampled rows of the timed buffers against the closed-form CPU oracle: per-token log-prob (abs), entropy
    (abs) and dlogits (row-relative).  vocab: the rows' column shards are gathered to rank 0, which checks whole
    rows; token: every rank checks rows of its own and the worst figure is taken."""
    import numpy as np

    from oracle import grpo_oracle as O

    dist, dev = job.dist, job.dev
    T = data["token_ids"].shape[1]
    n_local = data["token_ids"].numel()
    count = 64 if mode != "token" else max(8, 64 // job.world)
    rows = sample_rows(n_local, count).to(dev)
    x = data["logits"].view(n_local, -1)[rows]
    d = out["dlogits"].view(n_local, -1)[rows]
    if mode == "vocab" and job.world > 1:
        xs = torch.empty(job.world, *x.shape, dtype=x.dtype, device=dev)
        ds = torch.empty(job.world, *d.shape, dtype=d.dtype, device=dev)
        dist.all_gather_into_tensor(xs.view(-1), x.contiguous().view(-1))
        dist.all_gather_into_tensor(ds.view(-1), d.contiguous().view(-1))
        x = xs.permute(1, 0, 2).reshape(rows.numel(), -1)
        d = ds.permute(1, 0, 2).reshape(rows.numel(), -1)
    res = None
    if mode != "vocab" or job.rank == 0:
        pick = lambda t: t.reshape(n_local)[rows].double().cpu().numpy()  # noqa: E731
        advN = data["advantages"][:, None].expand(-1, T).reshape(n_local)
        an = O.analytic_rows(x.double().cpu().numpy(), data["token_ids"].reshape(n_local)[rows].long().cpu().numpy(),
                             pick(data["mask"]), pick(advN), pick(data["old_logps"]), pick(data["ref_logps"]),
                             data["total_valid"], beta=w.beta, epsilon_low=w.epsilon_low,
                             epsilon_high=w.epsilon_high, softcap=w.softcap)
        lp_abs = float(np.abs(pick(out["per_token_logps"]) - an["lp"]).max())
        ent_abs = float(np.abs(pick(out["token_entropy"]) - an["entropy_guard"]).max())
        dn = d.double().cpu().numpy()
        rowmax = np.abs(an["dlogits"]).max(axis=1)
        err = np.abs(dn - an["dlogits"]).max(axis=1)
        nz = rowmax > 0
        d_rel = float((err[nz] / rowmax[nz]).max()) if nz.any() else 0.0
        zero_ok = bool((err[~nz] == 0).all())
        res = [lp_abs, ent_abs, d_rel, 0.0 if zero_ok else 1.0]
    if mode == "token" and dist is not None and job.world > 1:
        t = torch.tensor(res, device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res = t.tolist()
    if res is None:
        return None
    total_rows = int(rows.numel()) * (job.world if mode == "token" else 1)
    return {"rows": total_rows, "lp_abs": res[0], "entropy_abs": res[1], "dlogits_rel": res[2],
            "zero_rows_exact": res[3] == 0.0, "gates": {"lp_abs": 2e-3, "entropy_abs": 5e-4, "dlogits_rel": 1e-2},
            "ok": bool(res[0] <= 2e-3 and res[1] <= 5e-4 and res[2] <= 1e-2 and res[3] == 0.0),
            "against": "closed-form f64 CPU oracle on sampled rows of the timed buffers"}


def run_workload(job: Job, name: str, steps: int, warmup: int, main: bool) -> dict:
    """Measure one workload at this job's GPU count.  main=False: the short form used for `extra`."""
    import mllm_jax_b200 as G
    from mllm_jax_b200 import _lib, synth

    args, world, rank, dev, dist = job.args, job.world, job.rank, job.dev, job.dist
    w = synth.parse_workload(name)
    if main and args.vocab:
        w = synth.scaled(w, vocab=args.vocab, name=w.name + f"-V{args.vocab}")
    if main and args.rows:
        w = synth.scaled(w, n_seqs=args.rows, name=w.name + f"-B{args.rows}")
    cfg = G.LossConfig(epsilon_low=w.epsilon_low, epsilon_high=w.epsilon_high, beta=w.beta, softcap=w.softcap)
    N, V = w.n_tokens, w.vocab
    mode = "single" if world == 1 and not job.self_exchange else args.parallelism
    if job.self_exchange:
        mode = "vocab"
    if mode == "vocab" and V % world:
        return {"workload": w.name, "skipped": f"vocabulary {V} does not split over {world} ranks"}
    if mode == "token" and w.n_seqs % world:
        return {"workload": w.name, "skipped": f"{w.n_seqs} sequences do not split over {world} ranks"}
    v_local = V // world if mode == "vocab" else V
    seqs_local = w.n_seqs // world if mode == "token" else w.n_seqs
    chunk_seqs, n_chunks = chunking(w, seqs_local, v_local)
    wc = w
    if n_chunks > 1:  # the buffer holds one chunk: generate that many sequences only
        total = chunk_seqs * (world if mode == "token" else 1)
        wc = synth.scaled(w, n_seqs=total, group=min(w.group, total))
    rows_chunk = chunk_seqs * w.seq_len  # rows of one launch on this rank

    exchange = None
    pending = []  # token-parallel: the loss all-reduce still in flight
    if mode == "single":
        data = synth.make_inputs(wc, seed=args.seed, device=str(dev))
        dlogits = torch.empty_like(data["logits"])
        first = G.grpo_value_and_grad(data["logits"], data["token_ids"], data["mask"], data["advantages"],
                                      data["total_valid"], data["old_logps"], data["ref_logps"], cfg=cfg,
                                      dlogits=dlogits)
        plan1 = first["problem"]  # buffers bound once (static shapes); a step relaunches on the same addresses

        def launch():
            plan1.run("mllm_grpo_fwd_bwd", reuse_args=True)
            return first
        parallelism = "single"
        kernel = "two_pass_kernel (mllm_grpo_fwd_bwd)"
    elif mode == "token":
        from mllm_jax_b200.vocab_parallel import TokenParallelLoss

        data = synth.make_inputs(wc, seed=args.seed, device=str(dev), row_shard=(rank, world))
        dlogits = torch.empty_like(data["logits"])
        tp = TokenParallelLoss(cfg)
        first = tp.value_and_grad(data["logits"], data["token_ids"], data["mask"], data["advantages"],
                                  data["total_valid"], data["old_logps"], data["ref_logps"], dlogits=dlogits)
        plan1 = first["problem"]

        def launch():
            # the one exchange: a scalar all-reduce, issued every step without stalling the compute stream (the
            # next step's kernel does not depend on it); the last one is waited for inside the timed region
            plan1.run("mllm_grpo_fwd_bwd", reuse_args=True)
            if pending:
                pending.pop().wait()
            first["loss"], work = tp.reduce_loss_async(first["local_loss"])
            pending.append(work)
            return first
        parallelism = default_parallelism(world, mode, seqs_local)
        kernel = "two_pass_kernel (mllm_grpo_fwd_bwd on this rank's rows)"
    else:
        from mllm_jax_b200.vocab_parallel import VocabParallelLoss

        data = synth.make_inputs(wc, seed=args.seed, device=str(dev), vocab_shard=(rank, world))
        dlogits = torch.empty_like(data["logits"])
        vp = VocabParallelLoss(V, cfg)
        call_args = (data["logits"], data["token_ids"], data["mask"], data["advantages"], data["total_valid"],
                     data["old_logps"], data["ref_logps"])
        vp_mode, vp_note = args.vp_mode, None
        if vp_mode == "fused":
            try:
                # buffers bound once (static shapes), every step relaunches on the same addresses
                plan = vp.plan_fused(*call_args, dlogits=dlogits)
                ok = torch.ones(1, device=dev)
            except Exception as exc:  # symmetric memory unavailable on this box
                vp_note = f"peer exchange buffers could not be set up ({type(exc).__name__}: {str(exc)[:80]})"
                ok = torch.zeros(1, device=dev)
            if world > 1:
                dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if ok.item() == 0:
                vp_mode = "nccl"
                vp_note = vp_note or "another rank could not set up the peer exchange buffers"
        if vp_mode == "fused":
            def launch():
                return vp.step_fused(plan)
            kernel = "two_pass_kernel<SHARDED> (mllm_grpo_fwd_bwd_sharded: exchange inside the kernel)"
        else:
            def launch():
                return vp.value_and_grad(*call_args, dlogits=dlogits)
            kernel = "row_stats_kernel + NCCL all-gather + combine_kernel + dlogits_kernel"
        parallelism = "sharded kernel, one shard exchanging with itself (tuning)" if job.self_exchange else \
            default_parallelism(world, mode, seqs_local) if vp_mode == "fused" and not vp_note else (
            f"vocab-parallel tp{world}, exchange: NCCL all-gather between kernels" + (f" [{vp_note}]" if vp_note else ""))

    def step():
        for _ in range(n_chunks):
            out = launch()
        return out

    def finish():  # token-parallel: the compute stream joins the last outstanding loss all-reduce
        if mode == "token" and pending:
            pending.pop().wait()

    for _ in range(max(warmup, 3)):
        out = step()
    finish()
    job.barrier()
    sampler = ClockSampler(job.local)
    if rank == 0 and main:
        sampler.start()
        time.sleep(0.15)
    launches0 = _lib.launch_count()
    job.barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        out = step()
    finish()
    ev1.record()
    job.barrier()
    launches = _lib.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 and main else None
    ms_per_step = job.max_over_ranks(ev0.elapsed_time(ev1)) / steps
    value = N / (ms_per_step * 1e-3)
    loss = float(out["loss"].item())
    status = int(out["problem"].device_status.item())

    # The dominant kernel alone: CUDA events around each launch of the entry point (the kernel plus the
    # 5 us loss reduction), averaged.
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    t_k = []
    for i in range(3 + min(steps, 10)):
        if dist is not None and mode == "vocab" and world > 1:
            dist.barrier()  # ranks enter the exchanging kernel together, as in the timed loop's steady state
        evs[0].record()
        launch()
        finish()
        evs[1].record()
        torch.cuda.synchronize()
        if i >= 3:
            t_k.append(evs[0].elapsed_time(evs[1]))
    ms_launch = job.max_over_ranks(sum(t_k) / len(t_k))
    peak = float(job.peaks["hbm_gbs"])
    bytes_launch = 6.0 * v_local * rows_chunk   # algorithmic: logits read twice + dlogits written once
    bytes_min = 4.0 * v_local * rows_chunk      # what has to cross HBM when the second read is served on chip
    ach = bytes_launch / (ms_launch * 1e-3) / 1e9
    one_kernel = "two_pass_kernel" in kernel
    roofline = {
        "bound": "hbm", "kernel": kernel, "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
        "peak_kind": job.peak_kind, "ms_per_launch": ms_launch, "algorithmic_bytes_per_launch": bytes_launch,
        # rows of 192 KB and more run as 6 CTAs x 128 threads and miss L2 on 5 % of their second reads
        "traffic": NCU_TRAFFIC_PER_ELEMENT["two_pass_kernel_softcap" if w.softcap else (
            "two_pass_kernel_long_rows" if (mode != "vocab" and 2 * v_local >= 192 * 1024) else "two_pass_kernel")] * v_local *
        rows_chunk if one_kernel else None,
        "traffic_note": "dram__bytes_read + dram__bytes_write per logit element from ncu captures of small cases of "
                        "the same kernel (profiles/), scaled by the elements of one launch: traffic grows in proportion",
        "note": "algorithmic = logits read twice + dlogits written once (6*V*N per GPU); the kernel's second read is "
                "served on chip and zero-gradient rows are not re-read, so its minimum DRAM traffic is 4*V*N and "
                "frac can exceed 1; frac_min_dram is the physical view",
        "min_dram_bytes_per_launch": bytes_min,
        "achieved_min_dram": bytes_min / (ms_launch * 1e-3) / 1e9,
        "frac_min_dram": bytes_min / (ms_launch * 1e-3) / 1e9 / peak,
        "frac_of_8TBs": ach / 8000.0,
        "step": {"ms_per_step": ms_per_step, "launches_per_step": n_chunks,
                 "frac": 6.0 * v_local * rows_chunk * n_chunks / (ms_per_step * 1e-3) / 1e9 / peak,
                 "frac_min_dram": 4.0 * v_local * rows_chunk * n_chunks / (ms_per_step * 1e-3) / 1e9 / peak},
    }

    if mode == "vocab" and one_kernel:
        # Exchange overhead: the same shard, taken as a vocabulary of its own, through the exchange-free entry point.
        local_ids = data["token_ids"] % v_local
        solo = G.grpo_value_and_grad(data["logits"], local_ids, data["mask"], data["advantages"],
                                     data["total_valid"], data["old_logps"], data["ref_logps"], cfg=cfg,
                                     dlogits=dlogits)["problem"]
        t_s = []
        for i in range(3 + min(steps, 10)):
            evs[0].record()
            solo.run("mllm_grpo_fwd_bwd", reuse_args=True)
            evs[1].record()
            torch.cuda.synchronize()
            if i >= 3:
                t_s.append(evs[0].elapsed_time(evs[1]))
        ms_solo = job.max_over_ranks(sum(t_s) / len(t_s))
        exchange = {"ms_sharded_launch": ms_launch, "ms_same_shard_without_exchange": ms_solo,
                    "overhead_ms": ms_launch - ms_solo, "overhead_frac": (ms_launch - ms_solo) / ms_launch,
                    "payload_bytes_per_token_per_rank": 32 * world,
                    "note": "same rows and columns through mllm_grpo_fwd_bwd (plan of an unsharded row of that "
                            "length) against mllm_grpo_fwd_bwd_sharded; each rank stores 4 (float, epoch) words "
                            "of 8 bytes per token into every rank's buffer"}
        out = launch()  # the timed path's outputs again (the solo run overwrote dlogits)
        torch.cuda.synchronize()

    parity = parity_check(job, w, data, out, mode, v_local)

    e2e = None
    if main and not args.no_e2e and n_chunks == 1:
        e2e = measure_e2e(data, launch, args, job, finish)
    result = {
        "workload": w.name, "rows": N, "vocab": V, "ms_per_step": ms_per_step, "value": value,
        "valid_tokens_per_s": value * float(data["mask"].mean().item()), "loss": loss, "device_status": status,
        "parallelism": parallelism, "roofline": roofline, "exchange": exchange, "parity": parity, "e2e": e2e,
        "gpu_launches": launches, "clocks": clocks, "steps": steps,
        "config": config_dict(w, world, mode, parallelism, args.seed),
    }
    return result


def measure_e2e(data, step_fn, args, job: Job, finish=lambda: None):
    """Same metric through the public API with HOST buffers: per step, copy the step's inputs (this
    rank's shard when N > 1) from pinned host memory, run fwd+bwd through `step_fn`, read the loss and
    the per-token log-probs back.  Time = max over ranks."""
    dist, dev = job.dist, job.dev
    from mllm_jax_b200 import host_io

    names = ("logits", "token_ids", "mask", "advantages", "old_logps", "ref_logps")
    host = {}
    # the staging buffers are allocated on the GPU's own NUMA node where sysfs names it (None: left where they fall)
    with host_io.near_gpu(dev.index if dev.index is not None else torch.cuda.current_device()) as numa_node:
        try:
            for k in names:
                host[k] = torch.empty(data[k].shape, dtype=data[k].dtype, pin_memory=True)
                host[k].copy_(data[k])
        except RuntimeError as e:  # not enough pinnable host memory
            return {"value": None, "unit": UNIT, "error": str(e)[:120]}
        torch.cuda.synchronize()
        n_local = data["token_ids"].numel()
        lp_host = torch.empty(data["token_ids"].shape, dtype=torch.float32, pin_memory=True)
        loss_host = torch.empty((), dtype=torch.float32, pin_memory=True)
    steps = max(2, min(args.steps, 5))
    h2d = sum(host[k].numel() * host[k].element_size() for k in names)
    d2h = lp_host.numel() * 4 + 4
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(1 + steps):
        if i == 1:
            job.barrier()
            ev0.record()
        for k in names:
            data[k].copy_(host[k], non_blocking=True)
        out = step_fn()
        finish()
        lp_host.copy_(out["per_token_logps"], non_blocking=True)
        loss_host.copy_(out["loss"], non_blocking=True)
        torch.cuda.synchronize()
    ev1.record()
    job.barrier()
    ms = job.max_over_ranks(ev0.elapsed_time(ev1))
    world = job.world
    token_mode = world > 1 and args.parallelism == "token"
    sec = ms * 1e-3 / steps
    return {"value": n_local * (world if token_mode else 1) / sec, "unit": UNIT, "h2d_bytes_per_step": h2d * world,
            "d2h_bytes_per_step": d2h * world, "ms_per_step": sec * 1e3, "steps": steps,
            "pinned_numa_node": numa_node,
            "note": "every rank copies its logits shard over its own PCIe link each step; dlogits stay on the "
                    "device for the lm_head backward"}


def main():
    args = parse()
    if args.impl == "reference":
        return run_reference(args)
    if args.fold_lm_head:
        line = run_fold_lm_head(Job(args), args, args.steps, args.warmup)
        print(json.dumps(line))
        return

    from mllm_jax_b200 import _lib, synth

    job = Job(args)
    lib = _lib.load()
    if args.plan:
        lib.mllm_grpo_set_plan_override(*[int(v) for v in args.plan.split(",")])
    res = run_workload(job, args.workload, args.steps, args.warmup, main=True)
    if "skipped" in res:
        raise SystemExit(res["skipped"])
    extra_names = args.extra if args.extra is not None else (DEFAULT_EXTRA if args.workload == "cfg1" else "none")
    extra = []
    for name in [n for n in extra_names.split(",") if n and n != "none" and n != args.workload]:
        gc.collect()
        torch.cuda.empty_cache()
        try:
            r = run_workload(job, name, steps=5, warmup=3, main=False)
        except torch.OutOfMemoryError as exc:
            r = {"workload": name, "skipped": f"out of device memory ({str(exc)[:60]})"}
            torch.cuda.empty_cache()
        keep = ("workload", "rows", "vocab", "ms_per_step", "value", "valid_tokens_per_s", "loss", "parallelism",
                "parity", "exchange", "skipped", "device_status")
        e = {k: r[k] for k in keep if k in r}
        if "roofline" in r:
            rf = r["roofline"]
            e.update(frac=rf["step"]["frac"], frac_min_dram=rf["step"]["frac_min_dram"], ms_per_launch=rf["ms_per_launch"],
                     launches_per_step=rf["step"]["launches_per_step"], chunks=r["config"]["chunks"])
        extra.append(e)

    fold = None
    if job.world == 1 and args.workload == "cfg1" and args.extra is None:
        # the row next to the path: lm_head folded into the forward (tensor-core kernel), measured briefly
        gc.collect()
        torch.cuda.empty_cache()
        try:
            f = run_fold_lm_head(job, args, steps=5, warmup=5)
            fold = {k: f[k] for k in ("metric", "value", "ms_per_step", "config", "roofline", "library_path", "weight_hv",
                                      "parity", "device_status")}
        except torch.OutOfMemoryError as exc:
            fold = {"skipped": f"out of device memory ({str(exc)[:60]})"}
    cpu = None
    if job.rank == 0 and job.world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(args, synth.parse_workload(args.workload))
    if job.dist is not None:
        job.dist.barrier()
        job.dist.destroy_process_group()
    if job.rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": job.world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": res["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16 in / f32 accumulate", "data": "synthetic",
            "config": res["config"], "loss": res["loss"], "device_status": res["device_status"],
            "valid_tokens_per_s": res["valid_tokens_per_s"], "roofline": res["roofline"], "exchange": res["exchange"],
            "parity": res["parity"], "cpu_baseline": cpu, "e2e": res["e2e"], "gpu_launches": res["gpu_launches"],
            "clocks": res["clocks"], "extra": extra, "fold_lm_head": fold,
        }))


def run_fold_lm_head(job, args, steps, warmup):
    """lm_head folded into the forward of the loss (1 GPU): hidden [N, H] x weight [V, H]^T -> per-token log-probs,
    entropy and loss with the logits held in tensor memory only, timed beside the library GEMM + loss kernel that
    materialises them.  Shapes: the workload's rows and vocabulary, H = 3584 (Qwen2.5-7B) unless --hidden."""
    import mllm_jax_b200 as G
    from mllm_jax_b200 import _lib, synth
    from mllm_jax_b200.linear_loss import lm_head_forward
    from oracle import grpo_oracle as O

    if job.world != 1:
        raise SystemExit("--fold-lm-head is a 1-GPU measurement")
    dev = job.dev
    w = synth.parse_workload(args.workload)
    if args.rows:
        w = synth.scaled(w, n_seqs=args.rows)
    if args.vocab:
        w = synth.scaled(w, vocab=args.vocab)
    B, T, V, H = w.n_seqs, w.seq_len, w.vocab, args.hidden
    N = B * T
    g = torch.Generator(device=dev).manual_seed(1234 + args.seed)
    hidden = torch.randn(B, T, H, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    weight = (torch.randn(V, H, generator=g, device=dev, dtype=torch.float32) * (w.sigma / H ** 0.5)).to(torch.bfloat16)
    side = synth.make_inputs(w, seed=args.seed, device=str(dev), want_logits=False)
    cfg = G.LossConfig(epsilon_low=w.epsilon_low, epsilon_high=w.epsilon_high, beta=w.beta, softcap=w.softcap)
    # old / ref log-probs around the true ones of THIS projection: one folded forward-only pass supplies them
    lp = lm_head_forward(hidden, weight, side["token_ids"], cfg=cfg)["per_token_logps"].clone()
    old = lp + (side["old_logps"] - side["exact_logps"])
    ref = lp + (side["ref_logps"] - side["exact_logps"])
    work = torch.empty(int(_lib.load().mllm_lm_head_partials_bytes(N, V)), dtype=torch.uint8, device=dev)
    call = (hidden, weight, side["token_ids"], side["mask"], side["advantages"], side["total_valid"], old, ref)

    def fused():
        return lm_head_forward(*call, cfg=cfg, workspace=work)

    logits = torch.empty(B, T, V, dtype=torch.bfloat16, device=dev)
    wt = weight.t()

    def library():
        torch.matmul(hidden, wt, out=logits)
        return G.grpo_token_loss_flat(logits, side["token_ids"], side["mask"], side["advantages"], side["total_valid"],
                                      old, ref, epsilon_low=w.epsilon_low, epsilon_high=w.epsilon_high, beta=w.beta,
                                      softcap=w.softcap)

    def timed(fn, steps, warmup):
        for _ in range(max(warmup, 3)):
            out = fn()
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(steps):
            out = fn()
        ev1.record()
        torch.cuda.synchronize()
        return ev0.elapsed_time(ev1) / steps, out

    sampler = ClockSampler(job.local)
    sampler.start()
    time.sleep(0.15)
    launches0 = _lib.launch_count()
    ms_fused, out = timed(fused, steps, warmup)
    launches = _lib.launch_count() - launches0
    clocks = sampler.stop()
    ms_lib, out_lib = timed(library, max(3, steps // 2), 3)
    # the same forward on the weight as a flax Dense kernel stores it ([H, V], MN-major tensor-core operand)
    w_hv = weight.t().contiguous()
    ms_hv, out_hv = timed(lambda: lm_head_forward(hidden, w_hv, *call[2:], cfg=cfg, workspace=work, weight_layout="hv"),
                          max(3, steps // 2), 3)
    hv_lp_diff = float((out_hv["per_token_logps"] - lm_head_forward(*call, cfg=cfg)["per_token_logps"]).abs().max().item())
    flops = 2.0 * N * V * H
    peak = float(job.peaks.get("bf16_tflops_sustained", 1400.0))
    tf = flops / (ms_fused * 1e-3) / 1e12
    # parity on sampled rows against float64 logits of the same operands
    rows = sample_rows(N, 48).to(dev)
    x64 = O.lm_head_logits(hidden.view(N, H)[rows].cpu(), weight.cpu()).numpy()
    pick = lambda t: t.reshape(N)[rows].double().cpu().numpy()  # noqa: E731
    import numpy as np
    advN = side["advantages"][:, None].expand(-1, T).reshape(N)
    an = O.analytic_rows(x64, side["token_ids"].reshape(N)[rows].long().cpu().numpy(), pick(side["mask"]), pick(advN),
                         pick(old), pick(ref), side["total_valid"], beta=w.beta, epsilon_low=w.epsilon_low,
                         epsilon_high=w.epsilon_high, softcap=w.softcap, want_grad=False)
    lp_abs = float(np.abs(pick(out["per_token_logps"]) - an["lp"]).max())
    ent_abs = float(np.abs(pick(out["token_entropy"]) - an["entropy_guard"]).max())
    terms_abs = float(np.abs(pick(out["problem"].loss_terms) - an["loss_terms"]).max())
    return ({
        "metric": "lm_head + GRPO loss forward tokens/s (logits never in HBM)", "value": N / (ms_fused * 1e-3),
        "unit": UNIT, "n_gpus": 1, "steps": steps, "warmup": max(warmup, 3), "ms_per_step": ms_fused,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 operands / f32 accumulate",
        "data": "synthetic",
        "config": {"workload": w.name + "-fold-lm-head", "rows": N, "vocab": V, "hidden": H,
                   "l2": "weight (%.2f GB) and hidden (%.2f GB) exceed the 126 MB L2" % (V * H * 2 / 1e9, N * H * 2 / 1e9)},
        "loss": float(out["loss"].item()), "device_status": int(out["problem"].device_status.item()),
        "roofline": {"bound": "tensor", "kernel": "lm_head_stats_kernel (tcgen05.mma 128x256x16 bf16, TMEM accumulators)",
                     "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak, "peak_kind": job.peak_kind +
                     " (library bf16 GEMM sustained)", "flops_per_launch": flops, "ms_per_launch": ms_fused,
                     "traffic": None,
                     "note": "ms_per_launch covers the tensor-core kernel plus the two small merge kernels"},
        "weight_hv": {"what": "same kernel on the [hidden, vocab] weight (MN-major operand, no transpose)",
                      "ms_per_step": ms_hv, "tflops": flops / (ms_hv * 1e-3) / 1e12, "lp_abs_vs_vh": hv_lp_diff},
        "library_path": {"what": "torch.matmul (library GEMM) writing bf16 logits + mllm_grpo_fwd reading them",
                         "ms_per_step": ms_lib, "tflops": flops / (ms_lib * 1e-3) / 1e12,
                         "logits_bytes": 2.0 * N * V, "loss": float(out_lib["loss"].item())},
        "parity": {"rows": int(rows.numel()), "lp_abs": lp_abs, "entropy_abs": ent_abs, "loss_terms_abs": terms_abs,
                   "ok": bool(lp_abs <= 2e-3 and ent_abs <= 5e-4),
                   "against": "closed-form f64 CPU oracle on float64 logits of the same bf16 operands"},
        "gpu_launches": launches, "clocks": clocks,
    })


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from mllm_jax_b200 import synth

    w = synth.parse_workload(args.workload)
    world = max(1, args.gpus)
    mode = "single" if world == 1 else args.parallelism
    t_all = time.perf_counter()
    cb = cpu_baseline(args, w, steps=args.steps, warmup=min(args.warmup, 2))
    value = cb["value"]
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": cb["ms_per_pass"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(w, world, mode, default_parallelism(world, mode, w.n_seqs // world if mode == "token"
                                                                    else w.n_seqs), args.seed),
        "note": "the reference's jnp path needs JAX, which is installed neither on the build host nor on the GPU hosts "
                "(probed); this arm times the line-for-line torch-CPU restatement on a bounded sample of the same "
                "workload (same vocabulary and distributions; the per-token cost does not depend on the row count)",
        "cpu_baseline": cb,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t_all,
    }))


if __name__ == "__main__":
    main()
