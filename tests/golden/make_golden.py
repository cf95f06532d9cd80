"""Regenerates the golden fixtures in this folder from the CPU oracle.

Run from the repository root:  python tests/golden/make_golden.py
Each .npz holds one small case in the reference layout: bf16 logits as bit patterns,
input_ids, labels, advantages, optional old / ref log-probs, the attributes, and the
oracle's float32 outputs (loss, per_token_logps, token_entropy, entropy, entropy_loss, dlogits).
The reference itself ships no vectors for this path and cannot run where this was written
(JAX unavailable), so these pin the oracle and the kernels to one another across machines.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import grpo_oracle as O  # noqa: E402
from tests.util import make_case  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = {
    # name: (make_case kwargs, attributes)
    "grpo_b2_l9_v1000": (dict(B=2, L=9, V=1000, seed=101, old="noisy", ref=True),
                         dict(beta=0.04, temperature=1.0, epsilon_low=0.2, epsilon_high=0.3, softcap=None)),
    "grpo_b3_l6_v4099_no_old": (dict(B=3, L=6, V=4099, seed=102, old="none"),
                                dict(beta=0.0, temperature=1.0, epsilon_low=0.2, epsilon_high=0.3, softcap=None)),
    "grpo_b2_l5_v2048_wide_clip": (dict(B=2, L=5, V=2048, seed=103, old="wide", ref=True),
                                   dict(beta=0.04, temperature=1.0, epsilon_low=0.2, epsilon_high=0.2, softcap=None)),
    "grpo_b2_l5_v3000_softcap30": (dict(B=2, L=5, V=3000, seed=104, old="noisy", ref=True, sigma=4.0),
                                   dict(beta=0.04, temperature=1.0, epsilon_low=0.2, epsilon_high=0.2, softcap=30.0)),
    "grpo_b2_l7_v129_temp07": (dict(B=2, L=7, V=129, seed=105, old="noisy"),
                               dict(beta=0.0, temperature=0.7, epsilon_low=0.2, epsilon_high=0.3, softcap=None)),
    "ppo_b2_l6_v777_token_adv": (dict(B=2, L=6, V=777, seed=106, old="wide", per_token_adv=True),
                                 dict(beta=0.0, temperature=1.0, epsilon_low=0.2, epsilon_high=0.2, softcap=None)),
}


def main():
    for name, (kw, attrs) in CASES.items():
        logits, inputs = make_case(**kw)
        out = O.reference_value_and_grad(logits, inputs, **attrs)
        rec = {
            "logits_bf16_bits": logits.view(torch.int16).numpy().astype(np.uint16),
            "input_ids": inputs["input_ids"].numpy(), "labels": inputs["labels"].numpy(),
            "advantages": inputs["advantages"].numpy(),
            "total_valid_token_count": np.float32(inputs["total_valid_token_count"]),
            "beta": np.float32(attrs["beta"]), "temperature": np.float32(attrs["temperature"]),
            "epsilon_low": np.float32(attrs["epsilon_low"]), "epsilon_high": np.float32(attrs["epsilon_high"]),
            "softcap": np.float32(attrs["softcap"] or 0.0),
            "loss": np.float32(out["loss"].item()), "per_token_logps": out["per_token_logps"].numpy(),
            "token_entropy": out["token_entropy"].numpy(), "entropy": out["entropy"].numpy(),
            "entropy_loss": out["entropy_loss"].numpy(), "dlogits": out["dlogits"].numpy(),
        }
        for k in ("old_per_token_logps", "ref_per_token_logps"):
            if k in inputs:
                rec[k] = inputs[k].numpy()
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
        print(name, "loss", float(rec["loss"]))


if __name__ == "__main__":
    main()
