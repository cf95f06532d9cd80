"""Helpers shared by the tests: seeded cases in the reference layout and tolerance checks.

Tolerances (the parity gate): per-token log-prob 2e-3 abs, loss 1e-4 rel, dlogits 1e-2 rel,
where "rel" for dlogits means, per row, max|d - ref| <= 1e-2 * max|ref| and, elementwise,
|d - ref| <= 1e-2*|ref| + one bf16 ulp of the row maximum.  Entropy: 5e-4 abs (the kernel
omits the reference's +1e-9 guard, worth at most V*1e-9).
"""
from __future__ import annotations

import numpy as np
import torch

LP_ATOL = 2e-3
LOSS_RTOL = 1e-4
DLOGITS_RTOL = 1e-2
ENT_ATOL = 5e-4


def make_case(B, L, V, seed=0, sigma=2.0, old="noisy", ref=False, per_token_adv=False, mask_kind="lengths",
              adv_scale=1.0):
    """Inputs in the reference layout: logits [B, L, V] bf16, input_ids/labels [B, L], advantages."""
    g = torch.Generator().manual_seed(seed)
    logits = (torch.randn(B, L, V, generator=g) * sigma).to(torch.bfloat16)
    input_ids = torch.randint(0, V, (B, L), generator=g, dtype=torch.int64).to(torch.int32)
    if mask_kind == "lengths":
        lens = torch.randint(max(1, L // 4), L + 1, (B,), generator=g)
        labels = (torch.arange(L)[None, :] < lens[:, None]).to(torch.int32)
        labels[:, 0] = 0  # prompt token
    elif mask_kind == "ones":
        labels = torch.ones(B, L, dtype=torch.int32)
    else:
        labels = (torch.rand(B, L, generator=g) < 0.6).to(torch.int32)
    if per_token_adv:
        adv = torch.randn(B, L - 1, generator=g) * adv_scale
    else:
        adv = torch.randn(B, generator=g) * adv_scale
    inputs = {"input_ids": input_ids, "labels": labels, "attention_mask": torch.ones(B, L, dtype=torch.int32),
              "advantages": adv, "total_valid_token_count": float(labels[:, 1:].sum().item()) or 1.0}
    if old != "none" or ref:
        x = logits.float()
        lp = torch.log_softmax(x[:, :-1], -1).gather(-1, input_ids[:, 1:].long()[..., None])[..., 0]
        if old == "noisy":
            inputs["old_per_token_logps"] = lp + 0.05 * torch.randn(B, L - 1, generator=g)
        elif old == "wide":  # many tokens outside the clip interval
            inputs["old_per_token_logps"] = lp + 0.4 * torch.randn(B, L - 1, generator=g)
        if ref:
            inputs["ref_per_token_logps"] = lp + 0.1 * torch.randn(B, L - 1, generator=g)
    return logits, inputs


def to_device(inputs, dev):
    return {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in inputs.items()}


def bf16_ulp(x: np.ndarray) -> np.ndarray:
    x = np.abs(x).astype(np.float64)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(x > 0, x, 1.0)))
    return np.where(x > 0, 2.0 ** (e - 7), 0.0)


def assert_dlogits_close(d: torch.Tensor, ref: torch.Tensor, rtol=DLOGITS_RTOL, what=""):
    d = d.detach().float().cpu().numpy().reshape(-1, d.shape[-1]).astype(np.float64)
    r = ref.detach().double().cpu().numpy().reshape(-1, ref.shape[-1])
    assert d.shape == r.shape, (d.shape, r.shape)
    rowmax = np.abs(r).max(axis=1)
    err = np.abs(d - r)
    # rows that must be exactly zero
    zero_rows = rowmax == 0
    assert (err[zero_rows] == 0).all(), f"{what}: rows with zero gradient are not exactly zero"
    nz = ~zero_rows
    if nz.any():
        rel_row = err[nz].max(axis=1) / rowmax[nz]
        assert rel_row.max() <= rtol, f"{what}: row-relative dlogits error {rel_row.max():.3e} > {rtol}"
        bound = rtol * np.abs(r[nz]) + bf16_ulp(rowmax[nz])[:, None]
        worst = (err[nz] - bound).max()
        assert worst <= 0, f"{what}: elementwise dlogits error exceeds bound by {worst:.3e}"


def assert_loss_close(a, b, rtol=LOSS_RTOL, what=""):
    a, b = float(a), float(b)
    assert abs(a - b) <= rtol * max(abs(b), 1e-12) + 1e-9, f"{what}: loss {a!r} vs oracle {b!r}"
