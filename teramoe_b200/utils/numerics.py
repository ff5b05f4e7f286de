"""bf16 numerics check: max-abs, cosine and the reference's calc_diff in one device pass.

The three criteria and their limits are the reference's acceptance test
(tests/test_teramoe_accuracy.py:60-82, :390-395): max_abs <= 1e-2, calc_diff <= 1e-5, cosine >= 0.99.
On CUDA the statistics come from the hand-written reduction kernel (csrc/comm.cu numerics_check).
"""
from __future__ import annotations

import torch


def numerics_report(a: torch.Tensor, b: torch.Tensor) -> dict:
    if a.shape != b.shape:
        raise ValueError(f"shape mismatch {tuple(a.shape)} vs {tuple(b.shape)}")
    if a.is_cuda:
        from .._build import load_ext
        if a.dtype != b.dtype or a.dtype not in (torch.bfloat16, torch.float32):
            a, b = a.float(), b.float()
        s = load_ext().numerics_check(a.contiguous(), b.contiguous()).tolist()
        mx, sab, saa, sbb, sp, sq = s
    else:
        x, y = a.double(), b.double()
        mx = float((x - y).abs().max()) if x.numel() else 0.0
        sab, saa, sbb = float((x * y).sum()), float((x * x).sum()), float((y * y).sum())
        sp, sq = float(((x + 1) * (y + 1)).sum()), float(((x + 1) ** 2 + (y + 1) ** 2).sum())
    cos = sab / max((saa * sbb) ** 0.5, 1e-30) if saa > 0 and sbb > 0 else (1.0 if saa == sbb else 0.0)
    diff = 1.0 - 2.0 * sp / sq if sq > 0 else 0.0
    return {"max_abs": mx, "cosine": cos, "calc_diff": diff}


def assert_close_bf16(a, b, name="tensor", max_abs=1e-2, calc_diff=1e-5, cosine=0.99) -> dict:
    r = numerics_report(a, b)
    ok = r["max_abs"] <= max_abs and r["calc_diff"] <= calc_diff and r["cosine"] >= cosine
    if not ok:
        raise AssertionError(f"{name}: {r} exceeds limits max_abs<={max_abs} calc_diff<={calc_diff} cosine>={cosine}")
    return r
