"""Acceptance rule of the GPU parity tests, in one place.

fp16 results: max-abs <= 2e-2 (times the largest reference magnitude for un-normalised outputs) and rel-L2 <= 1e-3
against the fp32 / fp64 oracle, the tolerance the benchmark specification states.

bf16 results cannot meet 1e-3: rounding the exact result to bf16 is already a rel-L2 of about 1.7e-3.  They are held to
that floor instead of to a flat number: with ``floor`` = rel-L2 of (oracle rounded to bf16) against the oracle, measured
on the very tensor under test, a result passes when

    rel-L2(kernel, oracle) <= K_BF16 * floor * sqrt(stages)

where ``stages`` counts the bf16 roundings between the inputs and that result which the algorithm cannot avoid on
16-bit tensor cores: the stored result itself plus every operand the kernel has to round before a tensor-core product
(P, dS, carried states ...); independent roundings add in quadrature.  ``stages`` is written next to every check.
The max-abs bound scales the same way from the 2e-2 of fp16 by the ratio of the two formats' rounding steps (8).

Every check can append its measured figures to the file named by AE_B200_PARITY_LOG (one JSON object per line).
"""
import json
import math
import os

import torch

from oracle import attention_oracle as orc

MAX_ABS, REL_L2 = 2e-2, 1e-3
K_BF16 = 1.15


def check(name, got, ref, dtype, stages=1, unnormalised=False, rel_limit=None):
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    mag = max(1.0, ref.abs().max().item()) if unnormalised else 1.0
    mx, rel = orc.error_stats(got, ref)
    if dtype == torch.bfloat16:
        _, floor = orc.error_stats(ref.to(torch.bfloat16), ref)
        lim_rel = K_BF16 * floor * math.sqrt(stages)
        lim_abs = 8 * MAX_ABS * mag
    else:
        floor = None
        lim_rel, lim_abs = REL_L2, MAX_ABS * mag
    if rel_limit is not None:  # a limit of its own, stated at the call (fp32 sums of many cancelling 16-bit terms)
        lim_rel, lim_abs = rel_limit, float("inf")
    log = os.environ.get("AE_B200_PARITY_LOG")
    if log:
        with open(log, "a") as f:
            f.write(json.dumps({"name": name, "dtype": str(dtype).replace("torch.", ""), "shape": list(got.shape),
                                "max_abs": mx, "rel_l2": rel, "floor": floor, "stages": stages,
                                "limit_rel": lim_rel, "limit_abs": lim_abs}) + "\n")
    assert mx <= lim_abs and rel <= lim_rel, (f"{name}: max-abs {mx:.3e} (limit {lim_abs:.3e}), rel-L2 {rel:.3e} "
                                              f"(limit {lim_rel:.3e}" + (f", bf16 floor {floor:.3e} x {stages} stages)"
                                                                         if floor else ")"))
    return mx, rel
