"""CPU oracle for the chunked linear-attention / SSD scan.  TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

The step-by-step recurrence the reference's kernels implement in chunked form
(attention_engine/core/template/tl_template/linear/linear_tl.py:172-207 state pass, :349-388 output pass):

    S_t = exp(a_t) S_{t-1} + k_t^T v_t ,     o_t = q_t S_t ,      a = decay_mod(decay), v = v_mod(v), ...

Parity: the reference checks this path only against third-party GPU kernels (mamba_ssm for Mamba2, absent here;
flash-linear-attention for simple_gla, bench_utils.py:552-566).  ``tests/golden/linear_scan.npz`` holds the output
of flash-linear-attention's own naive recurrent form (fla.ops.simple_gla.naive) run on CPU, which pins the
recurrence; ``tests/golden/mamba2.npz`` pins the Mamba2 mapping on top of it: the reference's own ``decay_mod`` /
``v_mod`` (attn_script/mamba2_ngroup1.py:26-33) evaluated by the reference's IR front end and fed to that recurrence.
The D_skip term has no counterpart in the reference (its harness passes D=None, bench_utils.py:304-308); it is the
benchmark configuration's ``o += D_skip[h] * x``.
"""
from __future__ import annotations

import torch


def linear_scan(q, k, v, a, dtype=torch.float64):
    """q [B, HQ, T, DK], k [B, HK, T, DK], v [B, H, T, DV], a [B, H, T] log-decay.  Returns o [B, H, T, DV]."""
    B, H, T, DV = v.shape
    q, k, v, a = q.to(dtype), k.to(dtype), v.to(dtype), a.to(dtype)
    q = q.repeat_interleave(H // q.shape[1], dim=1)
    k = k.repeat_interleave(H // k.shape[1], dim=1)
    S = torch.zeros(B, H, q.shape[-1], DV, dtype=dtype)
    outs = []
    for t in range(T):
        S = S * a[:, :, t].exp()[..., None, None] + k[:, :, t, :, None] * v[:, :, t, None, :]
        outs.append(torch.einsum("bhk,bhkv->bhv", q[:, :, t], S))
    return torch.stack(outs, dim=2)


def mamba2_ssd(x, dt, A, Bm, Cm, D_skip=None):
    """Mamba2 SSD in the reference's operator mapping (attn_script/mamba2_ngroup1.py:26-33, bench_utils.py:317-333):
    q = C, k = B, v = x * dt, a = dt * A; optional skip connection o += D_skip[h] * x.
    x [B, H, T, P], dt [B, H, T], A [H], Bm / Cm [B, G, T, N]."""
    a = dt.double() * A.double().view(1, -1, 1)
    v = x.double() * dt.double()[..., None]
    o = linear_scan(Cm, Bm, v, a)
    if D_skip is not None:
        o = o + D_skip.double().view(1, -1, 1, 1) * x.double()
    return o
