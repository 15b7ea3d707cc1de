"""Tile / stage sweep of the attention kernels and the tuned-config file.

Stands in for the reference's autotuner and its json cache (core/template/tl_template/attn/attn_tl.py:474-500:
a file holding a list of ``{problem keys..., "tuned_config": ...}`` entries, looked up by problem size, filled by
profiling when the entry is missing; candidate enumeration autotuner/decider.py:40-128,
autotuner/attnfwd_tunner.py:61-172).  The search space here is small because the kernels are hand-written
templates: ring depths of the streamed tiles, the number of row warpgroups, which form of the forward runs (one CTA
with two q tiles, or a CTA pair on tcgen05 cta_group::2) and which form of the backward (one kv-stationary pass with
fp32 dQ adds, or two passes without atomics).

``AttentionEngine(..., tune=True, tune_file=path)`` looks its problem up in ``path`` and, when it is not there, runs
``sweep`` on the current CUDA device (a few seconds: every candidate is compiled, timed with CUDA events on seeded
inputs of the problem's own shape, capped at ``max_rows`` batch x head rows) and appends the result.  Without
``tune`` an engine takes the entry of the package's own file (``tuned/sm_100a.json``, measured on a B200) when one
matches its head dims and dtype, else the built-in defaults.
"""
from __future__ import annotations

import json
import os
import time
from pathlib import Path

PACKAGE_FILE = Path(__file__).resolve().parent / "tuned" / "sm_100a.json"
SMEM_MAX = 232448


def problem_keys(B, Hq, Hkv, Sq, Skv, D, DV, dtype, mask_mode) -> dict:
    return {"batch": B, "heads": Hq, "kv_heads": Hkv, "seq_len": Sq, "seq_len_kv": Skv, "dim": D, "dimv": DV,
            "dtype": str(dtype).replace("torch.", ""), "mask_mode": mask_mode}


def lookup(path, keys: dict, exact: bool = True):
    """The tuned_config of the entry for ``keys``; with ``exact=False`` an entry that matches head dims, dtype and
    mask mode only (shapes the kernels do not depend on) is accepted."""
    path = Path(path)
    if not path.exists():
        return None
    try:
        entries = json.loads(path.read_text())
    except (OSError, ValueError):
        return None
    loose = ("dim", "dimv", "dtype", "mask_mode")
    for e in entries:
        if all(e.get(k) == v for k, v in keys.items()):
            return e["tuned_config"]
    if not exact:
        for e in entries:
            if all(e.get(k) == keys[k] for k in loose):
                return e["tuned_config"]
    return None


def store(path, keys: dict, tuned_config: dict, table: list):
    path = Path(path)
    entries = []
    if path.exists():
        try:
            entries = json.loads(path.read_text())
        except (OSError, ValueError):
            entries = []
    entries = [e for e in entries if not all(e.get(k) == v for k, v in keys.items())]
    entries.append({**keys, "tuned_config": tuned_config, "candidates": table})
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_suffix(f".tmp{os.getpid()}")
    tmp.write_text(json.dumps(entries, indent=1))
    os.replace(tmp, path)


def candidates(D: int, DV: int, n_final: int) -> dict:
    """Every configuration that fits in a CTA's shared memory, per kernel."""
    from .attn_engine import attn_bwd as ab
    ncs = n_final + 1
    fwd = [{"stages": st} for st in (2, 3, 4) if 2 * 128 * D * 2 + st * 128 * (D + DV) * 2 + 1536 <= SMEM_MAX]
    if DV == 128 and D in (64, 128):  # the forward over CTA pairs (falls back by itself under block lists)
        fwd.append({"fwd_pair": 1, "fwd_pair_stages": 5})
    fused = [{"mode": "fused", "fused_tile": [q, d, g]} for q in (2, 3, 4) for d in (1, 2) for g in (4,)
             if ab.fused_smem_bytes(D, DV, ncs, q, d) <= SMEM_MAX]
    split = []
    for bn, ks, vs in ((128, 3, 3), (128, 2, 2)):  # the dQ pass streams 128-row K / V tiles
        if bn * (ks * D + vs * DV) * 2 + 1536 <= SMEM_MAX:
            for dkv in ((128, 3, 2, 4, 0), (128, 2, 2, 4, 0), (128, 3, 3, 4, 0), (128, 2, 2, 2, 0)):
                smem = 128 * (D + DV) * 2 + dkv[0] * (dkv[1] * D + dkv[2] * DV) * 2 + 2 * dkv[0] * ncs * 4 + 256
                if smem <= SMEM_MAX:
                    split.append({"mode": "split", "dq_tile": [bn, ks, vs], "dkv_tile": list(dkv)})
    return {"fwd": fwd, "bwd": fused + split}


def sweep(score_mod, mask_mod, online_func, custom_io, keys: dict, mask_value="-inf", iters: int = 3,
          max_rows: int = 16, budget_s: float = 30.0, log=None) -> tuple:
    """Time every candidate on the current CUDA device.  Returns (tuned_config, table)."""
    import torch

    from .attn_engine.attn_engine import AttentionEngine
    from .core.utils import meta_tensor
    if not torch.cuda.is_available():
        raise RuntimeError("the sweep times kernels: it needs a CUDA device")
    dt = getattr(torch, keys["dtype"])
    Hq, Hkv, Sq, Skv, D, DV = (keys[k] for k in ("heads", "kv_heads", "seq_len", "seq_len_kv", "dim", "dimv"))
    B = max(1, min(keys["batch"], max_rows // max(1, Hkv)))  # the tile choice does not depend on the batch
    metas = (meta_tensor(B, Hq, Sq, D, dtype=dt), meta_tensor(B, Hkv, Skv, D, dtype=dt),
             meta_tensor(B, Hkv, Skv, DV, dtype=dt))
    g = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randn(B, Sq, Hq, D, device="cuda", dtype=dt, generator=g)
    k = torch.randn(B, Skv, Hkv, D, device="cuda", dtype=dt, generator=g)
    v = torch.randn(B, Skv, Hkv, DV, device="cuda", dtype=dt, generator=g)
    d_o = torch.randn(B, Sq, Hq, DV, device="cuda", dtype=dt, generator=g)
    customs = [torch.zeros([1 if isinstance(n, str) or n == 1 else n for n in sym.shape_idx] or [1], device="cuda")
               for sym in custom_io.input_tensors.values()]

    def build(cfg):
        return AttentionEngine(metas, custom_io, score_mod=score_mod, mask_mod=mask_mod, online_func=online_func,
                               mask_value=mask_value, tuned_config=cfg)

    def time_ms(fn):
        fn()
        torch.cuda.synchronize()
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b_.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b_) / iters

    t_end = time.time() + budget_s
    probe = build({})
    cands = candidates(D, DV, len(probe.lowered.final_names))
    table, best = [], {}
    for kind in ("fwd", "bwd"):
        best_ms = None
        for cand in cands[kind]:
            if time.time() > t_end and best_ms is not None:
                table.append({"kernel": kind, **cand, "ms": None, "note": "not timed: sweep budget used up"})
                continue
            try:
                eng = build({**best, **cand})
                if kind == "fwd":
                    ms = time_ms(lambda: eng._launch_fwd(q, k, v, customs))
                else:
                    o, finals = eng._launch_fwd(q, k, v, customs)
                    ms = time_ms(lambda: eng._launch_bwd(q, k, v, o, d_o, finals, customs))
                eng.check_status()
            except Exception as e:  # a candidate that does not compile or launch is recorded, not fatal
                table.append({"kernel": kind, **cand, "ms": None, "note": f"{type(e).__name__}: {e}"[:200]})
                continue
            table.append({"kernel": kind, **cand, "ms": round(ms, 4)})
            if log:
                log(f"{kind} {cand} {ms:.3f} ms")
            if best_ms is None or ms < best_ms:
                best_ms, pick = ms, cand
        if best_ms is not None:
            best.update(pick)
    best["swept_on"] = {"batch": B, "device": torch.cuda.get_device_name()}
    return best, table


def resolve(engine_kwargs: dict, keys: dict, tune: bool, tune_file: str) -> dict:
    """The tuned_config an engine starts from: the caller's file (swept and appended when ``tune`` and missing),
    else the package's file, else {} (built-in defaults)."""
    if tune_file:
        cfg = lookup(tune_file, keys)
        if cfg is None and tune:
            cfg, table = sweep(**engine_kwargs, keys=keys)
            store(tune_file, keys, cfg, table)
        if cfg is not None:
            return cfg
    elif tune:
        cfg, _ = sweep(**engine_kwargs, keys=keys)
        return cfg
    return lookup(PACKAGE_FILE, keys, exact=False) or {}


def main(argv=None):
    """``python -m attentionengine_b200.tune [--out FILE]``: sweep the three problem classes of the benchmark
    configurations (fp16 head dim 128 causal GQA; fp16 head dim 64 causal MHA; bf16 head dim 128 non-causal with an
    identity online function) on the current CUDA device and write the table the package ships."""
    import argparse
    import math

    import torch

    from . import examples as ex
    from .core import CustomIO
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(PACKAGE_FILE))
    args = ap.parse_args(argv)
    if os.path.exists(args.out):
        os.remove(args.out)
    scale = 1 / math.sqrt(128)
    problems = [
        ("cfg2", dict(score_mod=lambda s, c, b, h, q, kv: s * scale, mask_mod=ex.causal_mask,
                      online_func=ex.OnlineSoftmax(), custom_io=CustomIO({})),
         problem_keys(8, 32, 8, 8192, 8192, 128, 128, torch.float16, 1)),
        ("d64", dict(score_mod=lambda s, c, b, h, q, kv: s * 0.125, mask_mod=ex.causal_mask,
                     online_func=ex.OnlineSoftmax(), custom_io=CustomIO({})),
         problem_keys(4, 16, 16, 4096, 4096, 64, 64, torch.float16, 1)),
        ("cfg3", dict(score_mod=lambda s, c, b, h, q, kv: (s * scale).max(0) * (1.0 / 4096), mask_mod=None,
                      online_func=ex.OnlineIdentity(), custom_io=CustomIO({})),
         problem_keys(4, 32, 32, 4096, 4096, 128, 128, torch.bfloat16, 0)),
    ]
    for name, kwargs, keys in problems:
        cfg, table = sweep(**kwargs, keys=keys, log=lambda m, n=name: print(n, m, flush=True))
        store(args.out, keys, cfg, table)
        print(name, "->", cfg, flush=True)


if __name__ == "__main__":
    main()
