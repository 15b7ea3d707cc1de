"""The tuned-config file and the candidate enumeration of attentionengine_b200/tune.py (no GPU: the sweep itself
needs one and is exercised on a B200 by ``python -m attentionengine_b200.tune``)."""
import json

import torch

from attentionengine_b200 import tune
from attentionengine_b200.attn_engine import attn_bwd as ab

import helpers


def test_file_is_a_list_of_problem_entries_looked_up_by_keys(tmp_path):
    f = tmp_path / "tuned.json"
    k1 = tune.problem_keys(8, 32, 8, 8192, 8192, 128, 128, torch.float16, 1)
    k2 = tune.problem_keys(4, 16, 16, 4096, 4096, 64, 64, torch.float16, 1)
    assert tune.lookup(f, k1) is None
    tune.store(f, k1, {"stages": 2, "mode": "fused", "fused_tile": [2, 1, 4]}, [{"kernel": "fwd", "stages": 2, "ms": 1.0}])
    tune.store(f, k2, {"stages": 3, "mode": "split"}, [])
    tune.store(f, k1, {"stages": 2, "mode": "split"}, [])          # a second sweep of a problem replaces its entry
    entries = json.loads(f.read_text())
    assert len(entries) == 2 and all("tuned_config" in e and "candidates" in e for e in entries)
    assert tune.lookup(f, k1) == {"stages": 2, "mode": "split"} and tune.lookup(f, k2)["stages"] == 3
    other_shape = tune.problem_keys(1, 4, 4, 512, 512, 64, 64, torch.float16, 1)
    assert tune.lookup(f, other_shape) is None
    assert tune.lookup(f, other_shape, exact=False)["stages"] == 3  # same head dims / dtype / mask class


def test_candidates_fit_in_shared_memory():
    c = tune.candidates(128, 128, 1)
    # three stages do not fit at head dim 128; the forward over CTA pairs is a candidate at value head dim 128
    assert c["fwd"] == [{"stages": 2}, {"fwd_pair": 1, "fwd_pair_stages": 5}]
    assert {"mode": "fused", "fused_tile": [2, 1, 4]} in c["bwd"]
    assert all(ab.fused_smem_bytes(128, 128, 2, *x["fused_tile"][:2]) <= tune.SMEM_MAX for x in c["bwd"] if x["mode"] == "fused")
    c64 = tune.candidates(64, 64, 1)
    assert {"stages": 4} in c64["fwd"] and len(c64["bwd"]) > len(c["bwd"])
    assert not any("fwd_pair" in x for x in c64["fwd"])


def test_engine_takes_its_tile_choice_from_the_tune_file(tmp_path, monkeypatch):
    f = tmp_path / "tuned.json"
    keys = tune.problem_keys(1, 4, 2, 512, 512, 64, 64, torch.float16, 1)
    tune.store(f, keys, {"stages": 3, "mode": "split", "dq_tile": [128, 2, 2], "dkv_tile": [128, 2, 2, 4, 0]}, [])
    eng = helpers.softmax_engine(1, 4, 2, 512, 64, 64, torch.float16, True, tune_file=str(f))
    assert eng.kernels.stages == 3 and eng.bwd_mode == "split"
    assert ab.dq_tile_config(64, 64, eng.kernels.tuned) == (128, 2, 2)
    assert eng.kernels.bwd.dkv.cfg.stages == 2
    # the package's own table is the fallback; without it the built-in defaults apply
    monkeypatch.setattr(tune, "PACKAGE_FILE", tmp_path / "absent.json")
    plain = helpers.softmax_engine(1, 4, 2, 512, 64, 64, torch.float16, True)
    assert plain.tuned_config == {} and plain.kernels.stages == 2 and plain.bwd_mode is None


def test_batch_ranges_of_the_backward_launches():
    """The backward passes are launched as 4, 2 or 1 batch ranges: never more than asked for, only when the batch
    divides, and only while a range still brings the required number of CTAs per SM."""
    # the 8K GQA problem: 32 heads x 64 kv tiles per batch row, eight rounds of 148 SMs asked per range
    assert ab.batch_ranges(8, 32 * 64, 148, 4, min_rounds=8) == 4
    assert ab.batch_ranges(8, 32 * 64, 148, 2, min_rounds=8) == 2
    assert ab.batch_ranges(8, 32 * 64, 148, 1, min_rounds=8) == 1
    assert ab.batch_ranges(1, 32 * 64, 148, 4, min_rounds=8) == 1      # one batch row per rank at eight ranks
    assert ab.batch_ranges(6, 32 * 64, 148, 4, min_rounds=8) == 2      # 6 rows do not divide by 4
    assert ab.batch_ranges(4, 4 * 3, 148, 4, min_rounds=8) == 1        # small problems stay one launch
    # the scan's reverse pass: one CTA per (batch row, head), 80 heads
    assert ab.batch_ranges(8, 80, 148, 2) == 2 and ab.batch_ranges(8, 80, 148, 4) == 4
    assert ab.batch_ranges(2, 80, 148, 4) == 1                         # a single row would leave SMs empty
