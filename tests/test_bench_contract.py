"""The one JSON line bench.py prints: every key the benchmark contract names is present and consistent, for the
flagship and for the other configurations (--model).  Runs without a GPU: only the row builder, the synthetic
batches and the argument handling are exercised."""

import argparse
import importlib
import json
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture
def bench():
    sys.path.insert(0, ROOT)
    try:
        module = importlib.import_module("bench")
        yield importlib.reload(module)  # a fresh copy: select_model() rebinds module globals
    finally:
        sys.path.remove(ROOT)


def row_for(bench, **overrides):
    args = argparse.Namespace(gpus=2, steps=20, warmup=5, **overrides)
    clocks = {"sm_mhz": 1965.0, "sm_max_mhz": 1965.0, "reasons": [], "samples": 7}
    return bench.result_line(args, "ours", "ddp", 8.0, 8.1, 131072, 4, 8300, clocks, "bf16", {"kernels": "b200"})


def test_flagship_row_has_every_contract_key(bench):
    row = json.loads(json.dumps(row_for(bench)))  # it must survive serialisation
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches", "impl"):
        assert key in row, key
    assert row["metric"] == "gpt_85.8M_ddp_tokens_per_s" and row["unit"] == "tokens/s" and row["higher_is_better"] is True
    tokens = 16 * 512
    assert row["value"] == pytest.approx(tokens / 8.0e-3) and row["ms_per_step"] == 8.0
    assert row["vs_baseline"] == pytest.approx(row["value"] / 10265.0)
    assert row["config"]["global_batch"] == 16 and row["config"]["seq_len"] == 512 and row["config"]["parallelism"] == "ddp2"
    assert "l2" in row["config"] and row["scaling"] == "strong" and row["dtype"] == "bf16" and "synthetic" in row["data"]
    e2e = row["e2e"]
    assert e2e["unit"] == "tokens/s" and e2e["value"] == pytest.approx(tokens / 8.1e-3)
    assert (e2e["h2d_bytes_per_step"], e2e["d2h_bytes_per_step"]) == (131072, 4)
    assert row["gpu_launches"] == 8300 and row["clocks"]["sm_mhz"] == 1965.0


@pytest.mark.parametrize("name,label,batch,seq", [("1.3b", "1.3B", 64, 2048), ("pp24", "pp24L", 64, 1024)])
def test_other_configurations_are_named_and_have_no_published_baseline(bench, name, label, batch, seq):
    bench.select_model(name)
    row = row_for(bench)
    assert row["metric"] == f"gpt_{label}_ddp_tokens_per_s"
    assert row["vs_baseline"] is None
    assert (row["config"]["global_batch"], row["config"]["seq_len"]) == (batch, seq)
    assert row["value"] == pytest.approx(batch * seq / 8.0e-3)


def test_token_batches_are_pinned_free_rows_of_one_global_batch(bench, monkeypatch):
    monkeypatch.setattr(torch.Tensor, "pin_memory", lambda self: self)  # no CUDA runtime is needed for the check
    whole = bench.token_batches(2, 4, 0, 1, 65, 16)
    halves = [bench.token_batches(2, 2, rank, 2, 65, 16) for rank in (0, 1)]
    for step in range(2):
        x, y = whole[step]
        assert x.shape == (4, 16) and int(x.max()) < 65 and torch.equal(x[:, 1:], y[:, :-1])
        assert torch.equal(torch.cat([halves[0][step][0], halves[1][step][0]]), x)
        assert torch.equal(torch.cat([halves[0][step][1], halves[1][step][1]]), y)
