"""bench.py's `also` block on the host: a side measurement that fails must not cost the headline line (one GPU), and
a failed sharded-parity check must still come back with the line (under torchrun). The workloads are replaced by
stand-ins: nothing here touches a GPU."""
import argparse
import sys
import types

import pytest


@pytest.fixture()
def bench_mod(monkeypatch):
    import bench
    fake = types.ModuleType("bench_workloads")
    fake.calls = []

    def ok(name):
        def run(a, emit=False, **kw):
            fake.calls.append(name)
            if name == "decode":
                return [{"metric": "decode_tok_s", "value": float(b), "unit": "tok/s", "junk": 1} for b in kw["batches"]]
            return {"metric": name, "value": 1.0, "unit": "x", "junk": 1}
        return run
    fake.run_gemm, fake.run_q8_batch, fake.run_moe, fake.run_decode = ok("gemm"), ok("q8"), ok("moe"), ok("decode")
    monkeypatch.setitem(sys.modules, "bench_workloads", fake)
    return bench, fake


def _args():
    return argparse.Namespace(steps=2, warmup=1, prompt=16, batch=1)


def test_a_failing_side_measurement_is_recorded_and_the_rest_still_runs(bench_mod):
    bench, fake = bench_mod

    def boom(a, emit=False, **kw):
        raise RuntimeError("kernel declined")
    fake.run_moe = boom
    out = bench.also_block(_args(), 1, 0, 0)
    also = out["also"]
    assert also["mxfp4_moe_gptoss"] is None and "kernel declined" in also["mxfp4_moe_gptoss_error"]
    assert also["q4k_gemm_prefill"]["value"] == 1.0 and "junk" not in also["q4k_gemm_prefill"]      # trimmed to the kept keys
    assert also["llama8b_q4k_decode_b1"]["value"] == 1.0 and also["llama8b_q4k_decode_b64"]["value"] == 64.0
    assert "_exit" not in out


def test_under_torchrun_an_error_propagates_and_a_failed_parity_check_returns_with_exit_3(bench_mod):
    bench, fake = bench_mod
    fake.sharded_parity = lambda local: {"tp_err": 1e-6, "ep_err": 5e-3, "bar": 2e-3}
    out = bench.also_block(_args(), 2, 0, 0)
    assert out["_exit"] == 3 and out["sharded_parity"]["failed"] is True and "also" not in out
    fake.sharded_parity = lambda local: {"tp_err": 1e-6, "ep_err": 1e-4, "bar": 2e-3}

    def boom(a, emit=False, **kw):
        raise RuntimeError("rank lost")
    fake.run_q8_batch = boom
    with pytest.raises(RuntimeError):
        bench.also_block(_args(), 2, 0, 0)
    assert "gemm" not in fake.calls                     # the prefill GEMM is a one-GPU measurement
