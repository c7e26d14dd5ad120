"""CPU checks of the benchmark's reporting code: the roofline block carries every key the
measurement contract asks for, and every DRAM-traffic figure the benchmark reports is quoted
verbatim in the ncu summary under profiles/ that it names."""
import os

import bench

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INFO = {"gemm1_kernel_name": "fmoe_grouped_gemm_kernel", "gemm2_kernel_name": "fmoe_grouped_gemm_pair_kernel"}
PEAKS = dict(hbm_gbs=6457.4, bf16_burst=1655.9, bf16_sustained=1404.2, source="measured")
STAGES = {"sort": 0.02, "gather": 0.03, "gemm1": 1.6, "quant_y": 0.0, "gemm2": 0.85, "combine": 0.04}


def test_traffic_table_is_quoted_in_the_profiles():
    for name, t in bench.GEMM1_DRAM_TRAFFIC.items():
        path = os.path.join(ROOT, t["source"])
        assert os.path.exists(path), f"{name}: {t['source']} is missing"
        text = open(path).read()
        for q in t["quotes"]:
            assert q in text, f"{name}: '{q}' does not appear in {t['source']}"
        assert t["read"] > 0 and t["write"] >= 0


def test_tensor_bound_roofline_block():
    c = dict(bench.CONFIGS["C1"])
    clocks = {"sm_mhz": 1300.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 9}
    r = bench.roofline_entry(c, "C1", INFO, STAGES, clocks, 500.0, 2.6, PEAKS, None, False)
    for k in ("bound", "kernel", "achieved", "peak", "unit", "frac", "traffic", "peak_kind", "frac_of_burst",
              "frac_of_sustained", "frac_of_nominal", "step", "ms_per_launch", "traffic_source"):
        assert k in r, k
    assert r["bound"] == "tensor" and r["unit"] == "TFLOP/s"
    assert "sustained" in r["peak_kind"] and r["peak"] == PEAKS["bf16_sustained"]      # power-capped loop
    assert abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-12
    assert r["traffic"] == 1957748480 + 241425664
    assert abs(r["achieved"] - 4.0 * 4096 * 2 * 4096 * 14336 / 1.6e-3 / 1e12) < 1e-6
    # a short loop at full clock is compared with the burst figure; a resized workload has no traffic figure
    r2 = bench.roofline_entry(c, "C1", INFO, STAGES, {"sm_mhz": 1965.0, "sm_max_mhz": 1965.0, "reasons": []}, 100.0,
                              2.6, PEAKS, None, True)
    assert r2["peak"] == PEAKS["bf16_burst"] and r2["traffic"] is None


def test_fp8_roofline_uses_the_peak_measured_in_the_run():
    c = dict(bench.CONFIGS["C2"])
    fp8 = dict(burst=3100.0, sustained=2600.0, how="torch._scaled_mm")
    r = bench.roofline_entry(c, "C2", INFO, STAGES, None, 100.0, 2.8, PEAKS, fp8, False)
    assert r["peak"] == 3100.0 and "measured in this run" in r["peak_kind"]
    r = bench.roofline_entry(c, "C2", INFO, STAGES, None, 100.0, 2.8, PEAKS, None, False)
    assert r["peak"] == 2 * PEAKS["bf16_burst"] and "could not be measured" in r["peak_kind"]


def test_decode_roofline_is_against_hbm():
    c = dict(bench.CONFIGS["C3"])
    st = dict(STAGES, gemm1=0.155, gemm2=0.086)
    r = bench.roofline_entry(c, "C3", INFO, st, None, 50.0, 0.25, PEAKS, None, False)
    assert r["bound"] == "hbm" and r["unit"] == "GB/s" and r["peak"] == PEAKS["hbm_gbs"]
    assert abs(r["achieved"] - 8 * 2 * 14336 * 4096 / 0.155e-3 / 1e9) < 1e-6
    assert abs(r["step"]["achieved"] - 8 * 3 * 14336 * 4096 / 0.25e-3 / 1e9) < 1e-6
    assert 0 < r["frac_of_nominal"] < r["frac"]


def test_fine_grained_shape_reports_both_rooflines():
    c = dict(bench.CONFIGS["C4m"])
    r = bench.roofline_entry(c, "C4m", INFO, dict(STAGES, gemm1=2.2), None, 100.0, 4.2, PEAKS, None, False)
    assert r["bound"] == "tensor" and "hbm" in r
    assert abs(r["traffic"] - 8 * (1.035734e9 + 19.909376e6)) < 1 and "x8" in r["traffic_source"]
    c4 = dict(bench.CONFIGS["C4"])
    assert bench.roofline_entry(c4, "C4", INFO, dict(STAGES, gemm1=3.4), None, 100.0, 6.7, PEAKS, None, False)["traffic"] is None


def test_workload_config_names_the_workload_without_model_keys():
    cfg = bench.workload_config(bench.CONFIGS["C1"], 1)
    assert cfg["workload"] == "mixtral-8x7b-prefill-bf16" and "model" not in cfg
    assert bench.flops_per_step(bench.CONFIGS["C1"]) == 6.0 * 4096 * 2 * 4096 * 14336
