"""CPU: the host logic of bench.py that needs no device -- the traffic table, the config object
both arms print, the roofline arithmetic and the reference arm end to end on a tiny budget."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_traffic_table_names_every_workload():
    with open(os.path.join(ROOT, "profiles", "ncu_traffic.json")) as f:
        table = json.load(f)["workloads"]
    assert set(table) == set(bench.WORKLOADS)
    for name, rec in table.items():
        assert rec.get("dram_bytes") is not None or rec.get("reason"), name
    val, src = bench.ncu_traffic(bench.HEADLINE)
    assert val > 0 and src.startswith("profiles/") and os.path.exists(os.path.join(ROOT, src))


def test_both_arms_print_the_same_config():
    a = bench.config_for(bench.HEADLINE, 4, "strong")
    assert a == bench.config_for(bench.HEADLINE, 4, "strong")
    assert a["workload"] == bench.HEADLINE and "split over 4 ranks" in a["sharding"]
    assert bench.config_for(bench.HEADLINE, 1, "strong")["sharding"] == "none"
    assert "one named configuration per rank" in bench.config_for(bench.HEADLINE, 2, "weak")["sharding"]


def test_roofline_denominators(built_lib):
    peaks = {"hbm_gbs": 6500.0, "bf16_tflops": 1600.0, "bf16_tflops_sustained": 1400.0}
    d = bench.make_desc(bench.WORKLOADS["gemm_f16_4096"])
    ops, byts = bench.work_and_bytes(d)
    assert ops == 2.0 * 4096 ** 3 and byts == 3 * 4096 * 4096 * 2
    r = bench.roofline_for(d, ops, byts, 0.1, 1, peaks, "measured", False)
    assert r["bound"] == "tensor" and abs(r["frac"] - ops / 1e-4 / 1e12 / 1600.0) < 1e-12
    r = bench.roofline_for(d, ops, byts, 0.1, 1, peaks, "measured", True)
    assert r["peak"] == 1400.0 and "sustained" in r["peak_source"]
    r8 = bench.roofline_for(d, 8 * ops, 8 * byts, 0.1, 8, peaks, "measured", False)
    assert r8["peak"] == 8 * 1600.0
    di = bench.make_desc(bench.WORKLOADS["gemm_s8_8192"])
    oi, bi = bench.work_and_bytes(di)
    assumed = bench.roofline_for(di, oi, bi, 0.35, 1, peaks, "measured", False)
    assert assumed["peak"] == 3200.0 and "assumed" in assumed["peak_source"]
    measured = bench.roofline_for(di, oi, bi, 0.35, 1, peaks, "measured", False,
                                  {"int8_tops": 2950.0, "int8_tops_sustained": 2500.0})
    assert measured["peak"] == 2950.0 and "torch._int_mm" in measured["peak_source"]
    dc = bench.make_desc(bench.WORKLOADS["conv_c3a_n256_c64_56x56_k256_1x1"])
    oc, bc = bench.work_and_bytes(dc)
    assert bench.roofline_for(dc, oc, bc, 0.17, 1, peaks, "measured", False)["bound"] == "hbm"


def test_reference_arm_prints_one_line(oracle):
    out = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
         "--warmup", "0", "--workload", "conv_c1_n1_c64_56x56_k64_3x3"],
        capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["value"] > 0 and line["gpu_launches"] == 0
    assert line["config"] == bench.config_for("conv_c1_n1_c64_56x56_k64_3x3", 1, "strong")
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0
