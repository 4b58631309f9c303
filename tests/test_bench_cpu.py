"""Host-side pieces of bench.py that need no GPU: the per-workload table in the reference harness's CSV
format (bench/bench_util.hpp:142-154 of the reference: throughput from the p50), and the DRAM traffic
figure read from the committed profiler summary."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402


def test_csv_rows_are_per_call_and_throughput_comes_from_the_p50(tmp_path):
    bench.ROWS.clear()
    stats = {"p50_ms": 0.36, "p90_ms": 0.37, "p99_ms": 0.38, "min_ms": 0.35, "max_ms": 0.40, "mean_ms": 0.365}
    bench.ROWS.append((("gemv", 32, 1.0e9, 3.0e7), stats))          # 32 calls per timed step
    path = tmp_path / "t.csv"
    bench.write_csv(str(path))
    lines = path.read_text().splitlines()
    assert lines[0] == "name,p50_us,p90_us,p99_us,min_us,max_us,mean_us,gflops,gbps"
    name, p50, p90, p99, mn, mx, mean, gflops, gbps = lines[1].split(",")
    assert name == "gemv" and float(p50) == 11.25 and float(mn) == 10.938 and float(mx) == 12.5
    assert abs(float(gbps) - 3.0e7 / 11.25e-6 / 1e9) < 0.01 and abs(float(gflops) - 1.0e9 / 11.25e-6 / 1e9) < 0.01
    bench.ROWS.clear()


def test_traffic_is_read_from_the_committed_summary():
    t = bench.profile_traffic("gemv_w4a16_m1_cfg2")
    assert t is not None and 31_000_000 < t < 32_000_000            # one launch reads the packed weights once
    assert bench.profile_traffic("no_such_summary") is None
