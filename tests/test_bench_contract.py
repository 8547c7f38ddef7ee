"""The benchmark's reference arm runs on the CPU: check the JSON contract of its one output line."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--rows", "200000",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert out.returncode == 0, out.stderr
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "groupby-aggregate rows/sec" and d["unit"] == "rows/s"
    assert d["higher_is_better"] is True and d["value"] > 0
    # pandas is the reference's CPU path (cudf.pandas fallback): single-threaded; the C++ port rides along
    assert d["cpu_baseline"]["kind"] == "reference" and d["cpu_baseline"]["cores"] == 1
    assert "pandas" in d["cpu_baseline"]["engine"] and d["cpu_baseline"]["port_value"] > 0
    assert d["e2e"] == {"value": d["value"], "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"]


def test_other_ranks_of_the_reference_arm_exit_quietly():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                         capture_output=True, text=True, timeout=120, cwd=ROOT, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_pandas_expression_of_every_configuration_agrees_with_the_oracle():
    """The timed pandas expressions compute the same groups as the oracle (group count and, for C2, the means)."""
    import numpy as np
    sys.path.insert(0, ROOT)
    import bench
    import workloads
    from oracle import oracle
    for cfg in (1, 2, 3, 4, 5):
        w = workloads.make(cfg, 20_000, scale_domain=True)
        df, kn, vn = bench.pandas_frame(w)
        out = bench.pandas_groupby(w, df, kn, vn)
        okeys, ores = oracle.groupby(w.keys, w.requests, w.null_policy, row_filters=[f.mask for f in w.row_filters])
        assert len(out) == okeys[0].size, f"C{cfg}: {len(out)} pandas groups, {okeys[0].size} oracle groups"
        if cfg == 2:
            got = out.sort_index()["V0"].to_numpy(dtype=np.float64)
            order = np.lexsort([okeys[1].values(), okeys[0].values()])
            exp = ores[0][0].values()[order]
            assert np.allclose(got, exp, rtol=1e-5)
