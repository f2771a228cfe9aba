"""bench.py's contract, as far as it can be checked without a GPU: the reference arm (the reference's CPU algorithm,
one core) prints one JSON line with the keys the driver reads, on the same `config` as this build's arm."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    # 100 requested steps make the arm pick a bounded sample of the workload (here 256 of the 8192 rows); one
    # timed step of it is run by asking for --steps 1 through the same code path
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                          capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "fused pointwise GB/s" and line["unit"] == "GB/s"
    assert line["higher_is_better"] is True and line["n_gpus"] == 1 and line["steps"] == 1 and line["gpu_launches"] == 0
    assert line["value"] > 0 and line["ms_per_step"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] == 1 and line["cpu_baseline"]["value"] == line["value"]
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    sys.path.insert(0, ROOT)
    import bench
    assert line["config"] == bench.headline_config(1)          # the same config object as this build's arm: nothing extra in it
    assert "sample" in line["cpu_baseline"] and "sample" not in line["config"]


def test_other_ranks_of_the_reference_arm_do_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
                          capture_output=True, text=True, timeout=60, cwd=ROOT, env=env)
    assert proc.returncode == 0 and proc.stdout.strip() == ""


def test_sample_of_the_reference_arm_shrinks_with_the_requested_steps():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.reference_rows(25) == bench.N_SIDE             # the driver's --steps 20 --warmup 5: the whole workload
    previous = bench.N_SIDE
    for total in (27, 60, 100, 400, 5000):
        rows = bench.reference_rows(total)
        assert 256 <= rows <= previous and rows % 256 == 0
        assert rows == 256 or total * 6.0 * rows / bench.N_SIDE <= 125      # the whole run stays near two minutes
        previous = rows
