"""What the benchmark driver relies on and a CPU box can check: the reference arm answers with one JSON line and exit
code 0, and nothing else reaches stdout."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_and_exits_zero():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "3"],
                         capture_output=True, text=True, timeout=120, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-500:]
    lines = [l for l in out.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, out.stdout
    record = json.loads(lines[0])
    assert record["impl"] == "reference" and isinstance(record["unavailable"], str) and "\n" not in record["unavailable"]


def test_only_rank_zero_of_a_multi_rank_reference_call_prints():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                         capture_output=True, text=True, timeout=120, cwd=ROOT, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_flight_table_is_written_from_an_engines_report(tmp_path):
    sys.path.insert(0, ROOT)
    import bench

    class Engine:
        def flight_report(self):
            return [(0, 1 << 20, 0.5, 0.25), (1 << 20, 3 << 20, 1.0, 0.5)]

    path = str(tmp_path / "sub" / "flights.md")
    bench._write_flights(path, Engine(), "bert-tiny", "allreduce", 4, 12.5, 0, 1, "cpu")
    text = open(path).read()
    rows = [l for l in text.splitlines() if l.startswith("| 0 |") or l.startswith("| 1 |")]
    assert len(rows) == 2 and "| 1048576 | 4.0 | 0.50 | 0.250 |" in rows[0]
    # bus bandwidth of a 4-rank all-reduce: 2 * 3 / 4 * bytes / time
    assert rows[1].rstrip("|").split("|")[-1].strip() == str(round(1.5 * (2 << 20) * 4 / 0.5e-3 / 1e9))
    assert "busy 0.75 ms of the 12.50 ms step" in text and "ends 1.50 ms" in text
