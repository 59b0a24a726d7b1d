"""Self-launch, relaxed PS modes, failure detection, checkpoint reload across strategies, ad.function:
each as child processes (CPU ranks over gloo), failures made on the host."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
SCRIPT = os.path.join(HERE, "integration", "run_special.py")


def _launch(name, tmp_path, expect_ok=2):
    env = dict(os.environ, AUTODIST_MIN_LOG_LEVEL="ERROR", AUTODIST_TEST_TMP=str(tmp_path), AUTODIST_PG_TIMEOUT="120",
               AUTODIST_GATE_TIMEOUT="60")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_PORT", "AUTODIST_WORKER", "AUTODIST_STRATEGY_ID"):
        env.pop(k, None)
    r = subprocess.run([sys.executable, SCRIPT, name], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count(" ok") >= expect_ok, r.stdout + r.stderr[-2000:]


@pytest.mark.integration
@pytest.mark.parametrize("name,oks", [("selflaunch", 2), ("stale", 2), ("async", 2), ("failure", 1),
                                      ("crossload", 2), ("function", 2), ("twonode", 8), ("hetero", 3)])
def test_scenario(name, oks, tmp_path):
    _launch(name, tmp_path, oks)


@pytest.mark.integration
def test_two_train_ops_in_one_run_on_two_replicas(tmp_path, monkeypatch):
    """Parameter-server strategy (reduce to the owner, owner-side update, publish); the all-reduce form of the same program runs
    with ``AUTODIST_TWOOPTS=ar`` and, on one process, in ``tests/test_autodist.py``."""
    monkeypatch.setenv("AUTODIST_TWOOPTS", "ps")
    _launch("twoopts", tmp_path, 2)
