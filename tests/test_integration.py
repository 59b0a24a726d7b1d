"""Strategy x case matrix among CPU ranks over gloo; every (case) runs in fresh processes because a
process holds one AutoDist at a time and one process group (the reference's matrix does the same,
``tests/integration/test_all.py:55-69``)."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
RUNNER = os.path.join(HERE, "integration", "run_matrix.py")


def _run(case, nproc, only=""):
    env = dict(os.environ, AUTODIST_MIN_LOG_LEVEL="ERROR")
    env.pop("RANK", None)
    env.pop("WORLD_SIZE", None)
    r = subprocess.run([sys.executable, RUNNER, "--case", case, "--nproc", str(nproc), "--only", only],
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-4000:]
    return r.stdout


@pytest.mark.integration
@pytest.mark.parametrize("case", ["c0", "c1", "c2", "c3"])
def test_matrix_two_ranks(case):
    out = _run(case, 2)
    assert out.count(" ok") >= 28 and "FAIL" not in out


@pytest.mark.integration
def test_matrix_single_rank():
    out = _run("c0", 1, only="PS,AllReduce_None,PartitionedPS_proxy,Parallax_proxy")
    assert out.count(" ok") == 4


@pytest.mark.integration
def test_matrix_four_ranks():
    out = _run("c1", 4, only="AllReduce_chunk512,PartitionedPS_owners,UnevenPartitionedPS_proxy,PSLoadBalancing_proxy")
    assert out.count(" ok") == 16


@pytest.mark.integration
def test_matrix_unrolled_recurrent_case():
    out = _run("c4", 2, only="PS,AllReduce_None,PartitionedPS_proxy,Parallax_proxy,PartitionedAR,UnevenPartitionedPS_proxy,"
                             "RandomAxisPartitionAR")
    assert out.count(" ok") >= 7 and "FAIL" not in out
