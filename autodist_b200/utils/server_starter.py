"""Rank starter CLI.

The reference's ``autodist/utils/server_starter.py:48-125`` starts one TensorFlow server per node. Here a node needs
no server process: its ranks are the job. This CLI starts all ranks of the *local* node for a script, with the same
environment contract the coordinator uses, and stops the others when one of them fails:

    python -m autodist_b200.utils.server_starter --resource_spec spec.yml [--master_port 15000] script.py [args...]
"""
import argparse
import os
import signal
import subprocess
import sys

from autodist_b200 import const
from autodist_b200.resource_spec import ResourceSpec
from autodist_b200.utils.network import is_local_address


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--resource_spec", required=True)
    ap.add_argument("--master_addr", default=None)
    ap.add_argument("--master_port", type=int, default=const.DEFAULT_PORT_RANGE[0])
    ap.add_argument("--node", default=None, help="address of this node in the spec (default: the chief / a local address)")
    ap.add_argument("script")
    ap.add_argument("script_args", nargs=argparse.REMAINDER)
    args = ap.parse_args(argv)
    spec = ResourceSpec(args.resource_spec)
    replicas = spec.replica_devices
    node = args.node or next((h for h in sorted(spec.nodes) if is_local_address(h)), spec.chief)
    local = [r for r, d in enumerate(replicas) if d.rsplit(":", 2)[0] == node]
    if not local:
        sys.exit(f"no replica of the resource spec runs on node {node}")
    master = args.master_addr or ("127.0.0.1" if len(spec.nodes) == 1 else spec.chief)
    procs = []
    for r in local:
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(len(replicas)), LOCAL_RANK=str(int(replicas[r].rsplit(":", 1)[1])),
                   MASTER_ADDR=master, MASTER_PORT=str(args.master_port))
        procs.append(subprocess.Popen([sys.executable, args.script] + args.script_args, env=env, start_new_session=True))
    code = 0
    remaining = list(procs)
    while remaining:
        for p in list(remaining):
            rc = p.poll()
            if rc is None:
                continue
            remaining.remove(p)
            if rc != 0 and code == 0:
                code = rc
                for other in remaining:            # one rank failed: stop exactly the ranks started here
                    try:
                        os.killpg(os.getpgid(other.pid), signal.SIGTERM)
                    except (ProcessLookupError, PermissionError):
                        pass
        if remaining:
            try:
                remaining[0].wait(timeout=0.5)
            except subprocess.TimeoutExpired:
                pass
    sys.exit(code)


if __name__ == "__main__":
    main()
