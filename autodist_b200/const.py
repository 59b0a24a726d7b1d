"""Framework-wide constants and environment switches.

Parity with the reference's ``autodist/const.py:32-89``: same working directory
layout, same name prefixes and the same ``ENV`` variable names, so a resource
spec / strategy file / launch script written for the reference keeps working.
"""
import enum
import os

DEFAULT_WORKING_DIR = os.environ.get("AUTODIST_WORKING_DIR", "/tmp/autodist")
DEFAULT_SERIALIZATION_DIR = os.path.join(DEFAULT_WORKING_DIR, "strategies")
DEFAULT_LOG_DIR = os.path.join(DEFAULT_WORKING_DIR, "logs")
DEFAULT_TRACE_DIR = os.path.join(DEFAULT_WORKING_DIR, "traces")
DEFAULT_GRAPH_DIR = os.path.join(DEFAULT_WORKING_DIR, "graphs")
for _d in (DEFAULT_WORKING_DIR, DEFAULT_SERIALIZATION_DIR):
    os.makedirs(_d, exist_ok=True)

# Rendezvous ports are drawn from the same window the reference uses for its servers.
DEFAULT_PORT_RANGE = (15000, 16000)

AUTODIST_PREFIX = "AutoDist-"
AUTODIST_REPLICA_PREFIX = AUTODIST_PREFIX + "Replica-"
AUTODIST_TO_DELETE_SCOPE = "to-delete"

MAX_INT64 = 2 ** 63 - 1
MAX_INT32 = 2 ** 31 - 1
# Rank 0 of the job plays the role of the reference's collective group leader.
DEFAULT_GROUP_LEADER = 0


def _as_bool(default):
    return lambda raw: (raw if raw is not None else default) == "True"


def _as_str(default=""):
    return lambda raw: raw or default


class ENV(enum.Enum):
    """User-settable environment variables (same names as the reference).

    ``ENV.X.val`` parses the current process environment every time it is read,
    ``ENV.X.name`` is the variable's name (used when forwarding to workers).
    """

    AUTODIST_WORKER = (1, _as_str())
    AUTODIST_STRATEGY_ID = (2, _as_str())
    AUTODIST_MIN_LOG_LEVEL = (3, _as_str("INFO"))
    AUTODIST_IS_TESTING = (4, _as_bool("False"))
    AUTODIST_DEBUG_REMOTE = (5, _as_bool("False"))
    AUTODIST_PATCH_TF = (6, _as_bool("True"))        # kept by name: toggles optimizer patching
    AUTODIST_INTERNAL_TF = (7, _as_bool("False"))
    SYS_DATA_PATH = (8, _as_str())
    SYS_RESOURCE_PATH = (9, _as_str())
    # Additions of this framework.
    AUTODIST_RANK = (10, _as_str())                  # set by the launcher on spawned ranks
    AUTODIST_FETCH_MODE = (11, _as_str("replica0"))  # "replica0" (reference rule) or "local"
    AUTODIST_COMM = (12, _as_str("fused"))           # "fused" (own kernels) or "nccl" (baseline)
    AUTODIST_METRICS_FILE = (13, _as_str())          # JSONL step metrics of rank 0 ("%r" in the name = every rank)
    AUTODIST_STEP_TIMEOUT = (14, _as_str())          # seconds a training call may take before the watchdog fires
    AUTODIST_STEP_TIMEOUT_ACTION = (15, _as_str("report"))   # "report" (log + stack dump) or "abort" (exit code 70)

    @property
    def val(self):
        _, parse = self.value
        return parse(os.environ.get(self.name))
