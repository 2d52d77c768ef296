"""Start the ranks of a training script from the script itself.

``GPUS = 8`` in a config (or ``--set GPUS=8``) makes ``python -m kohakuwullm_b200.cli.train_lm_pipe ...`` spawn eight
ranks on this machine and run the same command line in each, so a launcher command is optional. No restarts
(``max_restarts=0``): a failed rank ends the run, and recovery is resuming from the last checkpoint. Already under a
launcher (``RANK`` in the environment) nothing is spawned. The rendezvous is a local c10d store on 127.0.0.1.
Reference: scripts/train/lm_pipe.py:360-369 (``elastic_launch(max_restarts=0)``).
"""

from __future__ import annotations

import os
import socket
import sys
import uuid


def under_launcher() -> bool:
    return "RANK" in os.environ and "WORLD_SIZE" in os.environ


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def self_launch(module: str, argv: list[str], nproc: int, timeout: float = 900.0) -> None:
    """Run ``python -m module *argv`` as ``nproc`` ranks on this machine and wait for them. Raises
    ``ChildFailedError`` (from torch's elastic agent) with the first failing rank's report when one fails."""
    from torch.distributed.launcher.api import LaunchConfig, elastic_launch

    config = LaunchConfig(min_nodes=1, max_nodes=1, nproc_per_node=nproc, run_id=f"kwu-{uuid.uuid4().hex[:8]}",
                          rdzv_backend="c10d", rdzv_endpoint=f"127.0.0.1:{_free_port()}", max_restarts=0,
                          monitor_interval=0.5, start_method="spawn", rdzv_configs={"timeout": int(timeout)},
                          local_addr="127.0.0.1")
    elastic_launch(config, sys.executable)("-m", module, *argv)


def maybe_self_launch(module: str, gpus: int, argv: list[str] | None = None) -> bool:
    """True when this process spawned the ranks (and they have finished): the caller returns without training."""
    if gpus and gpus > 1 and not under_launcher():
        self_launch(module, list(sys.argv[1:] if argv is None else argv), gpus)
        return True
    return False
