"""Job launcher: chooses the execution environment and starts the benchmark
driver, the counterpart of the reference's ``setup.sh`` (interactive choice of
LOCAL / POLARIS / AURORA exported as SYSTEM_ENVIRONMENT, testing/setup.sh:10-33)
and of its PBS runner scripts (``mpiexec --np N -ppn R ... ./out <n_iter> --overwrite b=... base=...``,
testing/custom_implementations/work_dir/all_reduce/runner_polaris_allreduce.sh:13-23).

    python -m configurable_hierarchical_allreduce_algorithms_b200.bench.launch [--env LOCAL|B200|MULTINODE]
        [--ranks-per-node R] [--num-nodes N] [--node-rank I] [--rdzv HOST:PORT] [--dry-run] -- <driver args>

  LOCAL      R x N gloo ranks on this machine's CPUs (oversubscribed), like SYSTEM_ENVIRONMENT=LOCAL
  B200       one rank per GPU of this machine over NVLink (default when GPUs are visible)
  MULTINODE  one rank per GPU on each of N machines; run once per machine with its --node-rank
The environment can also come from $SYSTEM_ENVIRONMENT.  Everything after ``--`` goes to ``bench/driver.py``.
"""
from __future__ import annotations

import argparse
import os
import shlex
import subprocess
import sys

PKG = __package__.rsplit(".", 1)[0]


def build_command(env: str, rpn: int, nodes: int, node_rank: int, rdzv: str, driver_args: list[str]) -> list[str]:
    base = [sys.executable, "-m", "torch.distributed.run"]
    if env == "LOCAL":
        cmd = base + ["--nnodes=1", f"--nproc-per-node={rpn * nodes}", "--master-addr", "127.0.0.1", "--master-port",
                      rdzv.split(":")[-1]]
        extra = ["backend=gloo", f"num_nodes={nodes}"]
    elif env == "B200":
        cmd = base + ["--nnodes=1", f"--nproc-per-node={rpn}", "--master-addr", "127.0.0.1", "--master-port",
                      rdzv.split(":")[-1]]
        extra = ["backend=gpu", "num_nodes=1"]
    elif env == "MULTINODE":
        host, port = rdzv.split(":")
        cmd = base + [f"--nnodes={nodes}", f"--node-rank={node_rank}", f"--nproc-per-node={rpn}", "--master-addr", host,
                      "--master-port", port]
        extra = ["backend=gpu", f"num_nodes={nodes}"]
    else:
        raise SystemExit(f"unknown environment {env!r}")
    have = {a.split("=")[0] for a in driver_args if "=" in a}
    return cmd + ["-m", f"{PKG}.bench.driver"] + driver_args + [e for e in extra if e.split("=")[0] not in have]


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    driver_args = []
    if "--" in argv:
        i = argv.index("--")
        argv, driver_args = argv[:i], argv[i + 1:]
    ap = argparse.ArgumentParser()
    ap.add_argument("--env", default=os.environ.get("SYSTEM_ENVIRONMENT", ""))
    ap.add_argument("--ranks-per-node", type=int, default=0)
    ap.add_argument("--num-nodes", type=int, default=1)
    ap.add_argument("--node-rank", type=int, default=0)
    ap.add_argument("--rdzv", default="127.0.0.1:29560")
    ap.add_argument("--dry-run", action="store_true")
    a = ap.parse_args(argv)
    ngpu = 0
    try:
        import torch
        ngpu = torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:  # noqa: BLE001
        pass
    env = (a.env or ("B200" if ngpu else "LOCAL")).upper()
    rpn = a.ranks_per_node or (ngpu if env != "LOCAL" and ngpu else 4)
    cmd = build_command(env, rpn, a.num_nodes, a.node_rank, a.rdzv, driver_args or ["4", "--overwrite"])
    print(f"SYSTEM_ENVIRONMENT={env} ranks/node={rpn} nodes={a.num_nodes}")
    print(" ".join(shlex.quote(c) for c in cmd))
    if a.dry_run:
        return 0
    return subprocess.call(cmd, env=dict(os.environ, SYSTEM_ENVIRONMENT=env))


if __name__ == "__main__":
    sys.exit(main())
