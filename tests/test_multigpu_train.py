"""Data-parallel and sharded-optimizer steps on real GPUs: this library's
collectives against the same step over torch.distributed (NCCL)."""
import os
import socket
import traceback

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.multigpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, P, port, mode, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), LOCAL_RANK=str(rank),
                          WORLD_SIZE=str(P))
        from configurable_hierarchical_allreduce_algorithms_b200.bench import train
        res = {}
        for impl, extra in (("ours", []), ("ours_kb", ["--algo", "radix_batch", "--k", "2", "--b", "2"]), ("nccl", [])):
            os.environ["MASTER_PORT"] = str(port + len(res) + 1)
            r = train.main(["--mode", mode, "--impl", impl.split("_")[0], "--tiny", "--steps", "6", "--warmup", "2"] + extra)
            res[impl] = r
        q.put((rank, "ok", res))
    except Exception:  # noqa: BLE001
        q.put((rank, "fail", traceback.format_exc()))


@pytest.mark.timeout(900)
@pytest.mark.parametrize("mode", ["dp", "zero"])
def test_training_step_matches_nccl(mode):
    from conftest import gpus_for_test
    P = gpus_for_test(4)
    if P < 2:
        pytest.skip("needs at least two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, P, port, mode, q)) for r in range(P)]
    for p in procs:
        p.start()
    res = [q.get(timeout=600) for _ in range(P)]
    for p in procs:
        p.join(60)
    bad = [r for r in res if r[1] != "ok"]
    assert not bad, "\n".join(f"rank {r[0]}:\n{r[2]}" for r in bad)
    r0 = [r for r in res if r[0] == 0][0][2]
    assert abs(r0["ours"]["loss"] - r0["nccl"]["loss"]) < 0.05, r0
    assert abs(r0["ours_kb"]["loss"] - r0["nccl"]["loss"]) < 0.05, r0
    assert r0["ours"]["collective_launches"] > 0
