"""Failure detection, exercised on the host only (gloo ranks, no GPU is faulted or hung).

* a peer that passes an inconsistent split matrix is caught by the debug check before data moves;
* a rank that raises before a collective makes its peers' collective end with an error through a
  short process-group timeout instead of waiting forever;
* a heartbeat through the store lets ranks learn between steps that a peer left.
"""
import datetime
import os

import pytest
import torch

from tests.dist_utils import run_distributed


def _split_mismatch(rank, world):
    import torch.distributed as dist
    from fluidmoe_b200.parallel import comm
    os.environ["FLUID_DEBUG_A2A_SPLITS"] = "1"
    x = torch.arange(8, dtype=torch.float32)
    ins = [4, 4]
    outs = [4, 4] if rank == 0 else [3, 5]      # rank 1 expects the wrong amount from rank 0
    try:
        comm.all_to_all(x, None, ins, outs)
    except comm.SplitMismatchError as e:
        return "caught: " + str(e)[:40]
    finally:
        os.environ["FLUID_DEBUG_A2A_SPLITS"] = "0"
    return "not caught"


def test_split_matrix_mismatch_is_detected_on_every_rank():
    res = run_distributed(_split_mismatch, 2)
    assert all(r.startswith("caught") for r in res), res


def _peer_dies(rank, world):
    import torch.distributed as dist
    # a second group with a short timeout, as a training job would use for its health checks
    g = dist.new_group(list(range(world)), timeout=datetime.timedelta(seconds=3))
    if rank == 1:
        return "left"          # leaves between steps: no collective of its own in flight
    try:
        dist.all_reduce(torch.ones(1), group=g)
    except Exception as e:  # noqa: BLE001 - gloo reports a timeout / connection error
        return "error:" + type(e).__name__
    return "completed"


def test_collective_with_missing_peer_errors_instead_of_hanging():
    res = run_distributed(_peer_dies, 2, timeout=120)
    assert res[1] == "left"
    assert res[0].startswith("error"), res


def _heartbeat(rank, world):
    import time
    import torch.distributed as dist
    from fluidmoe_b200.utils.health import Heartbeat
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, stale_after_s=1.0)
    hb.beat()
    dist.barrier()
    assert hb.missing() == []
    if rank == 1:
        time.sleep(2.5)         # stops beating
        return "silent"
    time.sleep(2.0)
    hb.beat()
    return hb.missing()


def test_heartbeat_reports_silent_rank():
    res = run_distributed(_heartbeat, 2, timeout=120)
    assert res[0] == [1], res
