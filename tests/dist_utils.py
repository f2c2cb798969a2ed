"""Spawn helper for multi-process CPU (gloo) tests."""
import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _to_plain(o):
    """Tensors cross the process boundary as numpy arrays (no shared-memory handles)."""
    if isinstance(o, torch.Tensor):
        return ("__tensor__", o.detach().cpu().numpy())
    if isinstance(o, dict):
        return {k: _to_plain(v) for k, v in o.items()}
    if isinstance(o, (list, tuple)):
        return type(o)(_to_plain(v) for v in o)
    return o


def _from_plain(o):
    if isinstance(o, tuple) and len(o) == 2 and isinstance(o[0], str) and o[0] == "__tensor__":
        return torch.from_numpy(o[1])
    if isinstance(o, dict):
        return {k: _from_plain(v) for k, v in o.items()}
    if isinstance(o, (list, tuple)):
        return type(o)(_from_plain(v) for v in o)
    return o


def _worker(rank, world, port, fn, args, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world), LOCAL_RANK=str(rank), FLUIDMOE_P2P_BACKEND="gloo")
    try:
        torch.set_num_threads(1)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        res = fn(rank, world, *args)
        q.put((rank, "ok", _to_plain(res)))
    except Exception:  # noqa: BLE001
        q.put((rank, "err", traceback.format_exc()))
    finally:
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:  # noqa: BLE001
                pass


def run_distributed(fn, world: int, *args, timeout: float = 240.0):
    """Run ``fn(rank, world, *args)`` in ``world`` gloo processes; return results by rank."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn, args, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            rank, status, payload = q.get(timeout=timeout)
            if status != "ok":
                raise AssertionError(f"rank {rank} failed:\n{payload}")
            results[rank] = _from_plain(payload)
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    return [results[r] for r in range(world)]
