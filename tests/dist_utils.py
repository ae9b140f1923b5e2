"""Run a function on several CPU ranks (gloo) and collect its return values."""
import os
import socket
import tempfile
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _entry(rank, world, port, fn, kwargs, outdir, backend):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.set_num_threads(1)
    try:
        if backend == "nccl":
            torch.cuda.set_device(rank)
        dist.init_process_group(backend, rank=rank, world_size=world)
        out = fn(rank, world, **kwargs)
        torch.save(out, os.path.join(outdir, f"out_{rank}.pt"))
    except Exception:
        with open(os.path.join(outdir, f"err_{rank}.txt"), "w") as f:
            f.write(traceback.format_exc())
        raise
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_distributed(fn, world: int, backend: str = "gloo", **kwargs):
    """``fn(rank, world, **kwargs)`` must be importable (module level).  Returns the list of outputs."""
    for attempt in range(4):
        with tempfile.TemporaryDirectory() as d:
            try:
                mp.spawn(_entry, args=(world, _free_port(), fn, kwargs, d, backend), nprocs=world, join=True)
            except Exception:
                errs = [open(os.path.join(d, f)).read() for f in sorted(os.listdir(d)) if f.startswith("err_")]
                if attempt < 3 and any("EADDRINUSE" in e for e in errs):
                    continue                      # the probed port was taken in the meantime: pick another one
                raise RuntimeError("distributed worker failed:\n" + "\n".join(errs))
            return [torch.load(os.path.join(d, f"out_{r}.pt"), weights_only=False) for r in range(world)]
