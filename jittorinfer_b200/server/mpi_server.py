"""Multi-GPU server ("llama-mpi-server"): one process per GPU, rank 0 serves HTTP.

The reference starts ``mpirun -np N llama-mpi-server`` and forces TP + EP + fused MoE on
(examples/mpi_server/server.cpp:888-916).  Here either run this module under torchrun,

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m jittorinfer_b200.server.mpi_server -c cfg.yaml

or let it spawn the ranks itself (``--nproc N``).  The data plane between ranks is the fused
peer-memory kernels (NCCL only bootstraps them); the control plane — rank 0 telling the others which
requests arrived — is a gloo broadcast per engine-loop iteration.
"""
from __future__ import annotations

import argparse
import os
import sys


def _rank_main(argv):
    import torch
    import torch.distributed as dist
    from .launch import main
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        dist.init_process_group("gloo")
    control = dist.new_group(backend="gloo")          # host-side task broadcasts
    # The process leaves through os._exit: a rank whose peers are gone must not wait in the process group's destructor.
    # The exit code and the traceback are therefore passed on by hand.
    rc = 1
    try:
        rc = int(main(argv, world=world, rank=rank, control_group=control) or 0)
    except SystemExit as e:
        rc = e.code if isinstance(e.code, int) else (0 if e.code is None else 1)
    except BaseException:
        import traceback
        traceback.print_exc()
        rc = 1
    finally:
        sys.stdout.flush()
        sys.stderr.flush()
        if dist.is_initialized():
            os._exit(rc)
    return rc


def cli(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="jittorinfer_b200.server.mpi_server", add_help=False)
    ap.add_argument("--nproc", type=int, default=0, help="spawn this many ranks locally (omit under torchrun / mpirun)")
    ap.add_argument("--master-port", type=int, default=29533)
    args, rest = ap.parse_known_args(argv)
    if "RANK" in os.environ and "WORLD_SIZE" in os.environ:
        return _rank_main(rest)
    if "OMPI_COMM_WORLD_RANK" in os.environ:          # started by mpirun, like the reference binary
        os.environ["RANK"] = os.environ["OMPI_COMM_WORLD_RANK"]
        os.environ["WORLD_SIZE"] = os.environ["OMPI_COMM_WORLD_SIZE"]
        os.environ["LOCAL_RANK"] = os.environ.get("OMPI_COMM_WORLD_LOCAL_RANK", os.environ["RANK"])
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", str(args.master_port))
        return _rank_main(rest)
    n = args.nproc
    if n <= 0:
        from ..config import load_yaml
        cfg_path = None
        for i, a in enumerate(rest):
            if a in ("-c", "--config") and i + 1 < len(rest):
                cfg_path = rest[i + 1]
        n = load_yaml(cfg_path).world_size
    import subprocess
    procs = []
    for r in range(n):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(n), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(args.master_port))
        procs.append(subprocess.Popen([sys.executable, "-m", "jittorinfer_b200.server.mpi_server"] + rest, env=env))
    rc = 0
    for p in procs:
        rc = p.wait() or rc
    return rc


if __name__ == "__main__":
    raise SystemExit(cli())
