"""``python -m jittorinfer_b200.server --config configs/x.yaml`` — the single-process server (llama-server).

For tensor/expert parallel serving start one process per GPU with
``python -m jittorinfer_b200.server.mpi_server --config ...`` (or torchrun): rank 0 serves HTTP.
"""
from .launch import main

if __name__ == "__main__":
    raise SystemExit(main())
