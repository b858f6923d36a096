"""``spike-run``: execute a compiled kernel from the command line.

    python -m nkipy_b200.spike.cli kernel.cubin -i x=data.npy [-i y=other_{rank}.npy]
        [--benchmark --warmup 5 --iterations 100 --mode device|host]
        [--save-trace --ntff-name out.json] [--output-dir out]
        [--core-id 0] [--num-cores N [--collective]] [--cc-enabled --rank-id R --world-size W]

Modes (same as the reference CLI, spike/src/spike/cli.py:81-429): single core; multi core
(`--num-cores N`: one worker per GPU — separate processes here, because one process drives
one GPU — each taking ``{rank}``-expanded inputs and writing ``core_{i}/name.npy``);
collective (`--collective`: the workers form a process group first).  Inputs not given
on the command line are filled with zeros.
"""

from __future__ import annotations

import argparse
import os
import subprocess
import sys
from typing import Dict

import numpy as np


def parse_inputs(specs, rank: int) -> Dict[str, np.ndarray]:
    out = {}
    for spec in specs or []:
        if "=" not in spec:
            raise SystemExit(f"bad -i argument {spec!r}; expected name=path.npy")
        name, path = spec.split("=", 1)
        out[name] = np.load(path.replace("{rank}", str(rank)))
    return out


def validate_env(args) -> None:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis is not None and args.num_cores > 1:
        n = len([v for v in vis.split(",") if v.strip() != ""])
        if args.num_cores > n:
            raise SystemExit(f"--num-cores {args.num_cores} exceeds CUDA_VISIBLE_DEVICES={vis!r} ({n} devices)")
    if args.cc_enabled and not (0 <= args.rank_id < args.world_size):
        raise SystemExit("--cc-enabled needs 0 <= --rank-id < --world-size")


def run_single(args, rank: int = 0) -> int:
    from .spike_model import SpikeModel
    from .spike_singleton import configure
    from .spike_tensor import SpikeTensor
    from ..core.dtypes import dtype_from_name

    if args.num_cores > 1:
        configure(device_ordinal=rank)
    model = SpikeModel.load_from_neff(args.neff, core_id=0 if args.num_cores > 1 else args.core_id,
                                      cc_enabled=args.cc_enabled or args.collective,
                                      rank_id=rank if args.num_cores > 1 else args.rank_id,
                                      world_size=args.num_cores if args.num_cores > 1 else args.world_size)
    given = parse_inputs(args.input, rank)
    inputs = {}
    for name in model.input_order:
        meta = model.input_info[name]
        dt = dtype_from_name(meta.dtype)
        key = name if name in given else name.replace(".must_alias_input", "")
        arr = given.get(key)
        if arr is None:
            arr = np.zeros(tuple(meta.shape), dtype=dt)
        if tuple(arr.shape) != tuple(meta.shape):
            raise SystemExit(f"input {name}: expected shape {tuple(meta.shape)}, file has {arr.shape}")
        inputs[name] = SpikeTensor.from_numpy(arr.astype(dt, copy=False), name)
    outputs = model.allocate_output_tensors()
    if args.benchmark:
        res = model.benchmark(inputs, outputs, args.warmup, args.iterations, args.mode)
        print(f"[core {rank}] {res}")
    else:
        model(inputs, outputs, save_trace=args.save_trace, ntff_name=args.ntff_name)
    out_dir = args.output_dir
    if out_dir:
        if args.num_cores > 1:
            out_dir = os.path.join(out_dir, f"core_{rank}")
        os.makedirs(out_dir, exist_ok=True)
        for name, t in outputs.items():
            np.save(os.path.join(out_dir, f"{name}.npy"), t.numpy())
    else:
        for name, t in outputs.items():
            a = t.numpy()
            print(f"[core {rank}] {name}: shape={a.shape} dtype={a.dtype} mean={a.astype(np.float64).mean():.6g}")
    return 0


def run_multi_core(args) -> int:
    procs = []
    for r in range(args.num_cores):
        env = dict(os.environ, SPIKE_RUN_WORKER_RANK=str(r))
        if args.collective:
            env.update(RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(args.num_cores),
                       MASTER_ADDR="127.0.0.1", MASTER_PORT=os.environ.get("MASTER_PORT", "29533"))
        procs.append(subprocess.Popen([sys.executable, "-m", "nkipy_b200.spike.cli", *sys.argv[1:]], env=env))
    return max(p.wait() for p in procs)


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="spike-run", description=__doc__.split("\n\n")[0])
    ap.add_argument("neff", help="compiled kernel (.cubin with its .json plan beside it)")
    ap.add_argument("-i", "--input", action="append", help="name=path.npy ({rank} is expanded per core)")
    ap.add_argument("--output-dir")
    ap.add_argument("--benchmark", action="store_true")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iterations", type=int, default=100)
    ap.add_argument("--mode", choices=["device", "host"], default="device")
    ap.add_argument("--save-trace", action="store_true")
    ap.add_argument("--ntff-name")
    ap.add_argument("--core-id", type=int, default=0)
    ap.add_argument("--cc-enabled", action="store_true")
    ap.add_argument("--rank-id", type=int, default=0)
    ap.add_argument("--world-size", type=int, default=1)
    ap.add_argument("--num-cores", type=int, default=1)
    ap.add_argument("--collective", action="store_true")
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    validate_env(args)
    worker = os.environ.get("SPIKE_RUN_WORKER_RANK")
    if args.num_cores > 1 and worker is None:
        return run_multi_core(args)
    return run_single(args, int(worker) if worker is not None else 0)


if __name__ == "__main__":
    sys.exit(main())
