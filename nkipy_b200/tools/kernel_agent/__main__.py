"""python -m nkipy_b200.tools.kernel_agent {discover,test,generate,list-ops,sweep,rerun}
(reference CLI: tools/kernel_agent/__main__.py:29-243)."""

from __future__ import annotations

import argparse
import json
import sys

from . import ops as ops_mod
from .generator import BedrockClient, TemplateClient, load_kernel
from .executor import run_kernel
from .sweep import rerun_failed, run_rerun, run_sweep


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="kernel_agent", description=__doc__)
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("list-ops", help="print the operation catalogue")
    d = sub.add_parser("discover", help="run every catalogue operation through numpy -> compile -> device")
    d.add_argument("--json", default=None, help="write the result table to this file")
    d.add_argument("--no-gpu", action="store_true")
    t = sub.add_parser("test", help="run a kernel file (kernel + make_inputs) through the pipeline")
    t.add_argument("file")
    t.add_argument("--no-gpu", action="store_true")
    g = sub.add_parser("generate", help="generate a kernel that uses the given operations")
    g.add_argument("ops", nargs="+")
    g.add_argument("--client", choices=["template", "bedrock"], default="template")
    g.add_argument("-o", "--output", default=None)
    s = sub.add_parser("sweep", help="generate and test random kernels")
    s.add_argument("--num-kernels", type=int, default=10, help="0: keep going until SIGINT / SIGTERM")
    s.add_argument("--timeout", type=int, default=120, help="seconds per kernel before it is abandoned")
    s.add_argument("--delay", type=float, default=0.0, help="pause between kernels, seconds")
    s.add_argument("--summary-interval", type=int, default=10)
    s.add_argument("--ops-per-kernel", type=int, default=4)
    s.add_argument("--out-dir", default="kernel_agent_sweep")
    s.add_argument("--seed", type=int, default=0)
    s.add_argument("--no-gpu", action="store_true")
    r = sub.add_parser("rerun", help="re-run a sweep: a .jsonl log (all of its kernels, or --only-failed) or a "
                                     "sweep directory (its failed kernels)")
    r.add_argument("out_dir", help="a sweep_*.jsonl log or a sweep directory")
    r.add_argument("--only-failed", action="store_true")
    r.add_argument("--timeout", type=int, default=120)
    r.add_argument("--no-gpu", action="store_true")
    args = ap.parse_args(argv)

    if args.cmd == "list-ops":
        for cat, names in ops_mod.TARGET_OPS.items():
            print(f"{cat}: {', '.join(names)}")
        return 0
    use_gpu = False if getattr(args, "no_gpu", False) else None
    if args.cmd == "discover":
        table = ops_mod.discover(use_gpu)
        n_pass = sum(v["status"] == "pass" for v in table.values())
        for k, v in table.items():
            print(f"{k:32s} {v['status']}" + (f"  ({v.get('error_stage')})" if v["status"] == "fail" else ""))
        print(f"{n_pass}/{len(table)} operations pass")
        if args.json:
            with open(args.json, "w") as f:
                json.dump(table, f, indent=1)
        return 0
    if args.cmd == "test":
        with open(args.file) as f:
            kernel, make_inputs = load_kernel(f.read())
        res = run_kernel(kernel, make_inputs(), use_gpu=use_gpu)
        print(json.dumps(res.as_dict(), indent=1))
        return 0 if res.passed else 1
    if args.cmd == "generate":
        client = TemplateClient() if args.client == "template" else BedrockClient()
        src = client.generate(args.ops, "")
        if args.output:
            with open(args.output, "w") as f:
                f.write(src)
        else:
            print(src)
        return 0
    if args.cmd == "sweep":
        summary = run_sweep(args.num_kernels or None, args.ops_per_kernel, args.out_dir, args.seed, use_gpu,
                            timeout=args.timeout, delay=args.delay, summary_interval=args.summary_interval,
                            verbose=True)
        print(f"{summary['passed']}/{summary['num_kernels']} kernels pass; log {summary['log']}")
        return 0 if summary["passed"] == summary["num_kernels"] else 1
    if args.cmd == "rerun":
        if args.out_dir.endswith(".jsonl"):
            summary = run_rerun(args.out_dir, use_gpu, timeout=args.timeout, only_failed=args.only_failed,
                                verbose=True)
        else:
            summary = rerun_failed(args.out_dir, use_gpu, timeout=args.timeout)
        print(f"{summary['passed']}/{summary['num_kernels']} kernels pass")
        return 0
    return 2


if __name__ == "__main__":
    sys.exit(main())
