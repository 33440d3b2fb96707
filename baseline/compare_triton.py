"""Same-GPU A/B of this library against the reference's Triton kernels.

    python baseline/compare_triton.py                 # both arms, prints a table and JSON
    python baseline/compare_triton.py --arm ours      # one arm (one JSON line)
    python baseline/compare_triton.py --arm triton
    python baseline/compare_triton.py --abba          # A B B A process order, paired ratio + CI

The reference package is expected under ``baseline/_ref`` (installed offline with
``pip install --no-index --no-build-isolation --no-deps --target baseline/_ref <reference>``;
the directory is git-ignored).  Both packages are called ``attnres``, so every arm runs in
its own process with only its own package on ``sys.path``.

Protocol (identical for both arms, through each package's public ``attnres()`` + autograd):
the reference's operator sweep (packed values [S, 16384, D], R = D) and its sliced low-rank shape
(S=16, D=4096, R=1024); forward+backward of a cell are captured together in one CUDA graph
after eager warm-up (which also lets Triton autotune), a 256 MB buffer is rewritten between
replays to evict L2, and the median of the replays is reported.  With ``--abba`` the arms run in
the order Triton, ours, ours, Triton (the ABBA order of the reference's own harness,
benchmarks/statistics.py:87-211, across processes here because both packages are named
``attnres``); the replays of an arm's two runs are pooled and the speed-up is the ratio of the
medians with a 95 % bootstrap interval (2 000 resamples of the replays, fixed seed).  Errors are measured against
the oracle (``oracle/attnres_oracle.py``) on the device at 2 048 rows: ``max_abs`` and
``relative_l2`` exactly as the reference defines them (validation/comparison.py:9-12).
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
CELLS = [(s, d, d) for d in (1024, 2048, 4096) for s in (2, 5, 9, 17, 25, 49)] + [(16, 4096, 1024)]
ROWS = 16384
ERROR_ROWS = 2048


def run_arm(arm: str, steps: int, cells) -> dict:
    package_dir = ROOT / "baseline" / "_ref" if arm == "triton" else ROOT / "fast-attnres_b200"
    sys.path[:] = [entry for entry in sys.path if "fast-attnres_b200" not in entry
                   and "baseline/_ref" not in entry]
    sys.path.insert(0, str(package_dir))
    sys.path.insert(1, str(ROOT))
    import torch
    import attnres as package
    from oracle import attnres_oracle as ao
    assert str(package_dir) in str(Path(package.__file__).resolve()), package.__file__
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    flush = torch.empty(256 * 1024 * 1024, device=device, dtype=torch.uint8)
    results = []
    for sources, width, rank in cells:
        scale = 1.0 if rank == width else rank ** -0.5
        generator = torch.Generator(device=device).manual_seed(20260827 + sources + width)
        # ---- errors at reduced rows
        values = torch.randn(sources, ERROR_ROWS, width, device=device, dtype=torch.bfloat16,
                             generator=generator).requires_grad_()
        query = (torch.randn(rank, device=device, generator=generator) * 0.02).to(
            torch.bfloat16).requires_grad_()
        upstream = torch.randn(ERROR_ROWS, width, device=device, dtype=torch.bfloat16,
                               generator=generator)
        out = package.attnres(values, query, scale=scale)
        grads = torch.autograd.grad(out, (values, query), upstream)
        expected = ao.oracle(values, query, scale=scale)
        expected_grads = torch.autograd.grad(expected, (values, query), upstream)
        errors = {name: ao.error_metrics(a, e) for name, a, e in
                  zip(("out", "dvalues", "dquery"), (out, *grads), (expected, *expected_grads))}
        del values, query, upstream, out, grads, expected, expected_grads
        # ---- timing at full rows
        values = torch.randn(sources, ROWS, width, device=device, dtype=torch.bfloat16,
                             generator=generator).requires_grad_()
        query = (torch.randn(rank, device=device, generator=generator) * 0.02).to(
            torch.bfloat16).requires_grad_()
        upstream = torch.randn(ROWS, width, device=device, dtype=torch.bfloat16,
                               generator=generator)

        def step():
            result = package.attnres(values, query, scale=scale)
            return torch.autograd.grad(result, (values, query), upstream)

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            kept = step()
        times = []
        for _ in range(steps + 2):
            flush.zero_()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            graph.replay()
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop))
        times = sorted(times[2:])
        ms = times[len(times) // 2]
        bytes_moved = ROWS * (6 * sources * width + 4 * width)
        results.append({"S": sources, "D": width, "R": rank, "fwd_bwd_ms": ms, "samples_ms": times,
                        "tokens_per_s": ROWS / (ms * 1e-3), "gbs": bytes_moved / ms / 1e6,
                        "errors": errors})
        del graph, kept, values, query, upstream
        torch.cuda.empty_cache()
    return {"arm": arm, "package": str(Path(package.__file__).resolve().parent),
            "torch": torch.__version__, "cells": results}


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawTextHelpFormatter)
    parser.add_argument("--arm", choices=("ours", "triton", "both"), default="both")
    parser.add_argument("--steps", type=int, default=7)
    parser.add_argument("--cells", default=None, help="subset, e.g. '9,2048,2048;16,4096,1024'")
    parser.add_argument("--abba", action="store_true",
                        help="run Triton, ours, ours, Triton and report paired ratios with a "
                             "bootstrap confidence interval")
    args = parser.parse_args()
    cells = CELLS if args.cells is None else [tuple(int(x) for x in c.split(","))
                                              for c in args.cells.split(";")]
    if args.arm != "both":
        print(json.dumps(run_arm(args.arm, args.steps, cells)), flush=True)
        return
    if not (ROOT / "baseline" / "_ref" / "attnres").exists():
        print(json.dumps({"unavailable": "baseline/_ref holds no reference install"}))
        return
    arms, runs = {}, []
    for arm in (("triton", "ours", "ours", "triton") if args.abba else ("triton", "ours")):
        command = [sys.executable, str(Path(__file__).resolve()), "--arm", arm, "--steps",
                   str(args.steps)] + (["--cells", args.cells] if args.cells else [])
        done = subprocess.run(command, capture_output=True, text=True)
        if done.returncode != 0:
            print(json.dumps({"arm": arm, "failed": done.stderr[-2000:]}))
            return
        runs.append((arm, json.loads(done.stdout.strip().splitlines()[-1])))
        arms.setdefault(arm, runs[-1][1])
    if args.abba:
        import numpy as np
        generator = np.random.default_rng(20260827)
        print("| S | D | R | Triton ms | ours ms | speed-up | 95 % interval |")
        print("|---|---|---|---|---|---|---|")
        for index, cell in enumerate(arms["triton"]["cells"]):
            pooled = {arm: np.array([x for name, run in runs if name == arm
                                     for x in run["cells"][index]["samples_ms"]])
                      for arm in ("triton", "ours")}
            ratio = np.median(pooled["triton"]) / np.median(pooled["ours"])
            draws = [np.median(generator.choice(pooled["triton"], pooled["triton"].size)) /
                     np.median(generator.choice(pooled["ours"], pooled["ours"].size))
                     for _ in range(2000)]
            low, high = np.percentile(draws, [2.5, 97.5])
            print(f"| {cell['S']} | {cell['D']} | {cell['R']} | {np.median(pooled['triton']):.3f} | "
                  f"{np.median(pooled['ours']):.3f} | {ratio:.2f}x | {low:.2f}x – {high:.2f}x |")
        print(json.dumps({"order": [name for name, _ in runs], "runs": [run for _, run in runs]}),
              flush=True)
        return
    print("| S | D | R | Triton ms | ours ms | speed-up | out rel-L2 (T / ours) | dV rel-L2 (T / ours) "
          "| dq rel-L2 (T / ours) | dq max-abs (T / ours) |")
    print("|---|---|---|---|---|---|---|---|---|---|")
    for t, o in zip(arms["triton"]["cells"], arms["ours"]["cells"]):
        te, oe = t["errors"], o["errors"]
        print(f"| {t['S']} | {t['D']} | {t['R']} | {t['fwd_bwd_ms']:.3f} | {o['fwd_bwd_ms']:.3f} | "
              f"{t['fwd_bwd_ms'] / o['fwd_bwd_ms']:.2f}x | "
              f"{te['out']['relative_l2']:.2e} / {oe['out']['relative_l2']:.2e} | "
              f"{te['dvalues']['relative_l2']:.2e} / {oe['dvalues']['relative_l2']:.2e} | "
              f"{te['dquery']['relative_l2']:.2e} / {oe['dquery']['relative_l2']:.2e} | "
              f"{te['dquery']['max_abs']:.2e} / {oe['dquery']['max_abs']:.2e} |")
    print(json.dumps(arms), flush=True)


if __name__ == "__main__":
    main()
