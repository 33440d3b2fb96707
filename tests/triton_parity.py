"""Error of this library and of the reference's Triton kernels against the oracle, on the
same GPU, the same seeded inputs and in one process.  TEST INFRASTRUCTURE.

    python tests/triton_parity.py [--cells quick|all|S,D,R;...] [--rows N] [--markdown]

Used by tests/test_dquery_accuracy_gpu.py (which runs it as a subprocess and asserts the
bounds) and, with ``--cells all --markdown``, to print the per-shape table kept in
baseline/triton_parity_b200.md.

The reference package is expected under ``baseline/_ref`` (``pip install --no-index
--no-build-isolation --no-deps --target baseline/_ref <reference>``).  Both packages are
called ``attnres``: the reference is imported under that name, this library under the
alias ``attnres_b200_package`` (its operators live in the ``attnres_b200::`` namespace, the
reference's in ``attnres::``, so they coexist).

Per shape, for out, dvalues and dquery: ``max_abs`` and ``relative_l2`` (definitions:
validation/comparison.py:9-12 of the reference) of Triton against the oracle, of this library
against the oracle, and of this library against Triton, plus whether the two implementations
agree inside rtol = atol = 0.05 (validation/protocol.json:12-15).

Bounds ("no worse than the reference kernel's own error"; every result is a BF16 rounding of
an FP32 value, and two correct FP32 evaluations round a few elements to neighbouring BF16
values):

    max_abs(ours)      <= max_abs(Triton) + one BF16 ulp at the largest expected magnitude
    relative_l2(ours)  <= relative_l2(Triton) + allowance
        out, dvalues:  allowance = 1.0e-5  (one element in 65 536 rounds to the neighbour)
        dquery:        allowance = ulp(rms(expected)) / ||expected||  (one of the R elements,
                       of typical magnitude, does)
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
REFERENCE_DIR = ROOT / "baseline" / "_ref"
SWEEP = [(s, d, d) for d in (1024, 2048, 4096) for s in (2, 5, 9, 17, 25, 49)] + [(16, 4096, 1024)]
QUICK = [(5, 1024, 1024), (49, 1024, 1024), (9, 2048, 2048), (25, 2048, 2048), (5, 4096, 4096),
         (17, 4096, 4096), (16, 4096, 1024)]
NAMES = ("out", "dvalues", "dquery")


def load_packages():
    """(reference package, this library) in one process."""
    sys.path[:] = [entry for entry in sys.path if "fast-attnres_b200" not in entry]
    for entry in (str(ROOT), str(REFERENCE_DIR)):
        if entry not in sys.path:
            sys.path.insert(0, entry)
    import attnres as reference
    assert str(REFERENCE_DIR) in str(Path(reference.__file__).resolve()), reference.__file__
    package_dir = ROOT / "fast-attnres_b200" / "attnres"
    spec = importlib.util.spec_from_file_location(
        "attnres_b200_package", package_dir / "__init__.py",
        submodule_search_locations=[str(package_dir)])
    ours = importlib.util.module_from_spec(spec)
    sys.modules["attnres_b200_package"] = ours
    spec.loader.exec_module(ours)
    return reference, ours


def bf16_ulp(magnitude: float) -> float:
    """Spacing of BF16 values at `magnitude` (8 significant bits)."""
    import math
    if magnitude <= 0.0:
        return 0.0
    return 2.0 ** (math.floor(math.log2(magnitude)) - 7)


def bounds(name: str, triton: dict, expected) -> dict:
    import torch
    ulp = bf16_ulp(float(expected.detach().float().abs().max()))
    norm = float(torch.linalg.vector_norm(expected.detach().float()).clamp_min(1e-20))
    typical = bf16_ulp(norm / expected.numel() ** 0.5)
    allowance = typical / norm if name == "dquery" else 1.0e-5
    return {"max_abs": triton["max_abs"] + ulp, "relative_l2": triton["relative_l2"] + allowance}


def run(cells, rows: int) -> dict:
    import torch
    reference, ours = load_packages()
    from oracle import attnres_oracle as ao
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    results = []
    for sources, width, rank in cells:
        began = time.perf_counter()
        scale = 1.0 if rank == width else rank ** -0.5
        generator = torch.Generator(device=device).manual_seed(20260827 + sources + width)
        values = torch.randn(sources, rows, width, device=device, dtype=torch.bfloat16,
                             generator=generator).requires_grad_()
        query = (torch.randn(rank, device=device, generator=generator) * 0.02).to(
            torch.bfloat16).requires_grad_()
        upstream = torch.randn(rows, width, device=device, dtype=torch.bfloat16,
                               generator=generator)

        def both(function):
            out = function(values, query, scale=scale)
            return (out.detach(), *torch.autograd.grad(out, (values, query), upstream))

        expected = both(ao.oracle)
        triton = both(reference.attnres)
        mine = both(ours.attnres)
        record = {"S": sources, "D": width, "R": rank, "rows": rows}
        for name, e, t, o in zip(NAMES, expected, triton, mine):
            t_err, o_err = ao.error_metrics(t, e), ao.error_metrics(o, e)
            limit = bounds(name, t_err, e)
            record[name] = {
                "triton": t_err, "ours": o_err, "ours_vs_triton": ao.error_metrics(o, t),
                "bound": limit,
                "within_bound": bool(o_err["max_abs"] <= limit["max_abs"]
                                     and o_err["relative_l2"] <= limit["relative_l2"]),
                "agree_rtol_atol_0.05": bool(torch.allclose(o.float(), t.float(), rtol=0.05,
                                                            atol=0.05)),
            }
        record["seconds"] = round(time.perf_counter() - began, 2)
        results.append(record)
        del values, query, upstream, expected, triton, mine
        torch.cuda.empty_cache()
    return {"torch": torch.__version__, "device": torch.cuda.get_device_name(device),
            "reference": str(Path(reference.__file__).resolve().parent), "cells": results}


def markdown(report: dict) -> str:
    lines = ["| S | D | R | tensor | Triton max-abs / rel-L2 | ours max-abs / rel-L2 | bound max-abs / "
             "rel-L2 | within | ours vs Triton max-abs | agree 0.05 |",
             "|---|---|---|---|---|---|---|---|---|---|"]
    for cell in report["cells"]:
        for name in NAMES:
            e = cell[name]
            lines.append(
                f"| {cell['S']} | {cell['D']} | {cell['R']} | {name} | "
                f"{e['triton']['max_abs']:.3g} / {e['triton']['relative_l2']:.2e} | "
                f"{e['ours']['max_abs']:.3g} / {e['ours']['relative_l2']:.2e} | "
                f"{e['bound']['max_abs']:.3g} / {e['bound']['relative_l2']:.2e} | "
                f"{'yes' if e['within_bound'] else 'NO'} | {e['ours_vs_triton']['max_abs']:.3g} | "
                f"{'yes' if e['agree_rtol_atol_0.05'] else 'NO'} |")
    return "\n".join(lines)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawTextHelpFormatter)
    parser.add_argument("--cells", default="quick")
    parser.add_argument("--rows", type=int, default=2048)
    parser.add_argument("--markdown", action="store_true", help="also print the table")
    args = parser.parse_args()
    if not (REFERENCE_DIR / "attnres").exists():
        print(json.dumps({"unavailable": "baseline/_ref holds no reference install"}))
        return
    cells = {"quick": QUICK, "all": SWEEP}.get(args.cells) or [
        tuple(int(x) for x in cell.split(",")) for cell in args.cells.split(";")]
    report = run(cells, args.rows)
    if args.markdown:
        print(markdown(report))
    print(json.dumps(report), flush=True)


if __name__ == "__main__":
    main()
