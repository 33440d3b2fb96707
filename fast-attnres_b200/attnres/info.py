"""``python -m attnres.info [--json]``: versions and the state of the CUDA library.

Counterpart of the reference's diagnostic command (src/attnres/info.py:23-107).  The
mapping carries the reference's keys (``package``, ``version``, ``python``, ``torch``,
``cuda_available``, ``cuda_runtime``, ``triton_available``, ``triton_version``) so scripts
written against it keep working, plus a ``library_*`` block for the sm_100a shared library
that does the work here.  Triton is reported but never imported or used.  The command runs
on a machine without a GPU and without the built library.
"""
from __future__ import annotations

import argparse
import importlib.metadata
import importlib.util
import json
import platform
import sys
from typing import Any


def _triton() -> tuple[bool, str | None]:
    """(installed, version) from package metadata only; Triton itself is not imported."""
    try:
        return True, importlib.metadata.version("triton")
    except importlib.metadata.PackageNotFoundError:
        pass
    try:
        return importlib.util.find_spec("triton") is not None, None
    except (ImportError, ValueError):
        return False, None


def collect_info() -> dict[str, Any]:
    """JSON-serialisable description of the package, the runtime and the CUDA library."""
    import torch

    from . import __version__, _native
    triton_available, triton_version = _triton()
    report: dict[str, Any] = {
        "package": "fast-attnres",
        "version": __version__,
        "python": platform.python_version(),
        "torch": str(torch.__version__),
        "cuda_available": bool(torch.cuda.is_available()),
        "cuda_runtime": torch.version.cuda,
        "triton_available": triton_available,
        "triton_version": triton_version,
        "backend": "sm_100a CUDA library (no Triton, no CPU fallback)",
        "library_path": str(_native.LIBRARY_PATH),
        "library_present": _native.LIBRARY_PATH.exists(),
        "library_abi": None,
        "library_error": None,
        "device": None,
        "compute_capability": None,
    }
    try:
        report["library_abi"] = int(_native.load().attnres_b200_abi_version())
    except Exception as error:  # missing or mismatched library
        report["library_error"] = str(error)
    if report["cuda_available"]:
        index = torch.cuda.current_device()
        report["device"] = torch.cuda.get_device_name(index)
        report["compute_capability"] = ".".join(map(str, torch.cuda.get_device_capability(index)))
    return report


collect = collect_info  # earlier name of the same function


def _format_human(info: dict[str, Any]) -> str:
    def yes_no(value: bool) -> str:
        return "yes" if value else "no"

    def shown(value: Any) -> str:
        return "unavailable" if value is None else str(value)

    library = (f"ABI {info['library_abi']}" if info["library_abi"] is not None
               else f"not loaded ({shown(info['library_error'])})")
    return "\n".join((
        f"{info['package']} {info['version']}",
        f"python: {info['python']}",
        f"torch: {info['torch']}",
        f"cuda available: {yes_no(info['cuda_available'])}",
        f"cuda runtime: {shown(info['cuda_runtime'])}",
        f"triton available: {yes_no(info['triton_available'])} (not used)",
        f"triton version: {shown(info['triton_version'])}",
        f"backend: {info['backend']}",
        f"library: {info['library_path']}",
        f"library state: {library}",
        f"device: {shown(info['device'])}",
        f"compute capability: {shown(info['compute_capability'])}",
        "attnres API: CUDA BF16 only",
    ))


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(prog="attnres.info", description=__doc__)
    parser.add_argument("--json", action="store_true", help="print the mapping as one JSON object")
    args = parser.parse_args(argv)
    info = collect_info()
    if args.json:
        json.dump(info, sys.stdout, sort_keys=True)
        sys.stdout.write("\n")
    else:
        sys.stdout.write(_format_human(info) + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())


__all__ = ["collect_info", "main"]
