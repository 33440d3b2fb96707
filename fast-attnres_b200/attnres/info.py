"""``python -m attnres.info [--json]``: versions and the state of the CUDA library.

Counterpart of the reference's diagnostic command (src/attnres/info.py:23-107), which
reports Triton; this one reports the sm_100a shared library instead.
"""
from __future__ import annotations

import argparse
import json
import platform
import sys


def collect() -> dict:
    import torch

    from . import __version__, _native
    report = {
        "attnres": __version__,
        "python": platform.python_version(),
        "torch": torch.__version__,
        "cuda_runtime": torch.version.cuda,
        "cuda_available": torch.cuda.is_available(),
        "library": str(_native.LIBRARY_PATH),
        "library_present": _native.LIBRARY_PATH.exists(),
    }
    try:
        report["library_abi"] = int(_native.load().attnres_b200_abi_version())
    except Exception as error:  # missing or mismatched library
        report["library_error"] = str(error)
    if torch.cuda.is_available():
        index = torch.cuda.current_device()
        report["device"] = torch.cuda.get_device_name(index)
        report["compute_capability"] = ".".join(map(str, torch.cuda.get_device_capability(index)))
    return report


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="attnres.info", description=__doc__)
    parser.add_argument("--json", action="store_true", help="print one JSON object")
    args = parser.parse_args(argv)
    report = collect()
    if args.json:
        print(json.dumps(report, sort_keys=True))
    else:
        for key, value in report.items():
            print(f"{key}: {value}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
