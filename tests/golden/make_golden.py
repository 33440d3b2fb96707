"""Regenerate ``reference_oracle.npz`` from the REFERENCE's own oracle.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/fast-attnres

It imports ``validation/oracle.py`` from that checkout (CPU, PyTorch), evaluates
forward and autograd gradients on seeded inputs and stores inputs and results as
BF16 bit patterns (uint16).  The tests then hold our oracle restatement to these
vectors bit for bit, without needing the reference at test time.
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

# name, S, N, D, R, eps, scale, seed, query_std, loss
CASES = [
    ("config1_cpu_oracle_run", 8, 2, 1024, 1024, 2**-23, 1.0, 0, 1.0, "square_mean"),
    ("tiny_sliced", 3, 2, 17, 5, 2**-23, 1.0, 23, 1.0, "upstream"),
    ("autocast_case", 5, 3, 17, 7, 2**-23, 0.7, 19, 1.0, "upstream"),
    ("negative_scale", 4, 3, 32, 16, 2**-10, -0.75, 20260827, 0.05, "upstream"),
    ("sliced_256_32", 9, 5, 256, 32, 2**-23, 1.0, 20260903, 0.25, "upstream"),
    ("installed_smoke", 2, 4, 64, 64, 2**-20, 0.75, 20260911, 1.0, "upstream"),
    ("odd_width", 7, 3, 257, 129, 2**-23, 1.0 / 8.0, 5, 0.25, "upstream"),
    ("single_source", 1, 3, 40, 8, 2**-23, 1.0, 6, 1.0, "upstream"),
    ("unit_width", 3, 2, 1, 1, 2**-23, 1.0, 7, 1.0, "upstream"),
]


def bits(tensor: torch.Tensor) -> np.ndarray:
    return tensor.detach().contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/fast-attnres")
    reference_root = Path(sys.argv[1])
    spec = importlib.util.spec_from_file_location(
        "reference_validation_oracle", reference_root / "validation" / "oracle.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    reference_oracle = module.oracle

    arrays: dict[str, np.ndarray] = {}
    names = []
    for name, S, N, D, R, eps, scale, seed, query_std, loss in CASES:
        torch.manual_seed(seed)
        values = torch.randn(S, N, D).to(torch.bfloat16).requires_grad_()
        query = (torch.randn(R) * query_std).to(torch.bfloat16).requires_grad_()
        out = reference_oracle(values, query, eps=eps, scale=scale)
        if loss == "square_mean":
            # the reference's CPU oracle run: loss = output.square().mean(); the upstream gradient
            # autograd hands the operator is d loss / d out in BF16.
            total = out.square().mean()
            upstream, = torch.autograd.grad(total, out, retain_graph=True)
        else:
            upstream = torch.randn(N, D).to(torch.bfloat16)
        dv, dq = torch.autograd.grad(out, (values, query), upstream)
        # The list form must give the same bits as the packed form.
        out_list = reference_oracle(tuple(values.unbind(0)), query, eps=eps, scale=scale)
        assert torch.equal(out_list, out)
        names.append(name)
        arrays[f"{name}.values"] = bits(values)
        arrays[f"{name}.query"] = bits(query)
        arrays[f"{name}.upstream"] = bits(upstream)
        arrays[f"{name}.out"] = bits(out)
        arrays[f"{name}.dv"] = bits(dv)
        arrays[f"{name}.dq"] = bits(dq)
        arrays[f"{name}.eps_scale"] = np.array([eps, scale], dtype=np.float64)
    arrays["names"] = np.array(names)
    arrays["torch_version"] = np.array(torch.__version__)
    np.savez_compressed(HERE / "reference_oracle.npz", **arrays)
    print(f"wrote {HERE / 'reference_oracle.npz'} with {len(names)} cases")


if __name__ == "__main__":
    main()
