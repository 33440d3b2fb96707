"""Host-side contract of ``attnres`` and ``LearnedQuery`` (no GPU needed).

The cases follow the reference's CPU contract tests (tests/test_api.py:16-61,
:90-109, :145-156, :224-277 and tests/test_info.py:27-38 of the reference).
"""
import inspect
import sys

import pytest
import torch

import attnres as package
from attnres import LearnedQuery, attnres
from attnres._sources import row_layout


def test_public_surface():
    assert set(package.__all__) == {"attnres", "LearnedQuery", "__version__"}
    parameters = inspect.signature(attnres).parameters
    assert list(parameters) == ["values", "query", "eps", "scale"]
    assert parameters["eps"].default == 2**-23 and parameters["scale"].default == 1.0
    assert parameters["eps"].kind is inspect.Parameter.KEYWORD_ONLY
    with pytest.raises(TypeError):
        attnres(torch.zeros(2, 3, 4, dtype=torch.bfloat16), torch.zeros(4, dtype=torch.bfloat16),
                keys=torch.zeros(2, 3, 4, dtype=torch.bfloat16))


def _sources(count, rows, width, *, grad=False):
    return [torch.randn(rows, width, dtype=torch.bfloat16, requires_grad=grad) for _ in range(count)]


@pytest.mark.parametrize("container", [list, tuple])
def test_cpu_source_lists_are_refused_without_importing_triton(monkeypatch, container):
    """The list path answers "CUDA required" for CPU tensors and never reaches for Triton (this
    package has none; the guard keeps it that way)."""
    import builtins
    real_import = builtins.__import__

    def watchful_import(name, *args, **kwargs):
        assert name.partition(".")[0] != "triton", f"attnres tried to import {name}"
        return real_import(name, *args, **kwargs)

    monkeypatch.setattr(builtins, "__import__", watchful_import)
    for stale in [name for name in sys.modules if name.partition(".")[0] == "triton"]:
        monkeypatch.delitem(sys.modules, stale)
    sources = container(_sources(3, 2, 8, grad=True))
    with pytest.raises(RuntimeError, match="CUDA"):
        attnres(sources, torch.randn(4, dtype=torch.bfloat16, requires_grad=True))


CPU_VALUES = torch.randn(5, 2, 13).to(torch.bfloat16)
CPU_QUERY = torch.randn(4).to(torch.bfloat16)


@pytest.mark.parametrize("values,query,error,text", [
    (CPU_VALUES, CPU_QUERY, RuntimeError, "CUDA"),
    (CPU_VALUES.float(), CPU_QUERY, TypeError, "BF16"),
    (CPU_VALUES, CPU_QUERY.float(), TypeError, "BF16"),
    ([CPU_VALUES[0].float(), CPU_VALUES[1].float()], CPU_QUERY, TypeError, "BF16"),
    (list(CPU_VALUES.unbind(0)), CPU_QUERY.double(), TypeError, "BF16"),
], ids=["cpu", "fp32-values", "fp32-query", "fp32-list", "fp64-query-list"])
def test_cpu_and_wrong_dtype_inputs_are_refused(values, query, error, text):
    with pytest.raises(error, match=text):
        attnres(values, query)


@pytest.mark.parametrize("as_list", [False, True], ids=["packed", "list"])
@pytest.mark.parametrize("keywords,error,text", [
    (dict(eps=0.0), ValueError, "eps"),
    (dict(eps=-1e-3), ValueError, "eps"),
    (dict(eps=float("inf")), ValueError, "eps"),
    (dict(scale=float("nan")), ValueError, "scale"),
    (dict(eps=True), TypeError, "eps"),
    (dict(scale="1"), TypeError, "scale"),
    (dict(scale=torch.tensor(1.0)), TypeError, "scale"),
    (dict(eps=2**-20, scale=0.75), RuntimeError, "CUDA"),     # valid scalars: the device is next
], ids=lambda value: "-".join(value) if isinstance(value, dict) else None)
def test_scalars_are_checked_before_the_device(keywords, error, text, as_list):
    values = torch.randn(4, 3, 9).to(torch.bfloat16)
    query = torch.randn(3).to(torch.bfloat16)
    with pytest.raises(error, match=text):
        attnres(tuple(values.unbind(0)) if as_list else values, query, **keywords)


def test_shape_and_container_errors():
    bf = torch.bfloat16
    query = torch.zeros(4, dtype=bf)
    with pytest.raises(TypeError, match="query must be a tensor"):
        attnres(torch.zeros(2, 3, 8, dtype=bf), [0.0] * 4)
    with pytest.raises(ValueError):
        attnres(torch.zeros(8, dtype=bf), query)                      # values rank < 2
    with pytest.raises(ValueError):
        attnres(torch.zeros(2, 3, 8, dtype=bf), torch.zeros(2, 2, dtype=bf))  # query rank
    with pytest.raises(ValueError):
        attnres(torch.zeros(130, 1, 8, dtype=bf), query)              # S > 129
    with pytest.raises(ValueError):
        attnres(torch.zeros(2, 1, 8193, dtype=bf), query)             # D > 8192
    with pytest.raises(ValueError):
        attnres(torch.zeros(2, 1, 3, dtype=bf), query)                # R > D
    with pytest.raises(ValueError):
        attnres(torch.zeros(2, 0, 8, dtype=bf), query)                # empty axis
    with pytest.raises(TypeError, match="list/tuple"):
        attnres({"a": torch.zeros(3, 8, dtype=bf)}, query)
    with pytest.raises(TypeError, match="only tensors"):
        attnres([torch.zeros(3, 8, dtype=bf), 1.0], query)
    with pytest.raises(ValueError, match="1<=S<=129"):
        attnres([], query)
    with pytest.raises(ValueError, match="1<=S<=129"):
        attnres([torch.zeros(1, 8, dtype=bf)] * 130, query)
    with pytest.raises(ValueError, match="same logical shape"):
        attnres([torch.zeros(3, 8, dtype=bf), torch.zeros(2, 8, dtype=bf)], query)
    with pytest.raises(ValueError, match="1<=R<=D"):
        attnres([torch.zeros(3, 2, dtype=bf)], query)
    with pytest.raises(ValueError):
        attnres([torch.zeros((), dtype=bf)], query)                   # source rank < 1
    with pytest.raises(TypeError, match="dtype/device"):
        attnres([torch.zeros(3, 8, dtype=bf), torch.zeros(3, 8)], query)


def test_learned_query_contract():
    module = LearnedQuery(16)
    assert module.query.dtype == torch.bfloat16 and module.query.shape == (16,)
    assert module().dtype == torch.bfloat16
    assert 0 < float(module.query.float().std()) < 0.1
    # Cast to FP32: the parameter is FP32, the query it hands out stays BF16 and
    # the gradient arrives in FP32.
    module = LearnedQuery(8).float()
    out = module()
    assert out.dtype == torch.bfloat16
    out.float().sum().backward()
    assert module.query.grad.dtype == torch.float32
    with pytest.raises(ValueError):
        LearnedQuery(0)
    with pytest.raises(TypeError):
        LearnedQuery(2.5)
    with pytest.raises(TypeError):
        LearnedQuery(True)
    with pytest.raises(ValueError):
        LearnedQuery(4, init_std=0.0)


def test_row_layout_flattens_affine_batches_and_copies_the_rest():
    # Same cases as tests/test_row_layout.py:7-41 of the reference.
    base = torch.arange(2 * 3 * 8, dtype=torch.float32)
    plain = base.view(2, 3, 8)
    tensor, row, feat = row_layout(plain)
    assert tensor is plain and (row, feat) == (8, 1)
    # singleton axes never constrain the layout
    single = base[:24].as_strided((3, 1, 8), (8, 16, 1))
    tensor, row, feat = row_layout(single)
    assert tensor is single and (row, feat) == (8, 1)
    # a broadcast row axis has stride 0
    broadcast = base[:8].expand(5, 8)
    tensor, row, feat = row_layout(broadcast)
    assert tensor is broadcast and (row, feat) == (0, 1)
    # a feature-strided view keeps its stride
    strided = base.view(6, 8)[:, ::2]
    tensor, row, feat = row_layout(strided)
    assert tensor is strided and (row, feat) == (8, 2)
    # a transposed batch is not affine: it is copied, and only then
    swapped = plain.transpose(0, 1)
    tensor, row, feat = row_layout(swapped)
    assert tensor is not swapped and tensor.is_contiguous() and (row, feat) == (8, 1)
    assert torch.equal(tensor, swapped)
    # a single vector
    tensor, row, feat = row_layout(base[:8])
    assert (row, feat) == (0, 1)


def test_accumulate_argument_checks():
    """`attnres_accumulate` validates like `attnres` and then checks the buffers (CPU only:
    nothing is launched)."""
    from attnres.accumulate import attnres_accumulate
    values = torch.zeros(3, 4, 16, dtype=torch.bfloat16)
    query = torch.zeros(8, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        attnres_accumulate(values, query, torch.zeros_like(values))
    with pytest.raises(RuntimeError, match="CUDA"):
        attnres_accumulate(list(values.unbind(0)), query, [torch.zeros(4, 16, dtype=torch.bfloat16)] * 3)
    with pytest.raises(ValueError):
        attnres_accumulate(values, query, torch.zeros_like(values), eps=0.0)
    from attnres.accumulate import _check_buffers
    good = [torch.zeros(4, 16, dtype=torch.bfloat16) for _ in range(3)]
    shapes = [(4, 16)] * 3
    _check_buffers(good, shapes, good[0].device)
    with pytest.raises(ValueError, match="one gradient buffer per source"):
        _check_buffers(good[:2], shapes, good[0].device)
    with pytest.raises(TypeError, match="BF16"):
        _check_buffers([g.float() for g in good], shapes, good[0].device)
    with pytest.raises(ValueError, match="shape"):
        _check_buffers([g[:2] for g in good], shapes, good[0].device)
    with pytest.raises(ValueError, match="contiguous"):
        _check_buffers([torch.zeros(16, 4, dtype=torch.bfloat16).T for _ in range(3)], shapes,
                       good[0].device)
    with pytest.raises(ValueError, match="own gradient buffer"):
        _check_buffers([good[0], good[0], good[1]], shapes, good[0].device)
    # overlapping views of one storage: each is contiguous with the right shape, but rows 2..3
    # of the first are rows 0..1 of the second
    storage = torch.zeros(6 * 16 + 4 * 16, dtype=torch.bfloat16)
    first, second = storage[:64].view(4, 16), storage[32:96].view(4, 16)
    with pytest.raises(ValueError, match="overlap"):
        _check_buffers([first, second, good[2]], shapes, good[0].device)
    # adjacent views of one storage do not overlap
    _check_buffers([storage[:64].view(4, 16), storage[64:128].view(4, 16), good[2]], shapes,
                   good[0].device)


def test_info_command_keeps_the_reference_keys_and_runs_without_a_gpu():
    """`python -m attnres.info [--json]` (tests/test_info.py:44-90 of the reference)."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    import attnres
    package_dir = Path(attnres.__file__).resolve().parents[1]
    for flags in ([], ["--json"]):
        done = subprocess.run([sys.executable, "-m", "attnres.info", *flags], cwd=package_dir,
                              capture_output=True, text=True, timeout=300)
        assert done.returncode == 0, done.stdout + done.stderr
        if flags:
            info = json.loads(done.stdout)
            assert info["package"] == "fast-attnres"
            assert info["version"] == attnres.__version__ == "2.0.1"
            assert info["torch"] == torch.__version__
            assert isinstance(info["cuda_available"], bool)
            assert isinstance(info["triton_available"], bool)
            assert info["library_present"] is True and info["library_abi"] == 3
        else:
            for text in ("fast-attnres 2.0.1", "torch:", "cuda available:", "triton available:",
                         "attnres API: CUDA BF16 only", "library state: ABI 3"):
                assert text in done.stdout


def test_fused_layer_norm_validates_like_attnres_on_cpu():
    """`attnres_layer_norm` runs the reference's argument checks first and then insists on
    CUDA tensors (nothing is launched on CPU)."""
    from attnres.fused import attnres_layer_norm
    values = torch.zeros(3, 4, 16, dtype=torch.bfloat16)
    query = torch.zeros(8, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        attnres_layer_norm(values, query)
    with pytest.raises(RuntimeError, match="CUDA"):
        attnres_layer_norm(list(values.unbind(0)), query, torch.ones(16), torch.zeros(16))
    with pytest.raises(TypeError):
        attnres_layer_norm(values.float(), query)
    with pytest.raises(ValueError):
        attnres_layer_norm(values, query, eps=0.0)
