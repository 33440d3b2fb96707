"""The package's example scripts run on a GPU (they assert their own results)."""
import importlib.util
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
EXAMPLES = Path(__file__).resolve().parents[1] / "fast-attnres_b200" / "examples"


@pytest.mark.parametrize("name", ["reads", "schedules_compile_graph", "training_extensions"])
def test_example_runs(name):
    spec = importlib.util.spec_from_file_location(f"example_{name}", EXAMPLES / f"{name}.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    summary = module.run("cuda")
    assert isinstance(summary, dict) and summary
