"""Shared test plumbing: the ``gpu`` marker, import paths, golden-fixture loading."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")
DTYPES = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


def from_raw(a: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    """Undo the uint16 bit-pattern storage the fixtures use for 16-bit floats."""
    if dtype in (torch.float16, torch.bfloat16):
        return torch.from_numpy(a.view(np.int16).copy()).view(dtype)
    return torch.from_numpy(a.copy())


def load_cases(name: str):
    """``{case: {field: ndarray}}`` from ``tests/golden/<name>.npz``."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    cases = {}
    for k in z.files:
        case, field = k.split("__")
        cases.setdefault(case, {})[field] = z[k]
    return cases


def same_values(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Equal as numbers (so -0.0 == +0.0), NaN nowhere."""
    return a.shape == b.shape and bool(torch.all(a.float() == b.float()))


@pytest.fixture(scope="session")
def cuda_device():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(scope="session", autouse=True)
def built_library():
    """Compile ``libactnn_b200.so`` when nvcc is around (a no-op if it is up to date)."""
    import shutil
    from actnn_b200.csrc import build as lib_build
    if os.path.exists(lib_build.NVCC) or shutil.which("nvcc"):
        lib_build.build()
    return lib_build.LIB


@pytest.fixture(autouse=True)
def fresh_scheme_registry():
    """The package keeps process-wide state the way the reference does (the configuration object
    and the list of every scheme ever created, which the per-layer allocation walks).  Every test
    starts from and leaves an empty registry and the default configuration, whatever ran before."""
    import actnn_b200
    from actnn_b200.conf import QuantizationConfig

    def reset():
        actnn_b200.config.__dict__.update(QuantizationConfig().__dict__)
        actnn_b200.QScheme.layers.clear()
        actnn_b200.QBNScheme.layers.clear()
        actnn_b200.QScheme.num_layers = 0
        actnn_b200.QScheme.prev_layer = None

    reset()
    yield
    reset()
