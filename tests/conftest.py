import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run with -m gpu on a B200)")


_PARITY_LOG = os.path.join(ROOT, "gpurun_out", "parity_achieved.jsonl")


def record_parity(kind: str, **numbers) -> None:
    """Append what a float parity check actually measured (raw max abs error, raw mean relative error, the floor that
    rounding the exact result to the output dtype sets, the bound applied) to gpurun_out/parity_achieved.jsonl, keyed
    by the running test.  Best effort: a read-only tree just skips the record."""
    import json
    try:
        os.makedirs(os.path.dirname(_PARITY_LOG), exist_ok=True)
        test = os.environ.get("PYTEST_CURRENT_TEST", "").split(" ")[0]
        with open(_PARITY_LOG, "a") as f:
            f.write(json.dumps({"test": test, "kind": kind, **{k: (float(v) if v is not None else None) for k, v in numbers.items()}}) + "\n")
    except OSError:
        pass


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from flash3dtransformer_b200.lib import _cabi
    _cabi.load()          # fails loudly if the extension was not built
    return torch.device("cuda:0")
