"""Test configuration: the `gpu` marker, import paths, and shared helpers.

`-m "not gpu"` covers the oracle against the golden vectors, the host logic and the C-ABI
surface; `-m gpu` holds the parity tests proper, which call the CUDA path through the C ABI.
The oracle (oracle/akl_oracle.py) is imported here as the checker only.
"""
import pathlib
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]
for p in (ROOT, ROOT / "tests", ROOT / "oracle"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (NVIDIA B200, sm_100a)")


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__ as entry

    package = entry.package()
    package.build()
    return package


@pytest.fixture(scope="session")
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def pytest_sessionfinish(session, exitstatus):
    """Write the measured parity figures the tests recorded (helpers.LEDGER) next to the other
    run outputs; nothing is written when no test recorded anything."""
    import json

    try:
        import helpers
    except Exception:  # noqa: BLE001
        return
    if not helpers.LEDGER:
        return
    out = ROOT / "gpurun_out"
    try:
        out.mkdir(exist_ok=True)
        path = out / "parity_ledger.json"
        old = json.loads(path.read_text()) if path.exists() else {}
        for section, entries in helpers.LEDGER.items():
            old.setdefault(section, {}).update(entries)
        path.write_text(json.dumps(old, indent=1, sort_keys=True))
    except OSError:
        pass
