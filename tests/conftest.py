import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "supersonic-moe_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(scope="session")
def built_library():
    """Path of libsmoe_b200.so; compiled with nvcc (no GPU needed) when it is not there yet."""
    so = os.path.join(PKG, "sonicmoe", "libsmoe_b200.so")
    if not os.path.exists(so):
        sys.path.insert(0, ROOT)
        import __graft_entry__
        __graft_entry__.build()
    return so


@pytest.fixture(scope="session", autouse=True)
def _library_present(built_library):
    return built_library


def pytest_sessionfinish(session, exitstatus):
    """With SMOE_PARITY_REPORT=<path>: the measured cosine / relative RMS error of every tensor that went through
    tests/parity_util.gate in this session (GPU vs fp32 gold, emulation vs gold, GPU vs emulation), as a table."""
    path = os.environ.get("SMOE_PARITY_REPORT")
    try:
        from parity_util import REPORT
    except Exception:
        return
    if not path or not REPORT:
        return
    with open(path, "w") as f:
        f.write("| tensor | gate | GPU vs fp32: cos | rrmse | emulation vs fp32: cos | rrmse | GPU vs emulation: cos | rrmse |\n")
        f.write("|---|---|---|---|---|---|---|---|\n")
        for name, kind, a, b, c, d, e, g in REPORT:
            f.write(f"| {name} | {kind} | {a:.5f} | {b:.5f} | {c:.5f} | {d:.5f} | {e:.5f} | {g:.5f} |\n")
