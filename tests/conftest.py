import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def built_library():
    """librode_b200.so, compiled on demand (nvcc cross-compiles without a GPU)."""
    from rode_b200 import build

    return build.build_library()


@pytest.fixture(scope="session")
def oracle_cpu():
    from oracle import cpu

    cpu.build()
    return cpu


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


# ---- tolerance head-room report ------------------------------------------------------------
# The full-size parity tests record how much of the tolerance each comparison used (ours and,
# where they can run, the reference's own kernels on the same inputs).  The rows are printed
# in the terminal summary and, when RODE_HEADROOM_JSON names a file, also written there.
_HEADROOM_ROWS = []


@pytest.fixture(scope="session")
def headroom():
    def record(config, impl, stats):
        _HEADROOM_ROWS.append({"config": config, "impl": impl, **stats})

    return record


def pytest_terminal_summary(terminalreporter):
    if not _HEADROOM_ROWS:
        return
    tr = terminalreporter
    tr.write_sep("-", "tolerance head-room (err / allowed; elements failing the literal 1e-5 rel / 1e-6 abs rule)")
    for r in _HEADROOM_ROWS:
        tr.write_line(f"{r['config']:<44} {r['impl']:<18} worst {r['worst_ratio']:.3f}   literal-rule failures "
                      f"{r['literal_fail']} of {r['elements']}   max err {r['max_err']:.3e}")
    path = os.environ.get("RODE_HEADROOM_JSON")
    if path:
        import json

        with open(path, "w") as f:
            json.dump(_HEADROOM_ROWS, f, indent=1)
