import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    import json
    with open(os.path.join(ROOT, "tests", "golden", "comet_golden.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def mtx_dir(golden, tmp_path_factory):
    """Write the golden matrices back out as MatrixMarket files."""
    d = tmp_path_factory.mktemp("mtx")
    for name, m in golden["matrices"].items():
        with open(d / name, "w") as f:
            f.write(m["banner"] + "\n%\n")
            f.write("%d %d %d\n" % tuple(m["size"]))
            for r, c, v in m["entries"]:
                f.write("%d %d\n" % (r, c) if v is None else "%d %d %r\n" % (r, c, v))
    return d
