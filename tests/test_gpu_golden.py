"""The reference's own integration tests, run through the C ABI of the CUDA
library (host memref entry points) and compared with their CHECK lines."""
import json
import os

import pytest

import comet_b200.api as gpu_api
from tests import golden_runner

pytestmark = pytest.mark.gpu

_G = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "comet_golden.json")))
_CASES = sorted(n for n, c in _G["cases"].items() if c["kind"] != "reader")


@pytest.mark.parametrize("name", _CASES)
def test_cuda_path_matches_reference_check_lines(name, golden, mtx_dir):
    case = golden["cases"][name]
    got = golden_runner.run_case(case, mtx_dir, gpu_api)
    assert golden_runner.normalise(got) == golden_runner.expected_text(case)
