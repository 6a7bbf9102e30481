"""The C++ layer classes (dl_cuda_b200/src/*.cuh: the reference's layer API on top of the C ABI),
driven by tests/cpp/layer_api_test, as the reference's tests/gpu_correctness_tests.cu drives its own."""
import subprocess
from pathlib import Path

import numpy as np
import pytest

from oracle import ref as refshim

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "tests" / "cpp" / "layer_api_test"


def run(*args):
    if not BIN.exists():
        from dl_cuda_b200 import build
        build.build_cpp_tests()
    res = subprocess.run([str(BIN), *map(str, args)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr


@pytest.mark.parametrize("mode", ["known_answer", "roundtrip", "chain", "optimizer"])
def test_layer_classes(mode):
    run(mode)


def test_checkpoint_bytes_and_curand_init_match_the_reference(tmp_path):
    mine = tmp_path / "mine.bin"
    run("checkpoint", mine, 3, 5, 3, 4, 1)
    data = mine.read_bytes()
    assert data[:4] == b"DLCU" and len(data) == 4 + 4 + 4 + 4 + 15 * 4
    header = np.frombuffer(data[4:16], np.int32)
    assert list(header) == [1, 1, 15]
    table = np.frombuffer(data[16:], np.float32).reshape(5, 3)
    # the cuRAND-initialised table of the SECOND reference layer built after set_global_init_seed(3)
    # (make_golden.py builds one layer before it)
    golden = np.load(ROOT / "tests" / "golden" / "embedding_layer_known_answer.npz")["curand_table_seed3"]
    assert np.array_equal(table.view(np.uint32), golden.view(np.uint32))
    if refshim.available():
        theirs = tmp_path / "theirs.bin"
        built_before = refshim.layers_built
        refshim.embedding_init(12345, 65, 64, 2048, theirs)
        mine2 = tmp_path / "mine2.bin"
        run("checkpoint", mine2, 12345, 65, 64, 2048, built_before)
        assert mine2.read_bytes() == theirs.read_bytes()
