"""GPU parity: tensor_gather against the reference's known answers, the CPU oracle, and numpy.take."""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_known_answers(gpu):
    cases = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "golden.json")))["gather_known_answers"]
    for case in cases:
        out = gpu.np_tensor_gather(np.array(case["source"], np.float32), case["indices"], case["axis"])
        assert sum(float(out[tuple(ix)]) for ix in case["sum_at"]) == case["expect"], case["src"]


@pytest.mark.parametrize("shape,axis,dtype", [((10,), 0, np.float32), ((32000, 768), 0, np.float32), ((5, 9), 1, np.int8),
                                              ((3, 4, 6), -2, np.float64), ((2, 3, 4, 5), 3, np.int32), ((6, 100, 33), 1, np.int8),
                                              ((4, 7, 16), 1, np.float32)])
def test_against_oracle(gpu, oracle, shape, axis, dtype):
    rng = np.random.default_rng(len(shape) * 13 + shape[0])
    src = rng.integers(-100, 100, shape).astype(dtype)
    idx = rng.integers(0, shape[axis], 37)
    out = gpu.np_tensor_gather(src, idx, axis)
    assert np.array_equal(out, oracle.tensor_gather(src, idx, axis))
    assert np.array_equal(out, np.take(src, idx, axis=axis))


def test_empty_and_out_of_range(gpu):
    assert gpu.np_tensor_gather(np.zeros((4, 3), np.float32), np.zeros(0, np.int64), 0).shape == (0, 3)
    with pytest.raises(gpu.SimpGpuError):
        gpu.np_tensor_gather(np.zeros((4, 3), np.float32), [1, 4], 0)    # reported, not a fault
    out = gpu.np_tensor_gather(np.arange(12, dtype=np.float32).reshape(4, 3), [3], 0)   # the library stays usable
    assert out.tolist() == [[9.0, 10.0, 11.0]]
