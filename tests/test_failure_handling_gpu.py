"""Host-side failure handling of the backend, exercised without making a GPU fail: an
environment hook in the style of the reference's YVEX_TEST_CUDA_LAUNCH_FAILURE /
_SYNC_FAILURE (src/backend/cuda/capability.c:763,806) makes the operator's launch or its
synchronisation REPORT a backend failure on the host. What is checked is the reference's
contract: typed error, the backend refuses every later operation (a failure is sticky,
capability.c:757-817), nothing falls back to a CPU path, a fresh backend works again."""
import os

import numpy as np
import pytest

import clori_b200
from clori_b200 import abi

pytestmark = pytest.mark.gpu


def attention(backend, check=False):
    q = np.array([[1, 0, 1, 0], [1, 0, 1, 0]], np.float32)
    k = np.array([[1, 0], [0, 1]], np.float32)
    v = np.array([[2, 4], [6, 8]], np.float32)
    r = clori_b200.attention_requirement(2, 2, 0, 2, 1, 2)
    out = backend.alloc("o", abi.DTYPE_F32, (2, 4))
    rc, facts = backend.attention_execute(r, backend.tensor("q", q), backend.tensor("k", k),
                                          backend.tensor("v", v), out, check=check)
    return rc, out


@pytest.mark.parametrize("variable", ["YVEX_B200_TEST_LAUNCH_FAILURE", "YVEX_B200_TEST_SYNC_FAILURE"])
def test_reported_failure_is_typed_and_sticky(library, variable):
    backend = clori_b200.Backend(0)
    try:
        rc, out = attention(backend)
        assert rc == abi.YVEX_OK and np.array_equal(out.read()[0], [2, 4, 2, 4])
        os.environ[variable] = "some.other.operator"          # names another operator: no effect
        assert attention(backend)[0] == abi.YVEX_OK
        os.environ[variable] = "cuda.transformer.gqa"
        with pytest.raises(clori_b200.operator.YvexError) as failure:
            attention(backend, check=True)
        assert failure.value.code == abi.YVEX_ERR_BACKEND and "injected" in failure.value.message
        del os.environ[variable]
        # the hook is gone, the refusal stays: every later operator and allocation is refused
        assert attention_refused(backend)
    finally:
        os.environ.pop(variable, None)
        backend.close()
    with clori_b200.Backend(0) as fresh:
        rc, out = attention(fresh)
        assert rc == abi.YVEX_OK and np.array_equal(out.read()[0], [2, 4, 2, 4])


def attention_refused(backend):
    try:
        rc, _ = attention(backend)
    except clori_b200.operator.YvexError as error:      # the allocation in front is refused already
        return error.code == abi.YVEX_ERR_BACKEND
    return rc == abi.YVEX_ERR_BACKEND
