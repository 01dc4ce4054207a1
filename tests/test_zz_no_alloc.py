"""The sort entry point for callers that cannot allocate device memory (a decode loop that may
not stall on the allocator, a plugin that only owns its input and output buffers) must give
exactly what the workspace version gives, call after call, while the two share nothing but
the library's built-in count table.  Collected last on purpose: a failure here cannot hide
the result of any other test."""
import numpy as np
import pytest
import torch

from lisa_b200 import _cabi, ops
from tests.gpu_util import dev_i32

pytestmark = pytest.mark.gpu


def _case(cuda, seed, tokens, experts, top_k):
    rng = np.random.default_rng(seed)
    return dev_i32(rng.integers(0, experts, size=(tokens, top_k)).astype(np.int32), cuda)


def test_static_scratch_sort_matches_workspace_sort_twice(cuda):
    # buffers the caller already owns: nothing is allocated between the two calls below
    outs = tuple(torch.empty(4096 * 8, dtype=torch.int32, device=cuda) for _ in range(3))
    for seed, (tokens, experts, top_k) in enumerate([(4096, 128, 8), (777, 512, 10)]):
        idx = _case(cuda, seed, tokens, experts, top_k)
        want = ops.moe_sort(idx, experts, top_k)
        views = tuple(o[: tokens * top_k] for o in outs)
        got = ops.moe_sort_static(idx, experts, top_k, out=views)
        torch.cuda.synchronize()
        for g, w in zip(got, want):
            assert torch.equal(g, w)  # integer work: exact


def test_static_scratch_sort_refuses_oversized_problems(cuda):
    idx = _case(cuda, 3, 4096, 4096, 8)  # 128 chunks x 4096 experts > 65536 counters
    with pytest.raises(_cabi.LisaError) as err:
        ops.moe_sort_static(idx, 4096, 8)
    assert err.value.code == _cabi.ERR_LIMIT
    assert "65536" in err.value.message
