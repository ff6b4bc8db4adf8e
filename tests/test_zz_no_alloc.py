"""The allocation-free attention entry point against the regular one (collected last on purpose).

``insg_gqa_decode_noalloc`` serves callers that cannot allocate device memory or pass a scratch buffer
(capture-time code, plug-in hosts with a foreign allocator): its split partials live in a fixed array
inside the library.  It must give what ``insg_gqa_decode`` gives, call after call, whether this file
runs alone in a fresh process or after every other test.
"""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def test_noalloc_matches_regular_entry_twice_in_a_row(cuda):
    from insignia_b200 import _lib, ops

    rng = np.random.default_rng(123)
    for call, tokens in enumerate((777, 3000)):  # two calls in a row share the static scratch
        q = torch.from_numpy(rng.standard_normal(4096).astype(np.float32)).cuda()
        k = torch.from_numpy(rng.standard_normal(tokens * 1024).astype(np.float32)).cuda()
        v = torch.from_numpy(rng.standard_normal(tokens * 1024).astype(np.float32)).cuda()
        want = ops.gqa_decode(q, k, v, tokens)
        got = ops.gqa_decode_noalloc(q, k, v, tokens)
        torch.cuda.synchronize()
        assert float((got - want).abs().max()) <= 3e-5, call  # the tolerance of the attention parity tests
        assert torch.equal(got, want), call                    # same kernel, same split order
        kb, vb = k.to(torch.bfloat16), v.to(torch.bfloat16)
        assert float((ops.gqa_decode_noalloc(q, kb, vb, tokens) - ops.gqa_decode(q, kb, vb, tokens)).abs().max()) <= 3e-5
    # sizes beyond the stated maximum are refused with a clear error, nothing is launched
    L = _lib.lib()
    rc = L.insg_gqa_decode_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), got.data_ptr(), 262145, 0, None)
    assert rc == -5 and b"262144" in L.insg_last_error()
