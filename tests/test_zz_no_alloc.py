"""hp_argmax_noalloc: the argmax entry point for callers that cannot allocate (its scratch is a fixed array inside
the library). Collected last on purpose. It must agree bit for bit with hp_argmax on consecutive calls that share
the built-in scratch, and must reject shapes beyond the built-in limits instead of launching."""
import ctypes

import numpy as np
import pytest
import torch

import hipster_b200 as hb
from hipster_b200 import kernels as K_
from oracle import orc

pytestmark = pytest.mark.gpu


def test_noalloc_argmax_matches_argmax_on_two_calls_in_a_row():
    rng = np.random.default_rng(7)
    first = rng.normal(size=(6, 248320)).astype(np.float32)
    second = rng.normal(size=(3, 70001)).astype(np.float32)
    first[2, 11] = first[2, 200000] = 40.0          # tie across partial blocks: the lower index must win
    second[0, 70000] = 40.0
    for a in (first, second):                        # the second call reuses the scratch the first one left behind
        t = torch.from_numpy(a).cuda()
        want_ids, want_vals = K_.argmax(t)
        got_ids, got_vals = K_.argmax_noalloc(t)
        torch.cuda.synchronize()
        assert torch.equal(got_ids, want_ids)
        assert np.array_equal(got_vals.cpu().numpy().view(np.uint32), want_vals.cpu().numpy().view(np.uint32))
        # and directly against independent checkers: the CPU oracle and numpy (first maximum = lowest index on ties)
        oi, ov = orc.argmax(a)
        assert np.array_equal(got_ids.cpu().numpy(), oi) and np.array_equal(got_vals.cpu().numpy().view(np.uint32), ov.view(np.uint32))
        assert np.array_equal(got_ids.cpu().numpy(), np.argmax(a, axis=1).astype(np.int32))
        if a is first:
            assert int(got_ids[2]) == 11            # the planted tie between columns 11 and 200000, in different partial blocks
    assert int(got_ids[0]) == 70000


def test_noalloc_argmax_rejects_shapes_beyond_the_builtin_scratch():
    L = hb.lib()
    max_rows, max_n = L.hp_argmax_noalloc_max_rows(), L.hp_argmax_noalloc_max_n()
    assert max_rows >= 32 and max_n >= 248320
    t = torch.zeros((1, 8), dtype=torch.float32, device="cuda")
    ids = torch.zeros(max_rows + 1, dtype=torch.int32, device="cuda")
    null = ctypes.c_void_p(0)
    rc = L.hp_argmax_noalloc(hb.ptr(t), max_rows + 1, 8, 8, hb.ptr(ids), null, null)
    assert rc == 1 and b"exceed" in L.hp_last_error()
    rc = L.hp_argmax_noalloc(hb.ptr(t), 1, max_n + 1, max_n + 1, hb.ptr(ids), null, null)
    assert rc == 1 and b"exceed" in L.hp_last_error()
