"""The allocation-free attention entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory themselves (a plug-in in a
host program that owns the memory pool, a real-time loop that must not enter the allocator),
so ``atom_flash_attention_static`` takes its split-K scratch from an array compiled into the
library.  Here it is called twice in a row, with different shapes so that the second call
finds the first one's leftovers in the shared array, and its output is compared with the
regular entry point's, which gets its scratch from the caller, and with a dense float reference.
A call that would need more
scratch than the array holds must be refused before anything runs.

This file is collected last, so a run that stops at the first failure has run all others.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
ERR_SCRATCH = 4
SCRATCH_FLOATS = 2 * 1024 * 1024


def _case(q_lens, ctx_lens, nh, nkv, hd, page, seed):
    from test_kernels_gpu import _paged_case, _ref_attention

    q, kp, vp, bt, dense = _paged_case(q_lens, ctx_lens, nh, nkv, hd, page, torch.bfloat16, seed)
    T = sum(q_lens)
    _case.dense_ref = _ref_attention(q, dense, q_lens, ctx_lens, nh, nkv, hd ** -0.5, 0)   # [T, nh, hd], dense float reference
    d = lambda x: x.to(DEV).contiguous()
    cu = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32, device=DEV)
    ctx = torch.tensor(ctx_lens, dtype=torch.int32, device=DEV)
    sot = torch.cat([torch.full((n,), i) for i, n in enumerate(q_lens)]).to(torch.int32).to(DEV)
    return d(q.reshape(T, nh * hd)), d(kp), d(vp), d(bt), cu, ctx, sot


def _static(lib):
    fn = lib.atom_flash_attention_static
    vp, i, i64, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
    fn.argtypes = [vp, vp, i64, vp, vp, vp, i, i, vp, vp, vp, i, i, i, i, i, f, i, i, i, i, vp]
    fn.restype = ctypes.c_int
    return fn


@pytest.mark.parametrize("hd", [64, 128])
def test_static_scratch_entry_point_matches_regular(hd):
    from atom_b200 import native

    lib = native.flash_lib(hd)
    fn = _static(lib)
    nh, nkv, page = 8, 2, 16
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row: first many short requests with 5 splits, then other lengths with 3
    for q_lens, ctx_lens, splits, seed in (([1, 1, 2, 1, 40], [900, 300, 77, 1, 40], 5, 1),
                                           ([1, 2, 1], [130, 700, 64], 3, 2)):
        q, kp, vp, bt, cu, ctx, sot = _case(q_lens, ctx_lens, nh, nkv, hd, page, seed)
        T, S = sum(q_lens), len(q_lens)
        tiles, has_short, _ = native.flash_plan(q_lens, nh // nkv, nkv, max(ctx_lens))
        plan = (tiles, has_short, splits)
        want = torch.empty((T, nh * hd), dtype=torch.bfloat16, device=DEV)
        scratch = torch.empty(native.flash_scratch_elems(T, nh, hd, splits), dtype=torch.float32, device=DEV)
        native.flash_attention(want, q, nh * hd, kp, vp, bt, cu, ctx, sot, T, S, nh, nkv, hd, hd ** -0.5, 0,
                               plan, scratch)
        got = torch.full_like(want, float("nan"))
        rc = fn(got.data_ptr(), q.data_ptr(), nh * hd, kp.data_ptr(), vp.data_ptr(), bt.data_ptr(),
                bt.shape[1], page, cu.data_ptr(), ctx.data_ptr(), sot.data_ptr(), T, S, nh, nkv, hd,
                hd ** -0.5, 0, tiles, int(has_short), splits, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
        # and against the dense reference that shares no kernel with either entry point
        ref = _case.dense_ref.reshape(T, nh * hd)
        assert (got.float().cpu() - ref).abs().max().item() <= 2e-2

    # beyond the array's size: refused, nothing written
    T_big = SCRATCH_FLOATS // (nh * 64 * (hd + 2)) + 1
    before = got.clone()
    rc = fn(got.data_ptr(), q.data_ptr(), nh * hd, kp.data_ptr(), vp.data_ptr(), bt.data_ptr(), bt.shape[1],
            page, cu.data_ptr(), ctx.data_ptr(), sot.data_ptr(), T_big, S, nh, nkv, hd, hd ** -0.5, 0, 0, 1, 64,
            stream)
    assert rc == ERR_SCRATCH
    torch.cuda.synchronize()
    assert torch.equal(got, before)
