"""The sampling entry point that allocates nothing, called through its exported C symbol.

Embedders that may not allocate device memory when they sample (a closed memory budget, a plugin
barred from the host's allocator, a real-time loop) call ``aien_sample_rows_static``: it draws
exactly what ``aien_sample_rows`` draws, on scratch the library keeps for itself.  Checked here:
two calls in a row give the tokens of the regular entry point, an oversized request is refused
with the size code and launches nothing.  This file sorts last so that a run that stops at the
first failure has already run everything else.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_sampling_matches_regular_entry_point():
    from aien_sovereign_core_mv_b200 import kernels as K
    lib = K.lib()
    fn = lib.aien_sample_rows_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 8
    stream = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(3)
    for call, (R, V) in enumerate([(5, 3001), (3, 70000)]):           # two calls in a row, the second dirtier and larger
        logits = torch.tensor(rng.standard_normal((R, V)).astype(np.float32) * 2.5).cuda()
        temp = torch.tensor([0.0, 0.7, 1.0, 1.4, 0.9][:R]).cuda()
        top_p = torch.tensor([1.0, 0.95, 1.0, 0.6, 0.9][:R]).cuda()
        top_k = torch.tensor([0, 0, 50, 0, 7][:R], dtype=torch.int32).cuda()
        seeds = torch.tensor([1, 2, 3, 4, 5][:R], dtype=torch.int64).cuda()
        rids = torch.tensor([10, 11, 12, 2 ** 35, 14][:R], dtype=torch.int64).cuda()
        pos = torch.full((R,), 17 + call, dtype=torch.int32).cuda()
        want = torch.empty(R, dtype=torch.int32, device="cuda")
        K.sample_rows(logits, temp, top_p, top_k, seeds, rids, pos, torch.empty(R * V, device="cuda"), want)
        got = torch.full((R,), -1, dtype=torch.int32, device="cuda")
        rc = fn(logits.data_ptr(), R, V, temp.data_ptr(), top_p.data_ptr(), top_k.data_ptr(), seeds.data_ptr(), rids.data_ptr(),
                pos.data_ptr(), got.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert got.cpu().tolist() == want.cpu().tolist()              # same draws, token for token
    # beyond the stated maximum: refused with the size code, output untouched
    R, V = 9, 151936
    logits = torch.zeros(R, V, device="cuda")
    got = torch.full((R,), -1, dtype=torch.int32, device="cuda")
    z = torch.zeros(R, device="cuda")
    zi = torch.zeros(R, dtype=torch.int32, device="cuda")
    zl = torch.zeros(R, dtype=torch.int64, device="cuda")
    rc = fn(logits.data_ptr(), R, V, z.data_ptr(), z.data_ptr(), zi.data_ptr(), zl.data_ptr(), zl.data_ptr(), zi.data_ptr(),
            got.data_ptr(), stream)
    torch.cuda.synchronize()
    assert rc == -3 and (got == -1).all()
