"""The allocation-free Q4_K decode entry point against the regular one, on a B200.

Collected last on purpose (file name): a run that stops at the first failure has then already
run every other test.

jl_matvec_q4k_noalloc serves callers that cannot allocate device memory while they run --
code inside a stream capture, a runtime whose memory planner forbids a late cudaMalloc -- so
its kernel scratch is a fixed array inside the library. The buffers it works on here are made
by torch BEFORE the calls; the calls themselves allocate nothing.
"""
import ctypes as C

import numpy as np
import pytest

from conftest import parity_err
from jitllm_b200 import Q4_K, Device, _lib, synth

pytestmark = pytest.mark.gpu
BAR = 2e-3


def test_noalloc_decode_matches_the_regular_entry_point_twice(orc):
    import torch

    lib = _lib.load()
    rng = synth.rng_for(0x5747)
    cases = [(4096, 4096), (1000, 2048)]
    with Device(0) as dev:
        for nrows, k in cases:
            assert k <= lib.jl_noalloc_max_k()
            w = synth.q4k_matrix(rng, nrows, k)
            w_dev = torch.from_numpy(w.reshape(-1)).cuda()           # raw ggml bytes on the device
            handle = dev.Upload(Q4_K, w, nrows, k)
            want = torch.empty(nrows, device="cuda", dtype=torch.float32)
            got = torch.full((nrows,), float("nan"), device="cuda", dtype=torch.float32)
            stream = torch.cuda.current_stream().cuda_stream
            # one call before free memory is measured: the first call on a device looks up the scratch's address and
            # may load the kernels' module, which is the driver's allocation, not the call's
            x0 = torch.zeros(k, device="cuda")
            assert lib.jl_matvec_q4k_noalloc(got.data_ptr(), w_dev.data_ptr(), x0.data_ptr(), nrows, k, stream) == _lib.OK
            torch.cuda.synchronize()
            for call in range(2):                                    # two calls in a row share the scratch
                x = synth.activations(rng, 1, k)[0]
                x_dev = torch.from_numpy(x).cuda()
                torch.cuda.synchronize()
                free_before = torch.cuda.mem_get_info()[0]
                rc = lib.jl_matvec_q4k_noalloc(got.data_ptr(), w_dev.data_ptr(), x_dev.data_ptr(), nrows, k, stream)
                assert rc == _lib.OK
                torch.cuda.synchronize()
                assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
                dev.MatVecDev(want, handle, x_dev, 1, stream)
                torch.cuda.synchronize()
                g, r = got.cpu().numpy(), want.cpu().numpy()
                assert np.isfinite(g).all()
                assert parity_err(g, r) <= BAR
                ref = orc.matmul_f64(Q4_K, w, x, nrows, k, 1)[0]
                assert parity_err(g, ref) <= BAR
                got.fill_(float("nan"))
            handle.free()


def test_noalloc_refuses_sizes_beyond_its_fixed_scratch():
    import torch

    lib = _lib.load()
    k = lib.jl_noalloc_max_k() + 256
    buf = torch.zeros(16 * (k // 256) * 144, device="cuda", dtype=torch.uint8)
    x = torch.zeros(k, device="cuda")
    out = torch.zeros(16, device="cuda")
    assert lib.jl_matvec_q4k_noalloc(out.data_ptr(), buf.data_ptr(), x.data_ptr(), 16, k, 0) == _lib.ENOMEM
    assert lib.jl_matvec_q4k_noalloc(out.data_ptr(), buf.data_ptr(), x.data_ptr(), 16, 100, 0) == _lib.EINVAL
