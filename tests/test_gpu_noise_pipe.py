"""Per-step noise pipeline of the flash scheduler (o1.c src/runtime/generate.c:1296, :1419-1439):
host-thread draws + device statistics / clamp against the serial host path."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,clip,threads", [(1 << 20 | 17, 2.5, 4), (3 * 64 * 3072, 8.0, 2), (100000, 0.0, 1)])
def test_noise_pipe_matches_host_path(pkg, dev, n, clip, threads):
    lib = pkg.lib
    seed = 4242 + 1                                     # the reference seeds the step generator with seed + 1
    pipe = C.c_void_p()
    assert lib.o1_noise_pipe_create(C.byref(pipe), seed, n, clip, threads) == 0, pkg.last_error()
    rng = lib.o1_torch_rng_create(seed)
    try:
        noise = torch.empty(n, dtype=torch.float32, device=dev)
        for step in range(4):
            pkg.check(lib.o1_noise_pipe_next(pipe, pkg.ptr(noise), None))
            got = noise.cpu().numpy()                   # synchronises the stream the pipe enqueued on
            want = np.empty(n, dtype=np.float32)
            lib.o1_torch_rng_randn(rng, want.ctypes.data_as(C.c_void_p), n)
            if clip > 0:
                lib.o1_noise_clamp_host(want.ctypes.data_as(C.c_void_p), n, clip)
            assert (got.view(np.uint32) == want.view(np.uint32)).all(), step
            if clip > 0 and clip < 4:
                assert (np.abs(got) == np.abs(got).max()).sum() > 10      # the clamp was exercised
    finally:
        lib.o1_torch_rng_free(rng)
        lib.o1_noise_pipe_free(pipe)


def test_noise_pipe_feeds_the_flash_scheduler_step(pkg, dev):
    """z_next = noise * s_noise * sigma_next + (1 - sigma_next) * (z - mo * sigma) with the pipe's noise equals
    the same step fed with host-generated noise (src/model/scheduler.c:71-99)."""
    lib = pkg.lib
    n = 16 * 3072
    g = torch.Generator().manual_seed(7)
    z = torch.randn(n, generator=g).to(dev)
    mo = torch.randn(n, generator=g).to(dev)
    pipe = C.c_void_p()
    assert lib.o1_noise_pipe_create(C.byref(pipe), 99, n, 8.0, 2) == 0
    rng = lib.o1_torch_rng_create(99)
    try:
        noise = torch.empty(n, dtype=torch.float32, device=dev)
        den = torch.empty_like(z)
        out_a, out_b = torch.empty_like(z), torch.empty_like(z)
        pkg.check(lib.o1_noise_pipe_next(pipe, pkg.ptr(noise), None))
        lib.hd_sched_denoised(pkg.ptr(z), pkg.ptr(mo), 0.7, pkg.ptr(den), n)
        lib.hd_sched_z_next(pkg.ptr(noise), pkg.ptr(den), 0.55, 7.5, pkg.ptr(out_a), n)
        host = np.empty(n, dtype=np.float32)
        lib.o1_torch_rng_randn(rng, host.ctypes.data_as(C.c_void_p), n)
        lib.o1_noise_clamp_host(host.ctypes.data_as(C.c_void_p), n, 8.0)
        hn = torch.from_numpy(host).to(dev)
        lib.hd_sched_z_next(pkg.ptr(hn), pkg.ptr(den), 0.55, 7.5, pkg.ptr(out_b), n)
        torch.cuda.synchronize()
        assert torch.equal(out_a, out_b)
    finally:
        lib.o1_torch_rng_free(rng)
        lib.o1_noise_pipe_free(pipe)
