"""GPU parity of the primitive-level C ABI (the hd_* functions of o1.c src/cuda/hd_cuda.h)
against the CPU oracle, and against the reference's own CUDA build when oracle/_ref holds it.
Tolerance classes are the reference's (docs/M1_NUMERICAL_CONTRACT.md:48-54): A exact, B pointwise,
C GEMM."""
import ctypes as C

import numpy as np
import pytest
import torch

import parity
from parity import np_ptr, seeded_bf16, torch_to_u16, u16_to_torch, assert_close

pytestmark = pytest.mark.gpu


_KEEP = []


@pytest.fixture(autouse=True)
def _release_device_temporaries():
    yield
    _KEEP.clear()


def dv(a, dev):
    """Host array -> device tensor that stays alive until the test ends (its address is handed to
    asynchronous kernels, so it must not return to the allocator mid-test)."""
    t = u16_to_torch(a, dev) if a.dtype == np.uint16 else torch.from_numpy(a).to(dev)
    _KEEP.append(t)
    return t


def empty_bf16(shape, dev):
    return torch.empty(shape, dtype=torch.bfloat16, device=dev)


def done(pkg, what):
    torch.cuda.synchronize()
    pkg.check_cuda_errbuf(what)


@pytest.mark.parametrize("rows,cols", [(7, 4096), (300, 4096), (1280 * 4, 128), (33, 96), (5, 100), (3, 8192)])
def test_rmsnorm(pkg, orc, dev, rows, cols):
    x, w = seeded_bf16((rows, cols), 1), seeded_bf16(cols, 2, 1.0, 0.1)
    y = empty_bf16((rows, cols), dev)
    pkg.lib.hd_rmsnorm(pkg.ptr(dv(x, dev)), pkg.ptr(dv(w, dev)), pkg.ptr(y), rows, cols, 1e-6)
    done(pkg, "rmsnorm")
    ref = np.empty_like(x)
    orc.orc_rmsnorm(np_ptr(x), np_ptr(w), np_ptr(ref), rows, cols, 1e-6)
    assert_close(torch_to_u16(y), ref, "B", "rmsnorm")
    r = parity.reflib()
    # The reference kernel reduces with a halving tree over min(cols,256) threads (norm.cu:31-35), which
    # only sums every element when that count is a power of two: compare against it for those shapes.
    if r is not None and (cols >= 256 or (cols & (cols - 1)) == 0):
        y2 = empty_bf16((rows, cols), dev)
        r.hd_rmsnorm(pkg.ptr(dv(x, dev)), pkg.ptr(dv(w, dev)), pkg.ptr(y2), rows, cols, 1e-6)
        torch.cuda.synchronize()
        assert_close(y, y2, "B", "rmsnorm vs reference CUDA")


@pytest.mark.parametrize("n", [1, 8, 1000, 4096 * 33 + 5])
def test_pointwise(pkg, orc, dev, n):
    a, b = seeded_bf16(n, 3, 0.0, 3.0), seeded_bf16(n, 4)
    ad, bd, y = dv(a, dev), dv(b, dev), empty_bf16(n, dev)
    ref = np.empty_like(a)
    r = parity.reflib()
    for name, fn, ofn, two in (("silu", pkg.lib.hd_silu, orc.orc_silu, False),
                               ("swiglu", pkg.lib.hd_swiglu, orc.orc_swiglu, True),
                               ("residual_add", pkg.lib.hd_residual_add, orc.orc_residual_add, True)):
        if two:
            fn(pkg.ptr(ad), pkg.ptr(bd), pkg.ptr(y), n)
            ofn(np_ptr(a), np_ptr(b), np_ptr(ref), n)
        else:
            fn(pkg.ptr(ad), pkg.ptr(y), n)
            ofn(np_ptr(a), np_ptr(ref), n)
        done(pkg, name)
        got = torch_to_u16(y)
        if name == "residual_add":
            assert (got == ref).all()               # one fp32 add + RNE: exact
        else:
            assert_close(got, ref, "B", name)
            assert np.abs(got.astype(np.int32) - ref.astype(np.int32)).max() <= 1   # expf ulp only
        if r is not None:
            y2 = empty_bf16(n, dev)
            rfn = getattr(r, "hd_" + name)
            rfn(pkg.ptr(ad), pkg.ptr(bd), pkg.ptr(y2), n) if two else rfn(pkg.ptr(ad), pkg.ptr(y2), n)
            torch.cuda.synchronize()
            assert torch.equal(y.view(torch.int16), y2.view(torch.int16)), f"{name} vs reference CUDA"


LINEAR_SHAPES = [(7, 5, 6, True), (1, 4096, 256, True), (1, 4096, 4096, True), (23, 1024, 4096, False),
                 (300, 4096, 1024, True), (129, 3072, 4096, True), (1037, 4096, 4096, False),
                 (1280, 1024, 3072, False), (257, 4096, 12288, False)]


@pytest.mark.parametrize("M,N,K,bias", LINEAR_SHAPES)
def test_linear(pkg, orc, dev, M, N, K, bias):
    x, w = seeded_bf16((M, K), 5), seeded_bf16((N, K), 6, 0.0, 0.02)
    b = seeded_bf16(N, 7, 0.0, 0.5) if bias else None
    y = empty_bf16((M, N), dev)
    pkg.lib.hd_linear(pkg.ptr(dv(x, dev)), pkg.ptr(dv(w, dev)), pkg.ptr(dv(b, dev)) if bias else None,
                      pkg.ptr(y), M, N, K, 1)
    done(pkg, "linear")
    ref = np.empty((M, N), dtype=np.uint16)
    orc.orc_linear(np_ptr(x), np_ptr(w), np_ptr(b) if bias else None, np_ptr(ref), M, N, K)
    assert_close(torch_to_u16(y), ref, "C", "linear")
    r = parity.reflib()
    if r is not None and M * N * K <= 1037 * 4096 * 4096:
        y2 = empty_bf16((M, N), dev)
        r.hd_linear_reference(pkg.ptr(dv(x, dev)), pkg.ptr(dv(w, dev)), pkg.ptr(dv(b, dev)) if bias else None,
                              pkg.ptr(y2), M, N, K, 1)
        torch.cuda.synchronize()
        assert_close(y, y2, "C", "linear vs reference CUDA kernel")


def test_linear_rejects_untransposed(pkg, dev):
    x = empty_bf16((4, 4), dev)
    pkg.lib.hd_cuda_clear_error()
    pkg.lib.hd_linear(pkg.ptr(x), pkg.ptr(x), None, pkg.ptr(x), 4, 4, 4, 0)
    assert b"transpose_w=0 unsupported" in pkg.lib.hd_cuda_last_error()   # gemm.cu:511-514
    pkg.lib.hd_cuda_clear_error()


@pytest.mark.parametrize("epi", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_epilogues(pkg, orc, dev, epi, bn):
    """The fused epilogues keep the reference's rounding points: compare with the unfused oracle chain."""
    if epi == 3 and bn == 128:
        pytest.skip("SwiGLU tiles are 256 wide")
    M, N, K = 300, 512, 768
    x, w, w2 = seeded_bf16((M, K), 8), seeded_bf16((N, K), 9, 0, 0.03), seeded_bf16((N, K), 10, 0, 0.03)
    bias, resid = seeded_bf16(N, 11), seeded_bf16((M, N), 12)
    y = dv(resid, dev).clone() if epi == 4 else empty_bf16((M, N), dev)
    rc = pkg.lib.o1_gemm(pkg.ptr(dv(x, dev)), K, pkg.ptr(dv(w, dev)), pkg.ptr(dv(w2, dev)), pkg.ptr(y), N, M, N,
                         K, epi, pkg.ptr(dv(bias, dev)), pkg.ptr(dv(resid, dev)), N, 0.25, bn)
    assert rc == 0, pkg.last_error()
    done(pkg, "gemm")
    acc = np.empty((M, N), dtype=np.uint16)
    ref = np.empty((M, N), dtype=np.uint16)
    orc.orc_linear(np_ptr(x), np_ptr(w), None, np_ptr(acc), M, N, K)
    if epi == 0:
        ref = acc
    elif epi == 1:
        orc.orc_linear(np_ptr(x), np_ptr(w), np_ptr(bias), np_ptr(ref), M, N, K)
    elif epi == 2:
        orc.orc_residual_add(np_ptr(acc), np_ptr(resid), np_ptr(ref), M * N)
    elif epi == 3:
        up = np.empty((M, N), dtype=np.uint16)
        orc.orc_linear(np_ptr(x), np_ptr(w2), None, np_ptr(up), M, N, K)
        orc.orc_swiglu(np_ptr(acc), np_ptr(up), np_ptr(ref), M * N)
    else:
        accf = parity.bf16_to_f32_np(x).astype(np.float64) @ parity.bf16_to_f32_np(w).astype(np.float64).T
        ref = parity.f32_to_bf16_np((parity.bf16_to_f32_np(resid) + 0.25 * accf).astype(np.float32))
    assert_close(torch_to_u16(y), ref, "C", f"gemm epi {epi}")


def test_gemm_pitched_operands(pkg, orc, dev):
    """x and y as column slices of wider buffers (how the block writes q|k|v side by side)."""
    M, N, K, ldx, ldy = 200, 256, 128, 320, 640
    xb, w = seeded_bf16((M, ldx), 13), seeded_bf16((N, K), 14, 0, 0.05)
    yb = torch.zeros(M, ldy, dtype=torch.bfloat16, device=dev)
    xd = dv(xb, dev)
    rc = pkg.lib.o1_gemm(C.c_void_p(xd.data_ptr() + 64 * 2), ldx, pkg.ptr(dv(w, dev)), None,
                         C.c_void_p(yb.data_ptr() + 128 * 2), ldy, M, N, K, 0, None, None, 0, 0.0, 0)
    assert rc == 0, pkg.last_error()
    done(pkg, "gemm pitched")
    xs = np.ascontiguousarray(xb[:, 64:64 + K])
    ref = np.empty((M, N), dtype=np.uint16)
    orc.orc_linear(np_ptr(xs), np_ptr(w), None, np_ptr(ref), M, N, K)
    got = torch_to_u16(yb)
    assert_close(np.ascontiguousarray(got[:, 128:128 + N]), ref, "C", "pitched gemm")
    assert not got[:, :128].any() and not got[:, 128 + N:].any()


def test_timestep_and_mrope(pkg, orc, dev):
    t = np.array([500.0, 3.0], dtype=np.float32)
    y = torch.empty(2, 256, device=dev)
    pkg.lib.hd_timestep_embed(pkg.ptr(dv(t, dev)), pkg.ptr(y), 2, 256)
    done(pkg, "timestep_embed")
    ref = np.empty((2, 256), dtype=np.float32)
    orc.orc_timestep_embed(np_ptr(t), np_ptr(ref), 2, 256)
    # t*freq reaches 500 rad; one ulp of expf in freq moves the angle by ~3e-5
    assert np.abs(y.cpu().numpy() - ref).max() <= 1e-4
    assert_close(y.cpu().numpy(), ref, "B", "timestep_embed")
    S = 23 + 48
    pos, _ = pkg.seq_t2i(23, 6, 8)
    sec = torch.tensor([24, 20, 20], dtype=torch.int64, device=dev)
    cs, sn = torch.empty(S, 128, device=dev), torch.empty(S, 128, device=dev)
    pkg.lib.hd_mrope_cos_sin(pkg.ptr(pos.to(dev)), 1, S, pkg.ptr(sec), 3, 128, 5e6, 1.0, 1, pkg.ptr(cs), pkg.ptr(sn))
    done(pkg, "mrope")
    rc_, rs_ = np.empty((S, 128), dtype=np.float32), np.empty((S, 128), dtype=np.float32)
    secn = np.array([24, 20, 20], dtype=np.int64)
    orc.orc_mrope_cos_sin(np_ptr(pos.numpy()), 1, S, np_ptr(secn), 3, 128, 5e6, 1.0, 1, np_ptr(rc_), np_ptr(rs_))
    assert np.abs(cs.cpu().numpy() - rc_).max() <= 5e-4 and np.abs(sn.cpu().numpy() - rs_).max() <= 5e-4
    # the compact per-forward table holds the same 64 angles
    tab = torch.empty(S, 128, device=dev)
    assert pkg.lib.o1_mrope_table(pkg.ptr(pos.to(dev)), S, 5e6, pkg.ptr(tab)) == 0
    done(pkg, "mrope_table")
    assert torch.equal(tab[:, :64], cs[:, :64]) and torch.equal(tab[:, 64:], sn[:, :64])
    r = parity.reflib()
    if r is not None:
        c2, s2 = torch.empty(S, 128, device=dev), torch.empty(S, 128, device=dev)
        r.hd_mrope_cos_sin(pkg.ptr(pos.to(dev)), 1, S, pkg.ptr(sec), 3, 128, 5e6, 1.0, 1, pkg.ptr(c2), pkg.ptr(s2))
        torch.cuda.synchronize()
        assert torch.equal(cs, c2) and torch.equal(sn, s2), "mrope table vs reference CUDA (same expressions)"


def test_rotary_and_fused_qk_norm_rope(pkg, orc, dev):
    T, gh, gw, H = 9, 5, 7, 6
    S = T + gh * gw
    pos, _ = pkg.seq_t2i(T, gh, gw)
    secn = np.array([24, 20, 20], dtype=np.int64)
    cs, sn = np.empty((S, 128), dtype=np.float32), np.empty((S, 128), dtype=np.float32)
    orc.orc_mrope_cos_sin(np_ptr(pos.numpy()), 1, S, np_ptr(secn), 3, 128, 5e6, 1.0, 1, np_ptr(cs), np_ptr(sn))
    x = seeded_bf16((H, S, 128), 15)
    y = empty_bf16((H, S, 128), dev)
    pkg.lib.hd_apply_rotary(pkg.ptr(dv(x, dev)), pkg.ptr(dv(cs, dev)), pkg.ptr(dv(sn, dev)), pkg.ptr(y), H, S, 128)
    done(pkg, "rotary")
    ref = np.empty_like(x)
    orc.orc_apply_rotary(np_ptr(x), np_ptr(cs), np_ptr(sn), np_ptr(ref), H, S, 128)
    assert (torch_to_u16(y) == ref).all()          # same table, same three roundings: exact
    # fused: seq-major [S, ld] in place == head_split -> rmsnorm -> rotary of the oracle
    ld = H * 128 + 256
    buf = seeded_bf16((S, ld), 16)
    w = seeded_bf16(128, 17, 1.0, 0.1)
    tab = torch.empty(S, 128, device=dev)
    pkg.lib.o1_mrope_table(pkg.ptr(pos.to(dev)), S, 5e6, pkg.ptr(tab))
    bd = dv(buf, dev)
    assert pkg.lib.o1_qk_norm_rope(pkg.ptr(bd), ld, S, H, pkg.ptr(dv(w, dev)), pkg.ptr(tab), 1e-6) == 0
    done(pkg, "qk_norm_rope")
    xs = np.ascontiguousarray(buf[:, :H * 128])
    hm, nr, ro = (np.empty((H, S, 128), dtype=np.uint16) for _ in range(3))
    orc.orc_head_split(np_ptr(xs), np_ptr(hm), S, H, 128)
    orc.orc_rmsnorm(np_ptr(hm), np_ptr(w), np_ptr(nr), H * S, 128, 1e-6)
    tabn = tab.cpu().numpy()
    cs2 = np.concatenate([tabn[:, :64], tabn[:, :64]], 1).copy()
    sn2 = np.concatenate([tabn[:, 64:], tabn[:, 64:]], 1).copy()
    orc.orc_apply_rotary(np_ptr(nr), np_ptr(cs2), np_ptr(sn2), np_ptr(ro), H, S, 128)
    want = np.empty((S, H * 128), dtype=np.uint16)
    orc.orc_head_merge(np_ptr(ro), np_ptr(want), S, H, 128)
    got = torch_to_u16(bd)
    assert_close(np.ascontiguousarray(got[:, :H * 128]), want, "B", "fused q/k norm + rope")
    assert (got[:, H * 128:] == buf[:, H * 128:]).all()      # columns beyond the heads untouched


def test_exact_copies(pkg, orc, dev):
    S, H, D = 37, 5, 128
    x = seeded_bf16((S, H, D), 18)
    a, b = empty_bf16((H, S, D), dev), empty_bf16((S, H, D), dev)
    pkg.lib.hd_head_split(pkg.ptr(dv(x, dev)), pkg.ptr(a), S, H, D)
    pkg.lib.hd_head_merge(pkg.ptr(a), pkg.ptr(b), S, H, D)
    done(pkg, "head split/merge")
    ref = np.empty((H, S, D), dtype=np.uint16)
    orc.orc_head_split(np_ptr(x), np_ptr(ref), S, H, D)
    assert (torch_to_u16(a) == ref).all() and (torch_to_u16(b) == x).all()
    # gather (OOB -> row 0) and tms substitution (embed.cu:15-58)
    rows, cols = 50, 256
    table = seeded_bf16((rows, cols), 19)
    idx = np.array([3, 0, 49, 50, -1, 7, 151673], dtype=np.int64)
    out = empty_bf16((len(idx), cols), dev)
    pkg.lib.hd_gather_rows(pkg.ptr(dv(table, dev)), pkg.ptr(dv(idx, dev)), pkg.ptr(out), len(idx), cols, rows)
    done(pkg, "gather")
    want = table[np.where((idx < 0) | (idx >= rows), 0, idx)]
    assert (torch_to_u16(out) == want).all()
    temb = seeded_bf16(cols, 20)
    out2 = empty_bf16((len(idx), cols), dev)
    pkg.lib.hd_apply_tms_condition(pkg.ptr(dv(idx, dev)), pkg.ptr(out), pkg.ptr(dv(temb, dev)), pkg.ptr(out2),
                                   len(idx), cols, 151673)
    done(pkg, "tms")
    want2 = want.copy()
    want2[6] = temb
    assert (torch_to_u16(out2) == want2).all()
    # vision rows (vision_kernels.cu:344-401)
    mask = np.array([0, 1, 1, 0, 0, 1, 0], dtype=np.uint8)
    emb = seeded_bf16((3, cols), 21)
    o3, o4 = empty_bf16((7, cols), dev), empty_bf16((7, cols), dev)
    pkg.lib.hd_vision_masked_scatter(pkg.ptr(out), pkg.ptr(dv(mask, dev)), pkg.ptr(dv(emb, dev)), pkg.ptr(o3), 7, cols)
    pkg.lib.hd_vision_deepstack_inject(pkg.ptr(out), pkg.ptr(dv(mask, dev)), pkg.ptr(dv(emb, dev)), pkg.ptr(o4), 7, cols)
    done(pkg, "vision rows")
    w3, w4 = want.copy(), want.copy()
    for k, r_ in enumerate(np.nonzero(mask)[0]):
        w3[r_] = emb[k]
        w4[r_] = parity.f32_to_bf16_np(parity.bf16_to_f32_np(want[r_]) + parity.bf16_to_f32_np(emb[k]))
    assert (torch_to_u16(o3) == w3).all() and (torch_to_u16(o4) == w4).all()


@pytest.mark.parametrize("n", [1, 7, 3072 * 64, 3072 * 64 + 3])
def test_scheduler_kernels(pkg, orc, dev, n):
    z, xc, xu = seeded_bf16(n, 22, 0, 4.0), seeded_bf16(n, 23), seeded_bf16(n, 24)
    sigma, sigma_next, g = 0.8769999742507935, 0.8569999933242798, 5.0
    zd, cd, ud = dv(z, dev), dv(xc, dev), dv(xu, dev)
    mc, mu, mo = (torch.empty(n, device=dev) for _ in range(3))
    zn = empty_bf16(n, dev)
    lib = pkg.lib
    lib.hd_sched_vcond(pkg.ptr(zd), pkg.ptr(cd), sigma, pkg.ptr(mc), n)
    lib.hd_sched_vcond(pkg.ptr(zd), pkg.ptr(ud), sigma, pkg.ptr(mu), n)
    lib.hd_sched_cfg_guided(pkg.ptr(mc), pkg.ptr(mu), g, pkg.ptr(mo), n)
    lib.hd_sched_flow_match_step(pkg.ptr(zd), pkg.ptr(mo), sigma, sigma_next, pkg.ptr(zn), n)
    fused = empty_bf16(n, dev)
    assert lib.o1_sched_cfg_flow_step(pkg.ptr(zd), pkg.ptr(cd), pkg.ptr(ud), sigma, sigma_next, g, pkg.ptr(fused), n) == 0
    done(pkg, "scheduler")
    assert torch.equal(zn.view(torch.int16), fused.view(torch.int16)), "fused step != unfused chain"
    omc, omu, omo = (np.empty(n, dtype=np.float32) for _ in range(3))
    ozn, ofz = np.empty(n, dtype=np.uint16), np.empty(n, dtype=np.uint16)
    orc.orc_sched_vcond(np_ptr(z), np_ptr(xc), sigma, np_ptr(omc), n)
    orc.orc_sched_vcond(np_ptr(z), np_ptr(xu), sigma, np_ptr(omu), n)
    orc.orc_sched_cfg_guided(np_ptr(omc), np_ptr(omu), g, np_ptr(omo), n)
    orc.orc_sched_flow_match_step(np_ptr(z), np_ptr(omo), sigma, sigma_next, np_ptr(ozn), n)
    orc.orc_sched_cfg_flow_step(np_ptr(z), np_ptr(xc), np_ptr(xu), sigma, sigma_next, g, np_ptr(ofz), n)
    assert (ozn == ofz).all()
    assert (mc.cpu().numpy() == omc).all()                      # one IEEE subtract and divide
    assert np.abs(mo.cpu().numpy() - omo).max() <= 4e-6 * max(1.0, float(np.abs(omo).max()))
    assert np.abs(torch_to_u16(zn).astype(np.int32) - ozn.astype(np.int32)).max() <= 1
    assert_close(torch_to_u16(zn), ozn, "B", "flow-match step")
    r = parity.reflib()
    if r is not None:
        m1, m2, m3 = (torch.empty(n, device=dev) for _ in range(3))
        z2 = empty_bf16(n, dev)
        r.hd_sched_vcond(pkg.ptr(zd), pkg.ptr(cd), sigma, pkg.ptr(m1), n)
        r.hd_sched_vcond(pkg.ptr(zd), pkg.ptr(ud), sigma, pkg.ptr(m2), n)
        r.hd_sched_cfg_guided(pkg.ptr(m1), pkg.ptr(m2), g, pkg.ptr(m3), n)
        r.hd_sched_flow_match_step(pkg.ptr(zd), pkg.ptr(m3), sigma, sigma_next, pkg.ptr(z2), n)
        torch.cuda.synchronize()
        assert torch.equal(mo, m3) and torch.equal(zn.view(torch.int16), z2.view(torch.int16)), \
            "scheduler chain vs reference CUDA kernels"
        assert torch.equal(fused.view(torch.int16), z2.view(torch.int16)), "fused step vs reference CUDA chain"


def test_flash_euler_and_unipc_kernels(pkg, orc, dev):
    n = 5000
    rng = np.random.default_rng(0)
    zf, mo, noise, old, conv = (rng.standard_normal(n).astype(np.float32) for _ in range(5))
    lib = pkg.lib
    den, zn = torch.empty(n, device=dev), torch.empty(n, device=dev)
    lib.hd_sched_denoised(pkg.ptr(dv(zf, dev)), pkg.ptr(dv(mo, dev)), 0.9, pkg.ptr(den), n)
    lib.hd_sched_z_next(pkg.ptr(dv(noise, dev)), pkg.ptr(den), 0.8, 8.0, pkg.ptr(zn), n)
    up = torch.empty(n, device=dev)
    zb = parity.f32_to_bf16_np(zf)
    lib.hd_sched_bf16_upcast(pkg.ptr(dv(zb, dev)), pkg.ptr(up), n)
    done(pkg, "flash euler")
    oden, ozn = np.empty(n, dtype=np.float32), np.empty(n, dtype=np.float32)
    orc.orc_sched_denoised(np_ptr(zf), np_ptr(mo), 0.9, np_ptr(oden), n)
    orc.orc_sched_z_next(np_ptr(noise), np_ptr(oden), 0.8, 8.0, np_ptr(ozn), n)
    assert np.abs(den.cpu().numpy() - oden).max() <= 1e-6 and np.abs(zn.cpu().numpy() - ozn).max() <= 4e-6
    assert (up.cpu().numpy() == parity.bf16_to_f32_np(zb)).all()
    c = (0.8, 0.9, 0.2, -0.11, 0.12, 0.4, 0.5, 1.3)
    out, oout = torch.empty(n, device=dev), np.empty(n, dtype=np.float32)
    for order in (1, 2):
        lib.hd_unipc_correct(pkg.ptr(dv(zf, dev)), pkg.ptr(dv(mo, dev)), pkg.ptr(dv(old, dev)), pkg.ptr(dv(conv, dev)),
                             *c, order, pkg.ptr(out), n)
        done(pkg, "unipc_correct")
        orc.orc_unipc_correct(np_ptr(zf), np_ptr(mo), np_ptr(old), np_ptr(conv), *c, order, np_ptr(oout), n)
        assert np.abs(out.cpu().numpy() - oout).max() <= 1e-5      # tests/unit/test_base_unipc_cuda.c:155
        lib.hd_unipc_predict(pkg.ptr(dv(zf, dev)), pkg.ptr(dv(mo, dev)), pkg.ptr(dv(old, dev)), c[0], c[1], c[2],
                             c[3], c[4], c[6], c[7], order, pkg.ptr(out), n)
        done(pkg, "unipc_predict")
        orc.orc_unipc_predict(np_ptr(zf), np_ptr(mo), np_ptr(old), c[0], c[1], c[2], c[3], c[4], c[6], c[7],
                              order, np_ptr(oout), n)
        assert np.abs(out.cpu().numpy() - oout).max() <= 1e-5
    lib.hd_unipc_convert(pkg.ptr(dv(zf, dev)), pkg.ptr(dv(mo, dev)), 0.7, pkg.ptr(out), n)
    done(pkg, "unipc_convert")
    orc.orc_unipc_convert(np_ptr(zf), np_ptr(mo), 0.7, np_ptr(oout), n)
    assert np.abs(out.cpu().numpy() - oout).max() <= 1e-6


def test_seeded_fill_is_bit_identical_on_host_and_device(pkg, orc, dev):
    n = 100003
    d16 = empty_bf16(n, dev)
    d32 = torch.empty(n, device=dev)
    assert pkg.lib.o1_fill_normal_bf16(pkg.ptr(d16), n, 99, 1.0, 0.02) == 0
    assert pkg.lib.o1_fill_normal_f32(pkg.ptr(d32), n, 99, 0.0, 1.0) == 0
    done(pkg, "fill")
    h16, h32 = np.empty(n, dtype=np.uint16), np.empty(n, dtype=np.float32)
    orc.orc_fill_normal_bf16(np_ptr(h16), n, 99, 1.0, 0.02)
    orc.orc_fill_normal_f32(np_ptr(h32), n, 99, 0.0, 1.0)
    assert (torch_to_u16(d16) == h16).all()
    assert (d32.cpu().numpy().view(np.uint32) == h32.view(np.uint32)).all()


@pytest.mark.parametrize("M,N,K,ldy,bn", [(300, 512, 256, 512 + 384, 0), (1024, 1024, 512, 1024, 256), (130, 256, 128, 256, 128)])
def test_projection_with_norm_and_rope_in_the_epilogue(pkg, dev, M, N, K, ldy, bn):
    """GEMM whose epilogue applies the per-head RMSNorm + rotary (epilogue 6) == plain GEMM followed by the
    in-place norm + rope kernel, bit for bit; columns of the output row beyond the projection stay untouched."""
    heads = N // 128
    x = dv(seeded_bf16((M, K), 71), dev)
    w = dv(seeded_bf16((N, K), 72, 0.0, 0.05), dev)
    nw = dv(seeded_bf16(128, 73, 1.0, 0.1), dev)
    pos, _ = pkg.seq_t2i(20, 10, (M - 20 + 9) // 10)
    tab = torch.empty(pos.shape[1], 128, device=dev)
    pkg.lib.o1_mrope_table(pkg.ptr(pos.to(dev)), pos.shape[1], 5e6, pkg.ptr(tab))
    assert pos.shape[1] >= M
    fill = seeded_bf16((M, ldy), 74)
    y_fused, y_plain = dv(fill, dev), dv(fill, dev)
    rc = pkg.lib.o1_gemm(pkg.ptr(x), K, pkg.ptr(w), None, pkg.ptr(y_fused), ldy, M, N, K, 6, pkg.ptr(nw), pkg.ptr(tab),
                         0, 1e-6, bn)
    assert rc == 0, pkg.last_error()
    rc = pkg.lib.o1_gemm(pkg.ptr(x), K, pkg.ptr(w), None, pkg.ptr(y_plain), ldy, M, N, K, 0, None, None, 0, 0.0, bn)
    assert rc == 0, pkg.last_error()
    assert pkg.lib.o1_qk_norm_rope(pkg.ptr(y_plain), ldy, M, heads, pkg.ptr(nw), pkg.ptr(tab), 1e-6) == 0
    done(pkg, "gemm + norm + rope")
    assert torch.equal(y_fused.view(torch.int16), y_plain.view(torch.int16))
    assert (torch_to_u16(y_fused)[:, N:] == fill[:, N:]).all()
    # shapes the tensor-core tiles do not cover refuse the fused epilogue instead of falling back silently
    assert pkg.lib.o1_gemm(pkg.ptr(x), K, pkg.ptr(w), None, pkg.ptr(y_fused), ldy, 4, N, K, 6, pkg.ptr(nw), pkg.ptr(tab),
                           0, 1e-6, 0) != 0


@pytest.mark.parametrize("M,qc,kc,K", [(300, 512, 128, 256), (1280, 4096, 1024, 4096), (4115, 1024, 256, 512)])
def test_qkv_projections_as_one_launch(pkg, dev, M, qc, kc, K):
    """o1_gemm_qkv (one launch over the three weight tensors, norm + rope on the q and k tiles) == three separate
    projections with the same epilogues, bit for bit; the row pitch may exceed the used columns."""
    ld = qc + 2 * kc + 128
    x = dv(seeded_bf16((M, K), 81), dev)
    wq, wk, wv = (dv(seeded_bf16((n, K), 82 + i, 0.0, 0.05), dev) for i, n in enumerate((qc, kc, kc)))
    nq, nk = dv(seeded_bf16(128, 86, 1.0, 0.1), dev), dv(seeded_bf16(128, 87, 1.0, 0.1), dev)
    pos, _ = pkg.seq_t2i(20, 10, (M - 20 + 9) // 10)
    tab = torch.empty(pos.shape[1], 128, device=dev)
    pkg.lib.o1_mrope_table(pkg.ptr(pos.to(dev)), pos.shape[1], 5e6, pkg.ptr(tab))
    fill = seeded_bf16((M, ld), 88)
    one, three = dv(fill, dev), dv(fill, dev)
    rc = pkg.lib.o1_gemm_qkv(pkg.ptr(x), K, pkg.ptr(wq), pkg.ptr(wk), pkg.ptr(wv), pkg.ptr(one), ld, M, qc, kc, K,
                             pkg.ptr(nq), pkg.ptr(nk), pkg.ptr(tab), 1e-6)
    assert rc == 0, pkg.last_error()
    P = lambda t, off: C.c_void_p(t.data_ptr() + off * 2)
    assert pkg.lib.o1_gemm(pkg.ptr(x), K, pkg.ptr(wq), None, P(three, 0), ld, M, qc, K, 6, pkg.ptr(nq), pkg.ptr(tab), 0, 1e-6, 0) == 0
    assert pkg.lib.o1_gemm(pkg.ptr(x), K, pkg.ptr(wk), None, P(three, qc), ld, M, kc, K, 6, pkg.ptr(nk), pkg.ptr(tab), 0, 1e-6, 0) == 0
    assert pkg.lib.o1_gemm(pkg.ptr(x), K, pkg.ptr(wv), None, P(three, qc + kc), ld, M, kc, K, 0, None, None, 0, 0.0, 0) == 0
    done(pkg, "qkv")
    assert torch.equal(one.view(torch.int16), three.view(torch.int16))
    assert (torch_to_u16(one)[:, qc + 2 * kc:] == fill[:, qc + 2 * kc:]).all()


@pytest.mark.parametrize("M,N,K,epi", [(4352, 4096, 512, 0), (4115, 4096, 256, 2), (4200, 3072, 320, 1), (8320, 4096, 192, 2)])
def test_gemm_on_cta_pairs_equals_single_cta_tiles(pkg, dev, M, N, K, epi):
    """The cta_group::2 form (two CTAs per 256 x 256 tile, each with half of the B tile) adds a row's K products in the
    same order as the one-CTA form: same bits, for an even and an odd number of row tiles, a partly filled last row
    tile and a ragged last K block, with the epilogues that take the pair form (plain, +bias, +residual)."""
    x = dv(seeded_bf16((M, K), 91), dev)
    w = dv(seeded_bf16((N, K), 92, 0.0, 0.05), dev)
    bias = dv(seeded_bf16(N, 93, 0.0, 0.5), dev) if epi == 1 else None
    resid = dv(seeded_bf16((M, N), 94), dev) if epi == 2 else None
    outs = []
    try:
        for mode in (0, 1):
            pkg.lib.o1_gemm_pair_mode(mode)
            y = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
            rc = pkg.lib.o1_gemm(pkg.ptr(x), K, pkg.ptr(w), None, pkg.ptr(y), N, M, N, K, epi,
                                 pkg.ptr(bias) if bias is not None else None,
                                 pkg.ptr(resid) if resid is not None else None, N, 0.0, 0)
            assert rc == 0, pkg.last_error()
            done(pkg, "gemm pair mode %d" % mode)
            outs.append(y)
    finally:
        pkg.lib.o1_gemm_pair_mode(1)
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    ref = x.float() @ w.float().t()
    if epi == 1: ref = (ref.bfloat16().float() + bias.float())
    if epi == 2: ref = (ref.bfloat16().float() + resid.float())
    err = (outs[1].float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)
    assert err < 1e-2, err     # the pair form really computed the product (fp32 reference, bf16 rounding of the result)
