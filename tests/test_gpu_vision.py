"""GPU parity of the vision tower (hd_vision_* of o1.c src/model/vision.h, src/cuda/vision_kernels.h) through the
C ABI: the stand-alone kernels and the ragged-edge GEMM shapes against the CPU oracle, the whole tower against the
oracle and -- when oracle/_ref holds it -- against the reference's own CUDA build of hd_vision_forward on the same
seeded weights and pixels.  Tolerances: pointwise B, GEMM C, one block D, whole tower V (tests/parity.py)."""
import ctypes as C

import numpy as np
import pytest
import torch

import parity
from parity import np_ptr, seeded_bf16, torch_to_u16, u16_to_torch, assert_close, metrics

pytestmark = pytest.mark.gpu

_KEEP = []


@pytest.fixture(autouse=True)
def _release_device_temporaries():
    yield
    _KEEP.clear()


def dv(a, dev):
    t = u16_to_torch(a, dev) if a.dtype == np.uint16 else torch.from_numpy(a).to(dev)
    _KEEP.append(t)
    return t


def empty_bf16(shape, dev):
    return torch.empty(shape, dtype=torch.bfloat16, device=dev)


def done(pkg, what):
    torch.cuda.synchronize()
    pkg.check_cuda_errbuf(what)


# ------------------------------------------------------------------ GEMM shapes of the tower
@pytest.mark.parametrize("M,N,K,bias", [
    (520, 4304, 1152, True),     # fc1: ragged right tile edge (4304 = 33 * 128 + 80)
    (520, 1152, 4304, True),     # fc2: ragged last K block (4304 = 67 * 64 + 16)
    (96, 3456, 1152, True),      # qkv
    (130, 4096, 4608, True),     # merger fc2
    (200, 4304, 4304, False),    # both edges ragged, no bias
    (9, 72, 40, True),           # smaller than one tile in every dimension
])
def test_linear_ragged_edges(pkg, orc, dev, M, N, K, bias):
    x, w = seeded_bf16((M, K), 11), seeded_bf16((N, K), 12, 0.0, 0.05)
    b = seeded_bf16(N, 13, 0.0, 0.5) if bias else None
    # canaries behind the output catch a store beyond column N or row M
    y = torch.full((M + 2, N), 777.0, dtype=torch.bfloat16, device=dev)
    pkg.lib.hd_linear(pkg.ptr(dv(x, dev)), pkg.ptr(dv(w, dev)), pkg.ptr(dv(b, dev)) if bias else None, pkg.ptr(y),
                      M, N, K, 1)
    done(pkg, "linear")
    ref = np.empty((M, N), dtype=np.uint16)
    orc.orc_linear(np_ptr(x), np_ptr(w), np_ptr(b) if bias else None, np_ptr(ref), M, N, K)
    assert_close(torch_to_u16(y[:M]), ref, "C", f"linear {M}x{N}x{K}")
    assert (y[M:] == 777.0).all(), "rows beyond M were written"


@pytest.mark.parametrize("exact", [0, 1])
def test_gemm_bias_gelu_epilogue(pkg, orc, dev, exact):
    M, N, K = 300, 4304, 1152
    x, w, b = seeded_bf16((M, K), 21), seeded_bf16((N, K), 22, 0.0, 0.05), seeded_bf16(N, 23, 0.0, 0.5)
    y = empty_bf16((M, N), dev)
    rc = pkg.lib.o1_gemm(pkg.ptr(dv(x, dev)), K, pkg.ptr(dv(w, dev)), None, pkg.ptr(y), N, M, N, K, pkg.EPI_BIAS_GELU,
                         pkg.ptr(dv(b, dev)), None, 0, float(exact), 0)
    assert rc == 0, pkg.last_error()
    done(pkg, "gemm+gelu")
    ref = np.empty((M, N), dtype=np.uint16)
    orc.orc_linear(np_ptr(x), np_ptr(w), np_ptr(b), np_ptr(ref), M, N, K)
    orc.orc_gelu(np_ptr(ref), np_ptr(ref), ref.size, exact)
    assert_close(torch_to_u16(y), ref, "C", "gemm + bias + gelu")


@pytest.mark.parametrize("M,N,K", [(520, 1152, 4304), (300, 1152, 1152)])
def test_gemm_bias_residual_epilogue(pkg, orc, dev, M, N, K):
    x, w, b = seeded_bf16((M, K), 24), seeded_bf16((N, K), 25, 0.0, 0.05), seeded_bf16(N, 26, 0.0, 0.5)
    res = seeded_bf16((M, N), 27)
    y = empty_bf16((M, N), dev)
    rc = pkg.lib.o1_gemm(pkg.ptr(dv(x, dev)), K, pkg.ptr(dv(w, dev)), None, pkg.ptr(y), N, M, N, K, pkg.EPI_BIAS_RESID,
                         pkg.ptr(dv(b, dev)), pkg.ptr(dv(res, dev)), N, 0.0, 0)
    assert rc == 0, pkg.last_error()
    done(pkg, "gemm+bias+residual")
    ref = np.empty((M, N), dtype=np.uint16)
    orc.orc_linear(np_ptr(x), np_ptr(w), np_ptr(b), np_ptr(ref), M, N, K)
    orc.orc_residual_add(np_ptr(res), np_ptr(ref), np_ptr(ref), ref.size)
    assert_close(torch_to_u16(y), ref, "C", "gemm + bias + residual")


# ------------------------------------------------------------------ stand-alone kernels
@pytest.mark.parametrize("rows,cols", [(520, 1152), (130, 4608), (7, 96), (3, 100)])
def test_layernorm(pkg, orc, dev, rows, cols):
    x, w, b = seeded_bf16((rows, cols), 3, 0.3, 1.5), seeded_bf16(cols, 4, 1.0, 0.1), seeded_bf16(cols, 5, 0.0, 0.1)
    y = empty_bf16((rows, cols), dev)
    pkg.lib.hd_vision_layernorm(pkg.ptr(dv(x, dev)), pkg.ptr(dv(w, dev)), pkg.ptr(dv(b, dev)), pkg.ptr(y), rows, cols, 1e-6)
    done(pkg, "layernorm")
    ref = np.empty_like(x)
    orc.orc_layernorm(np_ptr(x), np_ptr(w), np_ptr(b), np_ptr(ref), rows, cols, 1e-6)
    assert_close(torch_to_u16(y), ref, "B", "layernorm")
    r = parity.reflib()
    if r is not None and hasattr(r, "hd_vision_layernorm"):
        y2 = empty_bf16((rows, cols), dev)
        r.hd_vision_layernorm(pkg.ptr(dv(x, dev)), pkg.ptr(dv(w, dev)), pkg.ptr(dv(b, dev)), pkg.ptr(y2), rows, cols, 1e-6)
        torch.cuda.synchronize()
        assert_close(y, y2, "B", "layernorm vs reference CUDA")


def test_gelu_both_forms(pkg, orc, dev):
    x = parity.f32_to_bf16_np(np.linspace(-8, 8, 100003, dtype=np.float32))
    for exact, fn in ((0, "hd_vision_gelu"), (1, "hd_vision_gelu_exact")):
        y = empty_bf16(x.shape, dev)
        getattr(pkg.lib, fn)(pkg.ptr(dv(x, dev)), pkg.ptr(y), x.size)
        done(pkg, fn)
        ref = np.empty_like(x)
        orc.orc_gelu(np_ptr(x), np_ptr(ref), x.size, exact)
        assert_close(torch_to_u16(y), ref, "B", fn)
        r = parity.reflib()
        if r is not None and hasattr(r, fn):
            y2 = empty_bf16(x.shape, dev)
            getattr(r, fn)(pkg.ptr(dv(x, dev)), pkg.ptr(y2), x.size)
            torch.cuda.synchronize()
            assert (torch_to_u16(y) == torch_to_u16(y2)).mean() > 0.999, fn + " vs reference CUDA"


def test_tables_interp_and_rotary(pkg, orc, dev):
    gh, gw, H = 26, 20, 1152
    n = gh * gw
    idx, wgt = np.empty((4, n), np.int32), np.empty((4, n), np.float32)
    coords, inv = np.empty((2, n), np.int32), np.empty(18, np.float32)
    orc.orc_vision_tables(gh, gw, np_ptr(idx), np_ptr(wgt), np_ptr(coords), np_ptr(inv))
    # hd_vision_prepare_tables builds the same tables on the host and uploads them
    ws = pkg.VisionWorkspace()
    tables = torch.zeros(pkg.lib.hd_vision_tables_bytes(n), dtype=torch.uint8, device=dev)
    ws.tables, ws.tables_n = tables.data_ptr(), -1
    pkg.check(pkg.lib.hd_vision_prepare_tables(C.byref(ws), n, gh, gw), "prepare_tables")
    raw = tables.cpu().numpy()
    assert (raw[:16 * n].view(np.int32).reshape(4, n) == idx).all()
    assert (raw[16 * n:32 * n].view(np.float32).reshape(4, n) == wgt).all()
    assert (raw[32 * n:40 * n].view(np.int32).reshape(2, n) == coords).all()
    assert (raw[40 * n:40 * n + 72].view(np.float32) == inv).all()
    assert pkg.lib.hd_vision_prepare_tables(C.byref(ws), n, gh, gw) == 0          # same shape: nothing to do
    assert pkg.lib.hd_vision_prepare_tables(C.byref(ws), n, 13, 40) != 0          # odd grid is refused
    # interpolation
    pe = seeded_bf16((2304, H), 31, 0.0, 0.02)
    y = empty_bf16((n, H), dev)
    pkg.lib.hd_vision_pos_interp(pkg.ptr(dv(pe, dev)), C.c_void_p(ws.pos_idx), C.c_void_p(ws.pos_wgt), pkg.ptr(y), n, H)
    done(pkg, "pos_interp")
    pf = parity.bf16_to_f32_np(pe)
    ref = sum(wgt[k][:, None] * pf[idx[k]] for k in range(4))
    assert_close(torch_to_u16(y), ref.astype(np.float32), "B", "pos_interp")
    # rotary angles and tables
    rot = empty_bf16((n, 36), dev)
    cs, sn = torch.empty((n, 72), device=dev), torch.empty((n, 72), device=dev)
    pkg.lib.hd_vision_rot(C.c_void_p(ws.rot_inv), C.c_void_p(ws.rot_coords), pkg.ptr(rot), n, 18)
    pkg.lib.hd_vision_rot_cos_sin(pkg.ptr(rot), pkg.ptr(cs), pkg.ptr(sn), n, 18)
    done(pkg, "rot")
    ang = np.concatenate([coords[0][:, None] * inv[None], coords[1][:, None] * inv[None]], 1).astype(np.float32)
    ang16 = parity.f32_to_bf16_np(ang)
    assert (torch_to_u16(rot) == ang16).all()
    a = parity.bf16_to_f32_np(ang16).astype(np.float64)
    np.testing.assert_allclose(cs.cpu().numpy(), np.tile(np.cos(a), 2), atol=2e-6)
    np.testing.assert_allclose(sn.cpu().numpy(), np.tile(np.sin(a), 2), atol=2e-6)


def test_layout_kernels_are_index_maps(pkg, dev):
    n, heads, d = 37, 16, 72
    qkv = seeded_bf16((n, 3, heads, d), 41)
    q, k, v = (empty_bf16((heads, n, d), dev) for _ in range(3))
    pkg.lib.hd_vision_qkv_split(pkg.ptr(dv(qkv, dev)), pkg.ptr(q), pkg.ptr(k), pkg.ptr(v), n, heads, d)
    done(pkg, "qkv_split")
    for got, which in ((q, 0), (k, 1), (v, 2)):
        assert (torch_to_u16(got) == qkv[:, which].transpose(1, 0, 2)).all()
    sm = empty_bf16((n, heads * d), dev)
    pkg.lib.hd_vision_attn_merge(pkg.ptr(q), pkg.ptr(sm), heads, n, d)
    done(pkg, "attn_merge")
    assert (torch_to_u16(sm).reshape(n, heads, d) == qkv[:, 0]).all()
    gh, gw, hid = 6, 8, 1152
    grid = seeded_bf16((gh, gw, hid), 42)
    out = empty_bf16((gh // 2 * gw // 2, 4 * hid), dev)
    pkg.lib.hd_vision_spatial_merge(pkg.ptr(dv(grid, dev)), pkg.ptr(out), gh, gw, hid)
    done(pkg, "spatial_merge")
    ref = grid.reshape(gh // 2, 2, gw // 2, 2, hid).transpose(0, 2, 1, 3, 4).reshape(-1, 4 * hid)
    assert (torch_to_u16(out) == ref).all()


# ------------------------------------------------------------------ whole tower
@pytest.fixture(scope="module")
def tower(pkg, dev):
    vw = parity.VisionHostWeights()
    dev_w = [u16_to_torch(a, dev) for a in vw.arrays]
    binding = pkg.VisionBinding(*[t.data_ptr() for t in dev_w])
    return vw, dev_w, binding


def run_tower(pkg, dev, binding, px, gh, gw, lib=None, snaps=True):
    """hd_vision_forward of `lib` (this library by default): image_embeds, deepstack, block outputs 0 / 8 / 26."""
    lib = lib or pkg.lib
    n, m = gh * gw, gh * gw // 4
    ws = pkg.VisionWorkspace()
    space = torch.zeros(lib.hd_vision_workspace_bytes(n), dtype=torch.uint8, device=dev)
    tables = torch.zeros(lib.hd_vision_tables_bytes(n), dtype=torch.uint8, device=dev)
    ws.patch_out, ws.tables, ws.tables_n = space.data_ptr(), tables.data_ptr(), -1
    outs = {i: empty_bf16((n, 1152), dev) for i in ((0, 8, 26) if snaps else ())}
    for i, t in outs.items():
        ws.block_out_snaps[i] = t.data_ptr()
    rc = lib.hd_vision_prepare_tables(C.byref(ws), n, gh, gw)
    assert rc == 0, lib.hd_last_error()
    emb, ds = empty_bf16((m, 4096), dev), empty_bf16((3, m, 4096), dev)
    dsp = (C.c_void_p * 3)(*[ds[j].data_ptr() for j in range(3)])
    pxd = u16_to_torch(px, dev)
    rc = lib.hd_vision_forward(C.byref(binding), C.byref(ws), C.c_void_p(pxd.data_ptr()), n, gh, gw,
                               C.c_void_p(emb.data_ptr()), C.byref(dsp))
    assert rc == 0, lib.hd_last_error()
    torch.cuda.synchronize()
    err = lib.hd_cuda_last_error()
    assert not err, err
    return emb, ds, outs


@pytest.mark.parametrize("gh,gw", [(8, 12), (26, 20), (2, 2)])
def test_tower_against_oracle(pkg, orc, dev, tower, gh, gw):
    vw, _, binding = tower
    px = seeded_bf16((gh * gw, 1536), 7)
    emb, ds, outs = run_tower(pkg, dev, binding, px, gh, gw)
    emb_o, ds_o, blocks_o = parity.oracle_vision(vw, px, gh, gw, want_blocks=True)
    assert_close(torch_to_u16(outs[0]), blocks_o[0], "D", "block 0 output")
    assert_close(torch_to_u16(outs[8]), blocks_o[8], "E", "block 8 output")
    assert_close(torch_to_u16(outs[26]), blocks_o[26], "V", "block 26 output")
    assert_close(torch_to_u16(ds), ds_o, "V", "deepstack")
    assert_close(torch_to_u16(emb), emb_o, "V", "image_embeds")
    print("tower vs oracle %dx%d:" % (gh, gw), "b0", metrics(outs[0], blocks_o[0])[:2], "b26", metrics(outs[26], blocks_o[26])[:2],
          "emb", metrics(emb, emb_o)[:2])
    # the forward is deterministic and leaves nothing behind that a second call depends on
    emb2, ds2, _ = run_tower(pkg, dev, binding, px, gh, gw, snaps=False)
    assert torch.equal(emb, emb2) and torch.equal(ds, ds2)


def test_tower_against_reference_cuda_build(pkg, dev, tower):
    r = parity.reflib()
    if r is None or not hasattr(r, "hd_vision_forward"):
        pytest.skip("oracle/_ref/libo1ref.so (with src/model/vision.c) not built")
    _, _, binding = tower
    gh, gw = 26, 20
    px = seeded_bf16((gh * gw, 1536), 7)
    # pure-source reference path: hd_linear_reference (gemm.cu:35-90) + eager attention (sdpa = NULL), so every
    # arithmetic step of the comparison is the reference's own source
    r.hd_gemm_set_backend(0)
    emb_r, ds_r, outs_r = run_tower(pkg, dev, binding, px, gh, gw, lib=r)
    emb, ds, outs = run_tower(pkg, dev, binding, px, gh, gw)
    assert_close(outs[0], outs_r[0], "D", "block 0 output vs reference")
    assert_close(outs[8], outs_r[8], "E", "block 8 output vs reference")
    assert_close(outs[26], outs_r[26], "V", "block 26 output vs reference")
    assert_close(ds, ds_r, "V", "deepstack vs reference")
    assert_close(emb, emb_r, "V", "image_embeds vs reference")
    print("tower vs reference CUDA build: b0", metrics(outs[0], outs_r[0])[:2], "b26", metrics(outs[26], outs_r[26])[:2],
          "emb", metrics(emb, emb_r)[:2])


def test_forward_rejects_bad_arguments(pkg, dev, tower):
    _, _, binding = tower
    ws = pkg.VisionWorkspace()
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device=dev)
    ws.patch_out = buf.data_ptr()
    out = empty_bf16((4, 4096), dev)
    # tables not prepared
    assert pkg.lib.hd_vision_forward(C.byref(binding), C.byref(ws), pkg.ptr(buf), 16, 4, 4, pkg.ptr(out), None) != 0
    assert b"tables" in pkg.lib.hd_last_error()
    # odd grid
    assert pkg.lib.hd_vision_forward(C.byref(binding), C.byref(ws), pkg.ptr(buf), 15, 3, 5, pkg.ptr(out), None) != 0
    assert pkg.lib.hd_vision_forward(None, C.byref(ws), pkg.ptr(buf), 16, 4, 4, pkg.ptr(out), None) != 0


def test_edit_pipeline_tower_into_forward(pkg, orc, dev, tower):
    """The edit path end to end (o1.c src/runtime/generate.c:435-640 then hd_forward): one conditioning image goes
    through the vision tower, its image_embeds replace the <image_pad> rows of the text and the DeepStack tensors are
    added after decoder blocks 0..2; the target grid and one reference grid follow.  GPU pipeline against the oracle
    pipeline (orc_vision_forward -> orc_forward_visual)."""
    vw, _, binding = tower
    ch, cw = 4, 6                                           # merged vision tokens: 24 <image_pad> rows
    px = seeded_bf16((4 * ch * cw, 1536), 17)
    emb, ds, _ = run_tower(pkg, dev, binding, px, 2 * ch, 2 * cw, snaps=False)
    text = np.array([9906, 1917, 11, 151652] + [151655] * (ch * cw) + [151653, 151673], dtype=np.int64)
    refs = [(16, 4, 4, ch, cw)]
    gh = gw = 8
    _, pos, ar = pkg.seq_ref(text, refs, gh, gw)
    T, I = len(text), gh * gw + 16
    S = T + I
    L = 4
    w = pkg.Weights(n_layers=L, seed=1234, weight_set="B", device=dev)
    eng = pkg.Engine(w, T, I, ar_len=ar)
    vmask = np.zeros(S, dtype=np.uint8)
    vmask[:T] = (text == 151655)
    vin = seeded_bf16((I, 3072), 90)
    vis = (torch.from_numpy(vmask).to(dev), emb, [ds[k] for k in range(3)])
    out = eng.forward(torch.from_numpy(text).to(dev), pos.to(dev), u16_to_torch(vin, dev), 0.3, visual=vis)
    torch.cuda.synchronize()
    emb_o, ds_o = parity.oracle_vision(vw, px, 2 * ch, 2 * cw)
    hw = parity.HostWeights(pkg, L, 1234, "B")
    ref = parity.oracle_forward(hw, text, pos.numpy(), ar, vin, 0.3, visual=(vmask, emb_o, [ds_o[k] for k in range(3)]))
    print("edit pipeline vs oracle pipeline:", metrics(out, ref)[:2])
    assert_close(torch_to_u16(out), ref, "V", "tower -> forward")
    # the tower's outputs reach the prediction
    out_plain = eng.forward(torch.from_numpy(text).to(dev), pos.to(dev), u16_to_torch(vin, dev), 0.3)
    torch.cuda.synchronize()
    assert metrics(out_plain, out)[0] > 1e-2
