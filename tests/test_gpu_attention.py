"""Prefix-causal flash attention vs the eager restatement (o1.c src/cuda/attn.cu:22-113), class D
(the bar of tests/unit/test_sdpa_block.c:253), over ragged lengths, every kind of ar_len, both
operand layouts, and at full benchmark size on sampled query rows."""
import ctypes as C

import numpy as np
import pytest
import torch

import parity
from parity import np_ptr, seeded_bf16, torch_to_u16, u16_to_torch, assert_close

pytestmark = pytest.mark.gpu

@pytest.fixture(params=[1, 2], ids=["two-tile", "one-tile"])
def tile_mode(request, pkg):
    """Both attention kernels take every case of this module: 1 = two query tiles per CTA (what long sequences get),
    2 = one query tile per CTA with triple-buffered scores (what S < 8192 gets by default)."""
    pkg.lib.o1_attention_tile_mode(request.param)
    yield request.param
    pkg.lib.o1_attention_tile_mode(0)


CASES = [(23, 4, 1, 18), (23, 32, 8, 0), (128, 4, 4, 127), (129, 8, 2, 1), (300, 8, 2, 100), (300, 8, 2, 300),
         (1037, 8, 2, 18), (1280, 32, 8, 255), (257, 4, 1, 200)]


@pytest.mark.parametrize("S,H,KV,ar", CASES)
def test_flash_attention_seq_major(pkg, orc, dev, tile_mode, S, H, KV, ar):
    ld = (H + 2 * KV) * 128
    qkv = seeded_bf16((S, ld), 31, 0.0, 1.5)     # std 1.5: logits spread enough to exercise the mask
    d = u16_to_torch(qkv, dev)
    out = torch.zeros(S, H * 128, dtype=torch.bfloat16, device=dev)
    rc = pkg.lib.o1_flash_attention(C.c_void_p(d.data_ptr()), ld, C.c_void_p(d.data_ptr() + H * 256), ld,
                                    C.c_void_p(d.data_ptr() + (H + KV) * 256), ld, pkg.ptr(out), H * 128, S, H,
                                    KV, ar, 128 ** -0.5)
    assert rc == 0, pkg.last_error()
    torch.cuda.synchronize()
    ref = np.zeros((S, H * 128), dtype=np.uint16)
    orc.orc_attention_rows(np_ptr(qkv), ld, np_ptr(qkv[:, H * 128:]), ld, np_ptr(qkv[:, (H + KV) * 128:]), ld,
                           np_ptr(ref), H * 128, H, KV, S, 128, 128 ** -0.5, ar, None, 0)
    assert_close(torch_to_u16(out), ref, "D", "flash attention")
    # every head separately: a head-indexing bug cannot hide in the average
    got = torch_to_u16(out).reshape(S, H, 128)
    for h in range(H):
        assert_close(np.ascontiguousarray(got[:, h]), np.ascontiguousarray(ref.reshape(S, H, 128)[:, h]), "D",
                     f"head {h}")
    if ar > 1:
        # causal rows must not see later keys: changing keys/values >= ar leaves rows < ar unchanged
        d2 = d.clone()
        d2[ar:, H * 128:] = d2[ar:, H * 128:] * 0.5 + 1.0
        out2 = torch.zeros_like(out)
        pkg.lib.o1_flash_attention(C.c_void_p(d2.data_ptr()), ld, C.c_void_p(d2.data_ptr() + H * 256), ld,
                                   C.c_void_p(d2.data_ptr() + (H + KV) * 256), ld, pkg.ptr(out2), H * 128, S, H,
                                   KV, ar, 128 ** -0.5)
        torch.cuda.synchronize()
        assert torch.equal(out[:ar].view(torch.int16), out2[:ar].view(torch.int16))


@pytest.mark.parametrize("S,ar", [(23, 18), (300, 37), (640, 0)])
def test_sdpa_shim_head_major_and_mask_probe(pkg, orc, dev, tile_mode, S, ar):
    """hd_sdpa_* / hd_attention_eager keep the reference's head-major layouts and accept its mask tensor."""
    H, KV = 8, 2
    q, k, v = seeded_bf16((H, S, 128), 32), seeded_bf16((KV, S, 128), 33), seeded_bf16((KV, S, 128), 34)
    ref = np.empty((S, H, 128), dtype=np.uint16)
    orc.orc_attention(np_ptr(q), np_ptr(k), np_ptr(v), np_ptr(ref), H, KV, S, 128, 128 ** -0.5, ar)
    qd, kd, vd = (u16_to_torch(t, dev) for t in (q, k, v))
    plan = C.c_void_p()
    assert pkg.lib.hd_sdpa_create_prod(C.byref(plan), 1, H, KV, S, ar, 128, 128 ** -0.5) == 0
    out_hm = torch.zeros(H, S, 128, dtype=torch.bfloat16, device=dev)
    assert pkg.lib.hd_sdpa_execute(plan, pkg.ptr(qd), pkg.ptr(kd), pkg.ptr(vd), None, pkg.ptr(out_hm), None) == 0
    pkg.lib.hd_sdpa_destroy(plan)
    torch.cuda.synchronize()
    assert_close(torch_to_u16(out_hm.permute(1, 0, 2).contiguous()), ref, "D", "sdpa shim (split plan)")
    # plan without ar_len + the reference's additive mask tensor
    mask = np.empty((S, S), dtype=np.uint16)
    orc.orc_prefix_causal_mask(S, ar, np_ptr(mask))
    md = u16_to_torch(mask, dev)
    assert pkg.lib.hd_sdpa_create(C.byref(plan), 1, H, KV, S, S, 128, 128 ** -0.5) == 0
    out2 = torch.zeros_like(out_hm)
    assert pkg.lib.hd_sdpa_execute(plan, pkg.ptr(qd), pkg.ptr(kd), pkg.ptr(vd), pkg.ptr(md), pkg.ptr(out2), None) == 0
    pkg.lib.hd_sdpa_destroy(plan)
    torch.cuda.synchronize()
    assert torch.equal(out2.view(torch.int16), out_hm.view(torch.int16))
    out3 = torch.zeros(S, H, 128, dtype=torch.bfloat16, device=dev)
    pkg.lib.hd_attention_eager(pkg.ptr(qd), pkg.ptr(kd), pkg.ptr(vd), pkg.ptr(md), None, None, pkg.ptr(out3), H, KV,
                               S, 128, 128 ** -0.5)
    torch.cuda.synchronize()
    pkg.check_cuda_errbuf("attention_eager")
    assert_close(torch_to_u16(out3), ref, "D", "hd_attention_eager signature")
    r = parity.reflib()
    if r is not None and S <= 300:
        sc = torch.empty(H * S * S, dtype=torch.float32, device=dev)     # fp32 scores live in the same buffer
        pr = torch.empty(H * S * S, dtype=torch.bfloat16, device=dev)
        out4 = torch.zeros(S, H, 128, dtype=torch.bfloat16, device=dev)
        r.hd_attention_eager(pkg.ptr(qd), pkg.ptr(kd), pkg.ptr(vd), pkg.ptr(md), pkg.ptr(sc), pkg.ptr(pr),
                             pkg.ptr(out4), H, KV, S, 128, 128 ** -0.5)
        torch.cuda.synchronize()
        assert_close(out3, out4, "D", "flash vs reference CUDA eager attention")
        assert_close(torch_to_u16(out4), ref, "B", "oracle vs reference CUDA eager attention")


def test_non_prefix_causal_mask_is_rejected(pkg, orc, dev):
    """The O(S) probe that recovers ar_len from the reference's mask tensor refuses masks whose causal
    rows are not a prefix (here: rows 0..9 causal except row 4)."""
    S, H = 64, 4
    mask = np.empty((S, S), dtype=np.uint16)
    orc.orc_prefix_causal_mask(S, 10, np_ptr(mask))
    mask[4, :] = 0
    md = u16_to_torch(mask, dev)
    q = torch.zeros(H, S, 128, dtype=torch.bfloat16, device=dev)
    plan = C.c_void_p()
    assert pkg.lib.hd_sdpa_create(C.byref(plan), 1, H, H, S, S, 128, 0.088) == 0
    pkg.lib.hd_cuda_clear_error()
    rc = pkg.lib.hd_sdpa_execute(plan, pkg.ptr(q), pkg.ptr(q), pkg.ptr(q), pkg.ptr(md), pkg.ptr(q), None)
    pkg.lib.hd_sdpa_destroy(plan)
    assert rc != 0 and b"not prefix-causal" in pkg.lib.hd_cuda_last_error()
    pkg.lib.hd_cuda_clear_error()


def test_flash_attention_full_size_sampled_rows(pkg, orc, dev, tile_mode):
    """S = 16640 (256 text + 128x128 image tokens), 32/8 heads: sampled query rows against the oracle,
    plus the property that every output row is a convex combination of value rows."""
    S, H, KV, ar = 16640, 32, 8, 255
    ld = (H + 2 * KV) * 128
    d = torch.empty(S, ld, dtype=torch.bfloat16, device=dev)
    assert pkg.lib.o1_fill_normal_bf16(pkg.ptr(d), S * ld, 4242, 0.0, 1.0) == 0
    out = torch.zeros(S, H * 128, dtype=torch.bfloat16, device=dev)
    rc = pkg.lib.o1_flash_attention(C.c_void_p(d.data_ptr()), ld, C.c_void_p(d.data_ptr() + H * 256), ld,
                                    C.c_void_p(d.data_ptr() + (H + KV) * 256), ld, pkg.ptr(out), H * 128, S, H,
                                    KV, ar, 128 ** -0.5)
    assert rc == 0
    torch.cuda.synchronize()
    qkv = torch_to_u16(d)
    rows = np.array([0, 1, 127, 128, 254, 255, 256, 4351, 8191, 16511, 16512, 16639], dtype=np.int32)
    ref = np.zeros((S, H * 128), dtype=np.uint16)
    orc.orc_attention_rows(np_ptr(qkv), ld, np_ptr(qkv[:, H * 128:]), ld, np_ptr(qkv[:, (H + KV) * 128:]), ld,
                           np_ptr(ref), H * 128, H, KV, S, 128, 128 ** -0.5, ar, np_ptr(rows), len(rows))
    got = torch_to_u16(out)
    assert_close(np.ascontiguousarray(got[rows]), np.ascontiguousarray(ref[rows]), "D", "full-size sampled rows")
    v = d[:, (H + KV) * 128:].float()
    vmax, vmin = v.max(0).values.repeat_interleave(1), v.min(0).values
    o = out.float().reshape(S, H, 128)
    kvh = torch.arange(H, device=dev) // (H // KV)
    hi = vmax.reshape(KV, 128)[kvh] * 1.01 + 0.02
    lo = vmin.reshape(KV, 128)[kvh] * 1.01 - 0.02
    assert bool(((o <= hi) & (o >= lo)).all()) and bool(torch.isfinite(o).all())


@pytest.mark.parametrize("S,H,KV,ar,ways", [(1280, 32, 8, 255, 0), (2304, 20, 4, 18, 0), (2304, 20, 4, 18, 9),
                                            (2304, 20, 4, 2304, 0), (1037, 40, 8, 600, 0), (3000, 8, 2, 0, 3),
                                            (3000, 8, 2, 0, 12), (3000, 36, 4, 200, 2), (3000, 36, 4, 2900, 0), (1500, 150, 50, 1, 5)])
def test_flash_attention_key_split_tail(pkg, orc, dev, tile_mode, S, H, KV, ar, ways):
    """With scratch the items of the last, partly filled wave are cut along the keys and merged: same result as
    the oracle (class D) and close to the unsplit kernel; item counts here leave tails of different sizes, one
    case is fully causal (tail items with different key ranges), one has fewer items than SMs."""
    ld = (H + 2 * KV) * 128
    qkv = seeded_bf16((S, ld), 77, 0.0, 1.5)
    d = u16_to_torch(qkv, dev)
    args = (C.c_void_p(d.data_ptr()), ld, C.c_void_p(d.data_ptr() + H * 256), ld,
            C.c_void_p(d.data_ptr() + (H + KV) * 256), ld)
    plain = torch.zeros(S, H * 128, dtype=torch.bfloat16, device=dev)
    split = torch.zeros_like(plain)
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    assert pkg.lib.o1_flash_attention(*args, pkg.ptr(plain), H * 128, S, H, KV, ar, 128 ** -0.5) == 0
    pkg.lib.o1_attention_tail_ways(ways)            # 0: the library's own choice; n: forced
    try:
        assert pkg.lib.o1_flash_attention_ws(*args, pkg.ptr(split), H * 128, S, H, KV, ar, 128 ** -0.5,
                                             pkg.ptr(scratch), scratch.numel()) == 0, pkg.last_error()
        torch.cuda.synchronize()
    finally:
        pkg.lib.o1_attention_tail_ways(0)
    ref = np.zeros((S, H * 128), dtype=np.uint16)
    orc.orc_attention_rows(np_ptr(qkv), ld, np_ptr(qkv[:, H * 128:]), ld, np_ptr(qkv[:, (H + KV) * 128:]), ld,
                           np_ptr(ref), H * 128, H, KV, S, 128, 128 ** -0.5, ar, None, 0)
    assert_close(torch_to_u16(split), ref, "D", "key-split attention vs oracle")
    assert_close(torch_to_u16(split), torch_to_u16(plain), "C", "key-split vs unsplit")
    # (with 128-row items a fully causal first query tile sees a single key tile, which cannot be cut: no split then)
    if ways > 1 and not (tile_mode == 2 and 0 < ar < 256):
        assert not torch.equal(split.view(torch.int16), plain.view(torch.int16)), "the split path did not run"
    # too little scratch: falls back to the unsplit form, bit for bit
    small = torch.zeros_like(plain)
    assert pkg.lib.o1_flash_attention_ws(*args, pkg.ptr(small), H * 128, S, H, KV, ar, 128 ** -0.5, pkg.ptr(scratch),
                                         1024) == 0
    torch.cuda.synchronize()
    assert torch.equal(small.view(torch.int16), plain.view(torch.int16))


def _eager_numpy(q, k, v, mask, scaling):
    """softmax(q k^T * scaling + mask) v in fp64 with the probabilities rounded to bf16 (o1.c src/cuda/attn.cu:22-113);
    q [H,S,D], k/v [KV,S,D] as float arrays; returns probs [H,S,S], out [S,H,D]."""
    H, S, D = q.shape
    g = H // k.shape[0]
    probs = np.empty((H, S, S))
    out = np.empty((S, H, D))
    for h in range(H):
        sc = (q[h].astype(np.float64) @ k[h // g].astype(np.float64).T) * scaling + mask
        sc -= sc.max(axis=1, keepdims=True)
        p = np.exp(sc)
        p /= p.sum(axis=1, keepdims=True)
        p = parity.bf16_to_f32_np(parity.f32_to_bf16_np(p.astype(np.float32))).astype(np.float64)
        probs[h] = p
        out[:, h] = p @ v[h // g].astype(np.float64)
    return probs, out


@pytest.mark.parametrize("H,KV,S,D", [(2, 1, 3, 4), (4, 2, 37, 72), (4, 4, 50, 128)])
def test_attention_eager_general_path_fills_scores_and_probs(pkg, dev, H, KV, S, D):
    """hd_attention_eager for what the flash kernel does not cover (another head_dim, or a mask that is not
    prefix-causal): scores and probabilities are materialised as the reference does (src/cuda/attn.cu:129-174;
    the analytic case of its tests/unit/test_primitives.c:484-533 has head_dim 4 and a one-key mask)."""
    rng = np.random.default_rng(S)
    qh, kh, vh = seeded_bf16((H, S, D), 1), seeded_bf16((KV, S, D), 2), seeded_bf16((KV, S, D), 3)
    m = np.where(rng.random((S, S)) < 0.4, -3.3895e38, 0.0).astype(np.float32)
    m[:, 0] = 0.0                                                   # every row keeps one visible key
    mh = parity.f32_to_bf16_np(m)
    qd, kd, vd, md = (u16_to_torch(a, dev) for a in (qh, kh, vh, mh))
    scores = torch.zeros(H, S, S, dtype=torch.bfloat16, device=dev)
    probs = torch.zeros(H, S, S, dtype=torch.bfloat16, device=dev)
    out = torch.zeros(S, H, D, dtype=torch.bfloat16, device=dev)
    pkg.lib.hd_attention_eager(pkg.ptr(qd), pkg.ptr(kd), pkg.ptr(vd), pkg.ptr(md), pkg.ptr(scores), pkg.ptr(probs),
                               pkg.ptr(out), H, KV, S, D, D ** -0.5)
    torch.cuda.synchronize()
    pkg.check_cuda_errbuf("attention_eager")
    f = parity.bf16_to_f32_np
    want_p, want_o = _eager_numpy(f(qh), f(kh), f(vh), f(mh).astype(np.float64), D ** -0.5)
    assert_close(probs.float().cpu().numpy(), want_p.astype(np.float32), "B", "probs")
    assert_close(out.float().cpu().numpy(), want_o.astype(np.float32), "B", "out")
    assert float(scores.float().abs().max()) > 0
    # without the two buffers the general path cannot run: reported, nothing launched
    pkg.lib.hd_cuda_clear_error()
    pkg.lib.hd_attention_eager(pkg.ptr(qd), pkg.ptr(kd), pkg.ptr(vd), pkg.ptr(md), None, None, pkg.ptr(out), H, KV, S, D,
                               D ** -0.5)
    assert pkg.lib.hd_cuda_last_error() != b""
    pkg.lib.hd_cuda_clear_error()
