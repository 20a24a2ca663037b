"""CPU checks of the oracle's vision-tower restatement (o1.c src/model/vision.c, src/cuda/vision_kernels.cu):
closed forms for its pieces and an independent numpy restatement of the whole tower with the same bf16
rounding points.  (On the GPU box the same oracle is compared with the reference's own CUDA build of
hd_vision_forward, tests/test_gpu_vision.py.)"""
import math

import numpy as np
import pytest

import parity
from parity import np_ptr, seeded_bf16, bf16_to_f32_np as f32, f32_to_bf16_np as bf16, assert_close


def r(a):
    """fp32 array rounded to bf16 precision (kept as fp32)."""
    return f32(bf16(a))


def test_tables_against_the_rule(orc):
    """vision.c:215-280: token order is 2x2 block-major; corners / weights of the 48 x 48 grid; rotary (row, col)."""
    gh, gw = 26, 20          # the 416 x 320 conditioning image of docs/REF_IMAGE_NATIVE_IMPLEMENTATION.md
    n = gh * gw
    idx, wgt = np.empty((4, n), np.int32), np.empty((4, n), np.float32)
    coords, inv = np.empty((2, n), np.int32), np.empty(18, np.float32)
    orc.orc_vision_tables(gh, gw, np_ptr(idx), np_ptr(wgt), np_ptr(coords), np_ptr(inv))
    # first block = patches (0,0) (0,1) (1,0) (1,1); second block starts at column 2
    assert coords[:, :6].T.tolist() == [[0, 0], [0, 1], [1, 0], [1, 1], [0, 2], [0, 3]]
    assert coords[:, -1].tolist() == [gh - 1, gw - 1]
    assert sorted(map(tuple, coords.T.tolist())) == [(h, w) for h in range(gh) for w in range(gw)]
    np.testing.assert_allclose(wgt.sum(axis=0), 1.0, atol=1e-6)
    assert idx[:, 0].tolist() == [0, 1, 48, 49] and wgt[0, 0] == 1.0            # corner (0,0) exactly
    last = 47 * 48 + 47
    assert idx[:, -1].tolist() == [last, last, last, last]                        # clamped at the far corner
    for row in (5, 77, 333):
        h, w = coords[:, row]
        hf, wf = np.float32(h) * np.float32(47) / np.float32(gh - 1), np.float32(w) * np.float32(47) / np.float32(gw - 1)
        assert idx[0, row] == int(hf) * 48 + int(wf)
        assert abs(wgt[3, row] - (hf - int(hf)) * (wf - int(wf))) < 1e-6
    np.testing.assert_allclose(inv, [10000.0 ** (-2 * k / 36.0) for k in range(18)], rtol=1e-6)


@pytest.mark.parametrize("rows,cols", [(5, 1152), (3, 4608), (4, 96)])
def test_layernorm_closed_form(orc, rows, cols):
    x, w, b = seeded_bf16((rows, cols), 3, 0.3, 1.5), seeded_bf16(cols, 4, 1.0, 0.1), seeded_bf16(cols, 5, 0.0, 0.1)
    y = np.empty_like(x)
    orc.orc_layernorm(np_ptr(x), np_ptr(w), np_ptr(b), np_ptr(y), rows, cols, 1e-6)
    xf = f32(x).astype(np.float64)
    ref = (xf - xf.mean(1, keepdims=True)) / np.sqrt(xf.var(1, keepdims=True) + 1e-6) * f32(w) + f32(b)
    assert_close(y, ref.astype(np.float32), "B", "layernorm")
    orc.orc_layernorm(np_ptr(x), np_ptr(w), None, np_ptr(y), rows, cols, 1e-6)      # bias is optional
    assert_close(y, (ref - f32(b)).astype(np.float32), "B", "layernorm without bias")


def test_gelu_forms(orc):
    x = bf16(np.linspace(-6, 6, 4001, dtype=np.float32))
    y = np.empty_like(x)
    v = f32(x).astype(np.float64)
    orc.orc_gelu(np_ptr(x), np_ptr(y), x.size, 0)
    tanh_form = 0.5 * v * (1 + np.tanh(math.sqrt(2 / math.pi) * (v + 0.044715 * v ** 3)))
    assert_close(y, tanh_form.astype(np.float32), "B", "gelu tanh")
    orc.orc_gelu(np_ptr(x), np_ptr(y), x.size, 1)
    erf_form = np.array([0.5 * t * (1 + math.erf(t / math.sqrt(2))) for t in v])
    assert_close(y, erf_form.astype(np.float32), "B", "gelu erf")
    assert f32(y)[0] == 0.0 and f32(y)[-1] == 6.0


def test_rotary_f32_single_rounding(orc):
    heads, seq, dim = 2, 5, 72
    x = seeded_bf16((heads, seq, dim), 9)
    ang = np.random.default_rng(0).uniform(-3, 3, (seq, dim // 2)).astype(np.float32)
    cs, sn = np.tile(np.cos(ang), 2).astype(np.float32), np.tile(np.sin(ang), 2).astype(np.float32)
    y = np.empty_like(x)
    orc.orc_apply_rotary_f32(np_ptr(x), np_ptr(cs), np_ptr(sn), np_ptr(y), heads, seq, dim)
    xf = f32(x)
    rot = np.concatenate([-xf[..., dim // 2:], xf[..., :dim // 2]], -1)
    ref = bf16(xf * cs + rot * sn)
    assert np.abs(f32(y) - f32(ref)).max() <= 2 ** -7 * np.abs(f32(ref)).max()
    assert (y == ref).mean() > 0.99


def numpy_tower(vw, px, gh, gw):
    """The tower in numpy fp32 with bf16 rounding where vision.c stores bf16 tensors."""
    at = dict(zip(vw.names, vw.arrays))
    W = type("Lazy", (), {"__getitem__": lambda self, name: f32(at[name])})()   # fp32 view of one tensor at a time
    n, H, D = gh * gw, 1152, 72
    lin = lambda x, p: r(r(x @ W[p + ".weight"].T) + W[p + ".bias"])
    def ln(x, p):
        mean, ex2 = x.mean(1, keepdims=True), (x * x).mean(1, keepdims=True)
        return r((x - mean) / np.sqrt(ex2 - mean * mean + 1e-6) * W[p + ".weight"] + W[p + ".bias"])
    gelu_t = lambda v: r(0.5 * v * (1 + np.tanh(0.7978845608028654 * (v + 0.044715 * v ** 3))))
    gelu_e = lambda v: r(0.5 * v * (1 + np.vectorize(math.erf)(v * 0.7071067811865476))).astype(np.float32)
    idx, wgt = np.empty((4, n), np.int32), np.empty((4, n), np.float32)
    coords, inv = np.empty((2, n), np.int32), np.empty(18, np.float32)
    parity.oracle().orc_vision_tables(gh, gw, np_ptr(idx), np_ptr(wgt), np_ptr(coords), np_ptr(inv))
    x = r(f32(px) @ W["model.visual.patch_embed.proj.weight"].T + W["model.visual.patch_embed.proj.bias"])
    pos = r(sum(wgt[k][:, None] * W["model.visual.pos_embed.weight"][idx[k]] for k in range(4)))
    x = r(x + pos)
    ang = r(np.concatenate([coords[0][:, None] * inv[None], coords[1][:, None] * inv[None]], 1).astype(np.float32))
    cs, sn = np.tile(np.cos(ang), 2), np.tile(np.sin(ang), 2)
    rope = lambda t: r(t * cs[:, None] + np.concatenate([-t[..., D // 2:], t[..., :D // 2]], -1) * sn[:, None])
    blocks, deep = [], []
    for i in range(27):
        p = f"model.visual.blocks.{i}"
        qkv = lin(ln(x, p + ".norm1"), p + ".attn.qkv").reshape(n, 3, 16, D)
        q, k, v = rope(qkv[:, 0]), rope(qkv[:, 1]), qkv[:, 2]
        s = np.einsum("shd,thd->hst", q, k) * np.float32(1 / math.sqrt(D))
        pr = np.exp(s - s.max(-1, keepdims=True))
        pr = r(pr / pr.sum(-1, keepdims=True))
        att = r(np.einsum("hst,thd->shd", pr, v)).reshape(n, H)
        a = r(x + lin(att, p + ".attn.proj"))
        f1 = gelu_t(lin(ln(a, p + ".norm2"), p + ".mlp.linear_fc1"))
        x = r(a + lin(f1, p + ".mlp.linear_fc2"))
        blocks.append(x)
        if i in (8, 16, 24):
            dp = f"model.visual.deepstack_merger_list.{i // 8 - 1}"
            t = ln(x.reshape(n // 4, 4608), dp + ".norm")
            deep.append(lin(gelu_e(lin(t, dp + ".linear_fc1")), dp + ".linear_fc2"))
    mp = "model.visual.merger"
    t = ln(x, mp + ".norm").reshape(n // 4, 4608)
    emb = lin(gelu_e(lin(t, mp + ".linear_fc1")), mp + ".linear_fc2")
    return emb, np.stack(deep), np.stack(blocks)


@pytest.fixture(scope="module")
def vw():
    return parity.VisionHostWeights()


def test_tower_against_numpy_restatement(orc, vw):
    gh, gw = 4, 6
    px = seeded_bf16((gh * gw, 1536), 7)
    emb, ds, blocks = parity.oracle_vision(vw, px, gh, gw, want_blocks=True)
    emb_np, ds_np, blocks_np = numpy_tower(vw, px, gh, gw)
    # two restatements differ by summation order: single bf16 ulps after one block (GEMM class), more after 27
    assert_close(blocks[0], blocks_np[0], "C", "block 0 output")
    assert_close(blocks[8], blocks_np[8], "E", "block 8 output")
    assert_close(blocks[26], blocks_np[26], "V", "block 26 output")
    assert_close(ds, ds_np, "V", "deepstack")
    assert_close(emb, emb_np, "V", "image_embeds")
    # a second image size and repeatability
    emb2, _ = parity.oracle_vision(vw, px, gh, gw)
    assert (emb2 == emb).all()
    assert orc.orc_vision_forward(vw.pointer_table(), np_ptr(px), 3, 4, np_ptr(emb), None, None) == -1   # odd grid
