"""hd_forward and the CFG denoise step through the C ABI against the CPU oracle (and the reference's
CUDA build when present): few-layer stacks at small geometry, then a short latent chain."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import parity
from parity import np_ptr, seeded_bf16, torch_to_u16, u16_to_torch, assert_close

pytestmark = pytest.mark.gpu


def make_ids(T, seed):
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, 151000, size=T).astype(np.int64)
    ids[-1] = 151673                     # tms token closes the text block (sequence.c:67-100)
    return ids


@pytest.mark.parametrize("wset,n_layers", [("B", 2), ("A", 3)])
def test_forward_vs_oracle(pkg, dev, wset, n_layers):
    T, gh, gw = 19, 6, 8
    I = gh * gw
    w = pkg.Weights(n_layers=n_layers, seed=1234, weight_set=wset, device=dev)
    eng = pkg.Engine(w, T, I)
    pos, ar = pkg.seq_t2i(T, gh, gw)
    ids = make_ids(T, 1)
    vin = seeded_bf16((I, 3072), 43)
    names = ("after_timestep_conditioning", "after_target_embedding", "after_block_0_input", "after_block_0",
             "before_final_norm", "after_final_norm", "after_final_head")
    out, diag = eng.forward(torch.from_numpy(ids).to(dev), pos.to(dev), u16_to_torch(vin, dev), 0.5,
                            diag_names=names)
    out2 = eng.forward(torch.from_numpy(ids).to(dev), pos.to(dev), u16_to_torch(vin, dev), 0.5)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16)), "diagnostics changed the result"
    hw = parity.HostWeights(pkg, n_layers, 1234, wset)
    ref, hd = parity.oracle_forward(hw, ids, pos.numpy(), ar, vin, 0.5, dump=True)
    S = T + I
    assert_close(torch_to_u16(diag["after_block_0_input"]), hd[0], "C", "embedding + concat")
    # the tms row carries the timestep embedding, every other text row its table row
    emb = hw.embed_rows(ids)
    got_text = torch_to_u16(diag["after_timestep_conditioning"])
    assert (got_text[:-1] == emb[:-1]).all()
    assert_close(got_text[-1], hd[0][T - 1], "C", "t_emb row")
    assert_close(torch_to_u16(diag["after_block_0"]), hd[1], "D", "after block 0")
    assert_close(torch_to_u16(diag["before_final_norm"]), hd[n_layers], "D", "after last block")
    # final norm + head on the SAME hidden state: class C (one GEMM); end to end the head inherits the
    # stack's drift, which the reference bounds by a wider envelope (tests/unit/test_full_forward.c:446-486)
    fn = np.empty((S, 4096), dtype=np.uint16)
    gotf = torch_to_u16(diag["before_final_norm"])
    parity.oracle().orc_rmsnorm(np_ptr(gotf), np_ptr(hw.tensor(-1, "fnorm_w")), np_ptr(fn), S, 4096, 1e-6)
    assert_close(torch_to_u16(diag["after_final_norm"]), fn, "B", "final norm")
    head = np.empty((S, 3072), dtype=np.uint16)
    parity.oracle().orc_linear(np_ptr(fn), np_ptr(hw.tensor(-1, "fl_w")), np_ptr(hw.tensor(-1, "fl_b")),
                               np_ptr(head), S, 3072, 4096)
    assert_close(torch_to_u16(out), head, "C", "head on identical input")
    assert_close(torch_to_u16(out), ref, "E", "x_pred")
    assert_close(torch_to_u16(out)[T:], ref[T:], "E", "x_pred image rows")


def test_forward_vs_reference_cuda_build(pkg, dev):
    r = parity.reflib()
    if r is None:
        pytest.skip("oracle/_ref/libo1ref.so not built")
    T, gh, gw, L = 19, 6, 8, 2
    I, S = gh * gw, 19 + 48
    w = pkg.Weights(n_layers=L, seed=1234, weight_set="B", device=dev)
    eng = pkg.Engine(w, T, I)
    pos, ar = pkg.seq_t2i(T, gh, gw)
    ids = torch.from_numpy(make_ids(T, 1)).to(dev)
    vin = u16_to_torch(seeded_bf16((I, 3072), 43), dev)
    mine = eng.forward(ids, pos.to(dev), vin, 0.5)
    # reference hd_forward (src/model/forward.c:190) with its own workspace, eager attention, own GEMM kernel
    bs = C.c_int64(0)
    nbytes = r.hd_forward_workspace_bytes(S, I, 32, 8, 4096, 12288, 128, C.byref(bs))
    buf = torch.empty(nbytes + 256, dtype=torch.uint8, device=dev)
    ws = pkg.ForwardWorkspace()
    ws.hidden_a = buf.data_ptr()
    ws.block_scratch_bytes = bs.value
    mask = np.empty((S, S), dtype=np.uint16)
    parity.oracle().orc_prefix_causal_mask(S, ar, np_ptr(mask))
    md = u16_to_torch(mask, dev)
    sec = torch.tensor([24, 20, 20], dtype=torch.int64, device=dev)
    tt = torch.tensor([0.5], device=dev)
    out = torch.empty(S, 3072, dtype=torch.bfloat16, device=dev)
    r.hd_gemm_set_backend(0)
    rc = r.hd_forward(C.byref(w.binding), C.byref(ws), pkg.ptr(ids), T, pkg.ptr(pos.to(dev)), pkg.ptr(md),
                      pkg.ptr(vin), I, None, pkg.ptr(tt), pkg.ptr(sec), S, 32, 8, 4096, 12288, 128, pkg.TMS_ID,
                      None, pkg.ptr(out), None)
    torch.cuda.synchronize()
    assert rc == 0, r.hd_last_error()
    assert_close(mine, out, "E", "x_pred vs reference CUDA forward")


def test_cfg_denoise_chain_vs_oracle(pkg, orc, dev):
    """Three CFG flow-match steps (two forwards + fused scheduler update per step) on a seeded latent,
    device-resident and through the host-buffer entry point, against the same chain on the oracle.
    Staircase of o1.c docs/M1_7_TOLERANCES.md:61-91 for the first steps: nrmse <= 5e-3, cos >= 0.9999."""
    T, gh, gw, L, g = 12, 4, 6, 2, 5.0
    I = gh * gw
    w = pkg.Weights(n_layers=L, seed=1234, weight_set="B", device=dev)
    eng = pkg.Engine(w, T, I)
    pos, ar = pkg.seq_t2i(T, gh, gw)
    ids_c, ids_u = make_ids(T, 2), make_ids(T, 3)
    z0 = np.empty((I, 3072), dtype=np.uint16)
    assert orc.orc_initial_latent(123456, gh * 32, gw * 32, 32, 8.0, np_ptr(z0)) == 0
    sig = pkg.dev_sigmas()
    idc, idu, posd = torch.from_numpy(ids_c).to(dev), torch.from_numpy(ids_u).to(dev), pos.to(dev)
    z = u16_to_torch(z0, dev)
    zh = u16_to_torch(z0).pin_memory()
    zh_next = torch.empty_like(zh).pin_memory()
    zd_a, zd_b = torch.empty_like(z), torch.empty_like(z)
    hw = parity.HostWeights(pkg, L, 1234, "B")
    zo = z0.copy()
    for i in range(3):
        z = eng.denoise_step_cfg(idc, idu, posd, z, sig[i], sig[i + 1], g)
        eng.denoise_step_cfg_host(idc, idu, posd, zh, zd_a, sig[i], sig[i + 1], g, zd_b, zh_next)
        zh.copy_(zh_next)
        torch.cuda.synchronize()
        assert torch.equal(z.cpu().view(torch.int16), zh.view(torch.int16)), "host entry point differs"
        xc = parity.oracle_forward(hw, ids_c, pos.numpy(), ar, zo, 1.0 - np.float32(sig[i]))
        xu = parity.oracle_forward(hw, ids_u, pos.numpy(), ar, zo, 1.0 - np.float32(sig[i]))
        zn = np.empty_like(zo)
        orc.orc_sched_cfg_flow_step(np_ptr(zo), np_ptr(np.ascontiguousarray(xc[T:])),
                                    np_ptr(np.ascontiguousarray(xu[T:])), sig[i], sig[i + 1], g, np_ptr(zn), zo.size)
        zo = zn
        nrmse, cos, _, bad = parity.metrics(torch_to_u16(z), zo)
        assert bad == 0 and nrmse <= 5e-3 and cos >= 0.9999, (i, nrmse, cos)


def test_decode_to_rgb_and_gate(pkg, dev):
    """Final latent -> uint8 RGB on the device against the formula of o1.c src/runtime/decode.c:5-27, plus
    the non-finite count and range the reference's gate (generate.c:1474-1496) is built on."""
    gh, gw, p = 3, 5, 32
    z = seeded_bf16((gh * gw, 3 * p * p), 77, 0.0, 0.6)
    zf = parity.bf16_to_f32_np(z)
    rgb = torch.zeros(gh * p, gw * p, 3, dtype=torch.uint8, device=dev)
    stats = torch.zeros(3, dtype=torch.int32, device=dev)
    nb, mn, mx = C.c_int(), C.c_float(), C.c_float()
    zd = u16_to_torch(z, dev)
    rc = pkg.lib.o1_decode_to_rgb(pkg.ptr(zd), gh, gw, p, 3, pkg.ptr(rgb), pkg.ptr(stats), C.byref(nb), C.byref(mn),
                                  C.byref(mx))
    assert rc == 0, pkg.last_error()
    img = zf.reshape(gh, gw, 3, p, p).transpose(0, 3, 1, 4, 2).reshape(gh * p, gw * p, 3)
    want = np.clip(np.floor((img + 1.0) / 2.0 * 255.0 + 0.5), 0, 255)          # roundf: half away from zero, v >= 0
    neg = (img + 1.0) / 2.0 * 255.0 < 0
    want[neg] = 0
    assert (rgb.cpu().numpy() == want.astype(np.uint8)).all()
    assert nb.value == 0 and mn.value == zf.min() and mx.value == zf.max()
    z2 = z.copy()
    z2[3, 7] = 0x7FC0            # NaN
    z2[5, 9] = 0x7F80            # +inf
    zd2 = u16_to_torch(z2, dev)
    pkg.lib.o1_decode_to_rgb(pkg.ptr(zd2), gh, gw, p, 3, pkg.ptr(rgb), pkg.ptr(stats), C.byref(nb), C.byref(mn), C.byref(mx))
    assert nb.value == 2


def test_multi_reference_forward_with_visual_conditioning(pkg, orc, dev, golden):
    """Edit / personalise layout (workload c3 in miniature): text with <image_pad> runs, target grid,
    K = 4 reference grids with their own 3-axis positions from the hd_seq_build fixture; vision-tower outputs
    (image_embeds, DeepStack x3) scattered / added on the pad rows; reference rows taken from the x_embedder
    cache.  Against the oracle, and cache path == recompute path bit for bit."""
    g = np.load(os.path.join(golden, "seq_ref.npz"))
    T, gh, gw, S, ar, K = (int(v) for v in g["k4_meta"])
    ids_all, pos = g["k4_ids"], g["k4_pos"]
    geom = g["k4_geom"]
    I_tgt, n_ref = gh * gw, int(geom[:, 0].sum())
    I = I_tgt + n_ref                                  # every row after the text goes through x_embedder
    assert T + I == S
    text = np.ascontiguousarray(ids_all[:T])
    L = 4                                              # DeepStack touches blocks 0..2
    w = pkg.Weights(n_layers=L, seed=1234, weight_set="B", device=dev)
    eng = pkg.Engine(w, T, I, ar_len=ar)
    vmask = np.zeros(S, dtype=np.uint8)
    vmask[:T] = (text == 151655)
    V = int(vmask.sum())
    assert V == int((geom[:, 3] * geom[:, 4]).sum())
    emb = seeded_bf16((V, 4096), 81)
    dss = [seeded_bf16((V, 4096), 82 + k, 0.0, 0.5) for k in range(3)]
    vin = seeded_bf16((I, 3072), 90)                   # target latent rows, then reference pixel rows
    idsd, posd = torch.from_numpy(text).to(dev), torch.from_numpy(pos).to(dev)
    vind = u16_to_torch(vin, dev)
    vis = (torch.from_numpy(vmask).to(dev), u16_to_torch(emb, dev), [u16_to_torch(d, dev) for d in dss])
    out = eng.forward(idsd, posd, vind, 0.3, visual=vis)
    # x_embedder cache for the reference rows (computed once with the same weights)
    stage = torch.empty(n_ref, 1024, dtype=torch.bfloat16, device=dev)
    xe_ref = torch.empty(n_ref, 4096, dtype=torch.bfloat16, device=dev)
    ref_rows = vind[I_tgt:].contiguous()
    pkg.lib.hd_linear(pkg.ptr(ref_rows), C.c_void_p(w.addr(-1, "xe1_w")), None, pkg.ptr(stage), n_ref, 1024, 3072, 1)
    pkg.lib.hd_linear(pkg.ptr(stage), C.c_void_p(w.addr(-1, "xe2_w")), C.c_void_p(w.addr(-1, "xe2_b")), pkg.ptr(xe_ref),
                      n_ref, 4096, 1024, 1)
    eng.set_ref_cache(xe_ref)
    out_cached = eng.forward(idsd, posd, vind, 0.3, visual=vis)
    eng.set_ref_cache(None)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), out_cached.view(torch.int16)), "x_embedder cache changed the result"
    hw = parity.HostWeights(pkg, L, 1234, "B")
    ref = parity.oracle_forward(hw, text, pos, ar, vin, 0.3, visual=(vmask, emb, dss))
    assert_close(torch_to_u16(out), ref, "E", "multi-reference forward")
    # the visual inputs matter: without them the prediction differs
    out_plain = eng.forward(idsd, posd, vind, 0.3)
    torch.cuda.synchronize()
    assert parity.metrics(out_plain, out)[0] > 1e-2


def test_gguf_pack_to_device_and_resolve(pkg, dev, tmp_path):
    """hd_weights_to_device_gguf + hd_forward_resolve / hd_block_resolve: every tensor lands bit-exact (bf16
    unchanged, F32 / F16 rounded to bf16) at a 256-byte aligned address inside one arena, and the bindings
    point at the right tensors by manifest name; a pack lacking a tensor fails closed."""
    from test_abi_host import _small_pack
    path = str(tmp_path / "pack.gguf")
    tensors = _small_pack(pkg, path, n_layers=2)
    store = pkg.WeightStore()
    rc = pkg.lib.hd_weights_to_device_gguf(path.encode(), 0, C.byref(store))
    assert rc == 0, pkg.lib.hd_weights_last_error()
    assert store.n_allocs == len(tensors) and store.n_allocations == 1 and store.arena_ptr
    by_name = {}
    for i, (name, a) in enumerate(tensors):
        al = store.allocs[i]
        assert al.name.decode() == name and al.dev_ptr % 256 == 0 and al.nbytes == a.size * 2
        assert store.arena_ptr <= al.dev_ptr < store.arena_ptr + store.arena_bytes
        want = a.ravel() if a.dtype == np.uint16 else parity.f32_to_bf16_np(a.astype(np.float32).ravel())
        # read the tensor back through the library (bf16 -> fp32 is exact) and compare bit patterns
        up = torch.empty(a.size, dtype=torch.float32, device=dev)
        pkg.lib.hd_sched_bf16_upcast(C.c_void_p(al.dev_ptr), pkg.ptr(up), a.size)
        torch.cuda.synchronize()
        got = (up.cpu().numpy().view(np.uint32) >> 16).astype(np.uint16)
        assert (got == want).all(), name
        by_name[name] = (al.dev_ptr, want)
    fb = pkg.ForwardBinding()
    assert pkg.lib.hd_forward_resolve(C.byref(store), 2, C.byref(fb)) == 0, pkg.lib.hd_last_error()
    assert fb.n_layers == 2 and fb.embed_tokens == by_name[pkg.gguf_tensor_name(-1, "embed_tokens")][0]
    assert fb.blocks[1].down_proj == by_name[pkg.gguf_tensor_name(1, "down_proj")][0]
    assert fb.blocks[0].k_norm == by_name[pkg.gguf_tensor_name(0, "k_norm")][0]
    bb = pkg.BlockBinding()
    assert pkg.lib.hd_block_resolve(C.byref(store), 2, C.byref(bb)) == 6          # layer 2 is not in the pack
    assert b"missing weight model.language_model.layers.2." in pkg.lib.hd_last_error()
    fb3 = pkg.ForwardBinding()
    assert pkg.lib.hd_forward_resolve(C.byref(store), 3, C.byref(fb3)) == 6
    pkg.lib.hd_forward_binding_free(C.byref(fb))
    pkg.lib.hd_weight_store_free(C.byref(store))
    assert not store.arena_ptr
    assert pkg.lib.hd_weights_to_device_gguf(b"/nonexistent.gguf", 0, C.byref(store)) != 0


def test_forward_from_a_gguf_pack_and_header_only_layout(pkg, dev, tmp_path):
    """A pack of the real architecture (1 block) written from the seeded arena: loading it back gives the same
    forward bit for bit; the header-only store has the identical layout, and once its arena holds a copy of the
    loaded bytes (what a broadcast from the reading rank delivers) it gives the same forward too."""
    L, T, gh, gw = 1, 16, 4, 8
    I = gh * gw
    w = pkg.Weights(n_layers=L, seed=1234, weight_set="B", device=dev)
    tensors = []
    for layer, names in [(-1, pkg.GLOBAL_NAMES)] + [(l, pkg.SLOT_NAMES) for l in range(L)]:
        for name in names:
            bits = w.tensor(layer, name).contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
            tensors.append((pkg.gguf_tensor_name(layer, name), bits))
    path = str(tmp_path / "model.gguf")
    pkg.write_gguf(path, tensors, {"general.architecture": "hidream_o1", "hidream.num_layers": str(L)})
    pos, _ = pkg.seq_t2i(T, gh, gw)
    ids = np.arange(T, dtype=np.int64) + 7
    ids[-1] = pkg.TMS_ID
    idsd, posd = torch.from_numpy(ids).to(dev), pos.to(dev)
    vin = u16_to_torch(seeded_bf16((I, 3072), 43), dev)
    want = pkg.Engine(w, T, I).forward(idsd, posd, vin, 0.5)
    gw_ = pkg.GgufWeights(path, L, dev)
    try:
        got = pkg.Engine(gw_, T, I).forward(idsd, posd, vin, 0.5)
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
        lay = pkg.WeightStore()
        assert pkg.lib.o1_weights_gguf_layout(path.encode(), 0, C.byref(lay)) == 0, pkg.lib.hd_weights_last_error()
        try:
            assert lay.arena_bytes == gw_.store.arena_bytes and lay.n_allocs == gw_.store.n_allocs
            assert lay.host_bytes_loaded == 0
            for i in range(lay.n_allocs):
                assert lay.allocs[i].name == gw_.store.allocs[i].name
                assert lay.allocs[i].dev_ptr - lay.arena_ptr == gw_.store.allocs[i].dev_ptr - gw_.store.arena_ptr
            a = torch.as_tensor(pkg.model._DevBytes(gw_.store.arena_ptr, lay.arena_bytes), device=dev)
            b = torch.as_tensor(pkg.model._DevBytes(lay.arena_ptr, lay.arena_bytes), device=dev)
            b.copy_(a)                                        # stands in for the broadcast
            fb = pkg.ForwardBinding()
            assert pkg.lib.hd_forward_resolve(C.byref(lay), L, C.byref(fb)) == 0
            assert fb.blocks[0].q_proj - lay.arena_ptr == gw_.binding.blocks[0].q_proj - gw_.store.arena_ptr
            pkg.lib.hd_forward_binding_free(C.byref(fb))
            assert torch.equal(a, b)
        finally:
            pkg.lib.hd_weight_store_free(C.byref(lay))
    finally:
        gw_.close()


def test_cfg_step_replays_from_a_cuda_graph(pkg, dev):
    """One CFG denoise step (2 forwards + fused scheduler update) issues no allocation and no host
    synchronisation, so it can be captured once and replayed: the replay equals the eager step bit for bit,
    also after the latent buffer has been refilled."""
    T, gh, gw, L = 24, 8, 12, 2
    I = gh * gw
    w = pkg.Weights(n_layers=L, seed=1234, weight_set="B", device=dev)
    eng = pkg.Engine(w, T, I)
    pos, _ = pkg.seq_t2i(T, gh, gw)
    rng = np.random.default_rng(5)
    ids_c = rng.integers(0, 151000, size=T).astype(np.int64)
    ids_u = rng.integers(0, 151000, size=T).astype(np.int64)
    ids_c[-1] = ids_u[-1] = pkg.TMS_ID
    ic, iu, posd = torch.from_numpy(ids_c).to(dev), torch.from_numpy(ids_u).to(dev), pos.to(dev)
    z = u16_to_torch(seeded_bf16((I, 3072), 11, 0.0, 8.0), dev)
    eager = torch.empty_like(z)
    eng.denoise_step_cfg(ic, iu, posd, z, 0.8, 0.7, 5.0, eager)          # also the warm-up (tensor maps, attributes)
    torch.cuda.synchronize()
    out = torch.empty_like(z)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    try:
        with torch.cuda.stream(side):
            pkg.use_torch_stream()
            with torch.cuda.graph(graph, stream=side):
                eng.denoise_step_cfg(ic, iu, posd, z, 0.8, 0.7, 5.0, out)
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), eager.view(torch.int16))
        z2 = u16_to_torch(seeded_bf16((I, 3072), 12, 0.0, 8.0), dev)
        z.copy_(z2)
        graph.replay()
        torch.cuda.synchronize()
    finally:
        pkg.use_torch_stream()                                            # back to the default stream
    eng.denoise_step_cfg(ic, iu, posd, z2, 0.8, 0.7, 5.0, eager)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), eager.view(torch.int16))


def test_decode_to_rgb_against_the_reference_decode(pkg, dev, golden):
    """o1_decode_to_rgb byte for byte against hd_decode_to_rgb of o1.c src/runtime/decode.c:5-27: the committed
    fixture (values beyond [-1, 1], negative zero), and the reference function itself on a larger latent."""
    g = np.load(os.path.join(golden, "decode_ref.npz"))
    gh, gw, p = (int(v) for v in g["geom"])

    def run(z_bits, gh, gw):
        rgb = torch.zeros(gh * p, gw * p, 3, dtype=torch.uint8, device=dev)
        stats = torch.zeros(3, dtype=torch.int32, device=dev)
        nb, mn, mx = C.c_int(), C.c_float(), C.c_float()
        zd = u16_to_torch(z_bits, dev)
        rc = pkg.lib.o1_decode_to_rgb(pkg.ptr(zd), gh, gw, p, 3, pkg.ptr(rgb), pkg.ptr(stats), C.byref(nb), C.byref(mn),
                                      C.byref(mx))
        assert rc == 0, pkg.last_error()
        return rgb.cpu().numpy()

    assert (run(np.ascontiguousarray(g["z"]), gh, gw) == g["rgb"]).all()
    r = parity.reflib()
    if r is not None and hasattr(r, "hd_decode_to_rgb"):
        gh2, gw2 = 16, 24
        z = seeded_bf16((gh2 * gw2, 3 * p * p), 78, 0.0, 0.8)
        zf = np.ascontiguousarray(parity.bf16_to_f32_np(z))
        want = np.zeros((gh2 * p, gw2 * p, 3), dtype=np.uint8)
        r.hd_decode_to_rgb.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
        r.hd_decode_to_rgb.restype = None
        r.hd_decode_to_rgb(zf.ctypes.data_as(C.c_void_p), gh2, gw2, p, 3, want.ctypes.data_as(C.c_void_p))
        assert (run(z, gh2, gw2) == want).all()


def test_loader_against_the_reference_loader_and_converter(pkg, dev, golden, tmp_path):
    """The same pack through hd_weights_to_device_gguf of this library and of the reference's own loader
    (o1.c src/model/weights.c:519-669 + src/io/gguf.c, inside the reference-built checker library): same tensor
    names in the same order, same sizes, same offsets inside the arena, same device bytes.  Packs: one written by
    the reference's converter (fixture) and one written by write_gguf."""
    from test_abi_host import _small_pack
    r = parity.reflib()
    ours_path = str(tmp_path / "ours.gguf")
    _small_pack(pkg, ours_path, n_layers=2, with_f32=False)
    want = np.load(os.path.join(golden, "ref_convert_small.npz"))

    def dev_bytes(ptr_, n):
        return torch.as_tensor(pkg.model._DevBytes(ptr_, n), device=dev).cpu().numpy()

    for path in (os.path.join(golden, "ref_convert_small.gguf"), ours_path):
        mine = pkg.WeightStore()
        assert pkg.lib.hd_weights_to_device_gguf(path.encode(), 0, C.byref(mine)) == 0, pkg.lib.hd_weights_last_error()
        try:
            if path.endswith("ref_convert_small.gguf"):
                for i in range(mine.n_allocs):
                    a = mine.allocs[i]
                    bits = want[a.name.decode()]
                    assert a.nbytes == bits.size * 2
                    assert (dev_bytes(a.dev_ptr, a.nbytes).view(np.uint16) == bits.ravel()).all(), a.name
            if r is None:
                continue
            theirs = pkg.WeightStore()
            r.hd_weights_to_device_gguf.argtypes = [C.c_char_p, C.c_int, C.c_void_p]
            r.hd_weights_last_error.restype = C.c_char_p
            assert r.hd_weights_to_device_gguf(path.encode(), 0, C.byref(theirs)) == 0, r.hd_weights_last_error()
            try:
                assert theirs.n_allocs == mine.n_allocs and theirs.arena_bytes == mine.arena_bytes
                for i in range(mine.n_allocs):
                    a, b = mine.allocs[i], theirs.allocs[i]
                    assert a.name == b.name and a.nbytes == b.nbytes
                    assert a.dev_ptr - mine.arena_ptr == b.dev_ptr - theirs.arena_ptr
                assert (dev_bytes(mine.arena_ptr, mine.arena_bytes) == dev_bytes(theirs.arena_ptr, theirs.arena_bytes)).all()
            finally:
                r.hd_weight_store_free.argtypes = [C.c_void_p]
                r.hd_weight_store_free(C.byref(theirs))
        finally:
            pkg.lib.hd_weight_store_free(C.byref(mine))
