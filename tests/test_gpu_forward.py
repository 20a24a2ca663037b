"""hd_forward and the CFG denoise step through the C ABI against the CPU oracle (and the reference's
CUDA build when present): few-layer stacks at small geometry, then a short latent chain."""
import ctypes as C

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
