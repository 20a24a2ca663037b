"""Sequence-parallel (Ulysses) stages on ONE GPU: P emulated ranks advanced in lock step, exchanges
done by copies.  The sharded forward must reproduce the single-rank hd_forward (same kernels, same
rounding points; only GEMM tile shapes change with the row count), for P = 1, 2, 4, 8."""
import numpy as np
import pytest
import torch

import parity
from parity import seeded_bf16, torch_to_u16, u16_to_torch, assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("P", [1, 2, 4, 8])
def test_sp_forward_matches_single_rank(pkg, dev, P):
    from o1c_b200 import sp
    T, gh, gw, L = 24, 8, 13, 2          # S = 128: every P divides it; shard 0 mixes text and image rows
    I, S = gh * gw, 24 + 8 * 13
    w = pkg.Weights(n_layers=L, seed=1234, weight_set="B", device=dev)
    pos, ar = pkg.seq_t2i(T, gh, gw)
    rng = np.random.default_rng(1)
    ids = rng.integers(0, 151000, size=T).astype(np.int64)
    ids[-1] = pkg.TMS_ID
    idsd, posd = torch.from_numpy(ids).to(dev), pos.to(dev)
    vin = u16_to_torch(seeded_bf16((I, 3072), 43), dev)
    ref = pkg.Engine(w, T, I).forward(idsd, posd, vin, 0.5)
    engines = [sp.EngineSP(w, T, I, P, r, None) for r in range(P)]
    out = sp.run_emulated(engines, idsd, posd, vin, 0.5)
    torch.cuda.synchronize()
    assert out.shape == ref.shape
    assert_close(out, ref, "B", f"SP{P} forward vs single rank")
    if P == 1:
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16))
    # and against the CPU oracle, as the unsharded forward is
    hw = parity.HostWeights(pkg, L, 1234, "B")
    oref = parity.oracle_forward(hw, ids, pos.numpy(), ar, torch_to_u16(vin), 0.5)
    assert_close(torch_to_u16(out), oref, "E", f"SP{P} forward vs oracle")


def test_sp_rejects_bad_geometry(pkg, dev):
    from o1c_b200 import sp
    w = pkg.Weights(n_layers=1, device=dev)
    with pytest.raises(ValueError):
        sp.EngineSP(w, 24, 103, 2, 0, None)          # S = 127 not divisible
    with pytest.raises(ValueError):
        sp.EngineSP(w, 24, 120, 16, 0, None)         # 16 does not divide the 8 KV heads


@pytest.mark.parametrize("P", [2, 4, 8])
def test_sp_direct_form_is_bit_identical_to_staged_form(pkg, dev, P):
    """Direct form: GEMM / attention epilogues store into the destination ranks' buffers through a pointer
    table (here all on one device), norm + rope run on the receiving side.  Same values as the staged form."""
    from o1c_b200 import sp
    T, gh, gw, L = 24, 8, 13, 2
    I = gh * gw
    w = pkg.Weights(n_layers=L, seed=1234, weight_set="B", device=dev)
    pos, _ = pkg.seq_t2i(T, gh, gw)
    rng = np.random.default_rng(1)
    ids = rng.integers(0, 151000, size=T).astype(np.int64)
    ids[-1] = pkg.TMS_ID
    idsd, posd = torch.from_numpy(ids).to(dev), pos.to(dev)
    vin = u16_to_torch(seeded_bf16((I, 3072), 43), dev)
    staged = sp.run_emulated([sp.EngineSP(w, T, I, P, r, None) for r in range(P)], idsd, posd, vin, 0.5)
    engines = [sp.EngineSP(w, T, I, P, r, direct=True) for r in range(P)]
    try:
        for e in engines:
            e.connect([x.region for x in engines])
        direct = sp.run_emulated(engines, idsd, posd, vin, 0.5)
        again = sp.run_emulated(engines, idsd, posd, vin, 0.5)     # buffers are reused from forward to forward
        torch.cuda.synchronize()
    finally:
        for e in engines:
            e.close()
    assert torch.equal(direct.view(torch.int16), staged.view(torch.int16))
    assert torch.equal(again.view(torch.int16), staged.view(torch.int16))


def test_one_call_forward_on_a_single_rank(pkg, dev):
    """o1_sp_forward (the whole sharded forward of a rank as ONE library call: the loop a C host would otherwise
    write around the stage functions) with a single rank must equal hd_forward bit for bit; the multi-rank form of
    the same call is checked on real GPUs by tests/dist_sp_direct_check.py."""
    from o1c_b200 import sp
    T, gh, gw, L = 24, 8, 13, 3
    I = gh * gw
    w = pkg.Weights(n_layers=L, seed=1234, weight_set="B", device=dev)
    pos, _ = pkg.seq_t2i(T, gh, gw)
    rng = np.random.default_rng(1)
    ids = rng.integers(0, 151000, size=T).astype(np.int64)
    ids[-1] = pkg.TMS_ID
    idsd, posd = torch.from_numpy(ids).to(dev), pos.to(dev)
    vin = u16_to_torch(seeded_bf16((I, 3072), 43), dev)
    ref = pkg.Engine(w, T, I).forward(idsd, posd, vin, 0.5)
    e = sp.EngineSP(w, T, I, 1, 0, direct=True)
    try:
        e.connect([e.region])
        out = e.forward_c(idsd, posd, vin, 0.5)
        again = e.forward_c(idsd, posd, vin, 0.25)
        again = e.forward_c(idsd, posd, vin, 0.5)
        torch.cuda.synchronize()
    finally:
        e.close()
    assert torch.equal(out.view(torch.int16), ref.view(torch.int16))
    assert torch.equal(again.view(torch.int16), ref.view(torch.int16))


def test_sp_direct_form_on_real_gpus(pkg):
    """The same comparison with one process per GPU (CUDA IPC mappings, peer stores over NVLink, the flag
    barrier): needs at least two GPUs."""
    import json
    import os
    import subprocess
    import sys
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    world = 4 if n >= 4 else 2
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29531",
           os.path.join(root, "tests", "dist_sp_direct_check.py"), "--text", "64", "--grid", "32", "--layers", "2",
           "--cfg", "--gguf"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=root)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("{")][-1]
    rep = json.loads(line)
    assert rep["ok"] and rep["direct_equals_staged"] and rep["c_driver_equals_staged"] and rep["device_error"] == 0
    assert rep["cfg_step"]["bit_identical_to_one_gpu_step"] and rep["gguf_broadcast"]["forward_identical_on_every_rank"]


@pytest.mark.parametrize("P,direct", [(2, False), (4, True)])
def test_sp_multi_reference_forward_with_visual_conditioning(pkg, dev, P, direct):
    """Edit / personalise layout on sharded rows: K = 4 reference grids behind the target grid, <image_pad> rows
    receive image_embeds and the three DeepStack adds on whichever rank holds them.  Against the unsharded
    hd_forward with the same visual inputs."""
    from o1c_b200 import sp
    refs = [(64, 8, 8, 4, 4), (64, 8, 8, 4, 6), (16, 4, 4, 2, 2), (96, 8, 12, 3, 5)]   # tokens, grid, cond grid
    T, gh, gw = 88, 16, 16
    ids = np.random.default_rng(3).integers(0, 151000, size=T).astype(np.int64)
    o = 8
    for (_, _, _, ch, cw) in refs:                     # <|vision_start|> + one <|image_pad|> run per reference
        ids[o] = 151652
        ids[o + 1:o + 1 + ch * cw] = 151655
        o += 1 + ch * cw + 3
    ids[-2], ids[-1] = 151669, pkg.TMS_ID
    _, pos_t, ar = pkg.seq_ref(ids.tolist(), refs, gh, gw)
    pos = pos_t.numpy()
    I = gh * gw + sum(r[0] for r in refs)
    S = T + I
    assert S % P == 0 and pos.shape[1] == S
    text = ids
    L = 4
    w = pkg.Weights(n_layers=L, seed=1234, weight_set="B", device=dev)
    vmask = np.zeros(S, dtype=np.uint8)
    vmask[:T] = (text == 151655)
    V = int(vmask.sum())
    emb = u16_to_torch(seeded_bf16((V, 4096), 81), dev)
    dss = [u16_to_torch(seeded_bf16((V, 4096), 82 + k, 0.0, 0.5), dev) for k in range(3)]
    vin = u16_to_torch(seeded_bf16((I, 3072), 90), dev)
    idsd, posd, maskd = torch.from_numpy(text).to(dev), torch.from_numpy(pos).to(dev), torch.from_numpy(vmask).to(dev)
    ref = pkg.Engine(w, T, I, ar_len=ar).forward(idsd, posd, vin, 0.3, visual=(maskd, emb, dss))
    engines = [sp.EngineSP(w, T, I, P, r, None, ar_len=ar, direct=direct) for r in range(P)]
    try:
        for e in engines:
            if direct:
                e.connect([x.region for x in engines])
            e.set_visual(maskd, emb, dss)
        assert sum(e.visual is not None for e in engines) >= 1
        out = sp.run_emulated(engines, idsd, posd, vin, 0.3)
        torch.cuda.synchronize()
    finally:
        for e in engines:
            e.close()
    assert_close(out, ref, "B", f"SP{P} multi-reference forward vs unsharded")
    plain = pkg.Engine(w, T, I, ar_len=ar).forward(idsd, posd, vin, 0.3)
    assert parity.metrics(plain, out)[0] > 1e-2           # the visual inputs were applied


def test_sp_barrier_gives_up_when_a_peer_never_arrives(pkg, dev):
    """The flag barrier's wait is bounded: with a peer whose flag nobody sets the kernel returns after about two
    seconds, the device error word carries code 30, and the context stays usable (the next kernels run)."""
    import ctypes as C
    import time
    from o1c_b200 import sp
    w = pkg.Weights(n_layers=1, device=dev)
    engines = [sp.EngineSP(w, 24, 104, 2, r, direct=True) for r in range(2)]
    try:
        for e in engines:
            e.connect([x.region for x in engines])
        e0 = engines[0]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        e0.barrier()                                  # rank 1 never runs its barrier: its flag stays 0
        torch.cuda.synchronize()
        waited = time.perf_counter() - t0
        assert 0.5 < waited < 10.0, waited
        assert pkg.lib.o1_device_error() == 30        # reads and clears the word
        assert pkg.lib.o1_device_error() == 0
        # rank 1 arrives late with the same epoch: rank 0's flag is already there, so this one passes
        engines[1].barrier()
        torch.cuda.synchronize()
        assert pkg.lib.o1_device_error() == 0
        a = torch.ones(1024, device=dev)
        assert float((a + a).sum()) == 2048.0
    finally:
        for e in engines:
            e.close()


def test_sp_direct_form_with_key_split_attention(pkg, dev):
    """Two ranks at S = 2560: each rank's 320 attention items (16 heads x 20 query tiles; sequences this short take
    the one-tile kernel) leave a tail of 24 behind the second wave, which is cut along the keys (two ranges each; the
    partial results fit the rank's idle SwiGLU buffer) and merged; the fully causal first query tile among them has a
    single key tile and leaves one empty partial.  In the direct form the merge kernel writes through the peer table.
    Direct == staged bit for bit (same split), and both agree with the unsharded forward, whose attention runs unsplit."""
    from o1c_b200 import sp
    P = 2
    T, gh, gw, L = 256, 48, 48, 1
    I = gh * gw
    w = pkg.Weights(n_layers=L, seed=1234, weight_set="B", device=dev)
    pos, _ = pkg.seq_t2i(T, gh, gw)
    rng = np.random.default_rng(2)
    ids = rng.integers(0, 151000, size=T).astype(np.int64)
    ids[-1] = pkg.TMS_ID
    idsd, posd = torch.from_numpy(ids).to(dev), pos.to(dev)
    vin = u16_to_torch(seeded_bf16((I, 3072), 44), dev)
    pkg.lib.o1_attention_tail_ways(2)                 # two key ranges per tail item wherever scratch and keys allow
    try:
        staged = sp.run_emulated([sp.EngineSP(w, T, I, P, r, None) for r in range(P)], idsd, posd, vin, 0.5)
        engines = [sp.EngineSP(w, T, I, P, r, direct=True) for r in range(P)]
        try:
            for e in engines:
                e.connect([x.region for x in engines])
            direct = sp.run_emulated(engines, idsd, posd, vin, 0.5)
            torch.cuda.synchronize()
        finally:
            for e in engines:
                e.close()
        pkg.lib.o1_attention_tail_ways(1)             # and the same sharded forward without any split
        unsplit = sp.run_emulated([sp.EngineSP(w, T, I, P, r, None) for r in range(P)], idsd, posd, vin, 0.5)
        torch.cuda.synchronize()
    finally:
        pkg.lib.o1_attention_tail_ways(0)
    ref = pkg.Engine(w, T, I).forward(idsd, posd, vin, 0.5)
    torch.cuda.synchronize()
    assert torch.equal(direct.view(torch.int16), staged.view(torch.int16))
    assert not torch.equal(staged.view(torch.int16), unsplit.view(torch.int16)), "the split path did not run"
    assert_close(staged, unsplit, "C", "split vs unsplit sharded forward")
    assert_close(direct, ref, "C", "sharded forward with key-split attention vs unsharded")
