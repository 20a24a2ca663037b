"""Parity at the sizes the benchmark runs, against the reference's own CUDA build (oracle/_ref/libo1ref.so:
cuBLASLt GEMMs + cuDNN two-pass SDPA, o1.c's production backend) on identical seeded inputs:

  * hd_linear at M in {4115, 4352, 16640} for the seven block shapes, the head and the x_embedder: class C.
    These row counts are what make the persistent GEMM visit several row-tile groups and a partial last group.
  * hd_forward at 16640 rows (3 blocks) and at 4352 rows with all 36 blocks: the checkpoints and the envelope
    of o1.c tests/unit/test_full_forward.c:446-486, block 0 additionally at class D.
  * the 28-step CFG flow-match chain at 4352 rows, 36 blocks, Dev sigmas, guidance 5: the loop of
    tests/unit/test_m1_7_dev.c:477-522 (with the second, unconditional forward and hd_sched_cfg_guided)
    on the reference side, o1_denoise_step_cfg on this side; z after every step against the staircase of
    docs/M1_7_TOLERANCES.md:61-91 (NRMSE / cosine per step range, max_abs <= 8 bf16 ulp of the tensor max).

Measured distances are appended to the file named by O1_PARITY_REPORT when that variable is set.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import parity
import refharness as rh
from parity import metrics_dev, u16_to_torch, seeded_bf16

pytestmark = pytest.mark.gpu

# o1.c tests/unit/test_full_forward.c:446-486: (max NRMSE, min cosine) per checkpoint
ENVELOPE = {"after_block_0_input": (5e-3, 0.9999), "after_block_0": (1e-2, 0.9999), "after_block_mid": (1e-2, 0.9999),
            "after_block_last": (3e-2, 0.999), "before_final_norm": (3e-2, 0.999), "after_final_norm": (0.1, 0.99),
            "output": (0.18, 0.99)}
# docs/M1_7_TOLERANCES.md:61-91
def staircase(step):
    return (5e-3, 0.9999) if step <= 15 else ((1e-2, 0.9995) if step <= 23 else (2.5e-2, 0.999))


@pytest.fixture(scope="module")
def ref():
    r = parity.reflib()
    if r is None:
        pytest.skip("oracle/_ref/libo1ref.so not built")
    return r


def _check(what, got, want, lim, rec):
    """Records the distance and notes a violated bar in rec["failed"] (asserted by _done once everything is measured)."""
    nrmse, cos, mx, bad = metrics_dev(got, want)
    rec[what] = {"nrmse": nrmse, "cos": cos, "max_abs": mx}
    if bad:
        rec.setdefault("failed", []).append(f"{what}: {bad} non-finite values")
    if not (nrmse <= lim[0] and cos >= lim[1]):
        rec.setdefault("failed", []).append(f"{what}: nrmse={nrmse:.3e} (<= {lim[0]}) cos={cos:.6f} (>= {lim[1]})")


def _done(rec):
    parity.report(rec)
    assert not rec.get("failed"), "\n".join(rec["failed"])


LINEAR_SHAPES = [("q_proj", 4096, 4096, False), ("k_proj", 1024, 4096, False), ("o_proj", 4096, 4096, False),
                 ("gate_proj", 12288, 4096, False), ("down_proj", 4096, 12288, False), ("head", 3072, 4096, True),
                 ("x_embed1", 1024, 3072, False), ("x_embed2", 4096, 1024, True)]


@pytest.mark.parametrize("M", [4115, 4352, 16640])
def test_linear_at_benchmark_rows_vs_reference_cublaslt(pkg, dev, ref, M):
    rt = ref.hd_gemm_runtime_init(0, 64 << 20)
    assert rt
    ref.hd_gemm_set_backend(1)
    rec = {"test": "hd_linear", "M": M}
    try:
        for i, (name, N, K, has_bias) in enumerate(LINEAR_SHAPES):
            x = u16_to_torch(seeded_bf16((M, K), 100 + i), dev)
            w = u16_to_torch(seeded_bf16((N, K), 200 + i, 0.0, 0.02), dev)
            b = u16_to_torch(seeded_bf16((N,), 300 + i, 0.0, 0.02), dev) if has_bias else None
            canary = 0x7FC1                                   # a NaN pattern: every element must be overwritten
            y = torch.full((M + 1, N), canary, dtype=torch.int16, device=dev).view(torch.bfloat16)
            yr = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            pkg.lib.hd_linear(pkg.ptr(x), pkg.ptr(w), pkg.ptr(b), pkg.ptr(y), M, N, K, 1)
            ref.hd_linear(pkg.ptr(x), pkg.ptr(w), pkg.ptr(b), pkg.ptr(yr), M, N, K, 1)
            torch.cuda.synchronize()
            pkg.check_cuda_errbuf(name)
            assert not ref.hd_cuda_last_error(), ref.hd_cuda_last_error()
            assert bool((y[M].view(torch.int16) == canary).all()), f"{name}: wrote past row M"
            _check(name, y[:M], yr, parity.TOL["C"], rec)
    finally:
        ref.hd_gemm_runtime_destroy(rt)
    _done(rec)


def _forward_pair(pkg, dev, w, T, gh, gw, names, z_seed=43):
    """hd_forward of this library and of the reference's production build on the same weights and inputs."""
    I = gh * gw
    eng = pkg.Engine(w, T, I)
    reng = rh.RefEngine(w.binding, T, gh, gw, dev, production=True)
    ids_c, _ = rh.seeded_ids(T)
    ids = ids_c.to(dev)
    z = rh.seeded_latent(I, z_seed).to(dev)
    pos, _ = pkg.seq_t2i(T, gh, gw)
    mine, md = eng.forward(ids, pos.to(dev), z, 0.5, diag_names=names)
    theirs = torch.empty_like(mine)
    rd = reng.forward(ids, z, 0.5, theirs, diag_names=names)
    torch.cuda.synchronize()
    reng.close()
    return mine, md, theirs, rd


@pytest.mark.parametrize("wset", ["B", "A"])
def test_forward_at_16640_rows_vs_reference_production_build(pkg, dev, ref, wset):
    T, gh, gw, L = 256, 128, 128, 3                  # 3 blocks: the first, the middle and the last hook are distinct
    w = pkg.Weights(n_layers=L, seed=1234, weight_set=wset, device=dev)
    names = ("after_block_0_input", "after_block_0", "after_block_mid", "after_block_last", "after_final_norm")
    mine, md, theirs, rd = _forward_pair(pkg, dev, w, T, gh, gw, names)
    rec = {"test": "forward", "rows": T + gh * gw, "layers": L, "weights": wset}
    for n in names:
        _check(n, md[n], rd[n], ENVELOPE[n], rec)
    _check("after_block_0 (class D)", md["after_block_0"], rd["after_block_0"], parity.TOL["D"], rec)
    _check("output", mine, theirs, ENVELOPE["output"], rec)
    _check("output image rows", mine[T:], theirs[T:], ENVELOPE["output"], rec)
    _done(rec)


@pytest.fixture(scope="module")
def weights36(pkg, dev):
    return {s: None for s in "AB"}


def _w36(pkg, dev, cache, wset):
    for k in cache:                                  # one 15 GB arena at a time
        if k != wset:
            cache[k] = None
    if cache[wset] is None:
        torch.cuda.empty_cache()
        cache[wset] = pkg.Weights(n_layers=36, seed=1234, weight_set=wset, device=dev)
    return cache[wset]


@pytest.mark.parametrize("wset", ["B", "A"])
def test_forward_all_36_blocks_at_4352_rows_vs_reference_production_build(pkg, dev, ref, weights36, wset):
    """All 36 blocks.  Weight set A (every tensor N(0, 0.02), norm gains included) keeps both branches of every
    block tiny, so the stack is nearly the identity and the envelope is met with orders of magnitude to spare.
    Set B (norm gains 1 + N(0, 0.02)) makes every block contribute O(1); with RANDOM weights two correct bf16
    implementations then drift apart faster than the envelope, which was measured on the trained model: the
    reference's own two backends (its source GEMM + eager attention against its cuBLASLt + cuDNN build) are
    compared on the same inputs, and this library has to stay within 1.5 x their distance (or the envelope)."""
    T, gh, gw = 256, 64, 64
    w = _w36(pkg, dev, weights36, wset)
    names = ("after_block_0_input", "after_block_0", "after_block_mid", "after_block_last", "before_final_norm",
             "after_final_norm")
    mine, md, theirs, rd = _forward_pair(pkg, dev, w, T, gh, gw, names)
    rec = {"test": "forward", "rows": T + gh * gw, "layers": 36, "weights": wset}
    spread = {}
    if wset == "B":
        src = rh.RefEngine(w.binding, T, gh, gw, dev, production=False)
        ids = rh.seeded_ids(T)[0].to(dev)
        z = rh.seeded_latent(gh * gw, 43).to(dev)
        out_src = torch.empty_like(theirs)
        sd = src.forward(ids, z, 0.5, out_src, diag_names=names)
        torch.cuda.synchronize()
        src.close()
        for n in names:
            spread[n] = metrics_dev(sd[n], rd[n])[0]
        spread["output"] = metrics_dev(out_src, theirs)[0]
        rec["reference_source_vs_production_nrmse"] = spread

    def lim(n):
        e = ENVELOPE[n]
        return (max(e[0], 1.5 * spread[n]), min(e[1], 1.0 - 2.0 * (1.5 * spread[n]) ** 2)) if n in spread else e
    for n in names:
        _check(n, md[n], rd[n], lim(n), rec)
    _check("after_block_0 (class D)", md["after_block_0"], rd["after_block_0"], parity.TOL["D"], rec)
    _check("output", mine, theirs, lim("output"), rec)
    _check("output image rows", mine[T:], theirs[T:], lim("output"), rec)
    _done(rec)


@pytest.mark.parametrize("wset,g", [("A", 5.0), ("A", 1.0), ("B", 1.0), ("B", 5.0)])
def test_chain_28_steps_at_4352_rows_vs_reference(pkg, dev, ref, orc, weights36, wset, g):
    """Free-running 28-step chains on both sides from the same initial latent (the reference's RNG restatement x 8);
    additionally every step is repeated from the REFERENCE's latent, which isolates one step's distance.

    guidance 1 is the composition the staircase was written for (one prediction per step: with g = 1 the guided
    output is the conditional one exactly), asserted as it stands for BASELINE's weights (set A) and with twice
    the NRMSE for set B, whose random unit-gain blocks drift faster than the trained model (see the forward test).
    guidance 5 combines two predictions as g x_c + (1-g) x_u, which multiplies their independent rounding
    noise by sqrt(g^2 + (g-1)^2) = 6.4 in the part (1 - sigma'/sigma) of z' that comes from the prediction: the
    staircase is scaled by max(1, that factor) per step for set A, and set B is measured and reported only.
    Set B's free-running chain is asserted through step 23: in the last four steps sigma'/sigma -> 0 turns z' into
    the prediction itself, and the random unit-gain network's sensitivity to its input takes over (the two
    chains decorrelate although every single step, taken from the reference's latent, stays at the forward's
    own distance); those steps are covered by the per-step checks on the reference's latent."""
    T, gh, gw = 256, 64, 64
    I = gh * gw
    w = _w36(pkg, dev, weights36, wset)
    eng = pkg.Engine(w, T, I)
    reng = rh.RefEngine(w.binding, T, gh, gw, dev, production=True)
    ids_c, ids_u = (t.to(dev) for t in rh.seeded_ids(T))
    pos, _ = pkg.seq_t2i(T, gh, gw)
    posd = pos.to(dev)
    z0 = np.empty((I, 3072), dtype=np.uint16)
    assert orc.orc_initial_latent(123456, gh * 32, gw * 32, 32, 8.0, parity.np_ptr(z0)) == 0
    sig = pkg.dev_sigmas()
    z_mine = u16_to_torch(z0, dev)
    z_ref = z_mine.clone()
    zn_mine, zn_ref, zn_forced = (torch.empty_like(z_mine) for _ in range(3))
    rec = {"test": "chain", "rows": T + I, "layers": 36, "weights": wset, "guidance": g, "steps": []}
    failures = []
    try:
        for i in range(28):
            reng.cfg_step(ids_c, ids_u, z_ref, zn_ref, sig[i], sig[i + 1], g)
            eng.denoise_step_cfg(ids_c, ids_u, posd, z_ref, sig[i], sig[i + 1], g, zn_forced)
            # the predictions behind that step, on identical input: the whole-model output envelope of
            # o1.c tests/unit/test_full_forward.c:484
            xp_mine = eng.xp.view(2, T + I, 3072)
            n_x, c_x, _, bad_x = metrics_dev(xp_mine[0], reng.xc)
            eng.denoise_step_cfg(ids_c, ids_u, posd, z_mine, sig[i], sig[i + 1], g, zn_mine)
            torch.cuda.synchronize()
            n_f, c_f, m_f, bad_f = metrics_dev(zn_forced, zn_ref)
            n_c, c_c, m_c, bad_c = metrics_dev(zn_mine, zn_ref)
            ulp = parity.bf16_ulp_of_max(zn_ref)
            rec["steps"].append({"step": i, "chain_nrmse": n_c, "chain_cos": c_c, "chain_max_abs_ulps": m_c / ulp,
                                 "single_nrmse": n_f, "single_cos": c_f, "single_max_abs_ulps": m_f / ulp,
                                 "x_pred_nrmse": n_x, "x_pred_cos": c_x})
            if bad_f or bad_c or bad_x:
                failures.append(f"step {i}: non-finite values")
            if not (n_x <= ENVELOPE["output"][0] and c_x >= ENVELOPE["output"][1]):
                failures.append(f"step {i} x_pred on the reference's latent: nrmse={n_x:.3e} cos={c_x:.6f}")
            amp = max(1.0, (1.0 - sig[i + 1] / sig[i]) * (g * g + (g - 1.0) * (g - 1.0)) ** 0.5) if g != 1.0 else 1.0
            k = amp * (2.0 if wset == "B" else 1.0)
            lim_n, lim_c = staircase(i)
            lim_n, lim_c = lim_n * k, 1.0 - (1.0 - lim_c) * k * k
            if wset == "A" or (g == 1.0 and i <= 23):
                if not (n_c <= lim_n and c_c >= lim_c and m_c <= 8 * k * ulp):
                    failures.append(f"step {i} chain: nrmse={n_c:.3e} (<= {lim_n:.3g}) cos={c_c:.6f} (>= {lim_c:.6f}) "
                                    f"max_abs={m_c / ulp:.1f} ulp (<= {8 * k:.0f})")
            z_mine, zn_mine = zn_mine, z_mine
            z_ref, zn_ref = zn_ref, z_ref
    finally:
        reng.close()
        parity.report(rec)
    assert not failures, "\n".join(failures)


def test_mask_rewritten_in_place_is_probed_again(pkg, dev, orc):
    """The reference passes attention structure as an [S,S] additive mask that a host may rewrite, or free and
    re-allocate at the same address, between requests (src/runtime/generate.c:1202-1209): nothing about a mask
    pointer may be remembered."""
    S, H, KV = 300, 4, 2
    qh, kh, vh = seeded_bf16((H, S, 128), 1), seeded_bf16((KV, S, 128), 2), seeded_bf16((KV, S, 128), 3)
    q, k, v = (u16_to_torch(a, dev) for a in (qh, kh, vh))
    mask = torch.empty(S, S, dtype=torch.bfloat16, device=dev)
    outs = {}
    for ar in (40, 200):
        m = np.empty((S, S), dtype=np.uint16)
        orc.orc_prefix_causal_mask(S, ar, parity.np_ptr(m))
        mask.copy_(u16_to_torch(m, dev))                              # same address, other causal prefix
        out = torch.empty(S, H, 128, dtype=torch.bfloat16, device=dev)      # hd_attention_eager writes seq-major
        pkg.lib.hd_attention_eager(pkg.ptr(q), pkg.ptr(k), pkg.ptr(v), pkg.ptr(mask), None, None, pkg.ptr(out), H, KV, S,
                                   128, 128 ** -0.5)
        torch.cuda.synchronize()
        pkg.check_cuda_errbuf("attention")
        want = np.empty((S, H, 128), dtype=np.uint16)
        orc.orc_attention(parity.np_ptr(qh), parity.np_ptr(kh), parity.np_ptr(vh), parity.np_ptr(want), H, KV, S, 128,
                          128 ** -0.5, ar)
        parity.assert_close(parity.torch_to_u16(out), want, "D", f"ar_len {ar}")
        outs[ar] = out
    assert parity.metrics(outs[40], outs[200])[0] > 1e-2


def test_split_pass_writes_only_its_rows(pkg, dev):
    """hd_sdpa_execute_split_pass (include/hd_cudnn_sdpa.h:77-82): pass 0 = causal rows [0, ar_len), pass 1 = the
    rest; both together equal hd_sdpa_execute_split, and each leaves the other's rows untouched."""
    S, H, KV, ar = 700, 8, 2, 300
    q = u16_to_torch(seeded_bf16((H, S, 128), 1), dev)
    k = u16_to_torch(seeded_bf16((KV, S, 128), 2), dev)
    v = u16_to_torch(seeded_bf16((KV, S, 128), 3), dev)
    plan = C.c_void_p()
    assert pkg.lib.hd_sdpa_create_split(C.byref(plan), 1, H, KV, S, ar, 128, 128 ** -0.5) == 0
    full = torch.empty(H, S, 128, dtype=torch.bfloat16, device=dev)
    assert pkg.lib.hd_sdpa_execute_split(plan, pkg.ptr(q), pkg.ptr(k), pkg.ptr(v), pkg.ptr(full), None) == 0
    canary = 0x7FC1
    two = torch.full((H, S, 128), canary, dtype=torch.int16, device=dev)
    assert pkg.lib.hd_sdpa_execute_split_pass(plan, 0, pkg.ptr(q), pkg.ptr(k), pkg.ptr(v), pkg.ptr(two), None) == 0
    torch.cuda.synchronize()
    assert bool((two[:, ar:] == canary).all()) and bool((two[:, :ar] == full.view(torch.int16)[:, :ar]).all())
    assert pkg.lib.hd_sdpa_execute_split_pass(plan, 1, pkg.ptr(q), pkg.ptr(k), pkg.ptr(v), pkg.ptr(two), None) == 0
    torch.cuda.synchronize()
    assert bool((two == full.view(torch.int16)).all())
    pkg.lib.hd_sdpa_destroy(plan)


def test_cfg_step_with_a_shorter_unconditional_prompt_vs_oracle(pkg, orc, dev):
    """The unconditional branch has its own token count, positions and causal prefix
    (o1.c src/runtime/generate.c:1111-1206, :1340-1356)."""
    Tc, Tu, gh, gw, L, g = 14, 6, 4, 6, 2, 5.0
    I = gh * gw
    w = pkg.Weights(n_layers=L, seed=1234, weight_set="B", device=dev)
    eng = pkg.Engine(w, Tc, I)                                  # sized for the longer sequence
    rng = np.random.default_rng(11)
    ids = {}
    for name, T in (("c", Tc), ("u", Tu)):
        a = rng.integers(0, 151000, size=T).astype(np.int64)
        a[-1] = pkg.TMS_ID
        ids[name] = a
    pos_c, ar_c = pkg.seq_t2i(Tc, gh, gw)
    pos_u, ar_u = pkg.seq_t2i(Tu, gh, gw)
    z0 = seeded_bf16((I, 3072), 21, 0.0, 8.0)
    s0, s1 = 0.9, 0.8
    zn = eng.denoise_step_cfg_branches((torch.from_numpy(ids["c"]).to(dev), pos_c.to(dev), ar_c),
                                       (torch.from_numpy(ids["u"]).to(dev), pos_u.to(dev), ar_u),
                                       u16_to_torch(z0, dev), s0, s1, g)
    torch.cuda.synchronize()
    hw = parity.HostWeights(pkg, L, 1234, "B")
    xc = parity.oracle_forward(hw, ids["c"], pos_c.numpy(), ar_c, z0, 1.0 - np.float32(s0))
    xu = parity.oracle_forward(hw, ids["u"], pos_u.numpy(), ar_u, z0, 1.0 - np.float32(s0))
    want = np.empty_like(z0)
    orc.orc_sched_cfg_flow_step(parity.np_ptr(z0), parity.np_ptr(np.ascontiguousarray(xc[Tc:])),
                                parity.np_ptr(np.ascontiguousarray(xu[Tu:])), s0, s1, g, parity.np_ptr(want), z0.size)
    nrmse, cos, _, bad = parity.metrics(parity.torch_to_u16(zn), want)
    assert bad == 0 and nrmse <= 5e-3 and cos >= 0.9999, (nrmse, cos)
    # and the equal-length entry point is the same function with both branches alike
    a = eng.denoise_step_cfg(torch.from_numpy(ids["c"]).to(dev), torch.from_numpy(ids["c"]).to(dev), pos_c.to(dev),
                             u16_to_torch(z0, dev), s0, s1, g)
    b = eng.denoise_step_cfg_branches((torch.from_numpy(ids["c"]).to(dev), pos_c.to(dev), ar_c),
                                      (torch.from_numpy(ids["c"]).to(dev), pos_c.to(dev), ar_c),
                                      u16_to_torch(z0, dev), s0, s1, g)
    torch.cuda.synchronize()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
