"""Pins the CPU oracle (oracle/o1_oracle.c) against the reference's own vectors:
the scheduler dumps, outputs of the reference's torch_rng.c / sequence.c /
scheduler.c captured in tests/golden/, torch's CPU generator, and closed-form
fp64 evaluations of the primitives (the style of o1.c tests/unit/test_primitives.c:142-555).
"""
import ctypes as C
import json
import os

import numpy as np
import pytest
import torch

import parity
from parity import np_ptr, bf16_to_f32_np, f32_to_bf16_np


def test_rng_matches_reference_torch_rng(orc, golden):
    g = np.load(os.path.join(golden, "rng_ref.npz"))
    for n in (1, 8, 15, 16, 17, 31, 32, 1024):
        out = np.empty(n, dtype=np.float32)
        orc.orc_torch_randn(123457, np_ptr(out), n)
        assert (out.view(np.uint32) == g[f"randn_{n}"].view(np.uint32)).all(), n
    u = np.empty(2000, dtype=np.uint32)
    orc.orc_torch_rng_u32(123457, np_ptr(u), 2000)
    assert (u == g["u32_2000"]).all()
    h = orc.orc_rng_create(1234)
    chain = np.empty((8, 64), dtype=np.float32)
    for i in range(8):
        orc.orc_rng_randn(h, np_ptr(chain[i]), 64)
    orc.orc_rng_free(h)
    assert (chain.view(np.uint32) == g["chain_1234_8x64"].view(np.uint32)).all()


def test_rng_matches_torch_cpu_generator(orc):
    # n < 16 takes torch's serial double path: bit-exact.  n >= 16 takes normal_fill, which torch
    # vectorises with its own logf/sincosf on AVX2 hosts: equal up to a few float ulps there.
    for n in (1, 8, 15, 16, 17, 31, 32, 1024, 4099):
        g = torch.Generator(device="cpu")
        g.manual_seed(123457)
        ref = torch.randn(n, generator=g, dtype=torch.float32).numpy()
        out = np.empty(n, dtype=np.float32)
        orc.orc_torch_randn(123457, np_ptr(out), n)
        if n < 16:
            assert (out.view(np.uint32) == ref.view(np.uint32)).all(), n
        else:
            assert np.abs(out - ref).max() <= 4e-6, n


def test_sigma_schedules(orc, golden):
    ref = json.load(open(os.path.join(golden, "sigmas_ref.json")))
    dump = json.load(open(os.path.join(golden, "scheduler_dump.json")))
    s = np.zeros(64, dtype=np.float32)
    assert orc.orc_sigmas_dev(np_ptr(s)) == 29
    assert (s[:29] == np.array(ref["dev"], dtype=np.float32)).all()
    assert orc.orc_sigmas_flash(28, 1.0, np_ptr(s)) == 29
    assert (s[:29] == np.array(ref["flash_28_1"], dtype=np.float32)).all()
    assert orc.orc_sigmas_flash(28, 3.0, np_ptr(s)) == 29
    assert (s[:29] == np.array(ref["flow_match_28_3"], dtype=np.float32)).all()
    assert orc.orc_sigmas_default(50, 3.0, np_ptr(s)) == 51
    assert (s[:51] == np.array(ref["default_50_3"], dtype=np.float32)).all()
    # against the Python-oracle dump the reference's own test uses (tolerance 1e-6 there)
    for rec in dump["matrix"]:
        if rec["tlist"]:
            n = orc.orc_sigmas_dev(np_ptr(s))
        elif rec["sched"] in ("flash", "flow_match"):
            n = orc.orc_sigmas_flash(rec["steps"], rec["shift"], np_ptr(s))
        else:
            n = orc.orc_sigmas_default(rec["steps"], rec["shift"], np_ptr(s))
        assert n == len(rec["sigmas"])
        assert np.abs(s[:n] - np.array(rec["sigmas"], dtype=np.float32)).max() <= 1e-6, rec["name"]
        for i, v in enumerate(rec["noisescale"]):
            assert abs(orc.orc_noise_scale(n, i, 8.0, 8.0) - v) <= 1e-6


def test_scheduler_steps_against_dump(orc, golden):
    """Replays tests/unit/scheduler_matrix.c: one generator seeded 1234, per recipe z, mo, unused
    (and noise for flash), one Euler step, compared with the dump's STEP line (<= 1e-5)."""
    dump = json.load(open(os.path.join(golden, "scheduler_dump.json")))["matrix"]
    h = orc.orc_rng_create(1234)
    N = 64
    checked = 0
    for rec in dump:
        z, mo, unused = (np.empty(N, dtype=np.float32) for _ in range(3))
        for a in (z, mo, unused):
            orc.orc_rng_randn(h, np_ptr(a), N)
        mo = (mo * np.float32(0.3)).astype(np.float32)
        s0, s1 = np.float32(rec["sigmas"][0]), np.float32(rec["sigmas"][1])
        want = np.array(rec["step"], dtype=np.float32)
        if rec["sched"] == "flash":
            noise = np.empty(N, dtype=np.float32)
            orc.orc_rng_randn(h, np_ptr(noise), N)
            orc.orc_noise_clamp(np_ptr(noise), N, 8.0)
            den, out = np.empty(N, dtype=np.float32), np.empty(N, dtype=np.float32)
            orc.orc_sched_denoised(np_ptr(z), np_ptr(mo), float(s0), np_ptr(den), N)
            orc.orc_sched_z_next(np_ptr(noise), np_ptr(den), float(s1), 8.0, np_ptr(out), N)
            assert np.abs(out - want[:N]).max() <= 1e-5, rec["name"]
            checked += 1
        elif rec["sched"] == "flow_match":
            # the device step works on bf16 z; the dump is fp32, so check the fp32 formula here
            out = z + (s1 - s0) * mo
            assert np.abs(out - want[:N]).max() <= 1e-5, rec["name"]
            # and the bf16 kernel restatement agrees with it to bf16 rounding
            zb = f32_to_bf16_np(z)
            zn = np.empty(N, dtype=np.uint16)
            orc.orc_sched_flow_match_step(np_ptr(zb), np_ptr(mo), float(s0), float(s1), np_ptr(zn), N)
            expect = f32_to_bf16_np(bf16_to_f32_np(zb) + (s1 - s0) * mo)
            assert np.abs(zn.astype(np.int32) - expect.astype(np.int32)).max() <= 1
            checked += 1
        else:
            break   # UniPC recipe: draws differ from here on, covered by test_unipc_pointwise
    orc.orc_rng_free(h)
    assert checked >= 4


def test_unipc_pointwise_against_fp64(orc):
    rng = np.random.default_rng(5)
    n = 257
    last, mo0, mo_old, conv = (rng.standard_normal(n).astype(np.float32) for _ in range(4))
    c = dict(sig_t=0.8, sig_s0=0.9, alpha_t=0.2, h_phi_1=-0.11, B_h=0.12, r0=0.4, r1=0.5, inv=1.3)
    out = np.empty(n, dtype=np.float32)
    for order in (1, 2):
        orc.orc_unipc_correct(np_ptr(last), np_ptr(mo0), np_ptr(mo_old), np_ptr(conv), c["sig_t"], c["sig_s0"],
                              c["alpha_t"], c["h_phi_1"], c["B_h"], c["r0"], c["r1"], c["inv"], order,
                              np_ptr(out), n)
        x_t = (c["sig_t"] / c["sig_s0"]) * last.astype(np.float64) - c["alpha_t"] * c["h_phi_1"] * mo0
        d1t = conv.astype(np.float64) - mo0
        corr = c["r1"] * d1t + (c["r0"] * (mo_old.astype(np.float64) - mo0) * c["inv"] if order == 2 else 0)
        assert np.abs(out - (x_t - c["alpha_t"] * c["B_h"] * corr)).max() <= 1e-5
        orc.orc_unipc_predict(np_ptr(last), np_ptr(mo0), np_ptr(mo_old), c["sig_t"], c["sig_s0"], c["alpha_t"],
                              c["h_phi_1"], c["B_h"], c["r1"], c["inv"], order, np_ptr(out), n)
        x_t = (c["sig_t"] / c["sig_s0"]) * last.astype(np.float64) - c["alpha_t"] * c["h_phi_1"] * mo0
        if order == 2:
            x_t = x_t - c["alpha_t"] * c["B_h"] * (c["r1"] * (mo_old.astype(np.float64) - mo0) * c["inv"])
        assert np.abs(out - x_t).max() <= 1e-5
    orc.orc_unipc_convert(np_ptr(last), np_ptr(mo0), 0.7, np_ptr(out), n)
    assert np.abs(out - (last.astype(np.float64) - 0.7 * mo0)).max() <= 1e-6


def test_seq_t2i_positions(orc, golden, pkg):
    g = np.load(os.path.join(golden, "seq_t2i.npz"))
    for tag in ("s23", "c0", "odd"):
        T, gh, gw, S, ar = (int(v) for v in g[f"{tag}_meta"][:5])
        pos = np.empty((3, S), dtype=np.float32)
        assert orc.orc_seq_t2i(T, gh, gw, 4096, np_ptr(pos)) == ar == T - 1
        assert (pos == g[f"{tag}_pos"]).all()
        p2, ar2 = pkg.seq_t2i(T, gh, gw)          # the host-side mirror used by the product path
        assert ar2 == ar and (p2.numpy() == g[f"{tag}_pos"]).all()
    # docs/M1_NUMERICAL_CONTRACT.md:9-18 / sequence.c:97-100: S=23, T=19, 2x2 grid
    pos = g["s23_pos"]
    assert list(pos[0, 19:]) == [4096] * 4 and list(pos[1, 19:]) == [4096, 4096, 4097, 4097]
    assert list(pos[2, 19:]) == [4096, 4097, 4096, 4097] and list(pos[0, :19]) == list(range(19))


def test_prefix_causal_mask_bits(orc):
    S, ar = 37, 11
    m = np.empty((S, S), dtype=np.uint16)
    orc.orc_prefix_causal_mask(S, ar, np_ptr(m))
    for r in range(S):
        for c in range(S):
            assert m[r, c] == (0xFF7F if (r < ar and c > r) else 0)   # sequence.c:22, :120-142


def test_bf16_rounding_rule(orc):
    # RNE by integer add, no NaN special case (cuda_internal.h:29-36)
    cases = {1.0: 0x3F80, 1.00390625: 0x3F80, 1.01171875: 0x3F82, -2.5: 0xC020, 3.3895314e38: 0x7F7F}
    for f, bits in cases.items():
        assert orc.orc_f32_to_bf16(f) == bits
    x = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    mine = f32_to_bf16_np(x)
    th = torch.from_numpy(x).bfloat16().view(torch.int16).numpy().view(np.uint16)
    assert (mine == th).all()
    assert all(orc.orc_f32_to_bf16(float(v)) == int(b) for v, b in zip(x[:64], mine[:64]))


def _bf(a):
    return f32_to_bf16_np(np.asarray(a, dtype=np.float32))


def test_primitives_against_fp64(orc):
    rng = np.random.default_rng(1)
    rows, cols = 5, 96
    x, w = _bf(rng.standard_normal((rows, cols))), _bf(1 + 0.1 * rng.standard_normal(cols))
    y = np.empty_like(x)
    orc.orc_rmsnorm(np_ptr(x), np_ptr(w), np_ptr(y), rows, cols, 1e-6)
    xf, wf = bf16_to_f32_np(x).astype(np.float64), bf16_to_f32_np(w).astype(np.float64)
    ref = wf * xf / np.sqrt((xf * xf).mean(-1, keepdims=True) + 1e-6)
    parity.assert_close(y, ref.astype(np.float32), "B", "rmsnorm")
    # silu / swiglu / residual
    g, u = _bf(rng.standard_normal(1000) * 3), _bf(rng.standard_normal(1000))
    out = np.empty_like(g)
    gf, uf = bf16_to_f32_np(g).astype(np.float64), bf16_to_f32_np(u).astype(np.float64)
    orc.orc_silu(np_ptr(g), np_ptr(out), 1000)
    parity.assert_close(out, (gf / (1 + np.exp(-gf))).astype(np.float32), "B", "silu")
    orc.orc_swiglu(np_ptr(g), np_ptr(u), np_ptr(out), 1000)
    parity.assert_close(out, (gf / (1 + np.exp(-gf)) * uf).astype(np.float32), "B", "swiglu")
    orc.orc_residual_add(np_ptr(g), np_ptr(u), np_ptr(out), 1000)
    assert (out == _bf(gf + uf)).all()
    # linear 7x5x6 (the shape of test_primitives.c:273-298), with and without bias
    M, N, K = 7, 5, 6
    a, b, bias = _bf(rng.standard_normal((M, K))), _bf(rng.standard_normal((N, K))), _bf(rng.standard_normal(N))
    yy = np.empty((M, N), dtype=np.uint16)
    ref = bf16_to_f32_np(a).astype(np.float64) @ bf16_to_f32_np(b).astype(np.float64).T
    orc.orc_linear(np_ptr(a), np_ptr(b), None, np_ptr(yy), M, N, K)
    parity.assert_close(yy, ref.astype(np.float32), "C", "linear")
    orc.orc_linear(np_ptr(a), np_ptr(b), np_ptr(bias), np_ptr(yy), M, N, K)
    parity.assert_close(yy, (ref + bf16_to_f32_np(bias)).astype(np.float32), "C", "linear+bias")
    # timestep embedding: cos half first (gemm.cu:531-545)
    t = np.array([500.0], dtype=np.float32)
    e = np.empty(256, dtype=np.float32)
    orc.orc_timestep_embed(np_ptr(t), np_ptr(e), 1, 256)
    f = np.exp(-np.log(10000.0) * np.arange(128) / 128.0)
    assert np.abs(e[:128] - np.cos(500.0 * f)).max() < 2e-4 and np.abs(e[128:] - np.sin(500.0 * f)).max() < 2e-4


def test_mrope_axis_selection_and_rotary(orc):
    S, D = 6, 128
    pos = np.stack([np.arange(S) + 1, (np.arange(S) + 1) * 10, (np.arange(S) + 1) * 100]).astype(np.float32)
    sec = np.array([24, 20, 20], dtype=np.int64)
    cs, sn = np.empty((S, D), dtype=np.float32), np.empty((S, D), dtype=np.float32)
    orc.orc_mrope_cos_sin(np_ptr(pos), 1, S, np_ptr(sec), 3, D, 5e6, 1.0, 1, np_ptr(cs), np_ptr(sn))
    for kk in range(64):
        axis = kk % 3 if (kk % 3 in (1, 2) and kk // 3 < 20) else 0     # rope.cu:43-57
        inv = np.exp(-np.log(5e6) * 2 * kk / D)
        for s in range(S):
            ang = inv * pos[axis, s]
            assert abs(cs[s, kk] - np.cos(ang)) < 1e-3 and abs(sn[s, kk + 64] - np.sin(ang)) < 1e-3
    assert (cs[:, :64] == cs[:, 64:]).all() and (sn[:, :64] == sn[:, 64:]).all()
    x = _bf(np.random.default_rng(2).standard_normal((2, S, D)))
    y = np.empty_like(x)
    orc.orc_apply_rotary(np_ptr(x), np_ptr(cs), np_ptr(sn), np_ptr(y), 2, S, D)
    xf = bf16_to_f32_np(x).astype(np.float64)
    rot = np.concatenate([-xf[..., 64:], xf[..., :64]], -1)
    parity.assert_close(y, (xf * cs + rot * sn).astype(np.float32), "B", "rotary")


def test_attention_against_fp64(orc):
    rng = np.random.default_rng(3)
    H, KV, S, D, ar = 4, 2, 33, 128, 9
    q, k, v = (_bf(rng.standard_normal((n, S, D))) for n in (H, KV, KV))
    out = np.empty((S, H, D), dtype=np.uint16)
    orc.orc_attention(np_ptr(q), np_ptr(k), np_ptr(v), np_ptr(out), H, KV, S, D, D ** -0.5, ar)
    qf, kf, vf = (bf16_to_f32_np(t).astype(np.float64) for t in (q, k, v))
    ref = np.empty((S, H, D))
    for h in range(H):
        sc = qf[h] @ kf[h // 2].T * D ** -0.5
        for r in range(ar):
            sc[r, r + 1:] = -np.inf
        p = np.exp(sc - sc.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        ref[:, h] = p @ vf[h // 2]
    parity.assert_close(out, ref.astype(np.float32), "D", "attention")


def test_block_against_fp64_composition(orc, pkg):
    """orc_decoder_block vs an unrounded fp64 composition of the same layer (class D, the
    reference's bar for a block output and its internals, tests/unit/test_block.c:281-302)."""
    hw = parity.HostWeights(pkg, 1, 77, "B")
    T, gh, gw = 6, 3, 4
    S = T + gh * gw
    pos, ar = pkg.seq_t2i(T, gh, gw)
    x = parity.seeded_bf16((S, pkg.HIDDEN), 5)
    out, ints = parity.oracle_block(hw, 0, x, pos.numpy(), ar)
    f = lambda n: bf16_to_f32_np(hw.tensor(0, n)).astype(np.float64)
    xf = bf16_to_f32_np(x).astype(np.float64)
    rms = lambda a, w: w * a / np.sqrt((a * a).mean(-1, keepdims=True) + 1e-6)
    ln = rms(xf, f("input_ln"))
    q = (ln @ f("q_proj").T).reshape(S, 32, 128)
    k = (ln @ f("k_proj").T).reshape(S, 8, 128)
    v = (ln @ f("v_proj").T).reshape(S, 8, 128)
    q, k = rms(q, f("q_norm")), rms(k, f("k_norm"))
    cs, sn = np.empty((S, 128), dtype=np.float32), np.empty((S, 128), dtype=np.float32)
    sec = np.array([24, 20, 20], dtype=np.int64)
    orc.orc_mrope_cos_sin(np_ptr(np.ascontiguousarray(pos.numpy())), 1, S, np_ptr(sec), 3, 128, 5e6, 1.0, 1,
                          np_ptr(cs), np_ptr(sn))
    rope = lambda a: a * cs[:, None, :] + np.concatenate([-a[..., 64:], a[..., :64]], -1) * sn[:, None, :]
    q, k = rope(q), rope(k)
    att = np.empty((S, 32, 128))
    for h in range(32):
        sc = q[:, h] @ k[:, h // 4].T * 128 ** -0.5
        for r in range(ar):
            sc[r, r + 1:] = -np.inf
        p = np.exp(sc - sc.max(-1, keepdims=True))
        att[:, h] = (p / p.sum(-1, keepdims=True)) @ v[:, h // 4]
    ah = att.reshape(S, 4096) @ f("o_proj").T
    arr = xf + ah
    post = rms(arr, f("post_ln"))
    g, u = post @ f("gate_proj").T, post @ f("up_proj").T
    mlp = (g / (1 + np.exp(-g)) * u) @ f("down_proj").T
    parity.assert_close(ints["ln0"], ln.astype(np.float32), "B", "ln0")
    parity.assert_close(ints["attn_hidden"], ah.astype(np.float32), "D", "attn_hidden")
    parity.assert_close(ints["mlp_out"], mlp.astype(np.float32), "D", "mlp_out")
    parity.assert_close(out, (arr + mlp).astype(np.float32), "D", "block out")


def test_weight_generator_host_matches_library(orc, pkg):
    # the library's host entry point and the oracle implement the same integer hash
    for seed, i in ((1, 0), (1234, 99), (2 ** 63 + 5, 2 ** 40 + 3)):
        a = pkg.lib.o1_hash_normal_host(seed, i)
        b = orc.orc_hash_normal(seed, i)
        assert np.float32(a).view(np.uint32) == np.float32(b).view(np.uint32)
    v = np.empty(200000, dtype=np.float32)
    orc.orc_fill_normal_f32(np_ptr(v), v.size, 9, 0.0, 1.0)
    assert abs(v.mean()) < 0.01 and abs(v.std() - 1.0) < 0.01


def test_lora_merge_against_fp64(orc):
    rng = np.random.default_rng(4)
    N, K, R = 48, 40, 8
    w = _bf(rng.standard_normal((N, K)) * 0.02)
    up, down = (rng.standard_normal(s).astype(np.float32) * 0.01 for s in ((N, R), (R, K)))
    ref = bf16_to_f32_np(w).astype(np.float64) + 0.5 * (up.astype(np.float64) @ down.astype(np.float64))
    orc.orc_lora_merge(np_ptr(w), np_ptr(up), np_ptr(down), N, K, R, 0.5)
    assert np.abs(w.astype(np.int32) - _bf(ref).astype(np.int32)).max() <= 1   # ties only


def test_initial_latent_layout(orc):
    # randn(1,3,H,W) seed+1 -> [tok, c*p*p + p1*p + p2], x noise_scale (generate.c:78-104, :1266)
    Hpx, Wpx, p = 64, 96, 32
    z = np.empty(((Hpx // p) * (Wpx // p), 3 * p * p), dtype=np.uint16)
    assert orc.orc_initial_latent(123456, Hpx, Wpx, p, 8.0, np_ptr(z)) == 0
    noise = np.empty(3 * Hpx * Wpx, dtype=np.float32)
    orc.orc_torch_randn(123457, np_ptr(noise), noise.size)
    img = noise.reshape(3, Hpx // p, p, Wpx // p, p)                     # c, h, p1, w, p2
    want = np.transpose(img, (1, 3, 0, 2, 4)).reshape(z.shape) * np.float32(8.0)
    assert (z == f32_to_bf16_np(want)).all()


def test_seq_ref_positions(orc, golden, pkg):
    """K-reference layout against hd_seq_build outputs (K = 1 is the case of tests/unit/test_seq_ref.c:97-119:
    target at (4096,4096,4096)..4127, the reference grid at max_pos+1 = 4128 on all three axes)."""
    g = np.load(os.path.join(golden, "seq_ref.npz"))
    for tag in ("k1", "k4"):
        T, gh, gw, S, ar, K = (int(v) for v in g[f"{tag}_meta"])
        geom = np.ascontiguousarray(g[f"{tag}_geom"], dtype=np.int32)
        want_ids, want_pos = g[f"{tag}_ids"], g[f"{tag}_pos"]
        text = np.ascontiguousarray(want_ids[:T], dtype=np.int64)
        ids, pos = np.empty(S, dtype=np.int64), np.empty((3, S), dtype=np.float32)
        got_ar = orc.orc_seq_ref(np_ptr(text), T, K, np_ptr(geom), gh, gw, 4096, 151652, 151655, np_ptr(ids),
                                 np_ptr(pos), S)
        assert got_ar == ar == T - 1
        assert (ids == want_ids).all() and (pos == want_pos).all()
        pids, ppos, par = pkg.seq_ref(text.tolist(), [tuple(int(x) for x in r) for r in geom], gh, gw)
        assert par == ar and (pids.numpy() == want_ids).all() and (ppos.numpy() == want_pos).all()
    k = g["k1_pos"]
    T = int(g["k1_meta"][0])
    assert list(k[:, T]) == [4096, 4096, 4096] and k[:, T:T + 1024].max() == 4127
    assert list(k[:, T + 1024]) == [4128, 4128, 4128] and list(k[:, -1]) == [4128, 4143, 4143]


def test_adaln_block_variant_reduces_to_the_plain_block(pkg, orc):
    """orc_decoder_block_adaln with shift = scale = 0 and gate = 1 is orc_decoder_block bit for bit; a real
    modulation changes the result; the modulation vectors are Linear(SiLU(t_emb))."""
    import parity
    H = pkg.HIDDEN
    hw = parity.HostWeights(pkg, 1, 1234, "B")
    T, gh, gw = 8, 4, 4
    pos, ar = pkg.seq_t2i(T, gh, gw)
    x = parity.seeded_bf16((T + gh * gw, H), 42)
    mod = np.zeros(6 * H, dtype=np.uint16)
    mod[2 * H:3 * H] = mod[5 * H:] = parity.f32_to_bf16_np(np.ones(H, np.float32))
    plain, _ = parity.oracle_block(hw, 0, x, pos.numpy(), ar, want_ints=False)
    ident, _ = parity.oracle_block(hw, 0, x, pos.numpy(), ar, want_ints=False, mod6=mod)
    assert (plain == ident).all()
    t_emb, mw, mb = parity.seeded_bf16(H, 51), parity.seeded_bf16((6 * H, H), 52, 0.0, 0.02), parity.seeded_bf16(6 * H, 53, 0.0, 0.1)
    mod6 = np.empty(6 * H, dtype=np.uint16)
    orc.orc_adaln_modulation(parity.np_ptr(t_emb), parity.np_ptr(mw), parity.np_ptr(mb), parity.np_ptr(mod6), H)
    te = parity.bf16_to_f32_np(t_emb).astype(np.float64)
    act = parity.bf16_to_f32_np(parity.f32_to_bf16_np((te / (1 + np.exp(-te))).astype(np.float32))).astype(np.float64)
    want = parity.bf16_to_f32_np(mw).astype(np.float64) @ act + parity.bf16_to_f32_np(mb)
    parity.assert_close(mod6, want.astype(np.float32), "C", "modulation vectors")
    moded, ints = parity.oracle_block(hw, 0, x, pos.numpy(), ar, mod6=mod6)
    assert parity.metrics(moded, plain)[0] > 1e-2
    # ln0 is the modulated norm: bf16(norm * (1 + scale) + shift)
    _, pints = parity.oracle_block(hw, 0, x, pos.numpy(), ar)
    f = parity.bf16_to_f32_np
    want_ln = f(pints["ln0"]) * (1.0 + f(mod6[H:2 * H])) + f(mod6[:H])
    assert (ints["ln0"] == parity.f32_to_bf16_np(want_ln.astype(np.float32))).all()


def _merged_close(got, ref, w0, max_frac):
    """Bit-identical except on rounding ties of the FP32 sum (neighbouring bf16 values, a vanishing fraction)."""
    g, r_, w = (parity.bf16_to_f32_np(a).astype(np.float64) for a in (got, ref, w0))
    neq = got != ref
    assert neq.mean() <= max_frac, f"{neq.mean():.2e} of the merged weights differ"
    assert (np.abs(g - r_) <= np.maximum(np.abs(w), np.abs(r_)) * 2.0 ** -7 + 1e-30).all()


def test_lora_oracle_against_the_reference_python_contract(orc, golden):
    """orc_lora_merge against weights merged by the reference's own Python (merge_linear of
    tools/lora/tests/test_lora_formula.py + the bf16 rounding of tools/lora/merge_gguf.py), fixture lora_ref.npz."""
    g = np.load(os.path.join(golden, "lora_ref.npz"))
    for i in range(int(g["n_cases"])):
        N, K, R, alpha, mult = g[f"c{i}_meta"]
        N, K, R = int(N), int(K), int(R)
        w = g[f"c{i}_w"].copy()
        up, down = np.ascontiguousarray(g[f"c{i}_up"]), np.ascontiguousarray(g[f"c{i}_down"])   # kept alive across the call
        orc.orc_lora_merge(np_ptr(w), np_ptr(up), np_ptr(down), N, K, R,
                           float(np.float32(mult) * np.float32(alpha) / np.float32(R)))
        assert (w != g[f"c{i}_w"]).mean() > 0.05
        _merged_close(w, g[f"c{i}_merged"], g[f"c{i}_w"], 1e-3)


def test_pack_written_by_the_reference_converter_is_parsed(pkg, golden):
    """Header of a pack the reference's own tools/hidream_convert.py wrote (fixture ref_convert_small.gguf):
    names in its production order, element counts, BF16 type, payload bytes at the offsets the header gives."""
    path = os.path.join(golden, "ref_convert_small.gguf")
    want = np.load(os.path.join(golden, "ref_convert_small.npz"))
    n = pkg.lib.o1_gguf_probe(path.encode(), -1, None, 0, None, None, None)
    assert n == len(want.files) == 33
    raw = open(path, "rb").read()
    seen = []
    for i in range(n):
        buf = C.create_string_buffer(256)
        numel, typ, off = C.c_int64(), C.c_int(), C.c_int64()
        assert pkg.lib.o1_gguf_probe(path.encode(), i, buf, 256, C.byref(numel), C.byref(typ), C.byref(off)) == n
        name = buf.value.decode()
        seen.append(name)
        bits = want[name]
        assert numel.value == bits.size and typ.value == 30 and off.value % 256 == 0
        assert raw[off.value:off.value + bits.size * 2] == bits.tobytes(), name
    assert seen[0] == "model.language_model.embed_tokens.weight" and set(seen) == set(want.files)


def test_pack_written_here_is_read_by_the_reference_reader(pkg, tmp_path):
    """write_gguf's output through the reference's own hd_gguf_open (src/io/gguf.c:212-305, inside the
    reference-built checker library): same tensor table, alignment, payload offsets and metadata."""
    r = parity.reflib()
    if r is None:
        pytest.skip("oracle/_ref/libo1ref.so not built")
    from test_abi_host import _small_pack

    class GgufTensor(C.Structure):        # hd_gguf_tensor, src/io/gguf.h
        _fields_ = [("name", C.c_char_p), ("n_dims", C.c_uint32), ("dims", C.c_uint64 * 8), ("type", C.c_uint32),
                    ("offset", C.c_uint64), ("nbytes", C.c_uint64)]

    class GgufFile(C.Structure):          # hd_gguf_file
        _fields_ = [("path", C.c_char_p), ("n_tensors", C.c_int64), ("tensors", C.POINTER(GgufTensor)),
                    ("alignment", C.c_uint64), ("tensor_data_off", C.c_uint64), ("payload_bytes", C.c_uint64),
                    ("arch", C.c_char_p), ("name", C.c_char_p), ("profile", C.c_char_p), ("variant", C.c_char_p),
                    ("revision", C.c_char_p), ("dtype", C.c_char_p), ("quantization", C.c_char_p),
                    ("num_layers", C.c_int64), ("layout_version", C.c_int64)]

    path = str(tmp_path / "pack.gguf")
    tensors = _small_pack(pkg, path, n_layers=2, with_f32=False)
    f = GgufFile()
    r.hd_gguf_open.argtypes = [C.c_char_p, C.POINTER(GgufFile)]
    r.hd_gguf_last_error.restype = C.c_char_p
    assert r.hd_gguf_open(path.encode(), C.byref(f)) == 0, r.hd_gguf_last_error()
    try:
        assert f.n_tensors == len(tensors) and f.alignment == 256 and f.arch == b"hidream_o1" and f.profile == b"dev"
        raw = open(path, "rb").read()
        for i, (name, a) in enumerate(tensors):
            t = f.tensors[i]
            assert t.name.decode() == name and t.type == 30 and t.nbytes == a.nbytes
            assert list(t.dims[:t.n_dims]) == list(a.shape)
            numel, typ, off = C.c_int64(), C.c_int(), C.c_int64()
            pkg.lib.o1_gguf_probe(path.encode(), i, None, 0, C.byref(numel), C.byref(typ), C.byref(off))
            assert off.value == f.tensor_data_off + t.offset and numel.value == a.size
            dst = np.empty(a.size, dtype=np.uint16)
            r.hd_gguf_read_tensor.argtypes = [C.POINTER(GgufFile), C.POINTER(GgufTensor), C.c_void_p]
            assert r.hd_gguf_read_tensor(C.byref(f), C.byref(t), dst.ctypes.data_as(C.c_void_p)) == 0
            assert (dst == a.ravel()).all() and raw[off.value:off.value + a.nbytes] == a.tobytes()
    finally:
        r.hd_gguf_close.argtypes = [C.POINTER(GgufFile)]
        r.hd_gguf_close(C.byref(f))
