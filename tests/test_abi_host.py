"""No-GPU checks of the C ABI and of the host logic: the library loads, exports every
function include/o1_b200.h declares, sizes/offsets are consistent, argument checks fail
the way o1.c's do (status code + message, src/model/block.c:146-157, forward.c:208-224),
and the Python mirror's structs match the C layout."""
import ctypes as C
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "o1_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b((?:hd|o1)_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol(pkg):
    names = declared_functions()
    assert len(names) > 70
    missing = [n for n in names if not hasattr(pkg.lib, n)]
    assert not missing, f"declared in include/o1_b200.h but not exported: {missing}"


def test_no_torch_or_oracle_linked_into_product(pkg):
    import subprocess
    out = subprocess.run(["ldd", pkg.LIB_PATH], capture_output=True, text=True).stdout
    assert "torch" not in out and "o1oracle" not in out and "o1ref" not in out
    assert "cublas" not in out and "cudnn" not in out       # no library GEMM/attention on the hot path


def test_struct_sizes_match_c_layout(pkg):
    p = C.sizeof(C.c_void_p)
    assert C.sizeof(pkg.BlockBinding) == 8 + 11 * p
    assert C.sizeof(pkg.BlockInternals) == 5 * p
    assert C.sizeof(pkg.ForwardBinding) == 11 * p + 8 + p
    assert C.sizeof(pkg.ForwardWorkspace) == 13 * p + 8 + p + 8 + p
    assert C.sizeof(pkg.ForwardDiagnostics) == 10 * p
    assert C.sizeof(pkg.LoraEntry) == 512 + 3 * 4 + 2 * 4 + 4 + 3 * p   # 4 bytes padding before pointers


def test_workspace_layout(pkg):
    lib = pkg.lib
    S, I = 1280, 1024
    bs = C.c_int64(0)
    total = lib.hd_forward_workspace_bytes(S, I, 32, 8, 4096, 12288, 128, C.byref(bs))
    assert bs.value == lib.hd_decoder_block_scratch_bytes(S, 32, 8, 4096, 12288, 128)
    # O(S) scratch: far below the reference's 2*heads*S*S bf16 score buffers (block.c:106-131)
    assert bs.value < 2 * 32 * S * S * 2
    offs = {}
    for name in ("hidden_a", "hidden_b", "h_text", "norm_out", "head_out", "t_emb", "te_hidden", "freq",
                 "freq_bf16", "t_scaled", "xe_stage", "xe_out", "block_scratch", "rope_table"):
        o = lib.hd_forward_ws_offset(name.encode(), S, S - I, I, 32, 8, 4096, 12288, 128, None)
        assert o >= 0 and o % 256 == 0 and o < total, name
        offs[name] = o
    assert len(set(offs.values())) == len(offs)
    assert offs["hidden_a"] == 0 and offs["hidden_b"] == S * 4096 * 2
    assert lib.hd_forward_ws_offset(b"nope", S, S - I, I, 32, 8, 4096, 12288, 128, None) == -1
    # scratch grows linearly in S
    b2 = lib.hd_decoder_block_scratch_bytes(2 * S, 32, 8, 4096, 12288, 128)
    assert abs(b2 - 2 * bs.value) < 8192


def test_argument_checks_fail_closed_without_touching_the_gpu(pkg):
    lib = pkg.lib
    bb = pkg.BlockBinding()
    rc = lib.hd_decoder_block(None, None, None, C.byref(bb), None, None, 0, None, None, 16, 32, 8, 4096,
                              12288, 128, None)
    assert rc == 6 and b"null argument" in lib.hd_last_error()          # HD_ERR_MISSING
    fb, ws = pkg.ForwardBinding(), pkg.ForwardWorkspace()
    rc = lib.hd_forward(C.byref(fb), C.byref(ws), None, 4, None, None, None, 4, None, None, None, 8, 32, 8,
                        4096, 12288, 128, pkg.TMS_ID, None, None, None)
    assert rc == 6
    plan = C.c_void_p()
    assert lib.hd_sdpa_create(C.byref(plan), 2, 32, 8, 64, 64, 128, 0.088) != 0     # batch != 1
    assert lib.hd_sdpa_create(C.byref(plan), 1, 32, 8, 64, 64, 64, 0.125) != 0      # head_dim != 128
    assert lib.hd_sdpa_create_split(C.byref(plan), 1, 32, 8, 64, 65, 128, 0.088) != 0
    assert lib.hd_sdpa_create_prod(C.byref(plan), 1, 32, 8, 64, 18, 128, 0.088) == 0
    lib.hd_sdpa_destroy(plan)
    lib.hd_cuda_clear_error()
    lib.hd_linear(None, None, None, None, 4, 4, 4, 1)
    assert b"bad args" in lib.hd_cuda_last_error()
    lib.hd_cuda_clear_error()
    assert lib.hd_cuda_last_error() == b""
    assert lib.hd_lora_merge_gpu(None, 0, None) == 0


def test_host_bf16_helpers(pkg):
    lib = pkg.lib
    assert lib.hd_f32_to_bf16(1.0) == 0x3F80 and lib.hd_f32_to_bf16(1.01171875) == 0x3F82
    assert lib.hd_bf16_to_f32(0xC020) == -2.5


def test_dev_sigmas_and_seeds(pkg, golden):
    import json
    ref = json.load(open(os.path.join(golden, "sigmas_ref.json")))["dev"]
    assert pkg.dev_sigmas() == ref
    seeds = {pkg.weight_seed(1234, l, n) for l in range(36) for n in pkg.SLOT_NAMES}
    seeds |= {pkg.weight_seed(1234, -1, n) for n in pkg.GLOBAL_NAMES}
    assert len(seeds) == 36 * 11 + 11
    assert pkg.tensor_shape("gate_proj") == (12288, 4096) and pkg.tensor_shape("k_proj") == (1024, 4096)


def test_importing_without_the_library_fails_loudly(pkg, tmp_path):
    import importlib.util
    import shutil
    dst = tmp_path / "o1.c_b200"
    shutil.copytree(os.path.join(ROOT, "o1.c_b200"), dst, ignore=shutil.ignore_patterns("*.so", "*.o", "csrc"))
    spec = importlib.util.spec_from_file_location("o1c_nolib", dst / "__init__.py",
                                                  submodule_search_locations=[str(dst)])
    mod = importlib.util.module_from_spec(spec)
    with pytest.raises(ImportError, match="no fallback"):
        spec.loader.exec_module(mod)


def test_host_rng_schedules_and_initial_latent_match_reference_vectors(pkg, golden):
    """The library's own host code for the step loop (not the oracle): MT19937 randn against the
    reference's torch_rng.c outputs, sigma schedules against scheduler.c outputs, initial latent layout."""
    import json
    import numpy as np
    lib = pkg.lib
    g = np.load(os.path.join(golden, "rng_ref.npz"))
    for n in (1, 8, 15, 16, 17, 31, 32, 1024):
        h = lib.o1_torch_rng_create(123457)
        out = np.empty(n, dtype=np.float32)
        lib.o1_torch_rng_randn(h, out.ctypes.data_as(C.c_void_p), n)
        lib.o1_torch_rng_free(h)
        assert (out.view(np.uint32) == g[f"randn_{n}"].view(np.uint32)).all(), n
    h = lib.o1_torch_rng_create(123457)
    assert [lib.o1_torch_rng_u32(h) for _ in range(2000)] == g["u32_2000"].tolist()
    lib.o1_torch_rng_free(h)
    h = lib.o1_torch_rng_create(1234)
    chain = np.empty((8, 64), dtype=np.float32)
    for i in range(8):
        lib.o1_torch_rng_randn(h, chain[i].ctypes.data_as(C.c_void_p), 64)
    lib.o1_torch_rng_free(h)
    assert (chain.view(np.uint32) == g["chain_1234_8x64"].view(np.uint32)).all()
    ref = json.load(open(os.path.join(golden, "sigmas_ref.json")))
    s = np.zeros(64, dtype=np.float32)
    p = s.ctypes.data_as(C.c_void_p)
    assert lib.o1_sigmas_dev(p) == 29 and s[:29].tolist() == ref["dev"]
    assert lib.o1_sigmas_flash(28, 1.0, p) == 29 and s[:29].tolist() == ref["flash_28_1"]
    assert lib.o1_sigmas_flash(28, 3.0, p) == 29 and s[:29].tolist() == ref["flow_match_28_3"]
    assert lib.o1_sigmas_default(50, 3.0, p) == 51 and s[:51].tolist() == ref["default_50_3"]
    assert lib.o1_noise_scale(29, 5, 8.0, 4.0) == np.float32(8.0 + (4.0 - 8.0) * 5 / 27)
    # initial latent: same as the oracle's restatement, and a torch-free layout check
    import parity
    Hpx, Wpx = 64, 96
    z = np.empty(((Hpx // 32) * (Wpx // 32), 3072), dtype=np.uint16)
    assert lib.o1_initial_latent_host(123456, Hpx, Wpx, 32, 8.0, z.ctypes.data_as(C.c_void_p)) == 0
    zo = np.empty_like(z)
    assert parity.oracle().orc_initial_latent(123456, Hpx, Wpx, 32, 8.0, parity.np_ptr(zo)) == 0
    assert (z == zo).all()
    assert lib.o1_initial_latent_host(1, 65, 96, 32, 8.0, z.ctypes.data_as(C.c_void_p)) == 6
    x = np.random.default_rng(0).standard_normal(5000).astype(np.float32) * 3
    a, b = x.copy(), x.copy()
    lib.o1_noise_clamp_host(a.ctypes.data_as(C.c_void_p), a.size, 1.5)
    parity.oracle().orc_noise_clamp(parity.np_ptr(b), b.size, 1.5)
    assert (a == b).all() and a.max() < x.max()


def _small_pack(pkg, path, n_layers=2, with_f32=True):
    import numpy as np
    rng = np.random.default_rng(3)
    tensors = []
    for name in pkg.GLOBAL_NAMES:
        tensors.append((pkg.gguf_tensor_name(-1, name), rng.integers(0, 65535, size=(3, 40), dtype=np.uint16)))
    for l in range(n_layers):
        for name in pkg.SLOT_NAMES:
            if with_f32 and name == "q_norm":
                a = rng.standard_normal(128).astype(np.float32)
            elif with_f32 and name == "k_norm":
                a = rng.standard_normal(128).astype(np.float16)
            else:
                a = rng.integers(0, 0x7F00, size=(5, 24), dtype=np.uint16)
            tensors.append((pkg.gguf_tensor_name(l, name), a))
    pkg.write_gguf(path, tensors, {"general.architecture": "hidream_o1", "hidream.profile": "dev",
                                   "hidream.num_layers": str(n_layers)})
    return tensors


def test_gguf_header_parse_without_gpu(pkg, tmp_path):
    import numpy as np
    path = str(tmp_path / "pack.gguf")
    tensors = _small_pack(pkg, path)
    n = pkg.lib.o1_gguf_probe(path.encode(), -1, None, 0, None, None, None)
    assert n == len(tensors)
    raw = open(path, "rb").read()
    for i, (name, a) in enumerate(tensors):
        buf = C.create_string_buffer(256)
        numel, typ, off = C.c_int64(), C.c_int(), C.c_int64()
        assert pkg.lib.o1_gguf_probe(path.encode(), i, buf, 256, C.byref(numel), C.byref(typ), C.byref(off)) == n
        assert buf.value.decode() == name and numel.value == a.size
        assert typ.value == {np.dtype(np.float32): 0, np.dtype(np.float16): 1, np.dtype(np.uint16): 30}[a.dtype]
        assert off.value % 256 == 0 and raw[off.value:off.value + a.nbytes] == a.tobytes()
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGUX" + raw[4:200])
    assert pkg.lib.o1_gguf_probe(str(bad).encode(), -1, None, 0, None, None, None) == -1
    assert b"bad magic" in pkg.lib.hd_weights_last_error()
    trunc = tmp_path / "trunc.gguf"
    trunc.write_bytes(raw[:60])
    assert pkg.lib.o1_gguf_probe(str(trunc).encode(), -1, None, 0, None, None, None) == -1


def test_bulk_and_threaded_rng_equals_the_scalar_stream(pkg):
    """The block-wise uniform fill and the threaded Box-Muller give the same stream as draw-by-draw
    generation (the oracle's generator, which is pinned to the reference's torch_rng.c), across state
    refills and when scalar draws are mixed in between."""
    import numpy as np
    import parity
    lib, orc = pkg.lib, parity.oracle()
    h, o = lib.o1_torch_rng_create(987654321), orc.orc_rng_create(987654321)
    try:
        for n, threads in ((100003, 4), (5, 1), (70000, 3), (16, 2), (623, 1), (1 << 18, 8)):
            a = np.empty(n, dtype=np.float32)
            b = np.empty(n, dtype=np.float32)
            lib.o1_torch_rng_randn_mt(h, a.ctypes.data_as(C.c_void_p), n, threads)
            orc.orc_rng_randn(o, parity.np_ptr(b), n)
            assert (a.view(np.uint32) == b.view(np.uint32)).all(), (n, threads)
            lib.o1_torch_rng_u32(h)                      # one scalar draw in between keeps the states aligned
            tmp = np.empty(1, dtype=np.float32)
            # the oracle has no raw-u32 entry on a stateful generator: a 1-element randn uses 4 draws, so
            # advance the library's generator by the 3 remaining ones
            orc.orc_rng_randn(o, parity.np_ptr(tmp), 1)
            for _ in range(3):
                lib.o1_torch_rng_u32(h)
    finally:
        lib.o1_torch_rng_free(h)
        orc.orc_rng_free(o)


def test_gguf_header_that_points_outside_the_file_fails_closed(pkg, tmp_path):
    """A corrupt or truncated pack must fail in the header check (HD_ERR_PARSE), before any device memory is
    sized from it: tensor offset + size beyond the file, a dims product that wraps 64 bits, a zero dim."""
    import struct
    import numpy as np
    path = str(tmp_path / "pack.gguf")
    tensors = _small_pack(pkg, path)
    raw = bytearray(open(path, "rb").read())
    name0 = tensors[0][0].encode()
    at = raw.find(name0) + len(name0)            # tensor record: n_dims u32, dims u64 x n, type u32, offset u64
    nd = struct.unpack_from("<I", raw, at)[0]
    off_at = at + 4 + 8 * nd + 4
    store = pkg.WeightStore()

    def probe(mutated):
        p = tmp_path / "m.gguf"
        p.write_bytes(bytes(mutated))
        assert pkg.lib.o1_gguf_probe(str(p).encode(), -1, None, 0, None, None, None) == -1
        assert pkg.lib.hd_weights_to_device_gguf(str(p).encode(), 0, C.byref(store)) == 2      # HD_ERR_PARSE
        assert not store.arena_ptr
        return pkg.lib.hd_weights_last_error()

    m = bytearray(raw)
    struct.pack_into("<Q", m, off_at, 1 << 40)                       # offset far beyond the file
    assert b"lies outside" in probe(m)
    m = bytearray(raw)
    struct.pack_into("<Q", m, at + 4, 1 << 62)                       # dims product wraps
    struct.pack_into("<Q", m, at + 12, 8)
    assert b"malformed" in probe(m)
    m = bytearray(raw)
    struct.pack_into("<Q", m, at + 4, 0)                             # empty dimension
    assert b"malformed" in probe(m)
    assert b"lies outside" in probe(raw[:len(raw) - 300])            # payload cut short


def test_sp_rejects_more_ranks_than_its_tables_hold(pkg):
    """heads and kv_heads divisible by 16 would pass the divisibility checks; the peer tables and the kernels'
    destination tables hold O1_SP_MAX_RANKS = 8 entries."""
    from o1c_b200 import sp as spmod
    ws = spmod.SpWs()
    ws.sp_size, ws.sp_rank, ws.S, ws.T, ws.row0, ws.rows = 16, 0, 16 * 128, 16, 0, 128
    ws.heads, ws.kv_heads, ws.hidden, ws.ff, ws.head_dim, ws.ar_len = 32, 16, 4096, 12288, 128, 15
    bb = pkg.BlockBinding()
    dummy = C.c_void_p(256)
    assert pkg.lib.o1_sp_block_pre(C.byref(bb), C.byref(ws), dummy) == 6                       # HD_ERR_MISSING
    assert pkg.lib.o1_sp_block_attn(C.byref(ws)) == 6
    assert b"bad" in pkg.lib.hd_last_error()


def test_reference_harness_mirrors_the_seeded_arena_rules(pkg):
    """tests/refharness.py regenerates the product's seeded weights without loading the product library;
    its seeds, shapes, arena offsets and sigma list must be the package's."""
    import refharness as rh
    assert rh.SLOT_NAMES == pkg.SLOT_NAMES and rh.GLOBAL_NAMES == pkg.GLOBAL_NAMES
    for l, names in ((-1, pkg.GLOBAL_NAMES), (0, pkg.SLOT_NAMES), (35, pkg.SLOT_NAMES)):
        for n in names:
            assert rh.weight_seed(1234, l, n) == pkg.weight_seed(1234, l, n)
            assert rh.tensor_shape(n) == pkg.tensor_shape(n)
    assert rh.dev_sigmas() == pkg.dev_sigmas()
    pos, ar = rh.seq_t2i(7, 3, 5)
    pos2, ar2 = pkg.seq_t2i(7, 3, 5)
    assert ar == ar2 and torch.equal(pos, pos2)
    assert C.sizeof(rh.ForwardBinding) == C.sizeof(pkg.ForwardBinding)
    assert C.sizeof(rh.ForwardWorkspace) == C.sizeof(pkg.ForwardWorkspace)
    assert C.sizeof(rh.BlockBinding) == C.sizeof(pkg.BlockBinding)
    assert C.sizeof(rh.ForwardDiagnostics) == C.sizeof(pkg.ForwardDiagnostics)
