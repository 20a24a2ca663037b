"""Checker-side helpers shared by the tests, smoke() and bench.py's cpu_baseline leg.

Binds the CPU oracle (oracle/libo1oracle.so) and, when it was built, the
reference's own CUDA build (oracle/_ref/libo1ref.so) with ctypes, regenerates
the seeded weights on the host, and implements the reference's comparison
metrics (NRMSE and cosine in fp64 over fp32-upcast values,
o1.c tests/unit/test_block.c:52-71) and tolerance classes
(docs/M1_NUMERICAL_CONTRACT.md:48-54, tests/unit/test_primitives.c:100-102).
"""
import ctypes as C
import os
import subprocess

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_LIB = os.path.join(ORACLE_DIR, "libo1oracle.so")
REF_LIB = os.path.join(ORACLE_DIR, "_ref", "libo1ref.so")

# class -> (max NRMSE, min cosine)
TOL = {"B": (2e-3, 0.99999), "C": (5e-3, 0.9999), "D": (1e-2, 0.999), "E": (2e-2, 0.995)}
# Vision tower after all 27 blocks (random weights amplify single bf16 ulps from block to block): the reference's
# own tower test asserts cosine > 0.99 on every stage (tests/unit/test_vision.c:280-566); kept tighter here.
TOL["V"] = (5e-2, 0.998)

_P, _i, _i64, _f, _sz, _u64 = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t, C.c_uint64


class BlockW(C.Structure):
    _fields_ = [(n, _P) for n in ("q_proj", "k_proj", "v_proj", "o_proj", "input_ln", "post_ln",
                                  "gate_proj", "up_proj", "down_proj", "q_norm", "k_norm")]


class Globals(C.Structure):
    _fields_ = [(n, _P) for n in ("te0_w", "te0_b", "te2_w", "te2_b", "xe1_w", "xe2_w", "xe2_b", "fl_w",
                                  "fl_b", "fnorm_w")]


_oracle = None


def oracle():
    """The CPU oracle library; built on first use if the .so is absent."""
    global _oracle
    if _oracle is not None:
        return _oracle
    if not os.path.exists(ORACLE_LIB):
        subprocess.run(["make", "-s", "-C", ORACLE_DIR, "oracle"], check=True)
    lib = C.CDLL(ORACLE_LIB)

    def sig(name, res, *args):
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, list(args)

    sig("orc_num_threads", _i)
    sig("orc_bf16_to_f32", _f, C.c_uint16)
    sig("orc_f32_to_bf16", C.c_uint16, _f)
    sig("orc_hash_normal", _f, _u64, _u64)
    sig("orc_fill_normal_bf16", None, _P, _sz, _u64, _f, _f)
    sig("orc_fill_normal_f32", None, _P, _sz, _u64, _f, _f)
    sig("orc_fill_normal_rows_bf16", None, _P, _i64, _i64, _i64, _u64, _f, _f)
    sig("orc_rmsnorm", None, _P, _P, _P, _i, _i, _f)
    sig("orc_silu", None, _P, _P, _sz)
    sig("orc_swiglu", None, _P, _P, _P, _sz)
    sig("orc_residual_add", None, _P, _P, _P, _sz)
    sig("orc_linear", None, _P, _P, _P, _P, _i, _i, _i)
    sig("orc_timestep_embed", None, _P, _P, _i, _i)
    sig("orc_mrope_cos_sin", None, _P, _i, _i, _P, _i, _i, _f, _f, _i, _P, _P)
    sig("orc_apply_rotary", None, _P, _P, _P, _P, _i, _i, _i)
    sig("orc_attention", None, _P, _P, _P, _P, _i, _i, _i, _i, _f, _i)
    sig("orc_attention_rows", None, _P, _i, _P, _i, _P, _i, _P, _i, _i, _i, _i, _i, _f, _i, _P, _i)
    sig("orc_head_split", None, _P, _P, _i, _i, _i)
    sig("orc_head_merge", None, _P, _P, _i, _i, _i)
    sig("orc_decoder_block", _i, _P, _P, _i, C.POINTER(BlockW), _P, C.POINTER(_P), _i, _i, _i, _i, _i, _i)
    sig("orc_decoder_block_adaln", _i, _P, _P, _i, C.POINTER(BlockW), _P, _P, C.POINTER(_P), _i, _i, _i, _i, _i, _i)
    sig("orc_adaln_modulation", None, _P, _P, _P, _P, _i)
    sig("orc_forward", _i, C.POINTER(Globals), C.POINTER(BlockW), _i, _P, _P, _i, _P, _i, _P, _i, _f,
        _i64, _P, _P, _i, _i, _i, _i, _i)
    sig("orc_forward_visual", _i, C.POINTER(Globals), C.POINTER(BlockW), _i, _P, _P, _i, _P, _i, _P, _i, _f,
        _i64, _P, _P, _i, _i, _i, _i, _i, _P, _P, _P)
    sig("orc_sched_vcond", None, _P, _P, _f, _P, _sz)
    sig("orc_sched_cfg_guided", None, _P, _P, _f, _P, _sz)
    sig("orc_sched_flow_match_step", None, _P, _P, _f, _f, _P, _sz)
    sig("orc_sched_denoised", None, _P, _P, _f, _P, _sz)
    sig("orc_sched_z_next", None, _P, _P, _f, _f, _P, _sz)
    sig("orc_sched_cfg_flow_step", None, _P, _P, _P, _f, _f, _f, _P, _sz)
    sig("orc_unipc_convert", None, _P, _P, _f, _P, _sz)
    sig("orc_unipc_correct", None, _P, _P, _P, _P, _f, _f, _f, _f, _f, _f, _f, _f, _i, _P, _sz)
    sig("orc_unipc_predict", None, _P, _P, _P, _f, _f, _f, _f, _f, _f, _f, _i, _P, _sz)
    sig("orc_sigmas_dev", _i, _P)
    sig("orc_sigmas_flash", _i, _i, _f, _P)
    sig("orc_sigmas_default", _i, _i, _f, _P)
    sig("orc_noise_scale", _f, _i, _i, _f, _f)
    sig("orc_noise_clamp", None, _P, _sz, _f)
    sig("orc_rng_create", _P, _u64)
    sig("orc_rng_randn", None, _P, _P, _i64)
    sig("orc_rng_free", None, _P)
    sig("orc_lora_merge", None, _P, _P, _P, _i, _i, _i, _f)
    sig("orc_torch_randn", None, _u64, _P, _i64)
    sig("orc_torch_rng_u32", None, _u64, _P, _i64)
    sig("orc_initial_latent", _i, _u64, _i, _i, _i, _f, _P)
    sig("orc_seq_t2i", _i, _i, _i, _i, _i, _P)
    sig("orc_prefix_causal_mask", None, _i, _i, _P)
    sig("orc_seq_ref", _i, _P, _i, _i, _P, _i, _i, _i, _i64, _i64, _P, _P, _i)
    sig("orc_layernorm", None, _P, _P, _P, _P, _i, _i, _f)
    sig("orc_gelu", None, _P, _P, _sz, _i)
    sig("orc_apply_rotary_f32", None, _P, _P, _P, _P, _i, _i, _i)
    sig("orc_vision_tables", None, _i, _i, _P, _P, _P, _P)
    sig("orc_vision_forward", _i, _P, _P, _i, _i, _P, _P, _P)
    _oracle = lib
    return lib


_ref = False


def reflib():
    """The reference's own sources built as a shared library (make -C oracle ref), or None.
    Loaded RTLD_LOCAL and linked -Bsymbolic, so its hd_* symbols stay apart from the product's."""
    global _ref
    if _ref is not False:
        return _ref
    if not os.path.exists(REF_LIB):
        _ref = None
        return None
    try:
        lib = C.CDLL(REF_LIB, mode=os.RTLD_LOCAL | os.RTLD_NOW)
    except OSError:
        _ref = None
        return None

    def sig(name, res, *args):
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, list(args)

    sig("hd_cuda_last_error", C.c_char_p)
    sig("hd_cuda_clear_error", None)
    sig("hd_last_error", C.c_char_p)
    sig("hd_gemm_runtime_init", _P, _i, _sz)
    sig("hd_gemm_runtime_destroy", None, _P)
    sig("hd_gemm_set_backend", None, _i)
    sig("hd_rmsnorm", None, _P, _P, _P, _i, _i, _f)
    sig("hd_silu", None, _P, _P, _sz)
    sig("hd_swiglu", None, _P, _P, _P, _sz)
    sig("hd_residual_add", None, _P, _P, _P, _sz)
    sig("hd_linear", None, _P, _P, _P, _P, _i, _i, _i, _i)
    sig("hd_linear_reference", None, _P, _P, _P, _P, _i, _i, _i, _i)
    sig("hd_timestep_embed", None, _P, _P, _i, _i)
    sig("hd_mrope_cos_sin", None, _P, _i, _i, _P, _i, _i, _f, _f, _i, _P, _P)
    sig("hd_apply_rotary", None, _P, _P, _P, _P, _i, _i, _i)
    sig("hd_attention_eager", None, _P, _P, _P, _P, _P, _P, _P, _i, _i, _i, _i, _f)
    sig("hd_head_split", None, _P, _P, _i, _i, _i)
    sig("hd_head_merge", None, _P, _P, _i, _i, _i)
    sig("hd_gather_rows", None, _P, _P, _P, _i, _i, _i64)
    sig("hd_apply_tms_condition", None, _P, _P, _P, _P, _i, _i, _i64)
    sig("hd_sched_vcond", None, _P, _P, _f, _P, _i)
    sig("hd_sched_flow_match_step", None, _P, _P, _f, _f, _P, _i)
    sig("hd_sched_cfg_guided", None, _P, _P, _f, _P, _i)
    sig("hd_sched_bf16_upcast", None, _P, _P, _i)
    sig("hd_sched_denoised", None, _P, _P, _f, _P, _i)
    sig("hd_sched_z_next", None, _P, _P, _f, _f, _P, _i)
    sig("hd_f32_convert_bf16", None, _P, _P, _i)
    sig("hd_sdpa_create_prod", _i, C.POINTER(_P), _i, _i, _i, _i, _i, _i, _f)
    sig("hd_sdpa_execute", _i, _P, _P, _P, _P, _P, _P, _P)
    sig("hd_sdpa_destroy", None, _P)
    sig("hd_decoder_block_scratch_bytes", _i64, _i64, _i, _i, _i, _i, _i)
    sig("hd_decoder_block", _i, _P, _P, _P, _P, _P, _P, _i64, _P, _P, _i64, _i, _i, _i, _i, _i, _P)
    sig("hd_forward_workspace_bytes", _i64, _i64, _i, _i, _i, _i, _i, _i, C.POINTER(_i64))
    sig("hd_forward", _i, _P, _P, _P, _i, _P, _P, _P, _i, _P, _P, _P, _i, _i, _i, _i, _i, _i, _i, _P, _P, _P)
    sig("hd_lora_merge_gpu", _i, _P, _sz, _P)
    if hasattr(lib, "hd_vision_forward"):
        sig("hd_vision_workspace_bytes", _i64, _i64)
        sig("hd_vision_tables_bytes", _i64, _i64)
        sig("hd_vision_prepare_tables", _i, _P, _i, _i, _i)
        sig("hd_vision_forward", _i, _P, _P, _P, _i, _i, _i, _P, _P)
        sig("hd_vision_layernorm", None, _P, _P, _P, _P, _i, _i, _f)
        sig("hd_vision_gelu", None, _P, _P, _sz)
        sig("hd_vision_gelu_exact", None, _P, _P, _sz)
        sig("hd_apply_rotary_f32", None, _P, _P, _P, _P, _i, _i, _i)
    _ref = lib
    return lib


def np_ptr(a):
    return C.c_void_p(a.ctypes.data)


# ----------------------------------------------------------------- bf16 <-> numpy / torch
def f32_to_bf16_np(a):
    """RNE by integer add (o1.c src/cuda/support.cu:21-28), numpy float32 -> uint16."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    u = u + (0x7FFF + ((u >> 16) & 1)).astype(np.uint32)
    return (u >> 16).astype(np.uint16)


def bf16_to_f32_np(a):
    return (a.astype(np.uint32) << 16).view(np.float32)


def torch_to_u16(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def u16_to_torch(a, device="cpu"):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16).to(device)


# ----------------------------------------------------------------- metrics
def metrics(got, ref):
    """(nrmse, cosine, max_abs, n_nonfinite) with fp64 accumulation. Inputs: numpy uint16 (bf16),
    numpy float32, or torch tensors."""
    def to64(x):
        if isinstance(x, torch.Tensor):
            return x.detach().float().cpu().numpy().astype(np.float64).ravel()
        if x.dtype == np.uint16:
            return bf16_to_f32_np(x).astype(np.float64).ravel()
        return x.astype(np.float64).ravel()
    g, r = to64(got), to64(ref)
    bad = int((~np.isfinite(g)).sum())
    d = g - r
    rms_ref = np.sqrt(np.mean(r * r))
    nrmse = float(np.sqrt(np.mean(d * d)) / (rms_ref if rms_ref > 0 else 1.0))
    den = np.sqrt((g * g).sum()) * np.sqrt((r * r).sum())
    cos = float((g * r).sum() / den) if den > 0 else (1.0 if not d.any() else 0.0)
    return nrmse, cos, float(np.abs(d).max()) if d.size else 0.0, bad


def metrics_dev(got, ref):
    """The same four numbers for two device tensors, reduced on the device in fp64 (tensors of 10^8
    elements: the host path would copy and convert them first)."""
    g, r = got.reshape(-1).double(), ref.reshape(-1).double()
    bad = int((~torch.isfinite(g)).sum().item())
    d = g - r
    rms_ref = float(torch.sqrt(torch.mean(r * r)).item())
    nrmse = float(torch.sqrt(torch.mean(d * d)).item()) / (rms_ref if rms_ref > 0 else 1.0)
    den = float((torch.sqrt((g * g).sum()) * torch.sqrt((r * r).sum())).item())
    cos = float((g * r).sum().item()) / den if den > 0 else (1.0 if not bool(d.any()) else 0.0)
    return nrmse, cos, float(d.abs().max().item()) if d.numel() else 0.0, bad


def bf16_ulp_of_max(ref):
    """ULP(m) = 2^(floor(log2 m) - 7) at the tensor's largest magnitude (o1.c docs/M1_7_TOLERANCES.md:77-80)."""
    import math
    m = float(ref.float().abs().max().item()) if isinstance(ref, torch.Tensor) else float(np.abs(ref).max())
    return 2.0 ** (math.floor(math.log2(m)) - 7) if m > 0 else 0.0


def report(record):
    """Appends one JSON line to the file named by O1_PARITY_REPORT (measured distances for the write-up)."""
    path = os.environ.get("O1_PARITY_REPORT")
    if path:
        import json
        with open(path, "a") as f:
            f.write(json.dumps(record) + "\n")


def assert_close(got, ref, cls, what=""):
    nrmse, cos, mx, bad = metrics(got, ref)
    lim_n, lim_c = TOL[cls]
    assert bad == 0, f"{what}: {bad} non-finite values"
    assert nrmse <= lim_n and cos >= lim_c, (
        f"{what}: class {cls} violated: nrmse={nrmse:.3e} (<= {lim_n}) cos={cos:.7f} (>= {lim_c}) "
        f"max_abs={mx:.3e}")
    return nrmse, cos


# ----------------------------------------------------------------- host weights
class HostWeights:
    """Host copy of the seeded weights of o1c_b200.Weights (same generator, same seeds)."""

    def __init__(self, pkg, n_layers, seed=1234, weight_set="A", std=0.02, **dims):
        self.pkg, self.n_layers, self.seed, self.weight_set, self.std = pkg, n_layers, seed, weight_set, std
        self.dims = dict(hidden=pkg.HIDDEN, heads=pkg.HEADS, kv_heads=pkg.KV_HEADS, head_dim=pkg.HEAD_DIM,
                         ff=pkg.FF, vocab=pkg.VOCAB)
        self.dims.update(dims)
        self._cache = {}

    def _mean(self, name):
        from_norm = name in ("input_ln", "post_ln", "q_norm", "k_norm", "fnorm_w")
        return 1.0 if (self.weight_set == "B" and from_norm) else 0.0

    def tensor(self, layer, name):
        key = (layer, name)
        if key not in self._cache:
            shape = self.pkg.tensor_shape(name, **self.dims)
            a = np.empty(shape, dtype=np.uint16)
            oracle().orc_fill_normal_bf16(np_ptr(a), a.size, self.pkg.weight_seed(self.seed, layer, name),
                                          self._mean(name), self.std)
            self._cache[key] = a
        return self._cache[key]

    def embed_rows(self, ids):
        """Rows of embed_tokens for the given ids (OOB -> row 0), without building the table."""
        H = self.dims["hidden"]
        out = np.empty((len(ids), H), dtype=np.uint16)
        seed = self.pkg.weight_seed(self.seed, -1, "embed_tokens")
        for i, t in enumerate(ids):
            t = int(t)
            if t < 0 or t >= self.dims["vocab"]:
                t = 0
            oracle().orc_fill_normal_rows_bf16(np_ptr(out[i:i + 1]), t, 1, H, seed, 0.0, self.std)
        return out

    def block_struct(self, layer):
        bw = BlockW()
        keep = []
        for n in self.pkg.SLOT_NAMES:
            a = self.tensor(layer, n)
            keep.append(a)
            setattr(bw, n, a.ctypes.data)
        bw._keep = keep
        return bw

    def globals_struct(self):
        g = Globals()
        keep = []
        for n in self.pkg.GLOBAL_NAMES:
            if n == "embed_tokens":
                continue
            a = self.tensor(-1, n)
            keep.append(a)
            setattr(g, n, a.ctypes.data)
        g._keep = keep
        return g

    def drop(self, layer):
        for n in self.pkg.SLOT_NAMES:
            self._cache.pop((layer, n), None)


def oracle_block(hw, layer, x_u16, pos_np, ar_len, want_ints=True, mod6=None):
    """orc_decoder_block (orc_decoder_block_adaln with mod6 [6*hidden] u16) on host arrays.
    Returns (out, dict of the five internals)."""
    d = hw.dims
    S = x_u16.shape[0]
    out = np.empty_like(x_u16)
    names = ("ln0", "attn_hidden", "attn_resid", "post_ln", "mlp_out")
    ints = {n: np.empty_like(x_u16) for n in names} if want_ints else {}
    arr = (C.c_void_p * 5)(*[ints[n].ctypes.data if want_ints else None for n in names])
    bw = hw.block_struct(layer)
    pos_np = np.ascontiguousarray(pos_np, dtype=np.float32)
    dims = (S, d["heads"], d["kv_heads"], d["hidden"], d["ff"], d["head_dim"])
    if mod6 is None:
        rc = oracle().orc_decoder_block(np_ptr(x_u16), np_ptr(pos_np), ar_len, C.byref(bw), np_ptr(out),
                                        arr if want_ints else None, *dims)
    else:
        rc = oracle().orc_decoder_block_adaln(np_ptr(x_u16), np_ptr(pos_np), ar_len, C.byref(bw), np_ptr(mod6),
                                              np_ptr(out), arr if want_ints else None, *dims)
    assert rc == 0
    return out, ints


def oracle_forward(hw, ids_np, pos_np, ar_len, vin_u16, t, dump=False, visual=None):
    """visual = (vmask uint8 [S], image_embeds u16 [V,H], [deepstack0, 1, 2] u16 [V,H]) or None."""
    d = hw.dims
    T, I = len(ids_np), vin_u16.shape[0]
    S = T + I
    out = np.empty((S, 3072), dtype=np.uint16)
    blocks = (BlockW * hw.n_layers)()
    keep = []
    for l in range(hw.n_layers):
        b = hw.block_struct(l)
        keep.append(b)
        for n in hw.pkg.SLOT_NAMES:
            setattr(blocks[l], n, getattr(b, n))
    g = hw.globals_struct()
    rows = hw.embed_rows(ids_np)
    ids64 = np.ascontiguousarray(ids_np, dtype=np.int64)
    pos_np = np.ascontiguousarray(pos_np, dtype=np.float32)
    hd = np.empty((hw.n_layers + 1, S, d["hidden"]), dtype=np.uint16) if dump else None
    vm = emb = ds = None
    if visual is not None:
        vm, emb, dss = visual
        vm = np.ascontiguousarray(vm, dtype=np.uint8)
        ds = (C.c_void_p * 3)(*[a.ctypes.data for a in dss])
    rc = oracle().orc_forward_visual(C.byref(g), blocks, hw.n_layers, np_ptr(ids64), np_ptr(rows), T,
                                     np_ptr(pos_np), ar_len, np_ptr(vin_u16), I, float(t), hw.pkg.TMS_ID,
                                     np_ptr(out), np_ptr(hd) if dump else None, d["heads"], d["kv_heads"],
                                     d["hidden"], d["ff"], d["head_dim"], np_ptr(vm) if visual else None,
                                     np_ptr(emb) if visual else None, ds)
    assert rc == 0
    return (out, hd) if dump else out


def seeded_bf16(n_or_shape, seed, mean=0.0, std=1.0):
    """Host bf16 array from the shared counter-based generator (activations, latents)."""
    a = np.empty(n_or_shape, dtype=np.uint16)
    oracle().orc_fill_normal_bf16(np_ptr(a), a.size, seed, mean, std)
    return a


# ----------------------------------------------------------------- smoke
def smoke_check(pkg, device):
    """One small decoder block and one fused CFG scheduler step on the GPU, checked
    against the CPU oracle (class D on the block output and internals, exact class B
    on the scheduler)."""
    torch.cuda.set_device(device)
    pkg.use_torch_stream()
    T, gh, gw = 24, 8, 12
    S = T + gh * gw
    w = pkg.Weights(n_layers=1, seed=1234, weight_set="B", device=device)
    eng = pkg.Engine(w, T, gh * gw)
    pos, ar_len = pkg.seq_t2i(T, gh, gw)
    x = seeded_bf16((S, pkg.HIDDEN), 42)
    xd = u16_to_torch(x, device)
    out, ints = eng.block(xd, pos.to(device), 0, internals=True)
    torch.cuda.synchronize()
    err = pkg.lib.o1_device_error()
    assert err == 0, f"device error word = {err}"
    hw = HostWeights(pkg, 1, 1234, "B")
    ref_out, ref_ints = oracle_block(hw, 0, x, pos.numpy(), ar_len)
    assert_close(torch_to_u16(out), ref_out, "D", "smoke block out")
    for n in ("attn_hidden", "mlp_out"):
        assert_close(torch_to_u16(ints[n]), ref_ints[n], "D", f"smoke {n}")
    n = 4096
    z, xc, xu = (seeded_bf16(n, 7), seeded_bf16(n, 8), seeded_bf16(n, 9))
    zd, cd, ud = (u16_to_torch(a, device) for a in (z, xc, xu))     # kept alive across the async launch
    zn = torch.empty(n, dtype=torch.bfloat16, device=device)
    rc = pkg.lib.o1_sched_cfg_flow_step(pkg.ptr(zd), pkg.ptr(cd), pkg.ptr(ud), 0.9, 0.8, 5.0, pkg.ptr(zn), n)
    assert rc == 0
    torch.cuda.synchronize()
    ref = np.empty(n, dtype=np.uint16)
    oracle().orc_sched_cfg_flow_step(np_ptr(z), np_ptr(xc), np_ptr(xu), 0.9, 0.8, 5.0, np_ptr(ref), n)
    assert_close(torch_to_u16(zn), ref, "B", "smoke scheduler")


# ----------------------------------------------------------------- vision tower (edit modes)
VISION_BLOCK_SLOTS = ("norm1.weight", "norm1.bias", "norm2.weight", "norm2.bias", "attn.qkv.weight", "attn.qkv.bias",
                      "attn.proj.weight", "attn.proj.bias", "mlp.linear_fc1.weight", "mlp.linear_fc1.bias",
                      "mlp.linear_fc2.weight", "mlp.linear_fc2.bias")
VISION_MERGER_SLOTS = ("norm.weight", "norm.bias", "linear_fc1.weight", "linear_fc1.bias", "linear_fc2.weight",
                       "linear_fc2.bias")


def vision_tensor_list():
    """(manifest name, shape) of the 351 vision tensors in hd_vision_binding order (o1.c src/model/vision.c:52-127)."""
    H, I, O, M = 1152, 4304, 4096, 4608
    out = [("model.visual.patch_embed.proj.weight", (H, 1536)), ("model.visual.patch_embed.proj.bias", (H,)),
           ("model.visual.pos_embed.weight", (2304, H))]
    bshape = ((H,), (H,), (H,), (H,), (3 * H, H), (3 * H,), (H, H), (H,), (I, H), (I,), (H, I), (H,))
    for i in range(27):
        out += [(f"model.visual.blocks.{i}.{s}", sh) for s, sh in zip(VISION_BLOCK_SLOTS, bshape)]
    for prefix, nd in [("model.visual.merger", H)] + [(f"model.visual.deepstack_merger_list.{j}", M) for j in range(3)]:
        mshape = ((nd,), (nd,), (M, M), (M,), (O, M), (O,))
        out += [(f"{prefix}.{s}", sh) for s, sh in zip(VISION_MERGER_SLOTS, mshape)]
    return out


class VisionHostWeights:
    """Seeded host copies of the vision tower's tensors: matrices and biases N(0, std), LayerNorm weights
    1 + N(0, std), from the counter-based generator shared with the device (seed + tensor index)."""

    def __init__(self, seed=4321, std=0.02):
        self.names, self.arrays = [], []
        for i, (name, shape) in enumerate(vision_tensor_list()):
            is_ln_w = name.endswith(("norm1.weight", "norm2.weight", "norm.weight"))
            self.names.append(name)
            self.arrays.append(seeded_bf16(shape, seed + i, 1.0 if is_ln_w else 0.0, std))

    def pointer_table(self):
        return (C.c_void_p * len(self.arrays))(*[a.ctypes.data for a in self.arrays])


def oracle_vision(vw, pixels_u16, grid_h, grid_w, want_blocks=False):
    """image_embeds [m,4096], deepstack [3,m,4096] (and every block's output [27,n,1152]) from the CPU oracle."""
    n = grid_h * grid_w
    m = n // 4
    emb = np.empty((m, 4096), dtype=np.uint16)
    ds = np.empty((3, m, 4096), dtype=np.uint16)
    blocks = np.empty((27, n, 1152), dtype=np.uint16) if want_blocks else None
    rc = oracle().orc_vision_forward(vw.pointer_table(), np_ptr(pixels_u16), grid_h, grid_w, np_ptr(emb), np_ptr(ds),
                                     np_ptr(blocks) if want_blocks else None)
    assert rc == 0
    return (emb, ds, blocks) if want_blocks else (emb, ds)
