"""Drives the reference's own CUDA build (oracle/_ref/libo1ref.so: o1.c's sources compiled unchanged,
cuBLASLt GEMMs + cuDNN SDPA) WITHOUT the product library: seeded weights come from the CPU oracle's
generator and are copied to the device, positions and sigmas from the oracle, structs are declared here
from the reference headers.  bench.py's reference arm and the size-parity checks are built on this, so a
process that only imports this module never maps libo1b200.so.

Checker-side code: only tests/, bench.py's reference arm and the parity probe use it.
"""
import ctypes as C

import numpy as np
import torch

import parity
from parity import np_ptr

HIDDEN, HEADS, KV_HEADS, HEAD_DIM, FF = 4096, 32, 8, 128, 12288
PATCH_DIM, XE_MID, VOCAB, TMS_ID = 3072, 1024, 151936, 151673
SLOT_NAMES = ["q_proj", "k_proj", "v_proj", "o_proj", "input_ln", "post_ln", "gate_proj", "up_proj",
              "down_proj", "q_norm", "k_norm"]
GLOBAL_NAMES = ["embed_tokens", "te0_w", "te0_b", "te2_w", "te2_b", "xe1_w", "xe2_w", "xe2_b", "fl_w",
                "fl_b", "fnorm_w"]
NORM_NAMES = {"input_ln", "post_ln", "q_norm", "k_norm", "fnorm_w"}
DIMARGS = (HEADS, KV_HEADS, HIDDEN, FF, HEAD_DIM)
DIAG_NAMES = ("after_embedding", "after_timestep_conditioning", "after_target_embedding", "after_block_0_input",
              "after_block_0", "after_block_mid", "after_block_last", "before_final_norm", "after_final_norm",
              "after_final_head")

_P = C.c_void_p


class BlockBinding(C.Structure):
    """hd_block_binding (o1.c src/model/block.h:48-62)."""
    _fields_ = [("layer_idx", C.c_int)] + [(n, _P) for n in SLOT_NAMES]


class ForwardBinding(C.Structure):
    """hd_forward_binding (src/model/forward.h:40-59)."""
    _fields_ = [(n, _P) for n in GLOBAL_NAMES] + [("n_layers", C.c_int), ("blocks", C.POINTER(BlockBinding))]


class ForwardWorkspace(C.Structure):
    """hd_forward_workspace (src/model/forward.h:66-93)."""
    _fields_ = [(n, _P) for n in ("hidden_a", "hidden_b", "h_text", "norm_out", "head_out", "t_emb", "te_hidden",
                                  "freq", "freq_bf16", "t_scaled", "xe_stage", "xe_out", "xe_ref")] + [
        ("n_ref", C.c_int), ("block_scratch", _P), ("block_scratch_bytes", C.c_int64), ("sdpa", _P)]


class ForwardDiagnostics(C.Structure):
    """hd_forward_diagnostics (src/model/forward.h:96-107)."""
    _fields_ = [(n, _P) for n in DIAG_NAMES]


def tensor_shape(name):
    return {
        "q_proj": (HEADS * HEAD_DIM, HIDDEN), "k_proj": (KV_HEADS * HEAD_DIM, HIDDEN),
        "v_proj": (KV_HEADS * HEAD_DIM, HIDDEN), "o_proj": (HIDDEN, HEADS * HEAD_DIM),
        "input_ln": (HIDDEN,), "post_ln": (HIDDEN,), "gate_proj": (FF, HIDDEN), "up_proj": (FF, HIDDEN),
        "down_proj": (HIDDEN, FF), "q_norm": (HEAD_DIM,), "k_norm": (HEAD_DIM,),
        "embed_tokens": (VOCAB, HIDDEN), "te0_w": (HIDDEN, 256), "te0_b": (HIDDEN,), "te2_w": (HIDDEN, HIDDEN),
        "te2_b": (HIDDEN,), "xe1_w": (XE_MID, PATCH_DIM), "xe2_w": (HIDDEN, XE_MID), "xe2_b": (HIDDEN,),
        "fl_w": (PATCH_DIM, HIDDEN), "fl_b": (PATCH_DIM,), "fnorm_w": (HIDDEN,),
    }[name]


def weight_seed(seed, layer, name):
    """Seed of one tensor's counter-based stream (the same rule as the product's seeded arena)."""
    idx = SLOT_NAMES.index(name) if layer >= 0 else GLOBAL_NAMES.index(name)
    return (int(seed) * 1000003 + (layer + 1) * 64 + idx) & 0xFFFFFFFFFFFFFFFF


def arena_layout(n_layers):
    """(layer, name) -> (byte offset, shape, numel), 256-byte aligned, globals first: the layout of the
    product's seeded arena, so both arms hold the same bytes at the same offsets."""
    entries = [(-1, n) for n in GLOBAL_NAMES] + [(l, n) for l in range(n_layers) for n in SLOT_NAMES]
    offsets, off = {}, 0
    for layer, name in entries:
        shape = tensor_shape(name)
        n = int(np.prod(shape))
        offsets[(layer, name)] = (off, shape, n)
        off += (n * 2 + 255) & ~255
    return offsets, off


class HostFilledWeights:
    """Seeded weights generated on the HOST by the oracle's counter-based generator and copied to the device
    through a pinned staging buffer; bit-identical to the arena the product fills on the device."""

    def __init__(self, n_layers, device, seed=1234, weight_set="A", std=0.02):
        self.n_layers, self.device = n_layers, torch.device(device)
        self.offsets, total = arena_layout(n_layers)
        self.arena = torch.empty(total, dtype=torch.uint8, device=self.device)
        orc = parity.oracle()
        chunk = 64 << 20                                   # elements per staging pass (128 MB)
        stage = torch.empty(chunk, dtype=torch.int16).pin_memory()
        stage_np = stage.numpy().view(np.uint16)
        for (layer, name), (o, shape, n) in self.offsets.items():
            mean = 1.0 if (weight_set == "B" and name in NORM_NAMES) else 0.0
            s = weight_seed(seed, layer, name)
            cols = shape[-1]
            rows = n // cols
            r0 = 0
            while r0 < rows:
                nr = min(rows - r0, max(1, chunk // cols))
                orc.orc_fill_normal_rows_bf16(np_ptr(stage_np), r0, nr, cols, s, mean, std)
                dst = self.arena[o + r0 * cols * 2: o + (r0 + nr) * cols * 2]
                dst.copy_(stage[:nr * cols].view(torch.uint8), non_blocking=True)
                torch.cuda.synchronize()
                r0 += nr
        self.binding, self._blocks = make_binding(self.arena.data_ptr(), self.offsets, n_layers)

    def nbytes(self):
        return self.arena.numel()


def make_binding(base, offsets, n_layers):
    blocks = (BlockBinding * n_layers)()
    for l in range(n_layers):
        blocks[l].layer_idx = l
        for name in SLOT_NAMES:
            setattr(blocks[l], name, base + offsets[(l, name)][0])
    b = ForwardBinding()
    for name in GLOBAL_NAMES:
        setattr(b, name, base + offsets[(-1, name)][0])
    b.n_layers = n_layers
    b.blocks = C.cast(blocks, C.POINTER(BlockBinding))
    return b, blocks


def seq_t2i(T, gh, gw):
    """Position ids fp32 [3,S] (torch, host) and ar_len from the oracle's restatement of hd_seq_t2i."""
    S = T + gh * gw
    pos = np.empty((3, S), dtype=np.float32)
    ar = parity.oracle().orc_seq_t2i(T, gh, gw, 4096, np_ptr(pos))
    return torch.from_numpy(pos), ar


def dev_sigmas():
    s = np.empty(29, dtype=np.float32)
    assert parity.oracle().orc_sigmas_dev(np_ptr(s)) == 29
    return [float(v) for v in s]


def seeded_ids(T, seed=7):
    """Two independent text id vectors of length T (cond, uncond), tms token last; the bench's convention."""
    g = torch.Generator().manual_seed(seed)
    ids_c = torch.randint(0, 151000, (T,), generator=g, dtype=torch.int64)
    ids_u = torch.randint(0, 151000, (T,), generator=g, dtype=torch.int64)
    ids_c[-1] = ids_u[-1] = TMS_ID
    return ids_c, ids_u


def seeded_latent(I, seed=43, std=8.0):
    """bf16 [I,3072] ~ N(0, std^2) from the shared counter-based generator (host)."""
    return parity.u16_to_torch(parity.seeded_bf16((I, PATCH_DIM), seed, 0.0, std))


def ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


class RefEngine:
    """hd_forward and the CFG flow-match step of the reference build for one T2I geometry.
    binding: a ForwardBinding-compatible ctypes struct whose pointers are device addresses of the weights.
    production=True: cuBLASLt + cuDNN two-pass SDPA (the reference's production backend);
    False: its 16x16 source GEMM + eager attention (slow; small shapes only)."""

    def __init__(self, binding, T, gh, gw, device, production=True):
        r = parity.reflib()
        if r is None:
            raise RuntimeError("oracle/_ref/libo1ref.so is not built")
        self.r, self.binding, self.device = r, binding, torch.device(device)
        self.T, self.I = T, gh * gw
        self.S = self.T + self.I
        dev_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        pos, self.ar = seq_t2i(T, gh, gw)
        self.pos = pos.to(self.device)
        bs = C.c_int64(0)
        nbytes = r.hd_forward_workspace_bytes(self.S, self.I, *DIMARGS, C.byref(bs))
        self.buf = torch.empty(nbytes + 256, dtype=torch.uint8, device=self.device)
        self.ws = ForwardWorkspace()
        self.ws.hidden_a, self.ws.block_scratch_bytes = self.buf.data_ptr(), bs.value
        self.rt, self.plan, self.production = None, None, production
        if production:
            self.rt = r.hd_gemm_runtime_init(dev_index, 64 << 20)
            if not self.rt:
                raise RuntimeError("hd_gemm_runtime_init failed")
            r.hd_gemm_set_backend(1)
            plan = C.c_void_p()
            if r.hd_sdpa_create_prod(C.byref(plan), 1, HEADS, KV_HEADS, self.S, self.ar, HEAD_DIM,
                                     HEAD_DIM ** -0.5) != 0:
                raise RuntimeError("hd_sdpa_create_prod failed: %s" % r.hd_cuda_last_error())
            self.plan = plan
            self.ws.sdpa = plan
        else:
            r.hd_gemm_set_backend(0)
        rows = torch.arange(self.S, device=self.device)
        # prefix-causal additive mask [S,S] bf16: 0 = visible, 0xFF7F = masked (src/runtime/sequence.c:22,120-142)
        self.mask = ((rows[None, :] > rows[:, None]) & (rows[:, None] < self.ar)).to(torch.int16) * -129
        self.sec = torch.tensor([24, 20, 20], dtype=torch.int64, device=self.device)
        self.tt = torch.zeros(1, device=self.device)
        self.xc = torch.empty(self.S, PATCH_DIM, dtype=torch.bfloat16, device=self.device)
        self.xu = torch.empty_like(self.xc)
        n = self.I * PATCH_DIM
        self.mc, self.mu, self.mo = (torch.empty(n, device=self.device) for _ in range(3))

    def close(self):
        self.r.hd_cuda_clear_error()          # e.g. the note cuBLASLt leaves when it falls back for one shape
        if self.plan:
            self.r.hd_sdpa_destroy(self.plan)
            self.plan = None
        if self.rt:
            self.r.hd_gemm_runtime_destroy(self.rt)
            self.rt = None

    def forward(self, ids, zin, t, out, diag_names=()):
        """x_pred [S,3072] of one branch; diag_names: hd_forward_diagnostics hooks to capture."""
        self.tt.fill_(float(t))
        self.r.hd_gemm_set_backend(1 if self.production else 0)      # a process-wide switch in the reference
        diag, bufs = None, {}
        if diag_names:
            diag = ForwardDiagnostics()
            for n in diag_names:
                rows = {"after_embedding": self.T, "after_timestep_conditioning": self.T,
                        "after_target_embedding": self.I}.get(n, self.S)
                cols = PATCH_DIM if n == "after_final_head" else HIDDEN
                bufs[n] = torch.empty(rows, cols, dtype=torch.bfloat16, device=self.device)
                setattr(diag, n, bufs[n].data_ptr())
        rc = self.r.hd_forward(C.byref(self.binding), C.byref(self.ws), ptr(ids), self.T, ptr(self.pos),
                               ptr(self.mask), ptr(zin), self.I, None, ptr(self.tt), ptr(self.sec), self.S,
                               *DIMARGS, TMS_ID, C.byref(diag) if diag else None, ptr(out), None)
        if rc != 0:
            raise RuntimeError("reference hd_forward failed: %s" % self.r.hd_last_error())
        return bufs

    def cfg_step(self, ids_c, ids_u, zin, zout, s0, s1, guidance):
        """hd_forward x2 -> hd_sched_vcond x2 -> hd_sched_cfg_guided -> hd_sched_flow_match_step: the composition
        of src/runtime/generate.c:1314-1360 with the flow-match update of :900-905."""
        r = self.r
        self.forward(ids_c, zin, 1.0 - s0, self.xc)
        self.forward(ids_u, zin, 1.0 - s0, self.xu)
        n = self.I * PATCH_DIM
        r.hd_sched_vcond(ptr(zin), ptr(self.xc[self.T:]), s0, ptr(self.mc), n)
        r.hd_sched_vcond(ptr(zin), ptr(self.xu[self.T:]), s0, ptr(self.mu), n)
        r.hd_sched_cfg_guided(ptr(self.mc), ptr(self.mu), guidance, ptr(self.mo), n)
        r.hd_sched_flow_match_step(ptr(zin), ptr(self.mo), s0, s1, ptr(zout), n)
