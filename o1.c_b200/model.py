"""Seeded random-init weights, sequence geometry and an Engine object that
drives hd_forward / hd_decoder_block / the CFG denoise step of libo1b200.so.

Mirrors, on the Python side, what o1.c's runtime does around the hot path:
weight arena + bindings (src/model/weights.c, forward.c:61-105), position ids
(src/runtime/sequence.c:67-160), sigma list (src/model/scheduler.c:26-64) and
the step loop (src/runtime/generate.c:1314-1455).
"""
import ctypes as C
import os

import torch

from . import (  # noqa: F401  (re-exported names)
    lib, ptr, check, check_cuda_errbuf, BlockBinding, BlockInternals, ForwardBinding,
    ForwardWorkspace, ForwardDiagnostics, LoraEntry, HIDDEN, HEADS, KV_HEADS, HEAD_DIM, FF, PATCH_DIM,
    XE_MID, VOCAB, TMS_ID, N_LAYERS,
)

SLOT_NAMES = ["q_proj", "k_proj", "v_proj", "o_proj", "input_ln", "post_ln", "gate_proj", "up_proj",
              "down_proj", "q_norm", "k_norm"]
GLOBAL_NAMES = ["embed_tokens", "te0_w", "te0_b", "te2_w", "te2_b", "xe1_w", "xe2_w", "xe2_b", "fl_w",
                "fl_b", "fnorm_w"]
NORM_NAMES = {"input_ln", "post_ln", "q_norm", "k_norm", "fnorm_w"}
DEV_TIMESTEPS = [999, 987, 974, 960, 945, 929, 913, 895, 877, 857, 836, 814, 790, 764, 737, 707, 675,
                 640, 602, 560, 515, 464, 409, 347, 278, 199, 110, 8]


def tensor_shape(name, hidden=HIDDEN, heads=HEADS, kv_heads=KV_HEADS, head_dim=HEAD_DIM, ff=FF,
                 vocab=VOCAB):
    """[out, in] shapes of the bound tensors (o1.c src/model/block.h:48-62, forward.h:40-59)."""
    return {
        "q_proj": (heads * head_dim, hidden), "k_proj": (kv_heads * head_dim, hidden),
        "v_proj": (kv_heads * head_dim, hidden), "o_proj": (hidden, heads * head_dim),
        "input_ln": (hidden,), "post_ln": (hidden,), "gate_proj": (ff, hidden), "up_proj": (ff, hidden),
        "down_proj": (hidden, ff), "q_norm": (head_dim,), "k_norm": (head_dim,),
        "embed_tokens": (vocab, hidden), "te0_w": (hidden, 256), "te0_b": (hidden,),
        "te2_w": (hidden, hidden), "te2_b": (hidden,), "xe1_w": (XE_MID, PATCH_DIM),
        "xe2_w": (hidden, XE_MID), "xe2_b": (hidden,), "fl_w": (PATCH_DIM, hidden), "fl_b": (PATCH_DIM,),
        "fnorm_w": (hidden,),
    }[name]


def weight_seed(seed, layer, name):
    """Seed of one tensor's counter-based stream. layer = -1 for the global tensors."""
    idx = (SLOT_NAMES.index(name) if layer >= 0 else GLOBAL_NAMES.index(name))
    return (int(seed) * 1000003 + (layer + 1) * 64 + idx) & 0xFFFFFFFFFFFFFFFF


def dev_sigmas():
    """28 Dev sigmas + trailing 0.0, fp32 (scheduler.c:26-64)."""
    return [float(torch.tensor(t, dtype=torch.float32) / 1000.0) for t in DEV_TIMESTEPS] + [0.0]


def seq_t2i(text_len, grid_h, grid_w, fix_point=4096):
    """Position ids fp32 [3, S] and ar_len for a T2I sequence (sequence.c:88-118, 120-142)."""
    S = text_len + grid_h * grid_w
    pos = torch.empty(3, S, dtype=torch.float32)
    t = torch.arange(text_len, dtype=torch.float32)
    pos[:, :text_len] = t
    hh = torch.arange(grid_h, dtype=torch.float32).repeat_interleave(grid_w)
    ww = torch.arange(grid_w, dtype=torch.float32).repeat(grid_h)
    pos[0, text_len:] = float(fix_point)
    pos[1, text_len:] = fix_point + hh
    pos[2, text_len:] = fix_point + ww
    return pos, text_len - 1


def seq_ref(text_ids, refs, grid_h, grid_w, fix_point=4096, vision_start_id=151652, image_pad_id=151655):
    """Token ids, position ids fp32 [3, S] and ar_len for a K-reference (edit / personalise) sequence
    (o1.c src/runtime/sequence.c:232-410).  `text_ids`: the expanded template -- K runs of
    <|vision_start|> + cond_h*cond_w <|image_pad|> -- followed by boi and the tms token.  `refs`: one
    (tokens, grid_h, grid_w, cond_h, cond_w) per reference.  Sequence = text | target grid | reference grids;
    the target grid sits at fix_point, each reference grid starts at (largest position so far) + 1 on all
    three axes, and every row from the tms token on attends to everything."""
    K, T = len(refs), len(text_ids)
    image_len = grid_h * grid_w
    S = T + image_len + sum(r[0] for r in refs)
    ids = list(int(t) for t in text_ids)
    ids += [vision_start_id] + [image_pad_id] * (image_len - 1)
    for r in refs:
        ids += [vision_start_id] + [image_pad_id] * (r[0] - 1)
    vs = [i for i, t in enumerate(ids) if t == vision_start_id]
    if len(vs) != 2 * K + 1:
        raise ValueError("expected %d vision-start tokens, found %d" % (2 * K + 1, len(vs)))
    pos = torch.zeros(3, S, dtype=torch.float32)
    max_pos, fp, st_pos = -1, fix_point, 0
    for v in range(2 * K + 1):
        skip = v >= K
        tlen = max(0, vs[v] + 1 - st_pos - (1 if skip else 0))
        st_idx = max_pos + 1 if max_pos >= 0 else 0
        pos[:, st_pos:st_pos + tlen] = torch.arange(st_idx, st_idx + tlen, dtype=torch.float32)
        max_pos = st_idx + tlen - 1
        gh, gw = (refs[v][3], refs[v][4]) if v < K else ((grid_h, grid_w) if v == K else
                                                         (refs[v - K - 1][1], refs[v - K - 1][2]))
        if skip:
            if fp > 0:
                fp -= st_idx
            base, fp = fp + st_idx, 0
        else:
            base = tlen + st_idx
        g0 = st_pos + tlen
        pos[0, g0:g0 + gh * gw] = float(base)
        pos[1, g0:g0 + gh * gw] = base + torch.arange(gh, dtype=torch.float32).repeat_interleave(gw)
        pos[2, g0:g0 + gh * gw] = base + torch.arange(gw, dtype=torch.float32).repeat(gh)
        max_pos = max(max_pos, base + max(gh, gw) - 1)
        st_pos += tlen + gh * gw
    if st_pos < S:
        pos[:, st_pos:] = torch.arange(max_pos + 1, max_pos + 1 + S - st_pos, dtype=torch.float32)
    return torch.tensor(ids, dtype=torch.int64), pos, T - 1


class Weights:
    """One 256-byte-aligned device arena of bf16 tensors, filled by the library's
    counter-based generator so that the CPU oracle can regenerate any tensor.

    weight_set "A": every tensor ~ N(0, std).  "B": RMSNorm weights are
    1 + N(0, std) instead, which keeps attention logits away from zero.
    """

    def __init__(self, n_layers=N_LAYERS, seed=1234, weight_set="A", std=0.02, device="cuda",
                 hidden=HIDDEN, heads=HEADS, kv_heads=KV_HEADS, head_dim=HEAD_DIM, ff=FF, vocab=VOCAB):
        self.n_layers, self.seed, self.weight_set, self.std = n_layers, seed, weight_set, std
        self.dims = dict(hidden=hidden, heads=heads, kv_heads=kv_heads, head_dim=head_dim, ff=ff,
                         vocab=vocab)
        self.device = torch.device(device)
        entries = [(-1, n) for n in GLOBAL_NAMES] + [(l, n) for l in range(n_layers) for n in SLOT_NAMES]
        self.offsets, off = {}, 0
        for layer, name in entries:
            shape = tensor_shape(name, **self.dims)
            n = 1
            for d in shape:
                n *= d
            self.offsets[(layer, name)] = (off, shape, n)
            off += (n * 2 + 255) & ~255
        self.arena = torch.empty(off, dtype=torch.uint8, device=self.device)
        assert self.arena.data_ptr() % 256 == 0
        with torch.cuda.device(self.device):
            from . import use_torch_stream
            use_torch_stream()
            for (layer, name), (o, shape, n) in self.offsets.items():
                mean = 1.0 if (weight_set == "B" and name in NORM_NAMES) else 0.0
                rc = lib.o1_fill_normal_bf16(C.c_void_p(self.arena.data_ptr() + o), n,
                                             weight_seed(seed, layer, name), mean, std)
                if rc != 0:
                    check_cuda_errbuf("fill_normal")
        self._blocks = (BlockBinding * n_layers)()
        for l in range(n_layers):
            self._blocks[l].layer_idx = l
            for name in SLOT_NAMES:
                setattr(self._blocks[l], name, self.addr(l, name))
        self.binding = ForwardBinding()
        for name in GLOBAL_NAMES:
            setattr(self.binding, name, self.addr(-1, name))
        self.binding.n_layers = n_layers
        self.binding.blocks = C.cast(self._blocks, C.POINTER(BlockBinding))

    def addr(self, layer, name):
        return self.arena.data_ptr() + self.offsets[(layer, name)][0]

    def tensor(self, layer, name):
        """bf16 torch view of one tensor inside the arena."""
        o, shape, n = self.offsets[(layer, name)]
        return self.arena[o:o + n * 2].view(torch.bfloat16).view(*shape)

    def block_binding(self, layer):
        return self._blocks[layer]

    def nbytes(self):
        return self.arena.numel()


class Engine:
    """Workspace + call wrappers for one sequence geometry on one GPU."""

    def __init__(self, weights, text_len, img_tokens, ar_len=None):
        self.w = weights
        self.T, self.I, self.S = text_len, img_tokens, text_len + img_tokens
        self.ar_len = text_len - 1 if ar_len is None else ar_len
        d = weights.dims
        self.dimargs = (d["heads"], d["kv_heads"], d["hidden"], d["ff"], d["head_dim"])
        self.device = weights.device
        bs = C.c_int64(0)
        nbytes = lib.hd_forward_workspace_bytes(self.S, self.I, *self.dimargs, C.byref(bs))
        self.block_scratch_bytes = bs.value
        self.ws_buf = torch.empty(nbytes + 256, dtype=torch.uint8, device=self.device)
        self.ws = ForwardWorkspace()
        self.ws.hidden_a = self.ws_buf.data_ptr()
        self.ws.block_scratch_bytes = bs.value
        plan = C.c_void_p()
        rc = lib.hd_sdpa_create_split(C.byref(plan), 1, d["heads"], d["kv_heads"], self.S, self.ar_len,
                                      d["head_dim"], float(d["head_dim"]) ** -0.5)
        if rc != 0:
            check_cuda_errbuf("sdpa_create")
        self.plan = plan
        self.ws.sdpa = plan
        self.xp = torch.empty(2 * self.S * PATCH_DIM, dtype=torch.bfloat16, device=self.device)
        self.timestep = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.sec = torch.tensor([24, 20, 20], dtype=torch.int64, device=self.device)

    def __del__(self):
        try:
            if getattr(self, "plan", None):
                lib.hd_sdpa_destroy(self.plan)
        except Exception:
            pass

    def ws_region(self, name, nbytes):
        bs = C.c_int64(0)
        off = lib.hd_forward_ws_offset(name.encode(), self.S, self.T, self.I, *self.dimargs, C.byref(bs))
        if off < 0:
            raise KeyError(name)
        return self.ws_buf[off:off + nbytes]

    def block(self, x, pos, layer, internals=False, mod6=None):
        """hd_decoder_block on x [S, hidden] bf16; returns out (and the five internals).  With mod6
        ([6*hidden] bf16: shift/scale/gate for the attention and the MLP branch) the adaLN variant runs."""
        out = torch.empty_like(x)
        scratch = self.ws_region("block_scratch", self.block_scratch_bytes)
        ints, bufs = None, {}
        if internals:
            ints = BlockInternals()
            for n in ("ln0", "attn_hidden", "attn_resid", "post_ln", "mlp_out"):
                bufs[n] = torch.empty_like(x)
                setattr(ints, n, bufs[n].data_ptr())
        bb = self.w.block_binding(layer)
        fn = lib.hd_decoder_block if mod6 is None else lib.o1_decoder_block_adaln
        rc = fn(ptr(x), ptr(pos), None, C.byref(bb), ptr(self.sec if mod6 is None else mod6), ptr(scratch),
                self.block_scratch_bytes, C.byref(ints) if ints else None, ptr(out), self.S, *self.dimargs, self.plan)
        check(rc, "hd_decoder_block")
        return (out, bufs) if internals else out

    def set_ref_cache(self, xe_ref):
        """Precomputed x_embedder rows of the trailing reference tokens (forward.h:79-88): the edit path
        feeds the same reference pixels every step, so their embedding is computed once."""
        self._xe_ref = xe_ref
        self.ws.xe_ref = xe_ref.data_ptr() if xe_ref is not None else None
        self.ws.n_ref = xe_ref.shape[0] if xe_ref is not None else 0

    def forward(self, ids, pos, vinputs, t, out=None, diag_names=(), visual=None):
        """hd_forward; t is the model timestep (1 - sigma). Returns x_pred [S, 3072] bf16.
        visual = (mask uint8 [S], image_embeds [V,H], (deepstack0, 1, 2)) device tensors, or None."""
        if out is None:
            out = torch.empty(self.S, PATCH_DIM, dtype=torch.bfloat16, device=self.device)
        self.timestep.fill_(float(t))
        diag, bufs = None, {}
        if diag_names:
            diag = ForwardDiagnostics()
            d = self.w.dims
            for n in diag_names:
                rows = {"after_embedding": self.T, "after_timestep_conditioning": self.T,
                        "after_target_embedding": self.I}.get(n, self.S)
                cols = PATCH_DIM if n == "after_final_head" else d["hidden"]
                bufs[n] = torch.empty(rows, cols, dtype=torch.bfloat16, device=self.device)
                setattr(diag, n, bufs[n].data_ptr())
        d = self.w.dims
        vc = None
        if visual is not None:
            from . import VisualCond
            vmask, emb, dss = visual
            vc = VisualCond(image_embeds=emb.data_ptr(), visual_mask=vmask.data_ptr(), v_tokens=emb.shape[0])
            for k in range(3):
                vc.deepstack[k] = dss[k].data_ptr()
        rc = lib.hd_forward(C.byref(self.w.binding), C.byref(self.ws), ptr(ids), self.T, ptr(pos), None,
                            ptr(vinputs), self.I, C.byref(vc) if vc else None, ptr(self.timestep), ptr(self.sec), self.S,
                            *self.dimargs, TMS_ID, C.byref(diag) if diag else None, ptr(out), None)
        check(rc, "hd_forward")
        return (out, bufs) if diag_names else out

    def denoise_step_cfg(self, ids_c, ids_u, pos, z, sigma, sigma_next, guidance, z_next=None):
        """One CFG flow-match step on device-resident latents z [I, 3072] bf16."""
        if z_next is None:
            z_next = torch.empty_like(z)
        self.timestep.fill_(1.0 - float(sigma))
        rc = lib.o1_denoise_step_cfg(C.byref(self.w.binding), C.byref(self.ws), ptr(ids_c), ptr(ids_u),
                                     self.T, ptr(pos), self.ar_len, ptr(z), self.I, ptr(self.timestep),
                                     float(sigma), float(sigma_next), float(guidance), ptr(self.xp),
                                     ptr(z_next), *self.dimargs, TMS_ID)
        check(rc, "o1_denoise_step_cfg")
        return z_next

    def denoise_step_cfg_ref(self, ids_c, ids_u, pos, vin, target_tokens, sigma, sigma_next, guidance, z_next):
        """CFG step of a reference / edit sequence: vin [I, 3072] = target latent rows then the static
        reference rows; only the first target_tokens rows are stepped into z_next."""
        self.timestep.fill_(1.0 - float(sigma))
        rc = lib.o1_denoise_step_cfg_ref(C.byref(self.w.binding), C.byref(self.ws), ptr(ids_c), ptr(ids_u), self.T,
                                         ptr(pos), self.ar_len, ptr(vin), self.I, target_tokens, None,
                                         ptr(self.timestep), float(sigma), float(sigma_next), float(guidance),
                                         ptr(self.xp), ptr(z_next), *self.dimargs, TMS_ID)
        check(rc, "o1_denoise_step_cfg_ref")
        return z_next

    def denoise_step_cfg_branches(self, cond, uncond, z, sigma, sigma_next, guidance, z_next=None):
        """CFG step whose branches have their own sequences: cond / uncond = (ids [T_b], pos [3, T_b + I],
        ar_len) with T_b <= the text length this engine was sized for."""
        from . import CfgBranch
        if z_next is None:
            z_next = torch.empty_like(z)
        self.timestep.fill_(1.0 - float(sigma))
        br = []
        for ids, pos, ar in (cond, uncond):
            assert ids.numel() <= self.T
            br.append(CfgBranch(ids=ids.data_ptr(), text_len=ids.numel(), pos_f32=pos.data_ptr(), ar_len=ar))
        rc = lib.o1_denoise_step_cfg_branches(C.byref(self.w.binding), C.byref(self.ws), C.byref(br[0]),
                                              C.byref(br[1]), ptr(z), self.I, self.I, ptr(self.timestep),
                                              float(sigma), float(sigma_next), float(guidance), ptr(self.xp),
                                              ptr(z_next), *self.dimargs, TMS_ID)
        check(rc, "o1_denoise_step_cfg_branches")
        return z_next

    def denoise_step_cfg_host(self, ids_c, ids_u, pos, z_host, z_dev, sigma, sigma_next, guidance,
                              z_next_dev, z_next_host):
        """Same step through host (pinned) latents: H2D, step, D2H, synchronise."""
        rc = lib.o1_denoise_step_cfg_host(C.byref(self.w.binding), C.byref(self.ws), ptr(ids_c),
                                          ptr(ids_u), self.T, ptr(pos), self.ar_len, ptr(z_host),
                                          ptr(z_dev), self.I, float(sigma), float(sigma_next),
                                          float(guidance), ptr(self.timestep), ptr(self.xp),
                                          ptr(z_next_dev), ptr(z_next_host), *self.dimargs, TMS_ID)
        check(rc, "o1_denoise_step_cfg_host")
        return z_next_host


# ------------------------------------------------------------------ GGUF packs
GGUF_NAMES = {
    "embed_tokens": "model.language_model.embed_tokens.weight", "te0_w": "model.t_embedder1.mlp.0.weight",
    "te0_b": "model.t_embedder1.mlp.0.bias", "te2_w": "model.t_embedder1.mlp.2.weight",
    "te2_b": "model.t_embedder1.mlp.2.bias", "xe1_w": "model.x_embedder.proj1.weight",
    "xe2_w": "model.x_embedder.proj2.weight", "xe2_b": "model.x_embedder.proj2.bias",
    "fl_w": "model.final_layer2.linear.weight", "fl_b": "model.final_layer2.linear.bias",
    "fnorm_w": "model.language_model.norm.weight",
    "q_proj": "self_attn.q_proj.weight", "k_proj": "self_attn.k_proj.weight", "v_proj": "self_attn.v_proj.weight",
    "o_proj": "self_attn.o_proj.weight", "input_ln": "input_layernorm.weight",
    "post_ln": "post_attention_layernorm.weight", "gate_proj": "mlp.gate_proj.weight",
    "up_proj": "mlp.up_proj.weight", "down_proj": "mlp.down_proj.weight", "q_norm": "self_attn.q_norm.weight",
    "k_norm": "self_attn.k_norm.weight",
}


def gguf_tensor_name(layer, name):
    """Manifest name of a bound tensor (o1.c src/model/forward.c:70-80, block.c:70-82)."""
    return GGUF_NAMES[name] if layer < 0 else f"model.language_model.layers.{layer}.{GGUF_NAMES[name]}"


def write_gguf(path, tensors, metadata=None, alignment=256):
    """Writes a GGUF v3 pack in the byte layout of o1.c's tools/hidream_convert.py:223-286: magic, version 3,
    string key/values + general.alignment (u32), tensor table (dims in torch order, F32 = 0 / F16 = 1 /
    BF16 = 30), data section aligned to `alignment`, every tensor at an aligned offset.
    tensors: list of (name, numpy array) with dtype float32, float16 or uint16 (bf16 bit patterns)."""
    import struct
    import numpy as np

    def s(b):
        b = b.encode() if isinstance(b, str) else b
        return struct.pack("<Q", len(b)) + b

    kv = [(k, v) for k, v in (metadata or {}).items()]
    head = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(kv) + 1)
    for k, v in kv:
        head += s(k) + struct.pack("<I", 8) + s(v)
    head += s("general.alignment") + struct.pack("<I", 4) + struct.pack("<I", alignment)
    table, off, offsets = b"", 0, []
    for name, a in tensors:
        t = {np.dtype(np.float32): 0, np.dtype(np.float16): 1, np.dtype(np.uint16): 30}[a.dtype]
        table += s(name) + struct.pack("<I", a.ndim) + b"".join(struct.pack("<Q", d) for d in a.shape)
        table += struct.pack("<I", t) + struct.pack("<Q", off)
        offsets.append(off)
        off += (a.nbytes + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(head + table)
        pos = f.tell()
        f.write(b"\0" * ((pos + alignment - 1) // alignment * alignment - pos))
        start = f.tell()
        for (name, a), o in zip(tensors, offsets):
            f.seek(start + o)
            f.write(np.ascontiguousarray(a).tobytes())
        f.truncate(start + off)


class _DevBytes:
    """Zero-copy torch view of raw device memory through the CUDA array interface."""

    def __init__(self, ptr_, nbytes):
        self.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (int(ptr_), False),
                                         "version": 2}


class GgufWeights:
    """A GGUF pack on the device (hd_weights_to_device_gguf + hd_forward_resolve).  With a process group only
    rank `src` reads the payload; the other ranks allocate the identical arena from the header and receive
    the bytes by one broadcast (o1.c src/model/weights.c:519-669 would read the file once per process)."""

    def __init__(self, path, n_layers, device, group=None, src=0):
        from . import WeightStore, ForwardBinding
        self.device = torch.device(device)
        idx = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.store, self.binding, self.n_layers = WeightStore(), ForwardBinding(), n_layers
        # the architecture is fixed on this path (o1.c src/model/block.h:48-62); a pack with other shapes
        # fails in the kernels' shape checks
        self.dims = dict(hidden=HIDDEN, heads=HEADS, kv_heads=KV_HEADS, head_dim=HEAD_DIM, ff=FF, vocab=VOCAB)
        reader = True
        if group is not None:
            import torch.distributed as dist
            reader = dist.get_rank() == src
        fn = lib.hd_weights_to_device_gguf if reader else lib.o1_weights_gguf_layout
        if fn(os.fsencode(path), idx, C.byref(self.store)) != 0:
            raise RuntimeError(lib.hd_weights_last_error().decode())
        if group is not None:
            import torch.distributed as dist
            arena = torch.as_tensor(_DevBytes(self.store.arena_ptr, self.store.arena_bytes), device=self.device)
            dist.broadcast(arena, src=src, group=group)
            torch.cuda.synchronize()
        if lib.hd_forward_resolve(C.byref(self.store), n_layers, C.byref(self.binding)) != 0:
            err = lib.hd_last_error().decode()
            lib.hd_weight_store_free(C.byref(self.store))
            raise RuntimeError(err)

    def block_binding(self, layer):
        return self.binding.blocks[layer]

    def nbytes(self):
        return int(self.store.arena_bytes)

    def close(self):
        lib.hd_forward_binding_free(C.byref(self.binding))
        lib.hd_weight_store_free(C.byref(self.store))
