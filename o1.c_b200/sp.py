"""Sequence-parallel (Ulysses) engine: drives the o1_sp_* stage functions of libo1b200.so and the two
all-to-all exchanges per block.  The reference is single-GPU; this is the added multi-GPU form of the
same forward.  Layout rules live in `layout()` and `shard_rows()` so they can be tested without a GPU.

Ranks of one forward form an SP group of size P (P divides the 8 KV heads).  With CFG the two branches
run on two SP groups; rank pairs with equal sp_rank exchange their predictions (all-gather) and apply the
identical fused scheduler update to their own rows of the latent.
"""
import ctypes as C

import torch

from . import lib, ptr, check, BlockBinding, ForwardBinding, PATCH_DIM, TMS_ID

c_int, c_void_p = C.c_int, C.c_void_p


class SpWs(C.Structure):
    """o1_sp_ws (include/o1_b200.h)."""
    _fields_ = [(n, c_int) for n in ("sp_size", "sp_rank", "S", "T", "row0", "rows", "heads", "kv_heads",
                                     "hidden", "ff", "head_dim", "ar_len")] + \
               [(n, c_void_p) for n in ("send", "gath", "attn", "recv", "ln", "ar", "post", "swi", "rope")]


class SpPeers(C.Structure):
    """o1_sp_peers (include/o1_b200.h): every SP rank's gath / recv / flag buffers as mapped here."""
    _fields_ = [("gath", c_void_p * 8), ("recv", c_void_p * 8), ("flags", c_void_p * 8), ("rope_full", c_void_p)]


class SpCtx(C.Structure):
    """o1_sp_ctx (include/o1_b200.h): everything o1_sp_forward needs for one rank."""
    _fields_ = [("ws", SpWs), ("peers", SpPeers), ("hid", c_void_p * 2), ("small", c_void_p), ("xe_stage", c_void_p),
                ("epoch", C.c_uint), ("visual_mask", c_void_p), ("image_embeds", c_void_p), ("deepstack", c_void_p * 3),
                ("embed_row0", c_int), ("visual_rows", c_int)]


class CfgPair(C.Structure):
    """o1_cfg_pair (include/o1_b200.h): prediction exchange with the CFG partner."""
    _fields_ = [("branch", c_int), ("xp_local", c_void_p * 2), ("xp_partner", c_void_p * 2), ("flags_local", c_void_p),
                ("flags_partner", c_void_p), ("step", C.c_uint)]


for _name, _res, _args in (("o1_peer_alloc", c_int, (C.POINTER(c_void_p), C.c_size_t)),
                           ("o1_peer_free", c_int, (c_void_p,)),
                           ("o1_peer_export", c_int, (c_void_p, C.POINTER(C.c_ubyte))),
                           ("o1_peer_open", c_int, (C.POINTER(C.c_ubyte), C.POINTER(c_void_p))),
                           ("o1_peer_close", c_int, (c_void_p,))):
    _f = getattr(lib, _name)
    _f.restype, _f.argtypes = _res, list(_args)

for _name, _args in (("o1_sp_rope_table", (C.POINTER(SpWs), c_void_p)),
                     ("o1_sp_rope_table_full", (C.POINTER(SpWs), C.POINTER(SpPeers), c_void_p)),
                     ("o1_sp_block_pre_direct", (C.POINTER(BlockBinding), C.POINTER(SpWs), C.POINTER(SpPeers),
                                                 c_void_p)),
                     ("o1_sp_block_attn_direct", (C.POINTER(BlockBinding), C.POINTER(SpWs), C.POINTER(SpPeers))),
                     ("o1_sp_barrier", (C.POINTER(SpWs), C.POINTER(SpPeers), C.c_uint)),
                     ("o1_sp_visual_scatter", (C.POINTER(SpWs), c_void_p, c_void_p, c_int, c_void_p, c_void_p)),
                     ("o1_sp_deepstack", (C.POINTER(SpWs), c_void_p, c_void_p, c_int, c_void_p, c_void_p)),
                     ("o1_sp_block_pre", (C.POINTER(BlockBinding), C.POINTER(SpWs), c_void_p)),
                     ("o1_sp_block_attn", (C.POINTER(SpWs),)),
                     ("o1_sp_block_post", (C.POINTER(BlockBinding), C.POINTER(SpWs), c_void_p, c_void_p)),
                     ("o1_sp_forward_begin", (C.POINTER(ForwardBinding), C.POINTER(SpWs), c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_void_p, c_int, c_void_p)),
                     ("o1_sp_forward_end", (C.POINTER(ForwardBinding), C.POINTER(SpWs), c_void_p, c_void_p,
                                            c_void_p)),
                     ("o1_sp_forward", (C.POINTER(ForwardBinding), C.POINTER(SpCtx), c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_int, c_void_p)),
                     ("o1_denoise_step_cfg_sp", (C.POINTER(ForwardBinding), C.POINTER(SpCtx), C.POINTER(CfgPair), c_void_p,
                                                 c_void_p, c_void_p, c_int, c_void_p, C.c_float, C.c_float, C.c_float,
                                                 c_int, c_void_p, c_void_p)),
                     ("o1_parallel_layout", (c_int, c_int, C.POINTER(c_int), C.POINTER(c_int), C.POINTER(c_int),
                                             C.POINTER(c_int)))):
    _f = getattr(lib, _name)
    _f.restype, _f.argtypes = c_int, list(_args)


def layout(world, cfg=True, max_sp=8):
    """rank -> (image index, cfg branch, sp_rank), plus sp_size, for `world` GPUs working on ONE image
    when possible: world 1 -> both branches on one GPU; 2 -> CFG pair; 4 -> CFG x SP2; 8 -> CFG x SP4.
    With cfg=True this is the library's o1_parallel_layout (which honours O1_CFG_SPLIT / O1_SP_DEGREE)."""
    if world == 1 or not cfg:
        sp = min(world, max_sp)
        return {r: (r // sp, None, r % sp) for r in range(world)}, sp
    out, sp_size = {}, None
    for r in range(world):
        img, br, sr, sp = c_int(), c_int(), c_int(), c_int()
        n = lib.o1_parallel_layout(world, r, C.byref(img), C.byref(br), C.byref(sr), C.byref(sp))
        if n < 0:
            raise ValueError(f"no layout for {world} GPUs with the O1_CFG_SPLIT / O1_SP_DEGREE in the environment")
        out[r] = (img.value, None if br.value < 0 else br.value, sr.value)
        sp_size = sp.value
    return out, sp_size


def shard_rows(S, T, P, r):
    """Rows, text rows and image rows (as half-open ranges) of SP rank r; S must be a multiple of P."""
    if S % P:
        raise ValueError(f"sequence length {S} is not a multiple of the SP degree {P}")
    rows = S // P
    row0 = r * rows
    t0, t1 = min(row0, T), min(row0 + rows, T)
    i0, i1 = max(row0, T) - T, max(row0 + rows, T) - T
    return (row0, row0 + rows), (t0, t1), (i0, i1)


class EngineSP:
    """One SP rank of one forward.

    Staged form: `exchange(src, dst)` performs the equal-split all-to-all of the contiguous tensor `src`
    into `dst` (same shape): torch.distributed.all_to_all_single in a real job, a peer-copy emulation in
    single-process tests.

    Direct form (`direct=True`, exchange unused): gath / recv / flags live in one peer-visible region
    (`self.region`); after `connect()` has been given every rank's region base, the q/k/v GEMM and
    attention epilogues store straight into the peers' buffers and `barrier()` orders the ranks."""

    def __init__(self, weights, text_len, img_tokens, sp_size, sp_rank, exchange=None, ar_len=None, direct=False):
        self.w, self.P, self.r, self.exchange = weights, sp_size, sp_rank, exchange
        self.direct, self.peers, self.region, self.epoch, self._opened = direct, None, None, 0, []
        self.visual = None
        d = weights.dims
        self.T, self.I, self.S = text_len, img_tokens, text_len + img_tokens
        (self.row0, _), (self.t0, self.t1), (self.i0, self.i1) = shard_rows(self.S, self.T, sp_size, sp_rank)
        self.rows = self.S // sp_size
        H, ff, hd = d["hidden"], d["ff"], d["head_dim"]
        qc, kc = d["heads"] * hd, d["kv_heads"] * hd
        if d["kv_heads"] % sp_size:
            raise ValueError("SP degree must divide the KV heads")
        self.C, self.Hc = (qc + 2 * kc) // sp_size, qc // sp_size
        dev = weights.device
        bf = dict(dtype=torch.bfloat16, device=dev)
        R, S = self.rows, self.S
        if direct:
            # one cudaMalloc'd region (exportable through CUDA IPC): gath | recv | flags
            self.gath_bytes = S * self.C * 2
            self.recv_bytes = S * self.Hc * 2
            self.region_bytes = self.gath_bytes + self.recv_bytes + 256
            reg = c_void_p()
            if lib.o1_peer_alloc(C.byref(reg), self.region_bytes) != 0:
                raise RuntimeError("peer region allocation failed")
            self.region = reg.value
            gath_ptr, recv_ptr = self.region, self.region + self.gath_bytes
            send_ptr = attn_ptr = 0
        else:
            self.send = torch.empty(sp_size, R, self.C, **bf)
            self.gath = self.send.view(S, self.C) if sp_size == 1 else torch.empty(S, self.C, **bf)
            self.attn = torch.empty(S, self.Hc, **bf)
            self.recv = (self.attn.view(sp_size, R, self.Hc) if sp_size == 1
                         else torch.empty(sp_size, R, self.Hc, **bf))
            gath_ptr, recv_ptr = self.gath.data_ptr(), self.recv.data_ptr()
            send_ptr, attn_ptr = self.send.data_ptr(), self.attn.data_ptr()
        self.ln, self.ar, self.post = (torch.empty(R, H, **bf) for _ in range(3))
        self.swi = torch.empty(R, ff, **bf)
        self.hid = [torch.empty(R, H, **bf) for _ in range(2)]
        self.rope = torch.empty(R, 128, dtype=torch.float32, device=dev)
        self.small = torch.empty(4 * H * 2 + 4096, dtype=torch.uint8, device=dev)
        self.xe_stage = torch.empty(max(1, self.i1 - self.i0), 1024, **bf)
        self.timestep = torch.zeros(1, dtype=torch.float32, device=dev)
        self.ws = SpWs(sp_size=sp_size, sp_rank=sp_rank, S=S, T=self.T, row0=self.row0, rows=R, heads=d["heads"],
                       kv_heads=d["kv_heads"], hidden=H, ff=ff, head_dim=hd,
                       ar_len=(text_len - 1 if ar_len is None else ar_len),
                       send=send_ptr, gath=gath_ptr, attn=attn_ptr,
                       recv=recv_ptr, ln=self.ln.data_ptr(), ar=self.ar.data_ptr(),
                       post=self.post.data_ptr(), swi=self.swi.data_ptr(), rope=self.rope.data_ptr())

    def set_visual(self, mask, image_embeds, deepstack):
        """Visual conditioning of the following forwards: mask uint8 [S] (device) marks the <image_pad> rows,
        image_embeds [V, hidden], deepstack = three [V, hidden] tensors; None switches it off.  Only ranks whose
        rows hold marked rows do any work; the count of marked rows before this rank's rows is taken once here."""
        if mask is None:
            self.visual = None
            return
        m = mask.to("cpu")
        first = int(m[:self.row0].sum())
        mine = int(m[self.row0:self.row0 + self.rows].sum())
        self.visual = (mask, image_embeds, list(deepstack), first) if mine else None

    def _visual_after_embed(self, cur, nxt):
        if self.visual is None:
            return cur, nxt
        mask, emb, _, first = self.visual
        check(lib.o1_sp_visual_scatter(C.byref(self.ws), ptr(mask), ptr(emb), first, ptr(cur), ptr(nxt)), "sp_scatter")
        return nxt, cur

    def _visual_after_block(self, l, cur, nxt):
        """cur holds the block's output; DeepStack writes the sum into the other buffer."""
        if self.visual is None or l >= 3:
            return cur, nxt
        mask, _, dss, first = self.visual
        check(lib.o1_sp_deepstack(C.byref(self.ws), ptr(mask), ptr(dss[l]), first, ptr(cur), ptr(nxt)), "sp_deepstack")
        return nxt, cur

    def connect(self, region_bases, opened=()):
        """region_bases[p]: base of SP rank p's region as mapped in this process (own region for p == r)."""
        pt = SpPeers()
        for p, base in enumerate(region_bases):
            pt.gath[p] = base
            pt.recv[p] = base + self.gath_bytes
            pt.flags[p] = base + self.gath_bytes + self.recv_bytes
        self.peers, self._opened = pt, list(opened)

    def barrier(self):
        self.epoch += 1
        check(lib.o1_sp_barrier(C.byref(self.ws), C.byref(self.peers), self.epoch), "sp_barrier")

    def close(self):
        for q in self._opened:
            lib.o1_peer_close(q)
        self._opened = []
        if self.region:
            lib.o1_peer_free(self.region)
            self.region = None

    # the forward is split into generator-style stages so that a single process can interleave several
    # emulated ranks; `forward()` runs them back to back for a real rank
    def stages(self, ids, pos, vin_local, t, out_local):
        ws, w = C.byref(self.ws), self.w
        self.timestep.fill_(float(t))
        if self.direct:
            yield from self._stages_direct(ids, pos, vin_local, out_local)
            return
        check(lib.o1_sp_rope_table(ws, ptr(pos)), "sp_rope_table")
        check(lib.o1_sp_forward_begin(C.byref(w.binding), ws, ptr(ids), ptr(vin_local), ptr(self.timestep),
                                      ptr(self.small), ptr(self.xe_stage), TMS_ID, ptr(self.hid[0])), "sp_begin")
        cur, nxt = self._visual_after_embed(*self.hid)
        for l in range(w.n_layers):
            bb = C.byref(w.block_binding(l))
            check(lib.o1_sp_block_pre(bb, ws, ptr(cur)), "sp_block_pre")
            yield ("a2a", self.send, self.gath.view(self.P, self.rows, self.C))
            check(lib.o1_sp_block_attn(ws), "sp_block_attn")
            yield ("a2a", self.attn.view(self.P, self.rows, self.Hc), self.recv)
            check(lib.o1_sp_block_post(bb, ws, ptr(cur), ptr(nxt)), "sp_block_post")
            cur, nxt = self._visual_after_block(l, nxt, cur)
        check(lib.o1_sp_forward_end(C.byref(w.binding), ws, ptr(cur), ptr(self.ln), ptr(out_local)), "sp_end")

    def _stages_direct(self, ids, pos, vin_local, out_local):
        ws, w, pt = C.byref(self.ws), self.w, C.byref(self.peers)
        check(lib.o1_sp_rope_table(ws, ptr(pos)), "sp_rope_table")      # own rows: norm + rope run in the sender's epilogue
        check(lib.o1_sp_forward_begin(C.byref(w.binding), ws, ptr(ids), ptr(vin_local), ptr(self.timestep),
                                      ptr(self.small), ptr(self.xe_stage), TMS_ID, ptr(self.hid[0])), "sp_begin")
        cur, nxt = self._visual_after_embed(*self.hid)
        for l in range(w.n_layers):
            bb = C.byref(w.block_binding(l))
            check(lib.o1_sp_block_pre_direct(bb, ws, pt, ptr(cur)), "sp_block_pre_direct")
            yield ("barrier", None, None)
            check(lib.o1_sp_block_attn_direct(bb, ws, pt), "sp_block_attn_direct")
            yield ("barrier", None, None)
            check(lib.o1_sp_block_post(bb, ws, ptr(cur), ptr(nxt)), "sp_block_post")
            cur, nxt = self._visual_after_block(l, nxt, cur)
        check(lib.o1_sp_forward_end(C.byref(w.binding), ws, ptr(cur), ptr(self.ln), ptr(out_local)), "sp_end")

    def ctx(self):
        """o1_sp_ctx of this rank (direct form, after connect())."""
        if getattr(self, "_ctx", None) is None:
            c = SpCtx()
            c.ws, c.peers = self.ws, self.peers
            c.hid[0], c.hid[1] = self.hid[0].data_ptr(), self.hid[1].data_ptr()
            c.small, c.xe_stage, c.epoch = self.small.data_ptr(), self.xe_stage.data_ptr(), self.epoch
            if self.visual is not None:
                mask, emb, dss, first = self.visual
                c.visual_mask, c.image_embeds, c.embed_row0 = mask.data_ptr(), emb.data_ptr(), first
                c.visual_rows = int(mask[self.row0:self.row0 + self.rows].sum().item())
                for k in range(3):
                    c.deepstack[k] = dss[k].data_ptr()
            self._ctx = c
        return self._ctx

    def forward_c(self, ids, pos, vin_local, t, out_local=None):
        """The same forward driven by ONE library call (o1_sp_forward) instead of the stage-by-stage loop."""
        if out_local is None:
            out_local = torch.empty(self.rows, PATCH_DIM, dtype=torch.bfloat16, device=self.w.device)
        self.timestep.fill_(float(t))
        c = self.ctx()
        c.epoch = max(c.epoch, self.epoch)          # one monotonic epoch sequence whichever path ran before
        check(lib.o1_sp_forward(C.byref(self.w.binding), C.byref(c), ptr(ids), ptr(pos), ptr(vin_local),
                                ptr(self.timestep), TMS_ID, ptr(out_local)), "o1_sp_forward")
        self.epoch = c.epoch
        return out_local

    def forward(self, ids, pos, vin_local, t, out_local=None):
        """x_pred rows of this rank, [rows, 3072] bf16."""
        if out_local is None:
            out_local = torch.empty(self.rows, PATCH_DIM, dtype=torch.bfloat16, device=self.w.device)
        if self.direct and self.peers is not None and getattr(self, "c_driver", False):
            return self.forward_c(ids, pos, vin_local, t, out_local)
        for kind, src, dst in self.stages(ids, pos, vin_local, t, out_local):
            if self.P == 1:
                continue
            if kind == "barrier":
                self.barrier()
            else:
                self.exchange(src, dst)
        return out_local


def nccl_exchange(group):
    """Equal-split all-to-all over a torch.distributed process group (NCCL over NVLink)."""
    import torch.distributed as dist

    def ex(src, dst):
        dist.all_to_all_single(dst.view(-1), src.view(-1), group=group)
    return ex


def connect_direct(engine, group):
    """Exchange CUDA IPC handles of the peer regions inside the SP process group (ranks in sp_rank order)
    and map them; every rank of the group must call this.  Returns True when every rank mapped every peer;
    otherwise every rank gets False with nothing left mapped (the caller then uses the staged exchange)."""
    import torch.distributed as dist
    h = (C.c_ubyte * 64)()
    ok = lib.o1_peer_export(engine.region, h) == 0
    handles = [None] * engine.P
    dist.all_gather_object(handles, bytes(h) if ok else None, group=group)
    bases, opened = [], []
    for p in range(engine.P):
        if p == engine.r:
            bases.append(engine.region)
            continue
        q = c_void_p()
        if not ok or handles[p] is None or \
                lib.o1_peer_open((C.c_ubyte * 64).from_buffer_copy(handles[p]), C.byref(q)) != 0:
            ok = False
            break
        bases.append(q.value)
        opened.append(q.value)
    flag = torch.tensor([1 if ok else 0], device=engine.w.device, dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)       # all ranks take the same branch
    if int(flag.item()) == 0:
        for q in opened:
            lib.o1_peer_close(q)
        return False
    engine.connect(bases, opened)
    torch.cuda.synchronize()
    dist.barrier(group=group)      # every region is zeroed and mapped before the first store into it
    return True


class CfgPairLink:
    """The CFG partner's prediction buffers and flags, mapped through CUDA IPC (o1_cfg_pair).  One region per
    rank: [parity 0 | parity 1] x [2 branches][local image rows][3072] bf16, then 256 bytes of flags."""

    def __init__(self, engine, branch, group):
        import torch.distributed as dist
        self.n_img = engine.i1 - engine.i0
        self.slot_bytes = 2 * self.n_img * PATCH_DIM * 2
        self.bytes = 2 * self.slot_bytes + 256
        reg = c_void_p()
        if lib.o1_peer_alloc(C.byref(reg), max(self.bytes, 512)) != 0:
            raise RuntimeError("pair region allocation failed")
        self.region, self.partner = reg.value, None
        h = (C.c_ubyte * 64)()
        ok = lib.o1_peer_export(self.region, h) == 0
        handles = [None, None]
        dist.all_gather_object(handles, bytes(h) if ok else None, group=group)
        other = handles[branch ^ 1]
        q = c_void_p()
        if ok and other is not None and lib.o1_peer_open((C.c_ubyte * 64).from_buffer_copy(other), C.byref(q)) == 0:
            self.partner = q.value
        flag = torch.tensor([1 if self.partner else 0], device=engine.w.device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        self.ok = int(flag.item()) == 1
        self.pair = CfgPair()
        if self.ok:
            p = self.pair
            p.branch = branch
            for k in range(2):
                p.xp_local[k] = self.region + k * self.slot_bytes
                p.xp_partner[k] = self.partner + k * self.slot_bytes
            p.flags_local, p.flags_partner = self.region + 2 * self.slot_bytes, self.partner + 2 * self.slot_bytes
            p.step = 0
            torch.cuda.synchronize()
            dist.barrier(group=group)

    def close(self):
        if self.partner:
            lib.o1_peer_close(self.partner)
            self.partner = None
        if self.region:
            lib.o1_peer_free(self.region)
            self.region = None


def run_emulated(engines, ids, pos, vin, t):
    """Single-process emulation of P ranks on one device: stages are advanced in lock step and each
    all-to-all is done by copies (slab d of rank s -> slab s of rank d).  Returns x_pred [S, 3072]."""
    P = len(engines)
    outs = [torch.empty(e.rows, PATCH_DIM, dtype=torch.bfloat16, device=e.w.device) for e in engines]
    gens = [e.stages(ids, pos, vin[e.i0:e.i1] if e.i1 > e.i0 else None, t, o) for e, o in zip(engines, outs)]
    while True:
        steps = []
        for g in gens:
            try:
                steps.append(next(g))
            except StopIteration:
                steps.append(None)
        if all(s is None for s in steps):
            break
        if steps[0][0] == "barrier":      # direct form: the lock-step order of one stream is the barrier
            continue
        for s in range(P):
            for d in range(P):
                steps[d][2][s].copy_(steps[s][1][d])
    return torch.cat(outs, 0)
