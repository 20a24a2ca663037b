"""Host-side multi-GPU logic on CPU ranks (gloo, world size 2 and 4): the rank layout, the row sharding,
the slab algebra of the two Ulysses exchanges (checked with real all_to_all_single calls on CPU tensors),
the CFG-pair all-gather, and failure detection on the host (a rank that never arrives makes the others'
collective end with an error instead of hanging)."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _init(rank, world, port, timeout_s=60):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=timeout_s))


def _load():
    import sys
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package
    load_package()
    from o1c_b200 import sp
    return sp


def _a2a(src, dst):
    """Equal-split all-to-all built from point-to-point calls (this gloo build has no alltoall):
    slab d of `src` goes to rank d, slab s of the result came from rank s."""
    rank, world = dist.get_rank(), dist.get_world_size()
    outs = [torch.empty_like(dst[s]) for s in range(world)]
    outs[rank].copy_(src[rank])
    reqs = []
    for peer in range(world):
        if peer == rank:
            continue
        reqs.append(dist.isend(src[peer].contiguous(), peer))
        reqs.append(dist.irecv(outs[peer], peer))
    for r in reqs:
        r.wait()
    return outs


def _worker_ulysses(rank, world, port, q):
    try:
        sp = _load()
        _init(rank, world, port)
        P, S, heads, kv, hd = world, 8 * world, 8, 4 if world <= 4 else 8, 2
        rows = S // P
        # global activations every rank can rebuild: value encodes (row, column)
        C = (heads + 2 * kv) * hd
        full = (torch.arange(S).view(S, 1) * 1000 + torch.arange(C).view(1, C)).float()
        qc, kc = heads * hd, kv * hd
        qcp, kcp = qc // P, kc // P
        Cp = qcp + 2 * kcp
        mine = full[rank * rows:(rank + 1) * rows]
        # what o1_sp_block_pre writes: slab d = my rows x (q heads of d | k heads of d | v heads of d)
        send = torch.stack([torch.cat([mine[:, d * qcp:(d + 1) * qcp],
                                       mine[:, qc + d * kcp:qc + (d + 1) * kcp],
                                       mine[:, qc + kc + d * kcp:qc + kc + (d + 1) * kcp]], 1) for d in range(P)])
        gath = torch.empty(P, rows, Cp)
        got = torch.stack(_a2a(send, gath)).view(S, Cp)
        want = torch.cat([full[:, rank * qcp:(rank + 1) * qcp], full[:, qc + rank * kcp:qc + (rank + 1) * kcp],
                          full[:, qc + kc + rank * kcp:qc + kc + (rank + 1) * kcp]], 1)
        ok1 = torch.equal(got, want)                     # all rows, my heads, in sequence order
        # second exchange: attn [S, Hc] row blocks -> recv slabs = my rows of every head group
        attn = full[:, rank * qcp:(rank + 1) * qcp].contiguous()
        recv = torch.stack(_a2a(attn.view(P, rows, qcp), torch.empty(P, rows, qcp)))
        back = torch.cat([recv[s] for s in range(P)], 1)                  # K blocks of o_proj's A operand
        ok2 = torch.equal(back, mine[:, :qc])
        # layout and sharding agree across ranks
        lay, spn = sp.layout(world, cfg=False)
        (r0, r1), (t0, t1), (i0, i1) = sp.shard_rows(S, 5, P, rank)
        ok3 = lay[rank] == (0, None, rank) and spn == world and (r1 - r0) == rows and (t1 - t0) + (i1 - i0) == rows
        q.put((rank, ok1 and ok2 and ok3, ""))
        dist.destroy_process_group()
    except Exception as e:      # noqa: BLE001
        q.put((rank, False, repr(e)))


def _worker_cfg_pair(rank, world, port, q):
    try:
        sp = _load()
        _init(rank, world, port)
        lay, spn = sp.layout(world, cfg=True)
        image, branch, spr = lay[rank]
        peers = [r for r, v in lay.items() if v[0] == image and v[2] == spr]      # the two CFG branches
        grp = None
        for key in sorted({(v[0], v[2]) for v in lay.values()}):
            members = [r for r, v in lay.items() if (v[0], v[2]) == key]
            g = dist.new_group(members)
            if rank in members:
                grp = g
        mine = torch.full((4, 3), float(branch))
        both = [torch.empty(4, 3) for _ in peers]
        dist.all_gather(both, mine, group=grp)
        ok = len(peers) == 2 and both[0].eq(0).all() and both[1].eq(1).all() and spn == max(1, world // 2)
        # both ranks now hold cond and uncond: the scheduler update is the same pure function on each
        z = torch.arange(12.).view(4, 3)
        zn = z + (0.8 - 0.9) * ((1 - 5.0) * (z - both[1]) / 0.9 + 5.0 * (z - both[0]) / 0.9)
        gathered = [torch.empty_like(zn) for _ in range(world)]
        dist.all_gather(gathered, zn)
        ok = ok and all(torch.equal(gathered[0], t) for t in gathered if t is not None)
        q.put((rank, bool(ok), ""))
        dist.destroy_process_group()
    except Exception as e:      # noqa: BLE001
        q.put((rank, False, repr(e)))


def _worker_missing_peer(rank, world, port, q):
    """Rank 1 joins the group and then leaves between steps without entering the collective: rank 0's
    all-reduce must end with an error inside the short process-group timeout."""
    try:
        _init(rank, world, port, timeout_s=5)
        dist.barrier()
        if rank == 1:
            q.put((rank, True, "left"))
            return
        try:
            dist.all_reduce(torch.ones(4))
            q.put((rank, False, "collective returned although the peer never arrived"))
        except Exception as e:      # noqa: BLE001
            q.put((rank, True, type(e).__name__))
    except Exception as e:      # noqa: BLE001
        q.put((rank, False, repr(e)))


def _run(worker, world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.kill()
    for rank, ok, msg in res:
        assert ok, f"rank {rank}: {msg}"


@pytest.mark.parametrize("world", [2, 4])
def test_ulysses_exchange_slabs(world):
    _run(_worker_ulysses, world)


@pytest.mark.parametrize("world", [2, 4])
def test_cfg_pair_gather_and_identical_update(world):
    _run(_worker_cfg_pair, world)


def test_peer_that_never_arrives_is_detected_on_the_host():
    _run(_worker_missing_peer, 2)


def test_layout_table():
    import sys
    sys.path.insert(0, ROOT)
    sp = _load()
    lay, p = sp.layout(8)
    assert p == 4 and lay[0] == (0, 0, 0) and lay[3] == (0, 0, 3) and lay[4] == (0, 1, 0) and lay[7] == (0, 1, 3)
    lay, p = sp.layout(2)
    assert p == 1 and lay == {0: (0, 0, 0), 1: (0, 1, 0)}
    lay, p = sp.layout(1)
    assert p == 1 and lay == {0: (0, None, 0)}
    lay, p = sp.layout(4)
    assert p == 2 and lay[1] == (0, 0, 1) and lay[2] == (0, 1, 0)
    lay, p = sp.layout(16)
    assert p == 8 and lay[15] == (0, 1, 7)
    # the library's environment knobs (a C host reads the same function: o1_parallel_layout)
    import ctypes as C
    import os
    lib = sp.lib

    def c_layout(world, rank):
        a, b, c, d = C.c_int(), C.c_int(), C.c_int(), C.c_int()
        n = lib.o1_parallel_layout(world, rank, C.byref(a), C.byref(b), C.byref(c), C.byref(d))
        return n, a.value, b.value, c.value, d.value
    try:
        os.environ["O1_SP_DEGREE"] = "2"
        assert c_layout(8, 5) == (2, 1, 0, 1, 2)            # two images in flight: pair x SP2 each
        os.environ["O1_CFG_SPLIT"] = "0"
        assert c_layout(8, 5) == (4, 2, -1, 1, 2)           # both branches on every GPU, SP2, four images
        os.environ["O1_SP_DEGREE"] = "3"
        assert c_layout(8, 0)[0] == -1                      # does not divide the KV heads
        del os.environ["O1_SP_DEGREE"]
        os.environ["O1_GPUS"] = "2"
        assert c_layout(8, 1) == (1, 0, -1, 1, 2) and c_layout(8, 2)[0] == -1
    finally:
        for k in ("O1_SP_DEGREE", "O1_CFG_SPLIT", "O1_GPUS"):
            os.environ.pop(k, None)
    assert c_layout(1, 0) == (1, 0, -1, 0, 1)
    assert sp.shard_rows(16640, 256, 8, 0) == ((0, 2080), (0, 256), (0, 1824))
    assert sp.shard_rows(16640, 256, 8, 7) == ((14560, 16640), (256, 256), (14304, 16384))
    with pytest.raises(ValueError):
        sp.shard_rows(127, 24, 2, 0)
