#!/usr/bin/env python
"""Benchmark of the HiDream-O1 denoising hot path on B200.

Metric: seconds per image for 28-step CFG text-to-image at 16384 image tokens
(+256 text tokens, 36 decoder blocks).  A "step" here is one denoise step: cond forward, uncond
forward, fused CFG + flow-match scheduler update.  sec/image = 28 x mean step time.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c0|c1|c2|c3|c4|vision|vision64|elementwise|block]
                  [--exchange direct|nccl]

Prints ONE JSON line (rank 0): value = s/image from CUDA-event step times with the latent resident on the
device (max over ranks); e2e = the same through pinned host latents (H2D + D2H inside the timed region);
kernels = per tensor-core kernel family launches / total ms / TFLOP/s from events the library records
around its own launches; roofline = the family with the largest event time against the measured cuBLAS
bf16 peak; cpu_baseline = the C/OpenMP oracle timed on one decoder block and extrapolated by FLOPs.
"""
import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

WORKLOADS = {
    # name: (text tokens, grid_h, grid_w)
    "c2": (256, 128, 128),   # the 2048 x 2048 image of the headline metric: 16384 image tokens
    "c1": (256, 64, 64),     # 4096 image tokens
    "c0": (256, 32, 32),     # 1024 image tokens
    "c3": (512, 128, 128),   # multi-reference edit: + 4 reference images of 64x64 tokens
    "c4": (256, 64, 64),     # c1 geometry after a rank-64 LoRA merge, one image per GPU (data parallel)
}
C3_REFS = [(4096, 64, 64, 8, 8)] * 4     # (tokens, grid_h, grid_w, cond_h, cond_w) per reference
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu capture summarised in
# profiles/traffic_S16640.md (same kernels, same shapes, 2 decoder blocks instead of 36)
NCU_TRAFFIC_BYTES = {("c2", "flash_attn"): 306400000, ("c2", "gemm_swiglu"): 1558000000,
                     ("c2", "gemm_resid"): 2950000000}
STEPS_PER_IMAGE = 28
GUIDANCE = 5.0


METRICS = {
    # BASELINE's names: its 1024^2 / 2048^2 images are the 64x64 / 128x128 token grids
    "c2": "sec/image 2048^2 28-step CFG T2I",
    "c1": "sec/image 1024^2 28-step CFG T2I",
    "c0": "sec/image 28-step CFG T2I at 1024 image tokens",
    "c3": "sec/image 2048^2 28-step CFG multi-reference edit (4 references)",
    "c4": "sec/image 1024^2 28-step CFG T2I, LoRA-merged weights",
}


def metric_name(workload):
    """The headline metric is quoted on c2; the other workloads carry their own name."""
    return METRICS[workload]


def workload_desc(workload, layers):
    """One string for both arms, so that their lines can be matched mechanically."""
    T, gh, gw = WORKLOADS[workload]
    I = gh * gw + (sum(r[0] for r in C3_REFS) if workload == "c3" else 0)
    return (f"{workload}: {I} image tokens ({gh}x{gw}" + (" target + 4 references of 64x64" if workload == "c3" else "")
            + f") + {T} text tokens, {layers} decoder blocks, CFG (2 forwards/step), guidance {GUIDANCE}, "
            "flow-match Euler, Dev sigmas")


def flops_block(S, ar):
    gemm = 385875968.0 * S
    keys = 0.5 * ar * (ar + 1.0) + (S - ar) * float(S)
    return gemm + 4.0 * 32 * 128 * keys


def flops_forward(T, I, layers):
    S = T + I
    return layers * flops_block(S, T - 1) + 2.0 * I * (3072 * 1024 + 1024 * 4096) + 2.0 * S * 4096 * 3072


class ClockSampler:
    """nvidia-smi sampled every 200 ms while the timed region runs (read-only queries)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], 0, set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["bf16_tflops"], d["bf16_tflops_sustained"], d["hbm_gbs"], "measured"
    return 1590.0, 1400.0, 6650.0, "fallback"


# --------------------------------------------------------------------------------------- ours
def run_ours(args):
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package

    rank, world, local = dist_env()
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pkg = load_package()
    pkg.use_torch_stream()
    lib = pkg.lib

    T, gh, gw = WORKLOADS[args.workload]
    I_tgt = gh * gw
    is_ref, is_lora = args.workload == "c3", args.workload == "c4"
    I = I_tgt + (sum(r[0] for r in C3_REFS) if is_ref else 0)      # rows that go through x_embedder
    S = T + I
    layers = args.layers
    w = pkg.Weights(n_layers=layers, seed=1234, weight_set="A", device=dev)
    g = torch.Generator().manual_seed(7 + (rank if is_lora else 0))
    ids_c = torch.randint(0, 151000, (T,), generator=g, dtype=torch.int64)
    ids_u = torch.randint(0, 151000, (T,), generator=g, dtype=torch.int64)
    ids_c[-1] = ids_u[-1] = pkg.TMS_ID
    if is_ref:
        # template with one <|vision_start|> + cond_h*cond_w <|image_pad|> run per reference, then boi + tms
        for ids in (ids_c, ids_u):
            o = 8
            for (_, _, _, ch, cw) in C3_REFS:
                ids[o] = 151652
                ids[o + 1:o + 1 + ch * cw] = 151655
                o += 1 + ch * cw + 3
            ids[-2] = 151669
        _, pos, ar = pkg.seq_ref(ids_c.tolist(), C3_REFS, gh, gw)
    else:
        pos, ar = pkg.seq_t2i(T, gh, gw)
    eng = pkg.Engine(w, T, I, ar_len=ar)
    posd = pos.to(dev)
    ids_c, ids_u = ids_c.to(dev), ids_u.to(dev)
    lora_ms = None
    if is_lora:
        lora_ms = merge_synthetic_lora(pkg, w, layers, dev)
    # seeded N(0, 8^2) latent, the scale of the reference's initial noise (generate.c:1266)
    z = torch.empty(I, 3072, dtype=torch.bfloat16, device=dev)
    assert lib.o1_fill_normal_bf16(pkg.ptr(z), z.numel(), 42 + 1 + (rank if is_lora else 0), 0.0, 8.0) == 0
    if is_ref:
        z[I_tgt:].mul_(0.125)               # reference pixel rows ~ N(0,1); the target latent stays ~ N(0,64)
    z_initial = z                              # all image rows (the sharded layouts below keep their own slice)
    z_next = z.clone() if is_ref else torch.empty_like(z)
    z_host = z.cpu().pin_memory()
    z_next_host = torch.empty_like(z_host).pin_memory()
    z_stage = torch.empty_like(z)
    sig = pkg.dev_sigmas()

    # parallel layout (o1c_b200.sp.layout): 2 GPUs = CFG pair; 4 / 8 GPUs = CFG pair x Ulysses SP 2 / 4 on ONE
    # image.  Rank pairs with equal sp_rank all-gather their predictions and apply the same scheduler kernel.
    from o1c_b200 import sp as spmod
    if is_lora:
        lay, sp_size = {r: (r, None, 0) for r in range(world)}, 1       # one image per GPU, no communication
    else:
        lay, sp_size = spmod.layout(world, cfg=True)
    image_id, branch, sp_rank = lay[rank]
    pair = world >= 2 and not is_lora
    cfg_group = sp_group = None
    if pair:
        for key in sorted({(v[0], v[2]) for v in lay.values()}):
            members = sorted(r for r, v in lay.items() if (v[0], v[2]) == key)
            grp = dist.new_group(members)
            if rank in members:
                cfg_group = grp
        for key in sorted({(v[0], v[1]) for v in lay.values()}):
            members = sorted(r for r, v in lay.items() if (v[0], v[1]) == key)
            grp = dist.new_group(members)
            if rank in members:
                sp_group = grp
    n_images = len({v[0] for v in lay.values()})
    if sp_size > 1:
        del eng
        torch.cuda.empty_cache()
        eng = None
        if args.exchange == "direct":
            # exchanges done by the producing kernels' epilogues (peer stores) + flag barriers
            eng = spmod.EngineSP(w, T, I, sp_size, sp_rank, ar_len=ar, direct=True)
            if not spmod.connect_direct(eng, sp_group):
                # peer memory cannot be mapped here (no CUDA IPC between these processes): same kernels, NCCL
                # all-to-all between the stages instead of peer stores
                eng.close()
                eng = None
                args.exchange = "nccl (peer mapping unavailable)"
        if eng is None:
            eng = spmod.EngineSP(w, T, I, sp_size, sp_rank, spmod.nccl_exchange(sp_group), ar_len=ar)
        i0, i1, n_text_local = eng.i0, eng.i1, eng.t1 - eng.t0
        z, z_next = z[i0:i1].contiguous(), z_next[i0:i1].contiguous()
        z_host = z.cpu().pin_memory()
        z_next_host = torch.empty_like(z_host).pin_memory()
        z_stage = torch.empty_like(z)
        xp_local = torch.empty(eng.rows, 3072, dtype=torch.bfloat16, device=dev)
        xp_pair = torch.empty(2, i1 - i0, 3072, dtype=torch.bfloat16, device=dev)
        n_step_local = max(0, min(I_tgt, i1) - i0)      # local image rows that are target (stepped) rows
        # whole step in one library call per rank (o1_denoise_step_cfg_sp): C-driven forward, predictions exchanged
        # with the CFG partner by peer copies + a two-rank flag barrier instead of an NCCL all-gather
        pair_link = None
        if eng.direct and eng.peers is not None and not args.py_driver:
            eng.c_driver = True
            link = spmod.CfgPairLink(eng, branch, cfg_group)
            if link.ok:
                pair_link = link
            else:
                link.close()
    else:
        pair_link = None
    xp_both = torch.empty(2, S, 3072, dtype=torch.bfloat16, device=dev) if (pair and sp_size == 1) else None

    def step_device(i, zin, zout):
        s0, s1 = sig[i % STEPS_PER_IMAGE], sig[i % STEPS_PER_IMAGE + 1]
        if is_ref and not pair:
            eng.denoise_step_cfg_ref(ids_c, ids_u, posd, zin, I_tgt, s0, s1, GUIDANCE, zout)
            return
        if not pair:
            eng.denoise_step_cfg(ids_c, ids_u, posd, zin, s0, s1, GUIDANCE, zout)
            return
        ids_b = ids_u if branch else ids_c
        if sp_size == 1:
            mine = xp_both[branch]
            eng.forward(ids_b, posd, zin, 1.0 - s0, out=mine)
            dist.all_gather_into_tensor(xp_both.view(-1), mine.view(-1), group=cfg_group)
            # reference rows (c3) are static: only the target rows are stepped
            rc = lib.o1_sched_cfg_flow_step(pkg.ptr(zin), pkg.ptr(xp_both[0, T:]), pkg.ptr(xp_both[1, T:]), s0, s1,
                                            GUIDANCE, pkg.ptr(zout), I_tgt * 3072)
        elif pair_link is not None:
            c = eng.ctx()
            c.epoch = max(c.epoch, eng.epoch)
            eng.timestep.fill_(1.0 - s0)
            rc = lib.o1_denoise_step_cfg_sp(C.byref(w.binding), C.byref(c), C.byref(pair_link.pair), pkg.ptr(ids_b),
                                            pkg.ptr(posd), pkg.ptr(zin) if zin.numel() else None, n_step_local,
                                            pkg.ptr(eng.timestep), s0, s1, GUIDANCE, pkg.TMS_ID, pkg.ptr(xp_local),
                                            pkg.ptr(zout) if zout.numel() else None)
            eng.epoch = c.epoch
            if rc != 0:
                raise RuntimeError("o1_denoise_step_cfg_sp: " + pkg.last_error())
        else:
            eng.forward(ids_b, posd, zin if zin.numel() else None, 1.0 - s0, out_local=xp_local)
            mine = xp_local[n_text_local:]
            dist.all_gather_into_tensor(xp_pair.view(-1), mine.reshape(-1), group=cfg_group)
            rc = lib.o1_sched_cfg_flow_step(pkg.ptr(zin), pkg.ptr(xp_pair[0]), pkg.ptr(xp_pair[1]), s0, s1,
                                            GUIDANCE, pkg.ptr(zout), n_step_local * 3072) if n_step_local else 0
        assert rc == 0

    def step_host(i):
        s0, s1 = sig[i % STEPS_PER_IMAGE], sig[i % STEPS_PER_IMAGE + 1]
        if not pair and not is_ref:
            eng.denoise_step_cfg_host(ids_c, ids_u, posd, z_host, z_stage, s0, s1, GUIDANCE, z_next, z_next_host)
            return
        z_stage.copy_(z_host, non_blocking=True)
        step_device(i, z_stage, z_next)
        z_next_host.copy_(z_next, non_blocking=True)
        torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up (>= 3), then exactly K timed steps between barriers
    warm = args.warmup if args.short else max(3, args.warmup)
    cur, nxt = z, z_next
    for i in range(warm):
        step_device(i, cur, nxt)
        cur, nxt = nxt, cur
    torch.cuda.synchronize()
    assert lib.o1_device_error() == 0, "kernel reported a bounded-wait timeout"
    barrier()
    sampler = ClockSampler(local if "CUDA_VISIBLE_DEVICES" not in os.environ else
                           int(os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local]))
    if rank == 0:
        sampler.start()
    lib.o1_launch_count(1)
    lib.o1_profile_enable(1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step_device(i, cur, nxt)
        cur, nxt = nxt, cur
    e1.record()
    barrier()
    lib.o1_profile_enable(0)
    launches = lib.o1_launch_count(0)
    ms_total = e0.elapsed_time(e1)
    t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    assert lib.o1_device_error() == 0, "kernel reported a bounded-wait timeout"
    assert bool(torch.isfinite(cur.float()).all()), "latent went non-finite"

    # per-kernel event times of this rank inside the timed region
    kinds = {}
    for kind, name in ((0, "gemm_store"), (1, "gemm_bias"), (2, "gemm_resid"), (3, "gemm_swiglu"), (5, "flash_attn")):
        ms, n, wk = C.c_double(), C.c_int64(), C.c_double()
        lib.o1_profile_summary(kind, C.byref(ms), C.byref(n), C.byref(wk))
        if n.value:
            kinds[name] = {"launches": n.value, "ms_total": round(ms.value, 3),
                           "tflops": round(wk.value / ms.value / 1e9, 1)}

    # ---- end to end through host buffers (H2D of the latent + D2H of the result inside the timed region)
    e2e_steps = 0 if args.short else args.steps            # the same number of steps as the device-timed region
    e2e_ms = float("nan")
    if e2e_steps:
        step_host(0)
        barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            step_host(i)
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    te = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms = float(te.item())

    # ---- parity of what was just timed (outside every timed region)
    parity_rec = None
    if not args.short and not args.no_parity:
        if sp_size > 1:
            # the sharded forward against the unsharded one on the same inputs, every rank on its own rows
            parity_rec = sharded_vs_unsharded(pkg, dist, dev, eng, w, T, I, ar, posd, ids_u if branch else ids_c,
                                              z_initial, xp_local, world)
        elif rank == 0 and args.workload in ("c1", "c2"):
            # one GPU, or a CFG pair (each rank runs the unsharded forward of one branch): the same kernels
            parity_rec = reference_probe(T, gh, gw, local)
    extras = None
    if world == 1 and args.workload == "c2" and not args.short and not args.no_extras and layers == 36:
        extras = other_workloads(pkg, w, dev)

    images = n_images                                # images in flight (1 unless more GPUs than one image uses)
    sec_per_image = ms_step * STEPS_PER_IMAGE / 1e3 / images
    e2e_sec = e2e_ms * STEPS_PER_IMAGE / 1e3 / images

    out = None
    if rank == 0:
        burst, sustained, hbm, src = measured_peaks()
        fl_step = 2 * flops_forward(T, I, layers)
        top = max(kinds.items(), key=lambda kv: kv[1]["ms_total"])
        per_launch_ms = top[1]["ms_total"] / top[1]["launches"]
        achieved = top[1]["tflops"]
        out = {
            "metric": metric_name(args.workload), "value": round(sec_per_image, 4), "unit": "s/image",
            "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": round(ms_step, 3),
            "higher_is_better": False, "scaling": "strong" if images == 1 else "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_desc(args.workload, layers),
                       "seq_len": S, "layers": layers, "steps_per_image": STEPS_PER_IMAGE,
                       "parallelism": "1 GPU" if world == 1 else
                                      (f"dp{images} (one image per GPU)" if is_lora else f"cfg pair x ulysses sp{sp_size}"
                                       + (f" x dp{images}" if images > 1 else "")),
                       "sp_driver": (None if sp_size == 1 else
                                     ("one o1_denoise_step_cfg_sp call per step (C loop, peer copies of the predictions)"
                                      if pair_link is not None else "stage functions driven from Python, NCCL all-gather of "
                                      "the predictions")),
                       "sp_exchange": (None if sp_size == 1 else
                                       ("peer stores from the GEMM / attention epilogues + flag barriers"
                                        if args.exchange == "direct" else "NCCL all-to-all"
                                        + (" (peer mapping unavailable)" if "unavailable" in args.exchange else ""))),
                       "weights": "random-init N(0,0.02) bf16, seed 1234",
                       "l2": "no flush needed: every step streams 2 x %.1f GB of weights (L2 is 126 MB)"
                             % (w.nbytes() / 1e9)},
            "steps_per_s": round(1e3 / ms_step * images, 4),
            "model_tflops_per_step": round(fl_step / 1e12, 2),
            "achieved_tflops_per_gpu": round(fl_step * images / ms_step / 1e9 / world, 1),
            "e2e": {"value": round(e2e_sec, 4), "unit": "s/image",
                    "h2d_bytes_per_step": (I * 3072 * 2 + 4) * (2 if pair else 1) * images,
                    "d2h_bytes_per_step": I * 3072 * 2 * (2 if pair else 1) * images},
            "gpu_launches": int(launches),
            "clocks": clocks,
            # step time x median SM clock under load: compares runs (and GPU counts) whose power-capped clocks differ
            "ms_per_step_x_sm_mhz": (round(ms_step * clocks["sm_mhz"], 1) if clocks and clocks.get("sm_mhz") else None),
            "parity": parity_rec,
            "roofline": {"bound": "tensor", "kernel": top[0], "achieved": achieved, "peak": sustained,
                         "unit": "TFLOP/s", "frac": round(achieved / sustained, 4),
                         "traffic": NCU_TRAFFIC_BYTES.get((args.workload, top[0])) if world == 1 else None,
                         "peak_source": f"{src} (sustained bf16; burst {burst})",
                         "ms_per_launch": round(per_launch_ms, 4)},
            "kernels": kinds,
        }
        if extras is not None:
            out["configs"] = extras
        if lora_ms is not None:
            out["lora_merge_ms"] = round(lora_ms, 2)
            out["config"]["lora"] = "rank 64, A,B ~ N(0,0.01), alpha 64, merged into the 7 linears of every block"
        if args.short:
            out["short_profiler_run"] = True
            out.pop("e2e")
        if world == 1 and not args.no_cpu_baseline and not args.short:
            out["cpu_baseline"] = cpu_baseline(pkg, fl_step)
    if world > 1:
        dist.destroy_process_group()
    return out


def reference_probe(T, gh, gw, device_index):
    """tests/parity_probe.py as a child process: a 2-block forward at this geometry through the library and
    through the reference's production CUDA build (when oracle/_ref holds it), x_pred compared."""
    cmd = [sys.executable, os.path.join(ROOT, "tests", "parity_probe.py"), "--text", str(T), "--grid-h", str(gh),
           "--grid-w", str(gw), "--layers", "2", "--device", str(device_index)]
    try:
        p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        line = [l for l in p.stdout.splitlines() if l.startswith("{")]
        return json.loads(line[-1]) if line else {"status": "error: no output", "stderr": p.stderr[-300:]}
    except Exception as ex:      # noqa: BLE001
        return {"status": f"error: {type(ex).__name__}: {ex}"}


def sharded_vs_unsharded(pkg, dist, dev, eng_sp, w, T, I, ar, posd, ids, z_full, xp_local, world):
    """x_pred of the sequence-parallel forward against the single-GPU forward of the same branch on the same
    (initial) latent: every rank runs the unsharded forward itself (it holds all weights) and compares its own
    rows; the squared sums are reduced over all ranks, i.e. over both branches and all row shards."""
    import torch
    t = 0.5
    z_local = z_full[eng_sp.i0:eng_sp.i1].contiguous()
    eng_sp.forward(ids, posd, z_local if z_local.numel() else None, t, out_local=xp_local)
    torch.cuda.synchronize()
    eng1 = pkg.Engine(w, T, I, ar_len=ar)
    full = eng1.forward(ids, posd, z_full, t)
    torch.cuda.synchronize()
    mine = xp_local.double()
    want = full[eng_sp.row0:eng_sp.row0 + eng_sp.rows].double()
    acc = torch.stack([((mine - want) ** 2).sum(), (want ** 2).sum(), (mine * want).sum(), (mine ** 2).sum(),
                       (~torch.isfinite(mine)).sum().double()])
    dist.all_reduce(acc)
    d2, r2, gr, g2, bad = (float(v) for v in acc)
    nrmse = (d2 / r2) ** 0.5 if r2 > 0 else 0.0
    cos = gr / ((g2 * r2) ** 0.5) if g2 > 0 and r2 > 0 else 0.0
    del eng1
    return {"against": "the unsharded forward of this library on the same inputs (all ranks, both branches)",
            "x_pred": {"nrmse": round(nrmse, 6), "cos": round(cos, 7), "nonfinite": int(bad)},
            "status": "pass" if (nrmse <= 2e-2 and cos >= 0.995 and bad == 0) else "FAIL"}


def other_workloads(pkg, w, dev):
    """Short live measurements of the other BASELINE workloads on this GPU with the weights already resident
    (3 timed steps after 2 warm-ups each, CUDA events); c4 runs last because the merge rewrites the weights."""
    import torch
    lib = pkg.lib
    res = {}
    sig = pkg.dev_sigmas()

    def time_steps(fn, warm=2, n=3):
        for i in range(warm):
            fn(i)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(n):
            fn(i)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    def t2i(workload, seed_off):
        T, gh, gw = WORKLOADS[workload]
        I = gh * gw
        pos, ar = pkg.seq_t2i(T, gh, gw)
        eng = pkg.Engine(w, T, I, ar_len=ar)
        g = torch.Generator().manual_seed(7)
        ic = torch.randint(0, 151000, (T,), generator=g, dtype=torch.int64)
        iu = torch.randint(0, 151000, (T,), generator=g, dtype=torch.int64)
        ic[-1] = iu[-1] = pkg.TMS_ID
        ic, iu, posd = ic.to(dev), iu.to(dev), pos.to(dev)
        z = torch.empty(I, 3072, dtype=torch.bfloat16, device=dev)
        lib.o1_fill_normal_bf16(pkg.ptr(z), z.numel(), 43 + seed_off, 0.0, 8.0)
        zn = torch.empty_like(z)
        ms = time_steps(lambda i: eng.denoise_step_cfg(ic, iu, posd, z, sig[i], sig[i + 1], GUIDANCE, zn))
        assert bool(torch.isfinite(zn.float()).all())
        return ms, 2 * flops_forward(T, I, w.n_layers)

    try:
        ms, fl = t2i("c1", 0)
        res["c1"] = {"metric": metric_name("c1"), "value": round(ms * STEPS_PER_IMAGE / 1e3, 4), "unit": "s/image",
                     "ms_per_step": round(ms, 3), "tflops": round(fl / ms / 1e9, 1),
                     "parity": "tests/test_gpu_scale_parity.py: 36-block forward and 28-step chain at these rows "
                               "against the reference CUDA build"}
        # c0: one decoder block at 256 + 1024 tokens
        T, gh, gw = WORKLOADS["c0"]
        eng = pkg.Engine(w, T, gh * gw)
        pos, ar = pkg.seq_t2i(T, gh, gw)
        x = torch.empty(eng.S, pkg.HIDDEN, dtype=torch.bfloat16, device=dev)
        lib.o1_fill_normal_bf16(pkg.ptr(x), x.numel(), 42, 0.0, 1.0)
        posd = pos.to(dev)
        ms = time_steps(lambda i: eng.block(x, posd, 0), warm=3, n=10)
        res["c0"] = {"metric": "ms per decoder block (256 text + 1024 image tokens)", "value": round(ms, 4), "unit": "ms",
                     "tflops": round(flops_block(eng.S, ar) / ms / 1e9, 1), "l2": "not flushed (back-to-back launches)",
                     "parity": "tests/test_gpu_block.py: this shape against the oracle and the reference CUDA build"}
        del eng
        # c3: K = 4 references, S = 33280
        T, gh, gw = WORKLOADS["c3"]
        I_tgt = gh * gw
        I = I_tgt + sum(r[0] for r in C3_REFS)
        g = torch.Generator().manual_seed(7)
        ic = torch.randint(0, 151000, (T,), generator=g, dtype=torch.int64)
        iu = torch.randint(0, 151000, (T,), generator=g, dtype=torch.int64)
        ic[-1] = iu[-1] = pkg.TMS_ID
        for ids in (ic, iu):
            o = 8
            for (_, _, _, ch, cw) in C3_REFS:
                ids[o] = 151652
                ids[o + 1:o + 1 + ch * cw] = 151655
                o += 1 + ch * cw + 3
            ids[-2] = 151669
        _, pos, ar = pkg.seq_ref(ic.tolist(), C3_REFS, gh, gw)
        eng = pkg.Engine(w, T, I, ar_len=ar)
        ic, iu, posd = ic.to(dev), iu.to(dev), pos.to(dev)
        z = torch.empty(I, 3072, dtype=torch.bfloat16, device=dev)
        lib.o1_fill_normal_bf16(pkg.ptr(z), z.numel(), 43, 0.0, 8.0)
        z[I_tgt:].mul_(0.125)
        zn = z.clone()
        ms = time_steps(lambda i: eng.denoise_step_cfg_ref(ic, iu, posd, z, I_tgt, sig[i], sig[i + 1], GUIDANCE, zn),
                        warm=1, n=2)
        res["c3"] = {"metric": metric_name("c3"), "value": round(ms * STEPS_PER_IMAGE / 1e3, 3), "unit": "s/image",
                     "ms_per_step": round(ms, 2), "tflops": round(2 * flops_forward(T, I, w.n_layers) / ms / 1e9, 1),
                     "seq_len": T + I,
                     "parity": "tests/test_gpu_forward.py: the K = 4 layout with visual conditioning against the oracle at "
                               "small size; the reference build cannot run this size (its S x S score buffers need 142 GB)"}
        del eng, z, zn
        torch.cuda.empty_cache()
        # c4: rank-64 LoRA merged into every block linear, then the c1 shapes
        merge_ms = merge_synthetic_lora(pkg, w, w.n_layers, dev)
        ms, fl = t2i("c4", 1)
        res["c4"] = {"metric": metric_name("c4"), "value": round(ms * STEPS_PER_IMAGE / 1e3, 4), "unit": "s/image",
                     "ms_per_step": round(ms, 3), "lora_merge_ms": round(merge_ms, 2), "images_per_gpu": 1,
                     "parity": "tests/test_gpu_lora.py: merge against the reference's Python contract fixture; "
                               "forward kernels as c1"}
    except Exception as ex:      # noqa: BLE001 -- the headline line must survive a failure here
        res["error"] = f"{type(ex).__name__}: {ex}"
    return res


def merge_synthetic_lora(pkg, w, layers, dev):
    """Workload c4: rank-64 adapters (A, B ~ N(0, 0.01), alpha = 64, multiplier 1) merged at load into
    every linear of every block through hd_lora_merge_gpu.  Returns the merge time in ms (CUDA events)."""
    import torch
    targets = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]
    R = 64
    ents = (pkg.LoraEntry * (layers * len(targets)))()
    keep = []
    k = 0
    for l in range(layers):
        for name in targets:
            N, K = pkg.tensor_shape(name)
            up = torch.empty(N, R, device=dev)
            down = torch.empty(R, K, device=dev)
            pkg.lib.o1_fill_normal_f32(pkg.ptr(up), up.numel(), 5000 + k * 2, 0.0, 0.01)
            pkg.lib.o1_fill_normal_f32(pkg.ptr(down), down.numel(), 5001 + k * 2, 0.0, 0.01)
            keep += [up, down]
            e = ents[k]
            e.rank, e.in_dim, e.out_dim, e.alpha, e.multiplier = R, K, N, 64.0, 1.0
            e.up_dev, e.down_dev, e.base_dev = up.data_ptr(), down.data_ptr(), w.addr(l, name)
            k += 1
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    rc = pkg.lib.hd_lora_merge_gpu(ents, len(ents), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    e1.record()
    torch.cuda.synchronize()
    assert rc == 0, pkg.last_error()
    return e0.elapsed_time(e1)


def cpu_baseline(pkg, flops_step, S_sample=(256, 32, 32)):
    """The C/OpenMP oracle timed on the host cores on one decoder block at 1280 tokens, extrapolated to
    the step by algorithmic FLOPs (the block is >99.9% of a forward)."""
    import numpy as np
    import parity
    T, gh, gw = S_sample
    S = T + gh * gw
    hw = parity.HostWeights(pkg, 1, 1234, "A")
    pos, ar = pkg.seq_t2i(T, gh, gw)
    x = parity.seeded_bf16((S, pkg.HIDDEN), 42)
    hw.block_struct(0)                       # generate weights outside the timed region
    t0 = time.perf_counter()
    parity.oracle_block(hw, 0, x, pos.numpy(), ar, want_ints=False)
    dt = time.perf_counter() - t0
    fl = flops_block(S, ar)
    sec_image = dt * (flops_step * STEPS_PER_IMAGE / fl)
    return {"value": round(sec_image, 1), "unit": "s/image", "cores": parity.oracle().orc_num_threads(),
            "kind": "port",
            "sample": f"1 decoder block at S={S} ({dt:.2f} s, {fl / dt / 1e9:.0f} GFLOP/s), "
                      f"extrapolated by algorithmic FLOPs to 28 CFG steps of the benchmark workload"}


# --------------------------------------------------------------------------------- reference
def run_reference(args):
    """The reference's own build of this path: its CUDA sources (cuBLASLt GEMMs + cuDNN SDPA) compiled
    unchanged into oracle/_ref/libo1ref.so, driven through hd_forward x2 -> hd_sched_vcond x2 ->
    hd_sched_cfg_guided -> hd_sched_flow_match_step (the composition of src/runtime/generate.c).
    The reference has no CPU implementation of this path; if its library is unavailable or fails,
    the C/OpenMP port is timed on the host cores instead.

    This arm never loads the product library: weights are generated on the host by the oracle's generator
    (bit-identical to the device-side fill of the other arm) and copied to the device, positions and sigmas
    come from the oracle, and the step is driven through tests/refharness.py."""
    rank, world, local = dist_env()
    if rank != 0:
        return None
    import torch
    import parity
    import refharness as rh
    if args.workload not in ("c0", "c1", "c2"):
        return {"impl": "reference", "unavailable": "the reference build cannot run this workload: its S x S score "
                                                    "buffers exceed the GPU's memory (c3) / it has no LoRA GPU merge that "
                                                    "is safe to run (c4: lora_merge.cu:86-93 reads beyond the adapter)"}
    T, gh, gw = WORKLOADS[args.workload]
    I, S, layers = gh * gw, T + gh * gw, args.layers
    fl_step = 2 * flops_forward(T, I, layers)
    base = {"metric": metric_name(args.workload), "unit": "s/image", "n_gpus": world, "steps": args.steps,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "impl": "reference"}
    err = None
    if parity.reflib() is not None and torch.cuda.is_available():
        try:
            torch.cuda.set_device(local)
            dev = torch.device("cuda", local)
            t0 = time.perf_counter()
            w = rh.HostFilledWeights(layers, dev, seed=1234, weight_set="A")
            fill_s = time.perf_counter() - t0
            reng = rh.RefEngine(w.binding, T, gh, gw, dev, production=True)
            ids_c, ids_u = (t.to(dev) for t in rh.seeded_ids(T, 7))
            z_host = rh.seeded_latent(I, 43, 8.0).pin_memory()
            z = z_host.to(dev)
            zn = torch.empty_like(z)
            z_stage = torch.empty_like(z)
            zn_host = torch.empty_like(z_host).pin_memory()
            sig = rh.dev_sigmas()

            def step(i, zin, zout):
                reng.cfg_step(ids_c, ids_u, zin, zout, sig[i % 28], sig[i % 28 + 1], GUIDANCE)

            # The reference's GEMM runtime picks its cuBLASLt algorithm per shape by timing candidates over its first
            # calls (src/cuda/gemm.cu:413-461): with 3 untimed steps the timed region still holds part of that search
            # (measured 939 ms/step against 795 once it has settled), so this arm always gets at least 8.
            warm = max(8, args.warmup)
            cur, nxt = z, zn
            for i in range(warm):
                step(i, cur, nxt)
                cur, nxt = nxt, cur
            torch.cuda.synchronize()
            sampler = ClockSampler(local if "CUDA_VISIBLE_DEVICES" not in os.environ else
                                   int(os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local]))
            sampler.start()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(args.steps):
                step(i, cur, nxt)
                cur, nxt = nxt, cur
            e1.record()
            torch.cuda.synchronize()
            clocks = sampler.stop()
            ms_step = e0.elapsed_time(e1) / args.steps
            assert bool(torch.isfinite(cur.float()).all()), "latent went non-finite"
            # end to end: the step's latent comes from pinned host memory and the result goes back, every step
            t0 = time.perf_counter()
            for i in range(args.steps):
                z_stage.copy_(z_host, non_blocking=True)
                step(i, z_stage, zn)
                zn_host.copy_(zn, non_blocking=True)
                torch.cuda.synchronize()
            e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
            reng.close()
            val = ms_step * STEPS_PER_IMAGE / 1e3
            base.update({
                "value": round(val, 4), "warmup": warm, "warmup_requested": args.warmup,
                "warmup_note": "at least 8 untimed steps: the reference's cuBLASLt algorithm search (src/cuda/gemm.cu:413-461) "
                               "runs over its first calls per shape and would otherwise fall into the timed region",
                "ms_per_step": round(ms_step, 3),
                "config": {"workload": workload_desc(args.workload, layers), "seq_len": S, "layers": layers,
                           "steps_per_image": STEPS_PER_IMAGE,
                           "backend": "reference CUDA build on this GPU: cuBLASLt GEMM + cuDNN SDPA (two-pass)",
                           "weights": "random-init N(0,0.02) bf16, seed 1234 (generated on the host by the oracle's "
                                      "generator in %.1f s, the same bytes as the other arm's device fill)" % fill_s,
                           "product_library_loaded": "libo1b200" in open("/proc/self/maps").read()},
                "achieved_tflops": round(fl_step / ms_step / 1e9, 1),
                "clocks": clocks,
                "ms_per_step_x_sm_mhz": (round(ms_step * clocks["sm_mhz"], 1) if clocks.get("sm_mhz") else None),
                "cpu_baseline": {"value": round(val, 4), "unit": "s/image", "cores": 0, "kind": "reference",
                                 "sample": "the reference has no CPU implementation of this path; this is its own "
                                           "CUDA build (oracle/_ref) on the same GPU, full workload"},
                "e2e": {"value": round(e2e_ms * STEPS_PER_IMAGE / 1e3, 4), "unit": "s/image",
                        "h2d_bytes_per_step": I * 3072 * 2, "d2h_bytes_per_step": I * 3072 * 2},
            })
            return base
        except Exception as ex:      # noqa: BLE001 -- report and fall through to the CPU port
            err = f"{type(ex).__name__}: {ex}"
    # CPU port of the path on the host cores (the oracle is test infrastructure; this is the one place besides
    # cpu_baseline() where the bench executes it)
    from __graft_entry__ import load_package
    cb = cpu_baseline(load_package(), fl_step)
    base.update({"value": cb["value"], "warmup": 0, "ms_per_step": round(cb["value"] / STEPS_PER_IMAGE * 1e3, 1),
                 "config": {"workload": workload_desc(args.workload, layers),
                            "backend": "C/OpenMP port on host cores" + (f" (reference CUDA build failed: {err})" if err else "")},
                 "cpu_baseline": cb,
                 "e2e": {"value": cb["value"], "unit": "s/image", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    return base


# --------------------------------------------------------------------------------------- vision tower
VISION_GRIDS = {"vision": (26, 20), "vision64": (64, 64)}   # patches: the documented 416 x 320 image; 1024 x 1024


def run_vision(args):
    """Times hd_vision_forward (27-block ViT of the edit modes) on one GPU: plain launches and CUDA-graph replay,
    next to the reference's CUDA build (cuBLASLt hd_linear + its eager attention) when oracle/_ref holds it."""
    import torch
    from __graft_entry__ import load_package
    import parity

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    pkg = load_package()
    pkg.use_torch_stream()
    lib = pkg.lib
    gh, gw = VISION_GRIDS[args.workload]
    n, m = gh * gw, gh * gw // 4
    tensors = []
    for i, (name, shape) in enumerate(parity.vision_tensor_list()):
        t = torch.empty(shape, dtype=torch.bfloat16, device=dev)
        mean = 1.0 if name.endswith(("norm1.weight", "norm2.weight", "norm.weight")) else 0.0
        assert lib.o1_fill_normal_bf16(pkg.ptr(t), t.numel(), 4321 + i, mean, 0.02) == 0
        tensors.append(t)
    binding = pkg.VisionBinding(*[t.data_ptr() for t in tensors])
    px = torch.empty((n, 1536), dtype=torch.bfloat16, device=dev)
    lib.o1_fill_normal_bf16(pkg.ptr(px), px.numel(), 7, 0.0, 1.0)
    emb = torch.empty((m, 4096), dtype=torch.bfloat16, device=dev)
    ds = torch.empty((3, m, 4096), dtype=torch.bfloat16, device=dev)
    dsp = (C.c_void_p * 3)(*[ds[j].data_ptr() for j in range(3)])

    def make_ws(l):
        ws = pkg.VisionWorkspace()
        space = torch.zeros(l.hd_vision_workspace_bytes(n), dtype=torch.uint8, device=dev)
        tables = torch.zeros(l.hd_vision_tables_bytes(n), dtype=torch.uint8, device=dev)
        ws.patch_out, ws.tables, ws.tables_n = space.data_ptr(), tables.data_ptr(), -1
        assert l.hd_vision_prepare_tables(C.byref(ws), n, gh, gw) == 0
        return ws, (space, tables)

    def forward(l, ws):
        rc = l.hd_vision_forward(C.byref(binding), C.byref(ws), C.c_void_p(px.data_ptr()), n, gh, gw,
                                 C.c_void_p(emb.data_ptr()), C.byref(dsp))
        assert rc == 0, l.hd_last_error()

    def timed(fn, reps):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
        torch.cuda.synchronize()
        ev[0].record()
        for i in range(reps):
            fn()
            ev[i + 1].record()
        torch.cuda.synchronize()
        return statistics.median(ev[i].elapsed_time(ev[i + 1]) for i in range(reps))

    ws, keep = make_ws(lib)
    reps = args.steps if args.short else max(args.steps, 10)
    for _ in range(args.warmup if args.short else max(args.warmup, 3)):
        forward(lib, ws)
    lib.o1_launch_count(1)
    forward(lib, ws)
    launches = int(lib.o1_launch_count(1))
    ms_plain = timed(lambda: forward(lib, ws), reps)
    if args.short:      # profiler runs: plain launches only, no graph, no reference arm; not a benchmark value
        return {"metric": "vision tower ms/forward", "value": round(ms_plain, 4), "unit": "ms", "short": True,
                "gpu_launches": launches}
    # the forward neither allocates nor synchronises, so it can be captured once and replayed
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        pkg.use_torch_stream()
        forward(lib, ws)
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            pkg.use_torch_stream()
            forward(lib, ws)
    pkg.use_torch_stream()
    ms_graph = timed(graph.replay, reps)
    assert lib.o1_device_error() == 0
    # algorithmic FLOPs: block GEMMs, attention at head_dim 72, patch embedding, four mergers
    gemm = 2.0 * n * (1152 * 3456 + 1152 * 1152 + 2 * 1152 * 4304) * 27 + 2.0 * n * 1536 * 1152
    attn = 4.0 * 16 * 72 * n * n * 27
    merg = 4 * 2.0 * m * (4608 * 4608 + 4096 * 4608)
    flops = gemm + attn + merg
    out = {"metric": "vision tower ms/forward", "value": round(ms_graph, 4), "unit": "ms", "n_gpus": 1, "steps": reps,
           "warmup": max(args.warmup, 3), "higher_is_better": False, "dtype": "bf16", "data": "synthetic",
           "config": {"workload": f"{args.workload}: Qwen3-VL tower, {gh}x{gw} patches ({n} tokens -> {m} merged), 27 blocks, "
                                  "random-init weights seed 4321", "mode": "CUDA-graph replay of hd_vision_forward"},
           "ms_plain_launches": round(ms_plain, 4), "gpu_launches": launches,
           "model_gflops_per_forward": round(flops / 1e9, 1), "achieved_tflops": round(flops / ms_graph / 1e9, 1)}
    r = parity.reflib()
    if r is not None and hasattr(r, "hd_vision_forward"):
        rt = r.hd_gemm_runtime_init(0, 64 << 20)
        if rt:
            r.hd_gemm_set_backend(1)
            rws, rkeep = make_ws(r)
            for _ in range(3):
                forward(r, rws)
            out["reference_cuda_build_ms"] = round(timed(lambda: forward(r, rws), reps), 4)
            out["reference_backend"] = "cuBLASLt hd_linear + the reference's eager attention (sdpa = NULL)"
            r.hd_gemm_runtime_destroy(rt)
    return out


# --------------------------------------------------------------------------------------- elementwise kernels
def run_elementwise(args):
    """HBM-bound kernels of the path at the c2 shapes (S = 16640), each timed alone with CUDA events against the
    measured copy bandwidth.  Every kernel cycles through four sets of buffers (> 1 GB in total) so that no launch
    finds its operands in the 126 MB L2."""
    import torch
    from __graft_entry__ import load_package

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    pkg = load_package()
    pkg.use_torch_stream()
    lib = pkg.lib
    S, H, NB = 16640, 4096, (1 if args.short else 4)     # profiler runs hold one buffer set (1.3 GB)
    _, _, hbm, src = measured_peaks()
    bf = lambda *shape: [torch.randn(*shape, device=dev, dtype=torch.float32).to(torch.bfloat16) for _ in range(NB)]
    x, y, x2 = bf(S, H), bf(S, H), bf(S, H)
    w = torch.ones(H, dtype=torch.bfloat16, device=dev)
    lb = torch.zeros(H, dtype=torch.bfloat16, device=dev)
    qk = bf(S, 40 * 128)                                       # 32 q heads + 8 k heads of one token row
    w128 = torch.ones(128, dtype=torch.bfloat16, device=dev)
    pos, _ = pkg.seq_t2i(256, 128, 128)
    cs = torch.empty(S, 128, dtype=torch.float32, device=dev)
    assert lib.o1_mrope_table(pkg.ptr(pos.to(dev)), S, 5000000.0, pkg.ptr(cs)) == 0
    n_lat = 16384 * 3072
    z, xc, xu, zn = bf(n_lat), bf(n_lat), bf(n_lat), bf(n_lat)
    g, u, sw = bf(S, 12288 // 4), bf(S, 12288 // 4), bf(S, 12288 // 4)   # a quarter of the SwiGLU width keeps the set at 1.2 GB
    P = pkg.ptr
    cases = [
        ("rmsnorm_vec_kernel [16640,4096]", 2 * S * H * 2 + H * 2,
         lambda i: lib.hd_rmsnorm(P(x[i]), P(w), P(y[i]), S, H, 1e-6)),
        ("qk_norm_rope_kernel 40 heads x 128", 2 * S * 40 * 128 * 2 + S * 512,
         lambda i: lib.o1_qk_norm_rope(P(qk[i]), 40 * 128, S, 40, P(w128), P(cs), 1e-6)),
        ("pointwise residual add [16640,4096]", 3 * S * H * 2,
         lambda i: lib.hd_residual_add(P(x[i]), P(x2[i]), P(y[i]), S * H)),
        ("pointwise SwiGLU [16640,3072]", 3 * S * 3072 * 2,
         lambda i: lib.hd_swiglu(P(g[i]), P(u[i]), P(sw[i]), S * 3072)),
        ("cfg_flow_step_kernel 50.3 M elements", 4 * n_lat * 2,
         lambda i: lib.o1_sched_cfg_flow_step(P(z[i]), P(xc[i]), P(xu[i]), 0.7, 0.65, 5.0, P(zn[i]), n_lat)),
        ("layernorm_reg_kernel<5> [16640,1152] (vision)", 2 * S * 1152 * 2,
         lambda i: lib.hd_vision_layernorm(P(x[i]), P(w), P(lb), P(y[i]), S, 1152, 1e-6)),
    ]
    reps = args.steps if args.short else max(args.steps, 12)
    rows = {}
    for name, nbytes, fn in cases:
        for i in range(args.warmup if args.short else max(args.warmup, 3)):
            fn(i % NB)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
        torch.cuda.synchronize()
        ev[0].record()
        for i in range(reps):
            fn(i % NB)
            ev[i + 1].record()
        torch.cuda.synchronize()
        pkg.check_cuda_errbuf(name)
        us = statistics.median(ev[i].elapsed_time(ev[i + 1]) for i in range(reps)) * 1e3
        rows[name] = {"us": round(us, 2), "algorithmic_MB": round(nbytes / 1e6, 1), "GBps": round(nbytes / us / 1e3, 1),
                      "frac_of_hbm_peak": round(nbytes / us / 1e3 / hbm, 3)}
    top = rows["rmsnorm_vec_kernel [16640,4096]"]
    return {"metric": "elementwise kernels, achieved HBM GB/s", "value": top["GBps"], "unit": "GB/s", "n_gpus": 1,
            "steps": reps, "warmup": max(args.warmup, 3), "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "elementwise: c2 shapes (S = 16640), four rotating buffer sets per kernel (no L2 reuse)"},
            "roofline": {"bound": "hbm", "kernel": "rmsnorm_vec_kernel", "achieved": top["GBps"], "peak": hbm, "unit": "GB/s",
                         "frac": top["frac_of_hbm_peak"], "traffic": None, "peak_source": src + " (STREAM-style copy)"},
            "kernels": rows, "gpu_launches": len(cases) * (reps + max(args.warmup, 3))}


# --------------------------------------------------------------------------------------- one decoder block
def run_block(args):
    """One decoder block at 256 text + 1024 image tokens (hidden 4096, 32 / 8 heads of 128, SwiGLU 12288): this
    library's block, its adaLN-modulated variant, the reference's CUDA build of hd_decoder_block (cuBLASLt + cuDNN
    SDPA) on the same GPU and weights, and the C/OpenMP oracle of the same block on the host cores."""
    import numpy as np
    import torch
    from __graft_entry__ import load_package
    import parity

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    pkg = load_package()
    pkg.use_torch_stream()
    T, gh, gw = WORKLOADS["c0"]
    w = pkg.Weights(n_layers=1, seed=1234, weight_set="A", device=dev)
    eng = pkg.Engine(w, T, gh * gw)
    S, H = eng.S, pkg.HIDDEN
    pos, ar = pkg.seq_t2i(T, gh, gw)
    posd = pos.to(dev)
    x = parity.u16_to_torch(parity.seeded_bf16((S, H), 42), dev)
    mod = parity.u16_to_torch(parity.seeded_bf16(6 * H, 5, 0.0, 0.3), dev)
    fl = flops_block(S, ar)
    reps = args.steps if args.short else max(args.steps, 20)
    warm = args.warmup if args.short else max(args.warmup, 3)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)       # written between runs: 2 x L2

    def timed(fn):
        for _ in range(warm):
            fn()
        ts = []
        for _ in range(reps):
            flush.fill_(1)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return statistics.median(ts)

    pkg.lib.o1_launch_count(1)
    eng.block(x, posd, 0)
    launches = int(pkg.lib.o1_launch_count(1))
    ms = timed(lambda: eng.block(x, posd, 0))
    ms_adaln = timed(lambda: eng.block(x, posd, 0, mod6=mod))
    assert pkg.lib.o1_device_error() == 0
    _, sus, _, src = measured_peaks()
    out = {"metric": "ms per decoder block (256 text + 1024 image tokens)", "value": round(ms, 4), "unit": "ms", "n_gpus": 1,
           "steps": reps, "warmup": warm, "higher_is_better": False, "dtype": "bf16", "data": "synthetic",
           "config": {"workload": "block: one decoder block, 256 text + 1024 image tokens (S = 1280), weights N(0,0.02) seed 1234, "
                                  "activations N(0,1) seed 42", "l2": "256 MB written between timed launches"},
           "block_gflop": round(fl / 1e9, 1), "achieved_tflops": round(fl / ms / 1e9, 1),
           "roofline": {"bound": "tensor", "kernel": "whole block (%d launches)" % launches, "achieved": round(fl / ms / 1e9, 1),
                        "peak": sus, "unit": "TFLOP/s", "frac": round(fl / ms / 1e9 / sus, 4), "traffic": None,
                        "peak_source": src + " (sustained bf16)"},
           "adaln_variant_ms": round(ms_adaln, 4), "gpu_launches": launches}
    if args.short:
        return out
    r = parity.reflib()
    if r is not None:
        sec = torch.tensor([24, 20, 20], dtype=torch.int64, device=dev)
        mask = np.empty((S, S), dtype=np.uint16)
        parity.oracle().orc_prefix_causal_mask(S, ar, parity.np_ptr(mask))
        md = parity.u16_to_torch(mask, dev)
        nbytes = r.hd_decoder_block_scratch_bytes(S, 32, 8, 4096, 12288, 128)
        scratch = torch.empty(nbytes + 256, dtype=torch.uint8, device=dev)
        o2 = torch.empty(S, H, dtype=torch.bfloat16, device=dev)
        bb = w.block_binding(0)
        plan = C.c_void_p()
        rt = r.hd_gemm_runtime_init(0, 64 << 20)
        if rt and r.hd_sdpa_create_prod(C.byref(plan), 1, 32, 8, S, ar, 128, 128 ** -0.5) == 0:
            r.hd_gemm_set_backend(1)

            def ref_block():
                rc = r.hd_decoder_block(pkg.ptr(x), pkg.ptr(posd), pkg.ptr(md), C.byref(bb), pkg.ptr(sec), pkg.ptr(scratch),
                                        nbytes, None, pkg.ptr(o2), S, 32, 8, 4096, 12288, 128, plan)
                assert rc == 0, r.hd_last_error()
            out["reference_cuda_build_ms"] = round(timed(ref_block), 4)
            out["reference_backend"] = "cuBLASLt + cuDNN SDPA (two-pass), hd_decoder_block"
            r.hd_sdpa_destroy(plan)
        if rt:
            r.hd_gemm_runtime_destroy(rt)
    if not args.no_cpu_baseline:
        hw = parity.HostWeights(pkg, 1, 1234, "A")
        xh = parity.seeded_bf16((S, H), 42)
        hw.block_struct(0)
        t0 = time.perf_counter()
        parity.oracle_block(hw, 0, xh, pos.numpy(), ar, want_ints=False)
        dt = time.perf_counter() - t0
        out["cpu_baseline"] = {"value": round(dt * 1e3, 1), "unit": "ms", "cores": parity.oracle().orc_num_threads(),
                               "kind": "port", "sample": "the whole block once, C/OpenMP oracle"}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + sorted(VISION_GRIDS) + ["elementwise", "block"])
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the parity check that follows the timed region")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the short measurements of the other workloads that follow the c2 run on one GPU")
    ap.add_argument("--exchange", choices=("direct", "nccl"), default="direct",
                    help="Ulysses exchanges at 4 / 8 GPUs: stores into the peers' buffers from the producing "
                         "kernels (default) or NCCL all-to-all between the stage kernels")
    ap.add_argument("--py-driver", action="store_true",
                    help="sharded runs: drive the stage functions from Python and all-gather the predictions with NCCL "
                         "instead of one o1_denoise_step_cfg_sp call per step")
    ap.add_argument("--short", action="store_true",
                    help="profiler runs only: take --warmup literally, skip the end-to-end and CPU legs "
                         "(a number from such a run is not a benchmark value)")
    args = ap.parse_args()
    if args.workload == "elementwise":
        out = run_elementwise(args)
    elif args.workload == "block":
        out = run_block(args)
    elif args.workload in VISION_GRIDS:
        out = run_vision(args)     # one GPU, both arms in one line
    else:
        out = run_reference(args) if args.impl == "reference" else run_ours(args)
    if out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
