"""Regenerates the fixtures in this folder.  Needs a checkout of the reference (o1.c; its location comes
from the environment variable O1_REFERENCE) and oracle/_ref/libo1ref.so (make -C oracle ref); neither is
needed to RUN the tests, which only read the files written here.

  scheduler_dump.json : the reference's own scheduler oracle dumps
                        (tests/unit/oracle_dump.txt, oracle_dump_matrix.txt) as JSON
  rng_ref.npz         : outputs of the reference's torch_rng.c (hd_torch_randn_f32,
                        hd_torch_rng_u32), seed 123457, n in {1,8,15,16,17,31,32,1024}
  seq_t2i.npz         : hd_seq_t2i position ids and mask-derived ar_len for three geometries
  seq_ref.npz         : hd_seq_build ids / position ids / ar_len for K = 1 and K = 4 references
  sigmas_ref.json     : hd_scheduler_derive_{dev,flash,flow_match,default} outputs
"""
import ctypes as C
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("O1_REFERENCE", "/root/reference")
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libo1ref.so")


def parse_dump(path):
    recs, cur = [], None
    for line in open(path):
        parts = line.split()
        if not parts or parts[0].startswith("#"):
            continue
        if parts[0] == "RECIPE":
            cur = {"name": parts[1], "steps": int(parts[2]), "shift": float(parts[3]), "sched": parts[4],
                   "tlist": parts[5] == "True"}
            recs.append(cur)
        elif parts[0] in ("SIGMAS", "NOISESCALE", "STEP"):
            cur[parts[0].lower()] = [float(x) for x in parts[1:]]
    return recs


class HdSequence(C.Structure):
    _fields_ = [("input_ids", C.c_void_p), ("pos_f32", C.POINTER(C.c_float)),
                ("mask_bf16", C.POINTER(C.c_uint16)), ("vinput_mask", C.c_void_p), ("sec", C.c_int64 * 3),
                ("text_len", C.c_int), ("image_len", C.c_int), ("img_begin", C.c_int), ("S", C.c_int),
                ("n_refs", C.c_int), ("ref_len", C.c_int * 20), ("ref_begin", C.c_int * 20)]


class HdTorchRng(C.Structure):
    _fields_ = [("seed_", C.c_uint64), ("left_", C.c_int), ("seeded_", C.c_int), ("next_", C.c_uint32),
                ("state", C.c_uint32 * 624)]


class HdScheduler(C.Structure):
    # src/model/scheduler.h: float sigmas[HD_SCHED_MAX_STEPS]; int num_steps; int step_index; float clip
    _fields_ = [("sigmas", C.c_float * 1024), ("tail", C.c_int * 8)]


def main():
    out = {}
    out["matrix"] = parse_dump(os.path.join(REF, "tests/unit/oracle_dump_matrix.txt"))
    out["plain"] = parse_dump(os.path.join(REF, "tests/unit/oracle_dump.txt"))
    json.dump(out, open(os.path.join(HERE, "scheduler_dump.json"), "w"))

    ref = C.CDLL(REF_LIB)
    # --- RNG
    rng = {}
    for n in (1, 8, 15, 16, 17, 31, 32, 1024):
        st = HdTorchRng()
        ref.hd_torch_rng_seed(C.byref(st), C.c_uint64(123457))
        a = np.empty(n, dtype=np.float32)
        ref.hd_torch_randn_f32(C.byref(st), a.ctypes.data_as(C.c_void_p), C.c_int64(n))
        rng[f"randn_{n}"] = a
    st = HdTorchRng()
    ref.hd_torch_rng_seed(C.byref(st), C.c_uint64(123457))
    ref.hd_torch_rng_u32.restype = C.c_uint32
    rng["u32_2000"] = np.array([ref.hd_torch_rng_u32(C.byref(st)) for _ in range(2000)], dtype=np.uint32)
    # a generator that carries state over several calls (z, mo, unused, noise of scheduler_matrix.c)
    st = HdTorchRng()
    ref.hd_torch_rng_seed(C.byref(st), C.c_uint64(1234))
    chain = np.empty((8, 64), dtype=np.float32)
    for i in range(8):
        ref.hd_torch_randn_f32(C.byref(st), chain[i].ctypes.data_as(C.c_void_p), C.c_int64(64))
    rng["chain_1234_8x64"] = chain
    np.savez_compressed(os.path.join(HERE, "rng_ref.npz"), **rng)

    # --- T2I sequences
    seqs = {}
    for tag, (T, hpx, wpx) in {"s23": (19, 64, 64), "c0": (256, 1024, 1024), "odd": (7, 96, 160)}.items():
        ids = (np.arange(T, dtype=np.int64) + 100)
        ids[-1] = 151673
        s = HdSequence()
        rc = ref.hd_seq_t2i(ids.ctypes.data_as(C.c_void_p), T, hpx, wpx, 32, 151655, 151656, 151652, 151673, 1,
                            1, 4096, C.byref(s))
        assert rc == 0
        S = s.S
        pos = np.ctypeslib.as_array(s.pos_f32, shape=(3 * S,)).copy().reshape(3, S)
        mask = np.ctypeslib.as_array(s.mask_bf16, shape=(S * S,)).copy().reshape(S, S)
        causal_rows = np.array([(mask[r, r + 1:] != 0).all() and (mask[r, :r + 1] == 0).all() if r < S - 1
                                else False for r in range(S)])
        full_rows = np.array([(mask[r] == 0).all() for r in range(S)])
        ar = int(causal_rows.sum())
        assert causal_rows[:ar].all() and full_rows[ar:].all(), "mask is not prefix-causal"
        assert set(np.unique(mask)) <= {0, 0xFF7F}
        seqs[f"{tag}_pos"] = pos
        seqs[f"{tag}_meta"] = np.array([T, hpx // 32, wpx // 32, S, ar, s.text_len, s.image_len, s.img_begin])
        ref.hd_sequence_free(C.byref(s))
    np.savez_compressed(os.path.join(HERE, "seq_t2i.npz"), **seqs)

    # --- K-reference sequences through hd_seq_build (needs the reference tokenizer, linked into libo1ref)
    class HdRequest(C.Structure):        # src/runtime/request.h:90-120 (leading fields; the rest zero)
        _fields_ = [("prompt", C.c_char_p), ("mode", C.c_int), ("profile", C.c_char_p), ("width", C.c_int),
                    ("height", C.c_int), ("seed", C.c_uint64), ("steps", C.c_int), ("guidance", C.c_float),
                    ("shift", C.c_float), ("scheduler", C.c_int), ("references", C.c_void_p),
                    ("reference_count", C.c_size_t), ("tail", C.c_uint8 * 128)]

    class HdRefGeom(C.Structure):
        _fields_ = [(n, C.c_int) for n in ("tokens", "grid_h", "grid_w", "cond_h", "cond_w")]

    refseq = {}
    cases = {"k1": ((1024, 1024), [(256, 16, 16, 12, 12)]),                 # tests/unit/test_seq_ref.c:97-119
             "k4": ((512, 512), [(64, 8, 8, 4, 4), (64, 8, 8, 4, 6), (16, 4, 4, 2, 2), (96, 8, 12, 3, 5)])}
    for tag, ((hpx, wpx), geoms) in cases.items():
        K = len(geoms)
        req = HdRequest(prompt=b"a red fox on the snow", reference_count=K)
        arr = (HdRefGeom * K)(*[HdRefGeom(*g_) for g_ in geoms])
        s = HdSequence()
        rc = ref.hd_seq_build(C.byref(req), 32, 151655, 151656, 151652, 151673, 1, 1, 4096, hpx, wpx, arr, C.byref(s))
        assert rc == 0, ref.hd_last_error
        S = s.S
        ids = np.ctypeslib.as_array(C.cast(s.input_ids, C.POINTER(C.c_int64)), shape=(S,)).copy()
        pos = np.ctypeslib.as_array(s.pos_f32, shape=(3 * S,)).copy().reshape(3, S)
        mask = np.ctypeslib.as_array(s.mask_bf16, shape=(S * S,)).copy().reshape(S, S)
        full_rows = (mask == 0).all(1)
        ar = int((~full_rows).sum())
        assert (~full_rows[:ar]).all() and full_rows[ar:].all()
        for r in range(ar):
            assert (mask[r, :r + 1] == 0).all() and (mask[r, r + 1:] == 0xFF7F).all()
        refseq[f"{tag}_ids"], refseq[f"{tag}_pos"] = ids, pos
        refseq[f"{tag}_geom"] = np.array(geoms, dtype=np.int32)
        refseq[f"{tag}_meta"] = np.array([s.text_len, hpx // 32, wpx // 32, S, ar, K])
        ref.hd_sequence_free(C.byref(s))
    np.savez_compressed(os.path.join(HERE, "seq_ref.npz"), **refseq)

    # --- sigma schedules straight from scheduler.c
    sig = {}
    for name, fn, args in (("dev", "hd_scheduler_derive_dev", ()),
                           ("flash_28_1", "hd_scheduler_derive_flash", (28, 1.0)),
                           ("flow_match_28_3", "hd_scheduler_derive_flow_match", (28, 3.0)),
                           ("default_50_3", "hd_scheduler_derive_default", (50, 3.0))):
        s = HdScheduler()
        f = getattr(ref, fn)
        if args:
            f.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_float]
            n = f(C.byref(s), args[0], args[1], 8.0)
        else:
            f.argtypes = [C.c_void_p, C.c_float]
            n = f(C.byref(s), 8.0)
        sig[name] = [float(np.float32(s.sigmas[i])) for i in range(n)]
    json.dump(sig, open(os.path.join(HERE, "sigmas_ref.json"), "w"))
    print("fixtures written to", HERE)


if __name__ == "__main__":
    sys.exit(main())
