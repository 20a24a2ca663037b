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
  lora_ref.npz        : merged weights from the reference's Python LoRA contract
                        (tools/lora/tests/test_lora_formula.py merge_linear + tools/lora/merge_gguf.py
                        f32_to_bf16_bytes, i.e. the "sequential-bf16-v1" merge of merge_gguf.py:164-171)
  decode_ref.npz      : hd_decode_to_rgb (src/runtime/decode.c) on a seeded latent
  ref_convert_small.gguf / .npz : a miniature model written by the reference's own converter
                        (tools/hidream_convert.py run on a small safetensors shard) and the bf16 bits it must hold
"""
import ctypes as C
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("O1_REFERENCE", os.path.join(ROOT, "..", "reference"))
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
    lora_fixture()
    decode_fixture(ref)
    converter_fixture()
    print("fixtures written to", HERE)


def _bf16_bits(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def lora_fixture():
    """W' = bf16(f32(W) + multiplier * alpha/rank * up @ down), computed by the reference's own Python:
    merge_linear of tools/lora/tests/test_lora_formula.py:20 on fp32 arrays (what merge_gguf.py:164-171
    evaluates) and the bf16 rounding of merge_gguf.py:44-49."""
    sys.path.insert(0, os.path.join(REF, "tools", "lora"))
    sys.path.insert(0, os.path.join(REF, "tools", "lora", "tests"))
    from test_lora_formula import merge_linear
    from merge_gguf import f32_to_bf16_bytes
    rng = np.random.default_rng(20240607)
    out = {}
    cases = [(96, 160, 8, 16.0, 1.0), (256, 128, 64, 64.0, 1.0), (48, 72, 4, 2.0, 0.8), (128, 384, 16, 16.0, -0.5)]
    for i, (N, K, R, alpha, mult) in enumerate(cases):
        w_bits = _bf16_bits(rng.standard_normal((N, K)).astype(np.float32) * 0.02)
        w_f32 = (w_bits.astype(np.uint32) << 16).view(np.float32).reshape(N, K)
        up = (rng.standard_normal((N, R)) * 0.05).astype(np.float32)
        down = (rng.standard_normal((R, K)) * 0.05).astype(np.float32)
        merged = merge_linear(w_f32, up, down, np.float32(alpha), np.float32(R), np.float32(mult))
        assert merged.dtype == np.float32
        bits = np.frombuffer(f32_to_bf16_bytes(merged), dtype=np.uint16).reshape(N, K)
        out[f"c{i}_w"], out[f"c{i}_up"], out[f"c{i}_down"], out[f"c{i}_merged"] = w_bits, up, down, bits
        out[f"c{i}_meta"] = np.array([N, K, R, alpha, mult], dtype=np.float64)
    out["n_cases"] = np.array(len(cases))
    np.savez_compressed(os.path.join(HERE, "lora_ref.npz"), **out)


def decode_fixture(ref):
    """hd_decode_to_rgb of src/runtime/decode.c:5-27 on a seeded latent that covers values beyond [-1, 1],
    exact .5 ties of the rounding and negative zero."""
    rng = np.random.default_rng(77)
    gh, gw, p = 3, 5, 32
    z = _bf16_bits(rng.standard_normal((gh * gw, 3 * p * p)).astype(np.float32) * 0.7)
    zf = (z.astype(np.uint32) << 16).view(np.float32)
    zf.reshape(-1)[:6] = [-1.0, 1.0, -0.0, 0.00392156862, 1.5, -1.5]      # 0.0039..: (v+1)/2*255 = 128.0 (a tie-free probe)
    z = _bf16_bits(zf)
    zf = (z.astype(np.uint32) << 16).view(np.float32).copy()
    rgb = np.zeros((gh * p, gw * p, 3), dtype=np.uint8)
    ref.hd_decode_to_rgb.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    ref.hd_decode_to_rgb.restype = None
    ref.hd_decode_to_rgb(zf.ctypes.data_as(C.c_void_p), gh, gw, p, 3, rgb.ctypes.data_as(C.c_void_p))
    np.savez_compressed(os.path.join(HERE, "decode_ref.npz"), z=z.reshape(gh * gw, 3 * p * p), rgb=rgb,
                        geom=np.array([gh, gw, p]))


def converter_fixture():
    """A two-block miniature (tiny shapes, real tensor names) stored as one safetensors shard, converted by the
    reference's own tools/hidream_convert.py.  F32 sources exercise its F32 -> BF16 path."""
    import subprocess
    import tempfile
    from safetensors.numpy import save_file
    rng = np.random.default_rng(5)
    names = ["model.language_model.embed_tokens.weight", "model.language_model.norm.weight",
             "model.t_embedder1.mlp.0.weight", "model.t_embedder1.mlp.0.bias", "model.t_embedder1.mlp.2.weight",
             "model.t_embedder1.mlp.2.bias", "model.x_embedder.proj1.weight", "model.x_embedder.proj2.weight",
             "model.x_embedder.proj2.bias", "model.final_layer2.linear.weight", "model.final_layer2.linear.bias"]
    slots = ["self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.o_proj.weight",
             "input_layernorm.weight", "post_attention_layernorm.weight", "mlp.gate_proj.weight", "mlp.up_proj.weight",
             "mlp.down_proj.weight", "self_attn.q_norm.weight", "self_attn.k_norm.weight"]
    for l in range(2):
        names += [f"model.language_model.layers.{l}.{s}" for s in slots]
    tensors = {}
    for i, n in enumerate(names):
        shape = (7, 24) if n.endswith("proj.weight") or "embed" in n or "linear.weight" in n or "mlp." in n else (40,)
        tensors[n] = (rng.standard_normal(shape) * 0.3).astype(np.float32)
    with tempfile.TemporaryDirectory() as d:
        save_file(tensors, os.path.join(d, "model-00001-of-00001.safetensors"))
        json.dump({"weight_map": {n: "model-00001-of-00001.safetensors" for n in names}},
                  open(os.path.join(d, "model.safetensors.index.json"), "w"))
        out = os.path.join(HERE, "ref_convert_small.gguf")
        subprocess.run([sys.executable, os.path.join(REF, "tools", "hidream_convert.py"), "--source", d, "--output", out],
                       check=True, stdout=subprocess.DEVNULL)
    np.savez_compressed(os.path.join(HERE, "ref_convert_small.npz"), **{n: _bf16_bits(a) for n, a in tensors.items()})


if __name__ == "__main__":
    sys.exit(main())
