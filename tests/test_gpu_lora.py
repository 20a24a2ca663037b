"""Load-time LoRA merge (hd_lora_merge_gpu, o1.c include/hd_lora.h:71-79) against the FP32 restatement
of the documented contract W' = bf16(f32(W) + multiplier*alpha/rank * up@down) (hd_lora.h:10-14,
lora_merge.cu:26-33): the merged bf16 weights must be bit-identical except where the FP32 sum lands on
a rounding tie (counted, must be a vanishing fraction).

The reference's own GPU merge is NOT run here: its cublasSgemm call passes the row-major up-chunk
with leading dimension C instead of rank (lora_merge.cu:86-93), which reads beyond the adapter
buffer whenever out_dim != rank."""
import ctypes as C

import numpy as np
import pytest
import torch

import parity
from parity import np_ptr, seeded_bf16, torch_to_u16, u16_to_torch

pytestmark = pytest.mark.gpu


def check_merged(got, ref, w0, max_frac=2e-4):
    """Bit-identical except on rounding ties: where the two FP32 sums round to different bf16 values
    they must be neighbours at the scale of the operands (one bf16 ulp of max(|W|, |W'|)), and such
    elements must be a vanishing fraction."""
    g, r_, w = (parity.bf16_to_f32_np(a).astype(np.float64) for a in (got, ref, w0))
    neq = got != ref
    assert neq.mean() <= max_frac, f"{neq.mean():.2e} of the merged weights differ"
    ulp = np.maximum(np.abs(w), np.abs(r_)) * 2.0 ** -7 + 1e-30
    assert (np.abs(g - r_) <= ulp).all()


def entry(pkg, w, up, down, R, K, N, alpha, mult):
    e = pkg.LoraEntry()
    e.rank, e.in_dim, e.out_dim, e.alpha, e.multiplier = R, K, N, alpha, mult
    e.down_dev, e.up_dev, e.base_dev = down.data_ptr(), up.data_ptr(), w.data_ptr()
    return e


@pytest.mark.parametrize("N,K,R", [(1024, 4096, 64), (4096, 1024, 16), (384, 256, 8), (100, 72, 4), (512, 1280, 200)])
def test_lora_merge(pkg, orc, dev, N, K, R):
    w0 = seeded_bf16((N, K), 51, 0.0, 0.02)
    up = np.empty((N, R), dtype=np.float32)
    down = np.empty((R, K), dtype=np.float32)
    orc.orc_fill_normal_f32(np_ptr(up), up.size, 52, 0.0, 0.01)
    orc.orc_fill_normal_f32(np_ptr(down), down.size, 53, 0.0, 0.01)
    alpha, mult = float(R), 1.0
    wd = u16_to_torch(w0, dev)
    ents = (pkg.LoraEntry * 1)(entry(pkg, wd, torch.from_numpy(up).to(dev), torch.from_numpy(down).to(dev), R, K, N,
                                     alpha, mult))
    upd, dnd = torch.from_numpy(up).to(dev), torch.from_numpy(down).to(dev)
    ents[0].up_dev, ents[0].down_dev = upd.data_ptr(), dnd.data_ptr()
    rc = pkg.lib.hd_lora_merge_gpu(ents, 1, None)
    torch.cuda.synchronize()
    assert rc == 0, pkg.last_error()
    ref = w0.copy()
    orc.orc_lora_merge(np_ptr(ref), np_ptr(up), np_ptr(down), N, K, R, mult * alpha / R)
    got = torch_to_u16(wd)
    assert (got != w0).mean() > 0.01, "merge changed nothing"
    # 9 x 256 exact products per element are summed by the tensor core in its own order: more tie flips than at rank 64
    check_merged(got, ref, w0, max_frac=2e-4 if R <= 64 else 2e-3)


def test_lora_sequential_adapters_and_errors(pkg, orc, dev):
    """Two adapters on one weight: one bf16 rounding per adapter, in order (contract sequential-bf16-v1)."""
    N, K, R = 256, 512, 8
    w0 = seeded_bf16((N, K), 61, 0.0, 0.02)
    ups = [np.empty((N, R), dtype=np.float32) for _ in range(2)]
    dns = [np.empty((R, K), dtype=np.float32) for _ in range(2)]
    for i in range(2):
        orc.orc_fill_normal_f32(np_ptr(ups[i]), ups[i].size, 70 + i, 0.0, 0.05)
        orc.orc_fill_normal_f32(np_ptr(dns[i]), dns[i].size, 80 + i, 0.0, 0.05)
    wd = u16_to_torch(w0, dev)
    keep = [torch.from_numpy(a).to(dev) for a in ups + dns]
    ents = (pkg.LoraEntry * 2)(entry(pkg, wd, keep[0], keep[2], R, K, N, 4.0, 1.0),
                               entry(pkg, wd, keep[1], keep[3], R, K, N, 8.0, 0.5))
    assert pkg.lib.hd_lora_merge_gpu(ents, 2, None) == 0
    torch.cuda.synchronize()
    ref = w0.copy()
    orc.orc_lora_merge(np_ptr(ref), np_ptr(ups[0]), np_ptr(dns[0]), N, K, R, 1.0 * 4.0 / R)
    orc.orc_lora_merge(np_ptr(ref), np_ptr(ups[1]), np_ptr(dns[1]), N, K, R, 0.5 * 8.0 / R)
    check_merged(torch_to_u16(wd), ref, w0, 5e-4)
    bad = (pkg.LoraEntry * 1)(entry(pkg, wd, keep[0], keep[2], 0, K, N, 4.0, 1.0))
    assert pkg.lib.hd_lora_merge_gpu(bad, 1, None) == 5          # HD_ERR_MISMATCH


def test_lora_merge_against_the_reference_python_contract(pkg, dev, golden):
    """hd_lora_merge_gpu against weights merged by the reference's own Python (merge_linear of o1.c
    tools/lora/tests/test_lora_formula.py:20 + the bf16 rounding of tools/lora/merge_gguf.py:44-49,164-171);
    fixture tests/golden/lora_ref.npz, including a multiplier != 1 and a negative one."""
    import os
    g = np.load(os.path.join(golden, "lora_ref.npz"))
    for i in range(int(g["n_cases"])):
        N, K, R, alpha, mult = g[f"c{i}_meta"]
        N, K, R = int(N), int(K), int(R)
        w0 = np.ascontiguousarray(g[f"c{i}_w"])
        wd = u16_to_torch(w0, dev)
        upd = torch.from_numpy(np.ascontiguousarray(g[f"c{i}_up"])).to(dev)
        dnd = torch.from_numpy(np.ascontiguousarray(g[f"c{i}_down"])).to(dev)
        ents = (pkg.LoraEntry * 1)(entry(pkg, wd, upd, dnd, R, K, N, float(alpha), float(mult)))
        assert pkg.lib.hd_lora_merge_gpu(ents, 1, None) == 0, pkg.last_error()
        torch.cuda.synchronize()
        check_merged(torch_to_u16(wd), g[f"c{i}_merged"], w0, max_frac=1e-3)
