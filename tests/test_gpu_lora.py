"""Load-time LoRA merge (hd_lora_merge_gpu, o1.c include/hd_lora.h:71-79) against the FP32 restatement
of src/model/lora_merge.cu:26-109: the merged bf16 weights must be bit-identical except where
scale*delta lands on a rounding tie of the FP32 sum (counted, must be a vanishing fraction)."""
import ctypes as C

import numpy as np
import pytest
import torch

import parity
from parity import np_ptr, seeded_bf16, torch_to_u16, u16_to_torch

pytestmark = pytest.mark.gpu


def entry(pkg, w, up, down, R, K, N, alpha, mult):
    e = pkg.LoraEntry()
    e.rank, e.in_dim, e.out_dim, e.alpha, e.multiplier = R, K, N, alpha, mult
    e.down_dev, e.up_dev, e.base_dev = down.data_ptr(), up.data_ptr(), w.data_ptr()
    return e


@pytest.mark.parametrize("N,K,R", [(1024, 4096, 64), (4096, 1024, 16), (384, 256, 8), (100, 72, 4)])
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
    diff = got.astype(np.int32) - ref.astype(np.int32)
    assert np.abs(diff).max() <= 1
    assert (diff != 0).mean() <= 2e-4, f"{(diff != 0).mean():.2e} of the weights differ by one bf16 ulp"
    r = parity.reflib()
    if r is not None:
        w2 = u16_to_torch(w0, dev)
        ents2 = (pkg.LoraEntry * 1)(entry(pkg, w2, upd, dnd, R, K, N, alpha, mult))
        assert r.hd_lora_merge_gpu(ents2, 1, None) == 0
        torch.cuda.synchronize()
        d2 = torch_to_u16(w2).astype(np.int32) - got.astype(np.int32)
        assert np.abs(d2).max() <= 1 and (d2 != 0).mean() <= 2e-4, "vs reference cublasSgemm merge"


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
    diff = torch_to_u16(wd).astype(np.int32) - ref.astype(np.int32)
    assert np.abs(diff).max() <= 1 and (diff != 0).mean() <= 5e-4
    bad = (pkg.LoraEntry * 1)(entry(pkg, wd, keep[0], keep[2], 0, K, N, 4.0, 1.0))
    assert pkg.lib.hd_lora_merge_gpu(bad, 1, None) == 5          # HD_ERR_MISMATCH
