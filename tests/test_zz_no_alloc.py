"""o1_lora_merge_static: the LoRA merge for hosts that must not allocate device memory (their own pool
owns all of HBM, or a cudaMalloc/cudaFree stall is unacceptable while other streams work).  It must give
what hd_lora_merge_gpu gives -- same check as tests/test_gpu_lora.py: identical bf16 weights except on
rounding ties of the FP32 sum -- on two calls in a row that reuse the library's built-in scratch with
different shapes and values, and it must refuse sizes beyond that scratch.

Collected last on purpose, so a run that stops at the first failure has already run everything else."""
import numpy as np
import pytest
import torch

import parity
from parity import np_ptr, seeded_bf16, torch_to_u16, u16_to_torch
from test_gpu_lora import check_merged, entry

pytestmark = pytest.mark.gpu


def _case(pkg, orc, dev, N, K, R, seed, scale_alpha):
    w0 = seeded_bf16((N, K), seed, 0.0, 0.02)
    up, down = np.empty((N, R), dtype=np.float32), np.empty((R, K), dtype=np.float32)
    orc.orc_fill_normal_f32(np_ptr(up), up.size, seed + 1, 0.0, 0.02)
    orc.orc_fill_normal_f32(np_ptr(down), down.size, seed + 2, 0.0, 0.02)
    upd, dnd = torch.from_numpy(up).to(dev), torch.from_numpy(down).to(dev)
    w_old, w_new = u16_to_torch(w0, dev), u16_to_torch(w0, dev)
    ents = (pkg.LoraEntry * 1)(entry(pkg, w_old, upd, dnd, R, K, N, scale_alpha, 1.0))
    assert pkg.lib.hd_lora_merge_gpu(ents, 1, None) == 0, pkg.last_error()
    rc = pkg.lib.o1_lora_merge_static(pkg.ptr(w_new), pkg.ptr(upd), pkg.ptr(dnd), N, K, R, scale_alpha / R, None)
    assert rc == 0, pkg.last_error()
    torch.cuda.synchronize()
    got, want = torch_to_u16(w_new), torch_to_u16(w_old)
    assert (got != w0).mean() > 0.01, "merge changed nothing"
    check_merged(got, want, w0)
    # and both agree with the FP32 restatement of the documented formula
    ref = w0.copy()
    orc.orc_lora_merge(np_ptr(ref), np_ptr(up), np_ptr(down), N, K, R, scale_alpha / R)
    check_merged(got, ref, w0)


def test_static_scratch_merge_matches_allocating_merge_twice_in_a_row(pkg, orc, dev):
    _case(pkg, orc, dev, 1024, 4096, 64, 900, 64.0)      # one chunk of 1024 rows
    _case(pkg, orc, dev, 4096, 12288, 16, 910, 8.0)      # several chunks; stale scratch from call 1 underneath
    _case(pkg, orc, dev, 384, 256, 8, 920, 4.0)          # smaller than what the scratch still holds


def test_static_scratch_merge_rejects_oversized(pkg, dev):
    w = torch.zeros(16, dtype=torch.bfloat16, device=dev)
    f = torch.zeros(16, device=dev)
    pkg.lib.hd_cuda_clear_error()
    assert pkg.lib.o1_lora_merge_static(pkg.ptr(w), pkg.ptr(f), pkg.ptr(f), 1, 262145, 1, 1.0, None) == 9
    assert b"exceeds the built-in scratch" in pkg.lib.hd_cuda_last_error()
    assert pkg.lib.o1_lora_merge_static(pkg.ptr(w), pkg.ptr(f), pkg.ptr(f), 1, 16, 4097, 1.0, None) == 9
    assert pkg.lib.o1_lora_merge_static(None, pkg.ptr(f), pkg.ptr(f), 1, 16, 1, 1.0, None) == 6
    pkg.lib.hd_cuda_clear_error()
