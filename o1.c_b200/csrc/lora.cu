// Load-time LoRA merge  W = bf16( f32(W) + s * up @ down ),  s = multiplier*alpha/rank
// (o1.c include/hd_lora.h:10-14, src/model/lora_merge.cu:26-109, where the
// delta is an FP32 cublasSgemm over row chunks followed by an add/cast pass).
//
// Here the delta is a tcgen05 GEMM whose epilogue does the read-modify-write
// of W, so W crosses HBM once in each direction and no FP32 delta buffer
// exists.  The adapters arrive as FP32; to keep FP32-grade products on a
// bf16 tensor core each value is split into three bf16 terms
// (a = a1 + a2 + a3, 24 mantissa bits) and all nine cross terms are laid
// side by side along the contraction axis:
//     A' = [a1 a1 a1 a2 a2 a2 a3 a3 a3]   (out_dim x 9R)
//     B' = [b1 b2 b3 b1 b2 b3 b1 b2 b3]   (in_dim  x 9R, i.e. down transposed)
// Every bf16 x bf16 product is exact in the FP32 accumulator.
#include "common.cuh"
#include "kernels.h"
#include "../../include/o1_b200.h"

namespace o1 {

__device__ __forceinline__ void split3(float a, uint16_t& h1, uint16_t& h2, uint16_t& h3) {
    h1 = f32_to_bf16(a);
    const float r1 = a - bf16_to_f32(h1);
    h2 = f32_to_bf16(r1);
    const float r2 = r1 - bf16_to_f32(h2);
    h3 = f32_to_bf16(r2);
}

// up [N,R] fp32 -> A' [N, 9*Rp]
__global__ void lora_split_up_kernel(const float* __restrict__ up, uint16_t* __restrict__ a, int N, int R,
                                     int Rp) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long)N * Rp) return;
    const int r = (int)(i % Rp);
    const long n = i / Rp;
    uint16_t h[3] = {0, 0, 0};
    if (r < R) split3(up[n * R + r], h[0], h[1], h[2]);
    uint16_t* row = a + n * 9 * Rp;
#pragma unroll
    for (int t = 0; t < 9; ++t) row[t * Rp + r] = h[t / 3];
}
// down [R,K] fp32 -> B' [K, 9*Rp].  down is read along k (its contiguous axis), B' is written along its
// rows (9*Rp contiguous values per k): a tile of 32 k x Rp ranks goes through shared memory as split terms.
__global__ void __launch_bounds__(256) lora_split_down_kernel(const float* __restrict__ down,
                                                              uint16_t* __restrict__ b, int K, int R, int Rp) {
    extern __shared__ uint16_t sm[];            // [3][32][Rp + 2]: term, k within the tile, rank (padded)
    const int k0 = blockIdx.x * 32;
    const int ldp = Rp + 2;
    for (int i = threadIdx.x; i < 32 * Rp; i += blockDim.x) {
        const int kk = i & 31, r = i >> 5;      // kk fastest: coalesced reads of down
        uint16_t h[3] = {0, 0, 0};
        if (r < R && k0 + kk < K) split3(down[(long)r * K + k0 + kk], h[0], h[1], h[2]);
#pragma unroll
        for (int t = 0; t < 3; ++t) sm[(t * 32 + kk) * ldp + r] = h[t];
    }
    __syncthreads();
    const int row_len = 9 * Rp;
    for (int i = threadIdx.x; i < 32 * row_len; i += blockDim.x) {
        const int kk = i / row_len, c = i - kk * row_len;   // c fastest: coalesced writes of B'
        if (k0 + kk >= K) break;
        const int t = c / Rp, r = c - t * Rp;
        b[(long)(k0 + kk) * row_len + c] = sm[((t % 3) * 32 + kk) * ldp + r];
    }
}
// shapes the tensor-core tiles do not cover
__global__ void lora_simt_kernel(uint16_t* __restrict__ w, const float* __restrict__ up,
                                 const float* __restrict__ down, int N, int K, int R, float scale) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long)N * K) return;
    const int k = (int)(i % K);
    const long n = i / K;
    float acc = 0.f;
    for (int r = 0; r < R; ++r) acc += up[n * R + r] * down[(long)r * K + k];
    w[i] = f32_to_bf16(bf16_to_f32(w[i]) + scale * acc);
}

}  // namespace o1

using namespace o1;

extern "C" {

hd_status hd_lora_merge_gpu(hd_lora_entry* entries, size_t count, void* stream) {
    if (count == 0) return HD_OK;
    if (!entries) { set_error("lora: null entries"); return HD_ERR_MISSING; }
    cudaStream_t st = (cudaStream_t)stream;
    uint16_t* stage = nullptr;
    size_t stage_cap = 0;
    hd_status rc = HD_OK;
    for (size_t i = 0; i < count && rc == HD_OK; ++i) {
        hd_lora_entry* e = &entries[i];
        const int R = (int)e->rank, K = (int)e->in_dim, N = (int)e->out_dim;
        if (R <= 0 || K <= 0 || N <= 0 || !e->up_dev || !e->down_dev || !e->base_dev) {
            set_error("lora: bad entry %zu", i);
            rc = HD_ERR_MISMATCH;
            break;
        }
        const float scale = e->multiplier * e->alpha / (float)e->rank;
        const int Rp = (R + 63) & ~63;
        const size_t split_smem = (size_t)3 * 32 * (Rp + 2) * sizeof(uint16_t);   // lora_split_down_kernel's tile
        if (!gemm_tc_supported(N, K, 9 * Rp, EPI_LORA) || split_smem > 200 * 1024) {
            const long tot = (long)N * K;
            lora_simt_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, st>>>(
                (uint16_t*)e->base_dev, (const float*)e->up_dev, (const float*)e->down_dev, N, K, R, scale);
            if (cudaGetLastError() != cudaSuccess) { set_error("lora: simt launch failed"); rc = HD_ERR_RUNTIME; }
            continue;
        }
        const size_t need = ((size_t)N + (size_t)K) * 9 * Rp * sizeof(uint16_t) + 512;
        if (need > stage_cap) {
            if (stage) { cudaStreamSynchronize(st); cudaFree(stage); stage = nullptr; }
            if (cudaMalloc(&stage, need) != cudaSuccess) {
                set_error("lora: staging cudaMalloc of %zu bytes failed", need);
                rc = HD_ERR_OOM;
                break;
            }
            stage_cap = need;
        }
        uint16_t* a = stage;
        uint16_t* b = stage + (((size_t)N * 9 * Rp + 127) & ~(size_t)127);
        const long na = (long)N * Rp;
        lora_split_up_kernel<<<(unsigned)((na + 255) / 256), 256, 0, st>>>((const float*)e->up_dev, a, N, R, Rp);
        if (split_smem > 48 * 1024 &&
            cudaFuncSetAttribute(lora_split_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)split_smem) !=
                cudaSuccess) {
            set_error("lora: shared-memory attribute for rank %d failed", R);
            rc = HD_ERR_RUNTIME;
            break;
        }
        lora_split_down_kernel<<<(unsigned)((K + 31) / 32), 256, split_smem, st>>>((const float*)e->down_dev, b, K, R, Rp);
        if (cudaGetLastError() != cudaSuccess) { set_error("lora: split launch failed"); rc = HD_ERR_RUNTIME; break; }
        // W[N,K] += scale * A'[N,9Rp] . B'[K,9Rp]^T, in place
        if (!gemm_bf16_ld(a, 9 * Rp, b, nullptr, e->base_dev, K, N, K, 9 * Rp, EPI_LORA, nullptr, nullptr,
                          0, scale, 0, st)) {
            rc = HD_ERR_RUNTIME;
            break;
        }
        // the staging buffer is reused by the next entry: stream order keeps that safe
    }
    if (stage) {
        cudaStreamSynchronize(st);
        cudaFree(stage);
    }
    return rc;
}

}  // extern "C"
