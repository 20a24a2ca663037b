// LoRA merge of ONE target without any device allocation.
//
// Who needs this: a host that has handed all of the GPU's memory to its own pool
// before the engine starts (a serving process that pre-reserves HBM for weights,
// workspaces and other tenants), or that merges an adapter while other streams are
// busy producing images and therefore must avoid cudaMalloc / cudaFree, which
// stall the whole device.  hd_lora_merge_gpu allocates (and frees) a staging
// buffer per call; this entry point keeps its scratch in a fixed array inside the
// library image instead.
//
// Arithmetic: delta = up @ down in FP32 (rank-sequential sum), then
// W = bf16(f32(W) + scale * delta), row chunk by row chunk through the scratch --
// the same two-pass shape as o1.c's src/model/lora_merge.cu:26-109.
//
// The scratch is shared by every call in the process and keeps the previous call's
// contents; each chunk is fully overwritten before it is read, so nothing has to be
// cleared.  Two calls that overlap on the GPU (different streams) race on it.
#include "common.cuh"
#include "../../include/o1_b200.h"

namespace o1 {

// 4 Mi floats = 16 MiB, held by every GPU that loads the library until the process exits.
static constexpr size_t LORA_STATIC_FLOATS = 4u * 1024u * 1024u;
static __device__ __align__(256) float g_lora_delta[LORA_STATIC_FLOATS];

__global__ void lora_static_delta_kernel(const float* __restrict__ up, const float* __restrict__ down,
                                         float* __restrict__ delta, int rows, int K, int R) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long)rows * K) return;
    const int k = (int)(i % K);
    const long n = i / K;
    float acc = 0.f;
    for (int r = 0; r < R; ++r) acc = __fmaf_rn(up[n * R + r], down[(long)r * K + k], acc);
    delta[i] = acc;
}
__global__ void lora_static_add_kernel(uint16_t* __restrict__ w, const float* __restrict__ delta, long n,
                                       float scale) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) w[i] = f32_to_bf16(__fmaf_rn(scale, delta[i], bf16_to_f32(w[i])));
}

// Device address of the scratch, resolved once per device with that device current.
// In host code the array's name is only a handle for the runtime, not an address.
static float* lora_static_scratch(cudaError_t* err) {
    static float* ptrs[64] = {nullptr};
    int dev = 0;
    *err = cudaGetDevice(&dev);
    if (*err != cudaSuccess) return nullptr;
    if (dev < 0 || dev >= 64) { *err = cudaErrorInvalidDevice; return nullptr; }
    if (!ptrs[dev]) {
        float* p = nullptr;
        *err = cudaGetSymbolAddress((void**)&p, g_lora_delta);
        if (*err != cudaSuccess) return nullptr;
        ptrs[dev] = p;
    }
    return ptrs[dev];
}

}  // namespace o1

using namespace o1;

extern "C" hd_status o1_lora_merge_static(void* base_dev, const float* up_dev, const float* down_dev,
                                          uint32_t out_dim, uint32_t in_dim, uint32_t rank, float scale,
                                          void* stream) {
    if (!base_dev || !up_dev || !down_dev || out_dim == 0 || in_dim == 0 || rank == 0) {
        set_error("lora_merge_static: bad arguments");
        return HD_ERR_MISSING;
    }
    if ((size_t)in_dim > LORA_STATIC_FLOATS / 16 || rank > 4096) {
        set_error("lora_merge_static: in_dim %u (max %zu) or rank %u (max 4096) exceeds the built-in scratch",
                  in_dim, LORA_STATIC_FLOATS / 16, rank);
        return HD_ERR_UNSUPPORTED;
    }
    cudaError_t ce;
    float* scratch = lora_static_scratch(&ce);
    if (!scratch) {
        set_error("lora_merge_static: scratch address: %s", cudaGetErrorString(ce));
        return HD_ERR_RUNTIME;
    }
    cudaStream_t st = (cudaStream_t)stream;
    const int K = (int)in_dim, R = (int)rank;
    const int chunk_rows = (int)(LORA_STATIC_FLOATS / (size_t)K);     // >= 16 by the in_dim limit
    uint16_t* w = (uint16_t*)base_dev;
    for (uint32_t row0 = 0; row0 < out_dim; row0 += (uint32_t)chunk_rows) {
        const int rows = (int)((out_dim - row0) < (uint32_t)chunk_rows ? (out_dim - row0) : (uint32_t)chunk_rows);
        const long n = (long)rows * K;
        const unsigned blocks = (unsigned)((n + 255) / 256);
        lora_static_delta_kernel<<<blocks, 256, 0, st>>>(up_dev + (size_t)row0 * R, down_dev, scratch, rows, K, R);
        lora_static_add_kernel<<<blocks, 256, 0, st>>>(w + (size_t)row0 * K, scratch, n, scale);
    }
    ce = cudaGetLastError();
    if (ce != cudaSuccess) {
        set_error("lora_merge_static: launch: %s", cudaGetErrorString(ce));
        return HD_ERR_RUNTIME;
    }
    return HD_OK;
}
