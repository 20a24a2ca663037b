// Shared helpers: bf16 conversion with the reference's rounding
// (src/cuda/cuda_internal.h:21-40 in o1.c: RNE by integer add, no NaN
// special case), 128-bit vector types, error slot, stream handling.
// On the device the rounding is the hardware conversion (cvt.rn.bf16.f32 /
// cvt.rn.bf16x2.f32: one instruction instead of five per value; the epilogues
// and elementwise kernels round several times per element).  It gives the
// same result as the integer form for every finite input and infinity; only
// NaN payloads differ (canonical NaN instead of a shifted payload).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace o1 {

__host__ __device__ __forceinline__ float bf16_to_f32(uint16_t b) {
    uint32_t u = ((uint32_t)b) << 16;
#ifdef __CUDA_ARCH__
    return __uint_as_float(u);
#else
    float f;
    __builtin_memcpy(&f, &u, 4);
    return f;
#endif
}
__host__ __device__ __forceinline__ uint16_t f32_to_bf16(float f) {
#ifdef __CUDA_ARCH__
    uint16_t r;
    asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f));
    return r;
#else
    uint32_t u;
    __builtin_memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
#endif
}
__host__ __device__ __forceinline__ float bf16_round(float f) {
    return bf16_to_f32(f32_to_bf16(f));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float bf16lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }

// ---- process-wide state (one stream, one error buffer: the reference's
// primitive ABI has no stream argument and reports through a message buffer)
cudaStream_t current_stream();
char* errbuf();             // 512 bytes
void set_error(const char* fmt, ...);
int* device_error_word();   // per-device int set by kernels whose bounded waits ran out
int sm_count();

#define O1_CUDA_OK(call, what)                                                     \
    do {                                                                           \
        cudaError_t e__ = (call);                                                  \
        if (e__ != cudaSuccess) o1::set_error("%s: %s", what, cudaGetErrorString(e__)); \
    } while (0)

}  // namespace o1
