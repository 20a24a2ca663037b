// Flow-matching scheduler device math (o1.c src/cuda/sched.cu:23-229):
// the flash Euler chain, v_cond folding, CFG combine, deterministic
// flow-match Euler step and the UniPC bh2 predictor/corrector pointwise
// updates, all fp32 in torch's left-to-right order, plus one fused kernel
// for the CFG + flow-match step that reads z and both predictions once.
#include "common.cuh"
#include "kernels.h"

namespace o1 {

#define O1_LAUNCH_CHECK(name)                                                        \
    do {                                                                             \
        cudaError_t e__ = cudaGetLastError();                                        \
        if (e__ != cudaSuccess) { set_error(name ": %s", cudaGetErrorString(e__)); return false; } \
    } while (0)

static inline unsigned nblocks(size_t n) { return (unsigned)((n + 255) / 256); }

// The three pointwise formulas, written with explicit roundings so that the
// stand-alone kernels and the fused step produce identical bits.  The fused
// multiply-adds are the ones nvcc forms for the reference's expressions
// (sched.cu:57-60, 121, 142-143: first product fused, second product rounded).
__device__ __forceinline__ float vcond_f(float z, float xp, float sigma) {
    return __fdiv_rn(__fsub_rn(z, xp), sigma);
}
__device__ __forceinline__ float cfg_f(float mc, float mu, float g) {
    return __fmaf_rn(__fsub_rn(1.0f, g), mu, __fmul_rn(g, mc));
}
__device__ __forceinline__ float flow_f(float z, float dt, float mo) { return __fmaf_rn(dt, mo, z); }

__global__ void upcast_kernel(const uint16_t* __restrict__ in, float* __restrict__ out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = bf16_to_f32(in[i]);
}
__global__ void denoised_kernel(const float* __restrict__ z, const float* __restrict__ mo, float sigma,
                                float* __restrict__ den, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) den[i] = __fmaf_rn(-mo[i], sigma, z[i]);
}
__global__ void z_next_kernel(const float* __restrict__ noise, const float* __restrict__ den,
                              float sigma_next, float s_noise, float* __restrict__ z_next, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n)
        z_next[i] = __fmaf_rn(__fmul_rn(sigma_next, noise[i]), s_noise,
                              __fmul_rn(__fsub_rn(1.0f, sigma_next), den[i]));
}
__global__ void vcond_kernel(const uint16_t* __restrict__ z, const uint16_t* __restrict__ xp,
                             float sigma, float* __restrict__ mo, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) mo[i] = vcond_f(bf16_to_f32(z[i]), bf16_to_f32(xp[i]), sigma);
}
__global__ void flow_step_kernel(const uint16_t* __restrict__ z, const float* __restrict__ mo, float dt,
                                 uint16_t* __restrict__ z_next, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) z_next[i] = f32_to_bf16(flow_f(bf16_to_f32(z[i]), dt, mo[i]));
}
__global__ void cfg_kernel(const float* __restrict__ mc, const float* __restrict__ mu, float g,
                           float* __restrict__ mo, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) mo[i] = cfg_f(mc[i], mu[i], g);
}

// z' = bf16( z + dt * ( (1-g) * (z-xu)/sigma + g * (z-xc)/sigma ) ), 8 elements
// per thread through 128-bit loads: 3 reads + 1 write of 2 bytes per element.
__global__ void __launch_bounds__(256)
cfg_flow_step_kernel(const uint4* __restrict__ z, const uint4* __restrict__ xc,
                     const uint4* __restrict__ xu, float sigma, float dt, float g,
                     uint4* __restrict__ z_next, size_t nvec) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        const uint4 a = z[i], b = xc[i], c = xu[i];
        const uint32_t av[4] = {a.x, a.y, a.z, a.w};
        const uint32_t bv[4] = {b.x, b.y, b.z, b.w};
        const uint32_t cv[4] = {c.x, c.y, c.z, c.w};
        uint32_t ov[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float r[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float zf = h ? bf16hi(av[j]) : bf16lo(av[j]);
                const float cf = h ? bf16hi(bv[j]) : bf16lo(bv[j]);
                const float uf = h ? bf16hi(cv[j]) : bf16lo(cv[j]);
                const float mo = cfg_f(vcond_f(zf, cf, sigma), vcond_f(zf, uf, sigma), g);
                r[h] = flow_f(zf, dt, mo);
            }
            ov[j] = pack_bf16x2(r[0], r[1]);
        }
        z_next[i] = make_uint4(ov[0], ov[1], ov[2], ov[3]);
    }
}
__global__ void cfg_flow_step_scalar_kernel(const uint16_t* __restrict__ z, const uint16_t* __restrict__ xc,
                                            const uint16_t* __restrict__ xu, float sigma, float dt,
                                            float g, uint16_t* __restrict__ z_next, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float zf = bf16_to_f32(z[i]);
    const float mo = cfg_f(vcond_f(zf, bf16_to_f32(xc[i]), sigma), vcond_f(zf, bf16_to_f32(xu[i]), sigma), g);
    z_next[i] = f32_to_bf16(flow_f(zf, dt, mo));
}

__global__ void unipc_convert_kernel(const float* __restrict__ sample, const float* __restrict__ mo,
                                     float sigma_cur, float* __restrict__ conv, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) conv[i] = sample[i] - sigma_cur * mo[i];
}
__global__ void unipc_correct_kernel(const float* __restrict__ last, const float* __restrict__ mo0,
                                     const float* __restrict__ mo_old, const float* __restrict__ conv,
                                     float sig_t, float sig_s0, float alpha_t, float h_phi_1, float B_h,
                                     float rhos_c0, float rhos_c1, float inv_rks0, int order_c,
                                     float* __restrict__ out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float x_t = (sig_t / sig_s0) * last[i] - alpha_t * h_phi_1 * mo0[i];
    const float D1_t = conv[i] - mo0[i];
    float corr;
    if (order_c == 2) {
        const float D1s = (mo_old[i] - mo0[i]) * inv_rks0;
        corr = rhos_c0 * D1s + rhos_c1 * D1_t;
    } else {
        corr = rhos_c1 * D1_t;
    }
    out[i] = x_t - alpha_t * B_h * corr;
}
__global__ void unipc_predict_kernel(const float* __restrict__ sample, const float* __restrict__ mo0,
                                     const float* __restrict__ mo_old, float sig_t, float sig_s0,
                                     float alpha_t, float h_phi_1, float B_h, float rhos_p,
                                     float inv_rks0, int order_p, float* __restrict__ out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float x_t = (sig_t / sig_s0) * sample[i] - alpha_t * h_phi_1 * mo0[i];
    if (order_p == 2) {
        const float D1s = (mo_old[i] - mo0[i]) * inv_rks0;
        x_t -= alpha_t * B_h * (rhos_p * D1s);
    }
    out[i] = x_t;
}

bool sched_bf16_upcast(const void* in, float* out, int n, cudaStream_t st) {
    if (!in || !out || n <= 0) { set_error("sched_bf16_upcast: bad args"); return false; }
    upcast_kernel<<<nblocks(n), 256, 0, st>>>((const uint16_t*)in, out, n);
    O1_LAUNCH_CHECK("sched_bf16_upcast");
    return true;
}
bool sched_denoised(const float* z, const float* mo, float sigma, float* den, int n, cudaStream_t st) {
    if (!z || !mo || !den || n <= 0) { set_error("sched_denoised: bad args"); return false; }
    denoised_kernel<<<nblocks(n), 256, 0, st>>>(z, mo, sigma, den, n);
    O1_LAUNCH_CHECK("sched_denoised");
    return true;
}
bool sched_z_next(const float* noise, const float* den, float sigma_next, float s_noise,
                  float* z_next, int n, cudaStream_t st) {
    if (!noise || !den || !z_next || n <= 0) { set_error("sched_z_next: bad args"); return false; }
    z_next_kernel<<<nblocks(n), 256, 0, st>>>(noise, den, sigma_next, s_noise, z_next, n);
    O1_LAUNCH_CHECK("sched_z_next");
    return true;
}
bool sched_vcond(const void* z, const void* xp, float sigma, float* mo, int n, cudaStream_t st) {
    if (!z || !xp || !mo || n <= 0) { set_error("sched_vcond: bad args"); return false; }
    vcond_kernel<<<nblocks(n), 256, 0, st>>>((const uint16_t*)z, (const uint16_t*)xp, sigma, mo, n);
    O1_LAUNCH_CHECK("sched_vcond");
    return true;
}
bool sched_flow_match_step(const void* z, const float* mo, float sigma, float sigma_next,
                           void* z_next, int n, cudaStream_t st) {
    if (!z || !mo || !z_next || n <= 0) { set_error("sched_flow_match_step: bad args"); return false; }
    const float dt = sigma_next - sigma;
    flow_step_kernel<<<nblocks(n), 256, 0, st>>>((const uint16_t*)z, mo, dt, (uint16_t*)z_next, n);
    O1_LAUNCH_CHECK("sched_flow_match_step");
    return true;
}
bool sched_cfg_guided(const float* mc, const float* mu, float g, float* mo, int n, cudaStream_t st) {
    if (!mc || !mu || !mo || n <= 0) { set_error("sched_cfg_guided: bad args"); return false; }
    cfg_kernel<<<nblocks(n), 256, 0, st>>>(mc, mu, g, mo, n);
    O1_LAUNCH_CHECK("sched_cfg_guided");
    return true;
}
bool sched_cfg_flow_step(const void* z, const void* xc, const void* xu, float sigma, float sigma_next,
                         float g, void* z_next, size_t n, cudaStream_t st) {
    if (!z || !xc || !xu || !z_next || n == 0) { set_error("sched_cfg_flow_step: bad args"); return false; }
    const float dt = sigma_next - sigma;
    const uintptr_t al = (uintptr_t)z | (uintptr_t)xc | (uintptr_t)xu | (uintptr_t)z_next;
    if ((al & 15) == 0 && (n % 8) == 0) {
        const size_t nvec = n / 8;
        size_t want = (nvec + 255) / 256;
        const size_t cap = (size_t)sm_count() * 16;
        cfg_flow_step_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, st>>>(
            (const uint4*)z, (const uint4*)xc, (const uint4*)xu, sigma, dt, g, (uint4*)z_next, nvec);
    } else {
        cfg_flow_step_scalar_kernel<<<nblocks(n), 256, 0, st>>>(
            (const uint16_t*)z, (const uint16_t*)xc, (const uint16_t*)xu, sigma, dt, g,
            (uint16_t*)z_next, n);
    }
    O1_LAUNCH_CHECK("sched_cfg_flow_step");
    return true;
}
bool unipc_convert(const float* sample, const float* mo, float sigma_cur, float* conv, int n,
                   cudaStream_t st) {
    if (!sample || !mo || !conv || n <= 0) { set_error("unipc_convert: bad args"); return false; }
    unipc_convert_kernel<<<nblocks(n), 256, 0, st>>>(sample, mo, sigma_cur, conv, n);
    O1_LAUNCH_CHECK("unipc_convert");
    return true;
}
bool unipc_correct(const float* last, const float* mo0, const float* mo_old, const float* conv,
                   float sig_t, float sig_s0, float alpha_t, float h_phi_1, float B_h, float rhos_c0,
                   float rhos_c1, float inv_rks0, int order_c, float* out, int n, cudaStream_t st) {
    if (!last || !mo0 || !conv || !out || n <= 0) { set_error("unipc_correct: bad args"); return false; }
    unipc_correct_kernel<<<nblocks(n), 256, 0, st>>>(last, mo0, mo_old, conv, sig_t, sig_s0, alpha_t,
                                                     h_phi_1, B_h, rhos_c0, rhos_c1, inv_rks0,
                                                     order_c, out, n);
    O1_LAUNCH_CHECK("unipc_correct");
    return true;
}
bool unipc_predict(const float* sample, const float* mo0, const float* mo_old, float sig_t,
                   float sig_s0, float alpha_t, float h_phi_1, float B_h, float rhos_p,
                   float inv_rks0, int order_p, float* out, int n, cudaStream_t st) {
    if (!sample || !mo0 || !out || n <= 0) { set_error("unipc_predict: bad args"); return false; }
    unipc_predict_kernel<<<nblocks(n), 256, 0, st>>>(sample, mo0, mo_old, sig_t, sig_s0, alpha_t,
                                                     h_phi_1, B_h, rhos_p, inv_rks0, order_p, out, n);
    O1_LAUNCH_CHECK("unipc_predict");
    return true;
}

}  // namespace o1
