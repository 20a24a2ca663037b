// HBM-bound pointwise / row-reduction kernels of the decoder path:
// RMSNorm, SiLU / SwiGLU, residual add, 3-axis interleaved MRoPE tables and
// rotary apply, fused per-head q/k RMSNorm + rotary, head split / merge,
// embedding gather + timestep-token substitution, timestep sinusoid,
// vision-row scatter / DeepStack add, seeded initialisers.
//
// All follow the arithmetic and bf16 rounding points of o1.c's
// src/cuda/{norm,act,residual,rope,attn,embed}.cu and gemm.cu:531-545; what
// changes is the memory access: 128-bit loads/stores, warp-shuffle
// reductions, and fewer passes over HBM.
#include "common.cuh"
#include "kernels.h"

namespace o1 {

#define O1_LAUNCH_CHECK(name)                                                        \
    do {                                                                             \
        cudaError_t e__ = cudaGetLastError();                                        \
        if (e__ != cudaSuccess) { set_error(name ": %s", cudaGetErrorString(e__)); return false; } \
    } while (0)

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    f[0] = bf16lo(v.x); f[1] = bf16hi(v.x); f[2] = bf16lo(v.y); f[3] = bf16hi(v.y);
    f[4] = bf16lo(v.z); f[5] = bf16hi(v.z); f[6] = bf16lo(v.w); f[7] = bf16hi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 v;
    v.x = pack_bf16x2(f[0], f[1]); v.y = pack_bf16x2(f[2], f[3]);
    v.z = pack_bf16x2(f[4], f[5]); v.w = pack_bf16x2(f[6], f[7]);
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ------------------------------------------------------------------ RMSNorm
// y = bf16( (w * x) * rsqrt(mean(x^2) + eps) ), fp32 inside (norm.cu:12-48).
// One row per block; each thread keeps its slice of the row in registers
// between the reduction and the scaling pass, so HBM sees one read + one write.
template <int THREADS, int VEC_PER_THREAD>
__global__ void __launch_bounds__(THREADS)
rmsnorm_vec_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w,
                   uint16_t* __restrict__ y, int rows, int cols, float eps,
                   const uint16_t* __restrict__ scale, const uint16_t* __restrict__ shift) {
    const int row = blockIdx.x;
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * cols);
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * cols);
    const uint4* wr = reinterpret_cast<const uint4*>(w);
    const int nvec = cols >> 3;
    uint4 xv[VEC_PER_THREAD];
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < VEC_PER_THREAD; ++i) {
        const int idx = threadIdx.x + i * THREADS;
        if (idx < nvec) {
            xv[i] = xr[idx];
            float f[8];
            unpack8(xv[i], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) sq += f[j] * f[j];
        }
    }
    __shared__ float red[THREADS / 32];
    __shared__ float inv_s;
    sq = warp_sum(sq);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = (threadIdx.x < THREADS / 32) ? red[threadIdx.x] : 0.f;
        t = warp_sum(t);
        if (threadIdx.x == 0) inv_s = rsqrtf(t / (float)cols + eps);
    }
    __syncthreads();
    const float inv = inv_s;
#pragma unroll
    for (int i = 0; i < VEC_PER_THREAD; ++i) {
        const int idx = threadIdx.x + i * THREADS;
        if (idx < nvec) {
            float f[8], g[8];
            unpack8(xv[i], f);
            unpack8(wr[idx], g);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = g[j] * f[j] * inv;
            if (scale) {   // adaLN variant: the stored norm output, then * (1 + scale) + shift (NULL = o1.c's block)
                float sc[8], sh[8];
                unpack8(reinterpret_cast<const uint4*>(scale)[idx], sc);
                unpack8(reinterpret_cast<const uint4*>(shift)[idx], sh);
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = bf16_round(f[j]) * (1.0f + sc[j]) + sh[j];
            }
            yr[idx] = pack8(f);
        }
    }
}

// Any shape (scalar), one warp per row. Used for odd sizes only.
__global__ void rmsnorm_generic_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w,
                                       uint16_t* __restrict__ y, int rows, int cols, float eps,
                                       const uint16_t* __restrict__ scale, const uint16_t* __restrict__ shift) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const uint16_t* xr = x + (size_t)row * cols;
    uint16_t* yr = y + (size_t)row * cols;
    float sq = 0.f;
    for (int i = lane; i < cols; i += 32) { float v = bf16_to_f32(xr[i]); sq += v * v; }
    sq = warp_sum(sq);
    const float inv = rsqrtf(sq / (float)cols + eps);
    for (int i = lane; i < cols; i += 32) {
        float v = bf16_to_f32(w[i]) * bf16_to_f32(xr[i]) * inv;
        if (scale) v = bf16_round(v) * (1.0f + bf16_to_f32(scale[i])) + bf16_to_f32(shift[i]);
        yr[i] = f32_to_bf16(v);
    }
}

bool rmsnorm(const void* x, const void* w, void* y, int rows, int cols, float eps, cudaStream_t st) {
    return rmsnorm_mod(x, w, nullptr, nullptr, y, rows, cols, eps, st);
}
// scale / shift [cols] bf16 or both NULL: y = bf16(bf16(rmsnorm(x)) * (1 + scale) + shift)
bool rmsnorm_mod(const void* x, const void* w, const void* scale, const void* shift, void* y, int rows, int cols,
                 float eps, cudaStream_t st) {
    if (!x || !w || !y || rows <= 0 || cols <= 0 || (!scale != !shift)) { set_error("rmsnorm: bad args"); return false; }
    const bool aligned = ((((uintptr_t)x) | ((uintptr_t)y) | ((uintptr_t)w) | ((uintptr_t)scale) | ((uintptr_t)shift)) & 15) == 0;
    const uint16_t *sc = (const uint16_t*)scale, *sh = (const uint16_t*)shift;
    if (aligned && (cols % 8) == 0 && cols <= 128 * 8 * 8 && cols > 1024) {
        rmsnorm_vec_kernel<128, 8><<<rows, 128, 0, st>>>((const uint16_t*)x, (const uint16_t*)w,
                                                         (uint16_t*)y, rows, cols, eps, sc, sh);
    } else if (aligned && (cols % 8) == 0 && cols <= 1024) {
        rmsnorm_vec_kernel<32, 4><<<rows, 32, 0, st>>>((const uint16_t*)x, (const uint16_t*)w,
                                                       (uint16_t*)y, rows, cols, eps, sc, sh);
    } else {
        const int wpb = 4;
        rmsnorm_generic_kernel<<<(rows + wpb - 1) / wpb, wpb * 32, 0, st>>>(
            (const uint16_t*)x, (const uint16_t*)w, (uint16_t*)y, rows, cols, eps, sc, sh);
    }
    O1_LAUNCH_CHECK("rmsnorm");
    return true;
}

// ------------------------------------------------------------------ materialising attention (small / odd shapes)
// The path of o1.c's hd_attention_eager (src/cuda/attn.cu:22-174) for what the flash kernel does not cover: a head
// dimension other than 128 or an additive mask that is not prefix-causal.  One block per (head, query row): scores
// s_t = (q . k_t) * scaling + mask[s,t] in fp32 (stored as bf16), fp32 softmax with the row maximum subtracted,
// probabilities rounded to bf16 (and stored), out = sum_t p_t v_t accumulated in fp32 over the ROUNDED
// probabilities, written seq-major [seq, heads, dim].  O(seq^2) memory and time: meant for tests and small inputs.
__global__ void __launch_bounds__(128)
attention_rows_kernel(const uint16_t* __restrict__ q, const uint16_t* __restrict__ k, const uint16_t* __restrict__ v,
                      const uint16_t* __restrict__ mask, uint16_t* __restrict__ scores, uint16_t* __restrict__ probs,
                      uint16_t* __restrict__ out, int heads, int kv_heads, int seq, int dim, float scaling) {
    const int s = blockIdx.x, h = blockIdx.y, kh = h / (heads / kv_heads);
    const uint16_t* qr = q + ((size_t)h * seq + s) * dim;
    uint16_t* sc = scores + ((size_t)h * seq + s) * seq;
    uint16_t* pr = probs + ((size_t)h * seq + s) * seq;
    __shared__ float red[128];
    float mx = -INFINITY;
    for (int t = threadIdx.x; t < seq; t += blockDim.x) {
        const uint16_t* kr = k + ((size_t)kh * seq + t) * dim;
        float acc = 0.f;
        for (int i = 0; i < dim; ++i) acc += bf16_to_f32(qr[i]) * bf16_to_f32(kr[i]);
        acc = acc * scaling + bf16_to_f32(mask[(size_t)s * seq + t]);
        sc[t] = f32_to_bf16(acc);
        mx = fmaxf(mx, acc);          // the fp32 score itself is recomputed in the passes below
    }
    red[threadIdx.x] = mx;
    __syncthreads();
    for (int o = 64; o > 0; o >>= 1) {
        if (threadIdx.x < o) red[threadIdx.x] = fmaxf(red[threadIdx.x], red[threadIdx.x + o]);
        __syncthreads();
    }
    mx = red[0];
    __syncthreads();
    float sum = 0.f;
    for (int t = threadIdx.x; t < seq; t += blockDim.x) {
        const uint16_t* kr = k + ((size_t)kh * seq + t) * dim;
        float acc = 0.f;
        for (int i = 0; i < dim; ++i) acc += bf16_to_f32(qr[i]) * bf16_to_f32(kr[i]);
        acc = acc * scaling + bf16_to_f32(mask[(size_t)s * seq + t]);
        sum += expf(acc - mx);
    }
    red[threadIdx.x] = sum;
    __syncthreads();
    for (int o = 64; o > 0; o >>= 1) {
        if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    const float inv = 1.0f / red[0];
    __syncthreads();
    for (int t = threadIdx.x; t < seq; t += blockDim.x) {
        const uint16_t* kr = k + ((size_t)kh * seq + t) * dim;
        float acc = 0.f;
        for (int i = 0; i < dim; ++i) acc += bf16_to_f32(qr[i]) * bf16_to_f32(kr[i]);
        acc = acc * scaling + bf16_to_f32(mask[(size_t)s * seq + t]);
        pr[t] = f32_to_bf16(expf(acc - mx) * inv);
    }
    __syncthreads();
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        float acc = 0.f;
        for (int t = 0; t < seq; ++t) acc += bf16_to_f32(pr[t]) * bf16_to_f32(v[((size_t)kh * seq + t) * dim + d]);
        out[((size_t)s * heads + h) * dim + d] = f32_to_bf16(acc);
    }
}
bool attention_materialised(const void* q, const void* k, const void* v, const void* mask, void* scores, void* probs,
                            void* out, int heads, int kv_heads, int seq, int dim, float scaling, cudaStream_t st) {
    if (!q || !k || !v || !mask || !scores || !probs || !out || heads <= 0 || kv_heads <= 0 || (heads % kv_heads) != 0 ||
        seq <= 0 || dim <= 0 || heads > 65535) {
        set_error("attention_eager: bad args");
        return false;
    }
    dim3 grid(seq, heads);
    attention_rows_kernel<<<grid, 128, 0, st>>>((const uint16_t*)q, (const uint16_t*)k, (const uint16_t*)v,
                                                (const uint16_t*)mask, (uint16_t*)scores, (uint16_t*)probs,
                                                (uint16_t*)out, heads, kv_heads, seq, dim, scaling);
    O1_LAUNCH_CHECK("attention_eager");
    return true;
}

// ------------------------------------------------------------------ pointwise
template <int OP>  // 0 silu, 1 swiglu, 2 residual add
__global__ void pointwise_kernel(const uint16_t* __restrict__ a, const uint16_t* __restrict__ b,
                                 uint16_t* __restrict__ y, size_t n) {
    const size_t nvec = n >> 3;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        float fa[8], fb[8];
        unpack8(reinterpret_cast<const uint4*>(a)[i], fa);
        if (OP != 0) unpack8(reinterpret_cast<const uint4*>(b)[i], fb);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (OP == 0) {
                fa[j] = fa[j] * (1.0f / (1.0f + expf(-fa[j])));
            } else if (OP == 1) {
                const float sg = 1.0f / (1.0f + expf(-fa[j]));
                fa[j] = bf16_round(fa[j] * sg) * fb[j];
            } else {
                fa[j] = fa[j] + fb[j];
            }
        }
        reinterpret_cast<uint4*>(y)[i] = pack8(fa);
    }
    // tail (n % 8 elements)
    if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {
        const size_t i = (nvec << 3) + threadIdx.x;
        const float x = bf16_to_f32(a[i]);
        float r;
        if (OP == 0) r = x * (1.0f / (1.0f + expf(-x)));
        else if (OP == 1) r = bf16_round(x * (1.0f / (1.0f + expf(-x)))) * bf16_to_f32(b[i]);
        else r = x + bf16_to_f32(b[i]);
        y[i] = f32_to_bf16(r);
    }
}
template <int OP>
__global__ void pointwise_scalar_kernel(const uint16_t* __restrict__ a, const uint16_t* __restrict__ b,
                                        uint16_t* __restrict__ y, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float x = bf16_to_f32(a[i]);
    float r;
    if (OP == 0) r = x * (1.0f / (1.0f + expf(-x)));
    else if (OP == 1) r = bf16_round(x * (1.0f / (1.0f + expf(-x)))) * bf16_to_f32(b[i]);
    else r = x + bf16_to_f32(b[i]);
    y[i] = f32_to_bf16(r);
}
template <int OP>
static bool pointwise(const void* a, const void* b, void* y, size_t n, cudaStream_t st) {
    if (n == 0) return true;
    uintptr_t al = (uintptr_t)a | (uintptr_t)y | (OP ? (uintptr_t)b : 0);
    if ((al & 15) == 0) {
        size_t nvec = n >> 3;
        size_t want = (nvec + 255) / 256;
        int blocks = (int)(want < (size_t)(sm_count() * 16) ? (want ? want : 1) : (size_t)(sm_count() * 16));
        pointwise_kernel<OP><<<blocks, 256, 0, st>>>((const uint16_t*)a, (const uint16_t*)b,
                                                     (uint16_t*)y, n);
    } else {
        pointwise_scalar_kernel<OP><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(
            (const uint16_t*)a, (const uint16_t*)b, (uint16_t*)y, n);
    }
    return true;
}
bool silu(const void* x, void* y, size_t n, cudaStream_t st) {
    if (!x || !y) { set_error("silu: bad args"); return false; }
    pointwise<0>(x, nullptr, y, n, st);
    O1_LAUNCH_CHECK("silu");
    return true;
}
bool swiglu(const void* g, const void* u, void* y, size_t n, cudaStream_t st) {
    if (!g || !u || !y) { set_error("swiglu: bad args"); return false; }
    pointwise<1>(g, u, y, n, st);
    O1_LAUNCH_CHECK("swiglu");
    return true;
}
bool residual_add(const void* x, const void* a, void* y, size_t n, cudaStream_t st) {
    if (!x || !a || !y) { set_error("residual_add: bad args"); return false; }
    pointwise<2>(x, a, y, n, st);
    O1_LAUNCH_CHECK("residual_add");
    return true;
}

// ------------------------------------------------------------------ MRoPE
// Frequency index kk in [0, dim/2). Interleaved 3-axis selection
// (rope.cu:43-57): axis H if kk%3==1, W if kk%3==2, both only while
// kk/3 < section[axis]; everything else uses T.
__device__ __forceinline__ int mrope_axis(int kk, const int64_t* section, int n_section,
                                          int interleaved) {
    if (interleaved) {
        const int chunk = kk / 3, slot = kk % 3;
        if ((slot == 1 || slot == 2) && slot <= n_section - 1 && chunk < (int)section[slot]) return slot;
        return 0;
    }
    int acc = 0;
    for (int t = 0; t < n_section && t < 3; ++t) {
        if (kk < acc + (int)section[t]) return t;
        acc += (int)section[t];
    }
    return 0;
}

__global__ void mrope_cos_sin_kernel(const float* __restrict__ pos, const int64_t* __restrict__ section,
                                     float* __restrict__ cosd, float* __restrict__ sind, int bs,
                                     int seq, int dim, float theta, float scaling, int n_section,
                                     int interleaved) {
    const int s = blockIdx.x;
    const int b = blockIdx.y;
    const int half = dim / 2;
    for (int k = threadIdx.x; k < dim; k += blockDim.x) {
        const int kk = (k < half) ? k : (k - half);
        const int axis = mrope_axis(kk, section, n_section, interleaved);
        const float p = pos[((size_t)axis) * bs * seq + (size_t)b * seq + s];
        const float base = expf(-logf(theta) * (2.0f * (float)kk) / (float)dim);
        const float ang = base * p;
        const size_t o = ((size_t)b * seq + s) * dim + k;
        cosd[o] = cosf(ang) * scaling;
        sind[o] = sinf(ang) * scaling;
    }
}
bool mrope_cos_sin(const float* pos, int bs, int seq, const int64_t* section, int n_section,
                   int head_dim, float theta, float scaling, int interleaved, float* cosd,
                   float* sind, cudaStream_t st) {
    if (!pos || !section || !cosd || !sind || seq <= 0 || head_dim <= 0 || bs <= 0) {
        set_error("mrope: bad args");
        return false;
    }
    dim3 grid(seq, bs);
    mrope_cos_sin_kernel<<<grid, 128, 0, st>>>(pos, section, cosd, sind, bs, seq, head_dim, theta,
                                               scaling, n_section, interleaved);
    O1_LAUNCH_CHECK("mrope");
    return true;
}

// Compact per-forward table for head_dim 128, section [24,20,20] interleaved,
// attention_scaling 1: cs[s][kk] = cos, cs[s][64+kk] = sin, kk in [0,64).
// Layer-invariant, so it is built once per forward instead of once per block.
__global__ void mrope_table64_kernel(const float* __restrict__ pos, float* __restrict__ cs, int seq,
                                     float theta, int pos_stride) {
    const int s = blockIdx.x * 4 + (threadIdx.x >> 6);
    const int kk = threadIdx.x & 63;
    if (s >= seq) return;
    const int chunk = kk / 3, slot = kk % 3;
    int axis = 0;
    if (slot == 1 && chunk < 20) axis = 1;
    if (slot == 2 && chunk < 20) axis = 2;
    const float p = pos[(size_t)axis * pos_stride + s];
    const float base = expf(-logf(theta) * (2.0f * (float)kk) / 128.0f);
    const float ang = base * p;
    cs[(size_t)s * 128 + kk] = cosf(ang) * 1.0f;
    cs[(size_t)s * 128 + 64 + kk] = sinf(ang) * 1.0f;
}
bool mrope_table64(const float* pos, int seq, float theta, float* cs, cudaStream_t st) {
    if (!pos || !cs || seq <= 0) { set_error("mrope_table: bad args"); return false; }
    mrope_table64_kernel<<<(seq + 3) / 4, 256, 0, st>>>(pos, cs, seq, theta, seq);
    O1_LAUNCH_CHECK("mrope_table");
    return true;
}
bool mrope_table64_rows(const float* pos, int pos_stride, int row0, int rows, float theta, float* cs,
                        cudaStream_t st) {
    if (!pos || !cs || rows <= 0 || row0 < 0 || row0 + rows > pos_stride) { set_error("mrope_table: bad args"); return false; }
    mrope_table64_kernel<<<(rows + 3) / 4, 256, 0, st>>>(pos + row0, cs, rows, theta, pos_stride);
    O1_LAUNCH_CHECK("mrope_table");
    return true;
}

// rotate-half on head-major [heads, seq, dim] (rope.cu:97-134). f32_mode = 0
// reproduces the three bf16 roundings of the text path; 1 is the vision
// variant (single rounding).
__global__ void apply_rotary_kernel(const uint16_t* __restrict__ x, const float* __restrict__ cosd,
                                    const float* __restrict__ sind, uint16_t* __restrict__ y,
                                    long total, int seq, int dim, int f32_mode) {
    const long e = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= total) return;
    const int d = (int)(e % dim);
    const long hs = e / dim;
    const int s = (int)(hs % seq);
    const int half = dim / 2;
    const long src_half = hs * dim + ((d < half) ? d + half : d - half);
    const float x0 = bf16_to_f32(x[e]);
    const float xh = bf16_to_f32(x[src_half]);
    const float c = cosd[(long)s * dim + d];
    const float sn = sind[(long)s * dim + d];
    float v;
    if (f32_mode) {
        v = (d < half) ? (x0 * c - xh * sn) : (x0 * c + xh * sn);
    } else {
        const float a = bf16_round(x0 * c);
        const float b = bf16_round(xh * sn);
        v = (d < half) ? (a - b) : (a + b);
    }
    y[e] = f32_to_bf16(v);
}
bool apply_rotary(const void* x, const float* cosd, const float* sind, void* y, int heads, int seq,
                  int dim, int f32_mode, cudaStream_t st) {
    if (!x || !cosd || !sind || !y || heads <= 0 || seq <= 0 || dim <= 0) {
        set_error("apply_rotary: bad args");
        return false;
    }
    const long total = (long)heads * seq * dim;
    apply_rotary_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        (const uint16_t*)x, cosd, sind, (uint16_t*)y, total, seq, dim, f32_mode);
    O1_LAUNCH_CHECK("apply_rotary");
    return true;
}

// Fused per-head RMSNorm (weights w[128]) + rotary, in place, seq-major
// [S, ld] with head h at columns [h*128, h*128+128).  8 threads per head:
// thread t owns elements [8t, 8t+8) and [64+8t, 64+8t+8), which are exactly
// the rotate-half partners, so the rotation needs no exchange.  Rounding
// points: normed value -> bf16 (norm.cu:45-46), then the three roundings of
// rope.cu:123-133.
__global__ void __launch_bounds__(256)
qk_norm_rope_kernel(uint16_t* __restrict__ x, int ld, int S, int heads, int hpb, long blk_stride,
                    const uint16_t* __restrict__ w, const float* __restrict__ cs, float eps) {
    // One warp per token: lanes = (head within a quad) x 8, so one load instruction of the warp covers the low
    // halves of four adjacent heads and the next one their high halves -- 1 KB of contiguous memory per quad, and
    // the warp streams through its token's row.  The token's cos|sin values and the norm weights are loaded once
    // and reused for every head (the table row is twice the size of a head).
    const int s = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (s >= S) return;                          // whole warp
    const int lane = threadIdx.x & 31;
    const int hq = lane >> 3, t = lane & 7;
    float wl[8], wh[8], cc[8], ss[8];
    {
        unpack8(*reinterpret_cast<const uint4*>(w + 8 * t), wl);
        unpack8(*reinterpret_cast<const uint4*>(w + 64 + 8 * t), wh);
        const float4* c4 = reinterpret_cast<const float4*>(cs + (size_t)s * 128 + 8 * t);
        const float4* s4 = reinterpret_cast<const float4*>(cs + (size_t)s * 128 + 64 + 8 * t);
        const float4 ca = c4[0], cb = c4[1], sa = s4[0], sb = s4[1];
        cc[0] = ca.x; cc[1] = ca.y; cc[2] = ca.z; cc[3] = ca.w; cc[4] = cb.x; cc[5] = cb.y; cc[6] = cb.z; cc[7] = cb.w;
        ss[0] = sa.x; ss[1] = sa.y; ss[2] = sa.z; ss[3] = sa.w; ss[4] = sb.x; ss[5] = sb.y; ss[6] = sb.z; ss[7] = sb.w;
    }
    // G quads (16 heads) per trip: all 2*G 16-byte loads of a thread are issued before the first value is used
    constexpr int G = 4;
    for (int h0 = 0; h0 < heads; h0 += 4 * G) {
        uint16_t* base[G];
        uint4 vlo[G], vhi[G];
        bool on[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const int h = h0 + 4 * g + hq;
            on[g] = h < heads;
            const int hc = on[g] ? h : 0;
            base[g] = x + (size_t)(hc / hpb) * blk_stride + (size_t)s * ld + (hc % hpb) * 128;
            vlo[g] = on[g] ? *reinterpret_cast<const uint4*>(base[g] + 8 * t) : make_uint4(0, 0, 0, 0);
            vhi[g] = on[g] ? *reinterpret_cast<const uint4*>(base[g] + 64 + 8 * t) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float lo[8], hi[8];
            float sq = 0.f;
            unpack8(vlo[g], lo);
            unpack8(vhi[g], hi);
            // explicit roundings: the fused GEMM epilogue (EPI_QKNORM) sums in exactly this order
#pragma unroll
            for (int j = 0; j < 8; ++j) sq = __fadd_rn(sq, __fmaf_rn(hi[j], hi[j], __fmul_rn(lo[j], lo[j])));
            sq += __shfl_xor_sync(0xffffffffu, sq, 1);
            sq += __shfl_xor_sync(0xffffffffu, sq, 2);
            sq += __shfl_xor_sync(0xffffffffu, sq, 4);
            if (!on[g]) continue;
            const float inv = rsqrtf(sq / 128.0f + eps);
            float ol[8], oh[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float a = bf16_round(wl[j] * lo[j] * inv);
                const float b = bf16_round(wh[j] * hi[j] * inv);
                ol[j] = bf16_round(a * cc[j]) - bf16_round(b * ss[j]);
                oh[j] = bf16_round(b * cc[j]) + bf16_round(a * ss[j]);
            }
            *reinterpret_cast<uint4*>(base[g] + 8 * t) = pack8(ol);
            *reinterpret_cast<uint4*>(base[g] + 64 + 8 * t) = pack8(oh);
        }
    }
}
bool qk_norm_rope(void* x, int ld, int S, int heads, const void* w, const float* cs_table, float eps,
                  cudaStream_t st) {
    if (!x || !w || !cs_table || S <= 0 || heads <= 0 || (ld % 8) != 0 || (((uintptr_t)x) & 15)) {
        set_error("qk_norm_rope: bad args");
        return false;
    }
    return qk_norm_rope_blocked(x, ld, S, heads, heads, 0, w, cs_table, eps, st);
}
bool qk_norm_rope_blocked(void* x, int ld, int S, int heads, int hpb, long blk_stride, const void* w,
                          const float* cs_table, float eps, cudaStream_t st) {
    if (!x || !w || !cs_table || S <= 0 || heads <= 0 || hpb <= 0 || (heads % hpb) != 0 || (ld % 8) != 0 ||
        (blk_stride % 8) != 0 || (((uintptr_t)x) & 15)) {
        set_error("qk_norm_rope: bad args");
        return false;
    }
    qk_norm_rope_kernel<<<(unsigned)((S + 7) / 8), 256, 0, st>>>(
        (uint16_t*)x, ld, S, heads, hpb, blk_stride, (const uint16_t*)w, cs_table, eps);
    O1_LAUNCH_CHECK("qk_norm_rope");
    return true;
}

// ------------------------------------------------------------------ head split / merge
// [seq, heads, dim] <-> [heads, seq, dim], 16-byte chunks (attn.cu:180-218).
__global__ void head_perm_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, int seq,
                                 int heads, int dchunks, int merge) {
    const long total = (long)seq * heads * dchunks;
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int c = (int)(i % dchunks);
    const long r = i / dchunks;
    if (!merge) {  // i indexes the input [s, h, c]
        const int h = (int)(r % heads);
        const long s = r / heads;
        out[((long)h * seq + s) * dchunks + c] = in[i];
    } else {       // i indexes the output [s, h, c]
        const int h = (int)(r % heads);
        const long s = r / heads;
        out[i] = in[((long)h * seq + s) * dchunks + c];
    }
}
__global__ void head_perm_scalar_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out,
                                        int seq, int heads, int dim, int merge) {
    const long total = (long)seq * heads * dim;
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int d = (int)(i % dim);
    const long r = i / dim;
    const int h = (int)(r % heads);
    const long s = r / heads;
    const long hm = ((long)h * seq + s) * dim + d;
    if (!merge) out[hm] = in[i]; else out[i] = in[hm];
}
static bool head_perm(const void* in, void* out, int seq, int heads, int dim, int merge,
                      cudaStream_t st) {
    if (!in || !out || seq <= 0 || heads <= 0 || dim <= 0) { set_error("head_split/merge: bad args"); return false; }
    if ((dim % 8) == 0 && ((((uintptr_t)in) | ((uintptr_t)out)) & 15) == 0) {
        const long total = (long)seq * heads * (dim / 8);
        head_perm_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
            (const uint4*)in, (uint4*)out, seq, heads, dim / 8, merge);
    } else {
        const long total = (long)seq * heads * dim;
        head_perm_scalar_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
            (const uint16_t*)in, (uint16_t*)out, seq, heads, dim, merge);
    }
    O1_LAUNCH_CHECK("head_split/merge");
    return true;
}
bool head_split(const void* in, void* out, int seq, int heads, int dim, cudaStream_t st) {
    return head_perm(in, out, seq, heads, dim, 0, st);
}
bool head_merge(const void* in, void* out, int seq, int heads, int dim, cudaStream_t st) {
    return head_perm(in, out, seq, heads, dim, 1, st);
}

// ------------------------------------------------------------------ embedding
// mode 0: gather rows (OOB id -> row 0)                 (embed.cu:15-29)
// mode 1: out[row] = id==tms ? t_emb : emb[row]         (embed.cu:44-58)
// mode 2: both in one pass
__global__ void embed_rows_kernel(const uint16_t* __restrict__ table, const int64_t* __restrict__ idx,
                                  const uint16_t* __restrict__ emb, const uint16_t* __restrict__ t_emb,
                                  uint16_t* __restrict__ out, int M, int cols, int64_t nrows,
                                  int64_t tms_id, int mode) {
    const int row = blockIdx.x;
    int64_t id = idx[row];
    const uint16_t* src;
    if (mode == 0) {
        if (id < 0 || id >= nrows) id = 0;
        src = table + id * cols;
    } else if (mode == 1) {
        src = (id == tms_id) ? t_emb : emb + (size_t)row * cols;
    } else {
        if (id == tms_id) src = t_emb;
        else { if (id < 0 || id >= nrows) id = 0; src = table + id * cols; }
    }
    uint16_t* dst = out + (size_t)row * cols;
    if ((cols % 8) == 0 && ((((uintptr_t)src) | ((uintptr_t)dst)) & 15) == 0) {
        for (int c = threadIdx.x; c < cols / 8; c += blockDim.x)
            reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
    } else {
        for (int c = threadIdx.x; c < cols; c += blockDim.x) dst[c] = src[c];
    }
}
bool gather_rows(const void* table, const void* idx, void* out, int M, int cols, int64_t nrows,
                 cudaStream_t st) {
    if (!table || !idx || !out || M <= 0 || cols <= 0) { set_error("gather_rows: bad args"); return false; }
    embed_rows_kernel<<<M, 128, 0, st>>>((const uint16_t*)table, (const int64_t*)idx, nullptr, nullptr,
                                         (uint16_t*)out, M, cols, nrows, 0, 0);
    O1_LAUNCH_CHECK("gather_rows");
    return true;
}
bool tms_condition(const void* idx, const void* emb, const void* t_emb, void* out, int M, int H,
                   int64_t tms_id, cudaStream_t st) {
    if (!idx || !emb || !t_emb || !out || M <= 0 || H <= 0) { set_error("tms_condition: bad args"); return false; }
    embed_rows_kernel<<<M, 128, 0, st>>>(nullptr, (const int64_t*)idx, (const uint16_t*)emb,
                                         (const uint16_t*)t_emb, (uint16_t*)out, M, H, 0, tms_id, 1);
    O1_LAUNCH_CHECK("tms_condition");
    return true;
}
bool embed_text(const void* table, const void* idx, const void* t_emb, void* out, int M, int H,
                int64_t nrows, int64_t tms_id, cudaStream_t st) {
    if (!table || !idx || !t_emb || !out || M <= 0 || H <= 0) { set_error("embed_text: bad args"); return false; }
    embed_rows_kernel<<<M, 128, 0, st>>>((const uint16_t*)table, (const int64_t*)idx, nullptr,
                                         (const uint16_t*)t_emb, (uint16_t*)out, M, H, nrows, tms_id, 2);
    O1_LAUNCH_CHECK("embed_text");
    return true;
}

__global__ void scale_f32_kernel(const float* in, float* out, float s, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = in[i] * s;
}
bool scale_f32(const float* in, float* out, float s, int n, cudaStream_t st) {
    if (!in || !out || n <= 0) { set_error("scale_f32: bad args"); return false; }
    scale_f32_kernel<<<(n + 255) / 256, 256, 0, st>>>(in, out, s, n);
    O1_LAUNCH_CHECK("scale_f32");
    return true;
}
__global__ void f32_to_bf16_kernel(const float* in, uint16_t* out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = f32_to_bf16(in[i]);
}
bool f32_to_bf16_buf(const float* in, void* out, int n, cudaStream_t st) {
    if (!in || !out || n <= 0) { set_error("f32_convert_bf16: bad args"); return false; }
    f32_to_bf16_kernel<<<(n + 255) / 256, 256, 0, st>>>(in, (uint16_t*)out, n);
    O1_LAUNCH_CHECK("f32_convert_bf16");
    return true;
}
// [cos(t f_p) | sin(t f_p)], f_p = exp(-ln(1e4) p / half)   (gemm.cu:531-545)
__global__ void timestep_embed_kernel(const float* __restrict__ t, float* __restrict__ y, int N, int dim) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= N * dim) return;
    const int n = idx / dim, d = idx % dim, half = dim / 2;
    const int p = d < half ? d : d - half;
    const float freq = expf(-logf(10000.0f) * (float)p / (float)half);
    const float arg = t[n] * freq;
    float v = (d < half) ? cosf(arg) : sinf(arg);
    if ((dim % 2) && d == dim - 1) v = 0.0f;
    y[idx] = v;
}
bool timestep_embed(const float* t, float* y, int N, int dim, cudaStream_t st) {
    if (!t || !y || N <= 0 || dim <= 0) { set_error("timestep_embed: bad args"); return false; }
    timestep_embed_kernel<<<(N * dim + 255) / 256, 256, 0, st>>>(t, y, N, dim);
    O1_LAUNCH_CHECK("timestep_embed");
    return true;
}

// ------------------------------------------------------------------ vision rows
// k-th set mask row receives row k of `embeds` (scatter) or has row k of
// `ds` added (DeepStack); other rows are copied (vision_kernels.cu:344-401).
// The rank of a row is the count of set mask bytes before it, taken by one
// warp with a strided sum instead of a serial loop in every thread.
__global__ void vision_rows_kernel(const uint16_t* __restrict__ in, const uint8_t* __restrict__ mask,
                                   const uint16_t* __restrict__ src, uint16_t* __restrict__ out,
                                   int rows, int H, int add) {
    // prefix count of mask[0..row) by one warp, then the row op
    const int row = blockIdx.x;
    __shared__ int rank_s;
    if (threadIdx.x < 32) {
        int cnt = 0;
        for (int i = threadIdx.x; i < row; i += 32) cnt += mask[i] ? 1 : 0;
        cnt = (int)warp_sum((float)cnt);
        if (threadIdx.x == 0) rank_s = cnt;
    }
    __syncthreads();
    const bool m = mask[row] != 0;
    const uint16_t* a = in + (size_t)row * H;
    const uint16_t* b = src + (size_t)rank_s * H;
    uint16_t* o = out + (size_t)row * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        uint16_t v = a[c];
        if (m) v = add ? f32_to_bf16(bf16_to_f32(v) + bf16_to_f32(b[c])) : b[c];
        o[c] = v;
    }
}
bool masked_scatter(const void* h_text, const uint8_t* mask, const void* embeds, void* out, int T,
                    int H, cudaStream_t st) {
    if (!h_text || !mask || !embeds || !out || T <= 0 || H <= 0) { set_error("masked_scatter: bad args"); return false; }
    vision_rows_kernel<<<T, 256, 0, st>>>((const uint16_t*)h_text, mask, (const uint16_t*)embeds,
                                          (uint16_t*)out, T, H, 0);
    O1_LAUNCH_CHECK("masked_scatter");
    return true;
}
bool deepstack_inject(const void* in, const uint8_t* mask, const void* ds, void* out, int S, int H,
                      cudaStream_t st) {
    if (!in || !mask || !ds || !out || S <= 0 || H <= 0) { set_error("deepstack_inject: bad args"); return false; }
    vision_rows_kernel<<<S, 256, 0, st>>>((const uint16_t*)in, mask, (const uint16_t*)ds,
                                          (uint16_t*)out, S, H, 1);
    O1_LAUNCH_CHECK("deepstack_inject");
    return true;
}

// ------------------------------------------------------------------ seeded init
// Counter-based generator shared bit-for-bit with the CPU oracle: two
// splitmix64 hashes of (seed, index) give eight 16-bit uniforms whose sum is
// an Irwin-Hall(8) variate; centred and scaled it has unit variance.  Only
// integer arithmetic plus one exact int->float conversion and two IEEE
// multiplies/adds, so host and device agree exactly.
__host__ __device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
__host__ __device__ __forceinline__ float hash_normal(uint64_t seed, uint64_t i) {
    const uint64_t a = splitmix64(seed ^ (i * 2 + 0) * 0xD1B54A32D192ED03ull);
    const uint64_t b = splitmix64(seed ^ (i * 2 + 1) * 0xD1B54A32D192ED03ull);
    int sum = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        sum += (int)((a >> (16 * k)) & 0xFFFF);
        sum += (int)((b >> (16 * k)) & 0xFFFF);
    }
    // mean 8*32767.5 = 262140, variance 8*(65536^2-1)/12
    return ((float)(sum - 262140)) * (1.0f / 53509.9f);
}
__global__ void fill_normal_kernel(uint16_t* dst16, float* dst32, size_t n, uint64_t seed, float mean,
                                   float std) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float v = __fadd_rn(mean, __fmul_rn(std, hash_normal(seed, i)));
        if (dst16) dst16[i] = f32_to_bf16(v); else dst32[i] = v;
    }
}
bool fill_normal_bf16(void* dst, size_t n, uint64_t seed, float mean, float std, cudaStream_t st) {
    if (!dst) { set_error("fill_normal: bad args"); return false; }
    if (n == 0) return true;
    size_t want = (n + 255) / 256;
    int blocks = (int)(want < (size_t)(sm_count() * 32) ? want : (size_t)(sm_count() * 32));
    fill_normal_kernel<<<blocks, 256, 0, st>>>((uint16_t*)dst, nullptr, n, seed, mean, std);
    O1_LAUNCH_CHECK("fill_normal");
    return true;
}
bool fill_normal_f32(float* dst, size_t n, uint64_t seed, float mean, float std, cudaStream_t st) {
    if (!dst) { set_error("fill_normal: bad args"); return false; }
    if (n == 0) return true;
    size_t want = (n + 255) / 256;
    int blocks = (int)(want < (size_t)(sm_count() * 32) ? want : (size_t)(sm_count() * 32));
    fill_normal_kernel<<<blocks, 256, 0, st>>>(nullptr, dst, n, seed, mean, std);
    O1_LAUNCH_CHECK("fill_normal");
    return true;
}

// out[c, r] = in[r, c]  (small matrices: LoRA down-projection transpose)
__global__ void transpose_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out, int rows,
                                 int cols) {
    __shared__ uint16_t tile[32][33];
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int r = r0 + j, c = c0 + threadIdx.x;
        if (r < rows && c < cols) tile[j][threadIdx.x] = in[(size_t)r * cols + c];
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int c = c0 + j, r = r0 + threadIdx.x;
        if (r < rows && c < cols) out[(size_t)c * rows + r] = tile[threadIdx.x][j];
    }
}
bool transpose_bf16(const void* in, void* out, int rows, int cols, cudaStream_t st) {
    if (!in || !out || rows <= 0 || cols <= 0) { set_error("transpose: bad args"); return false; }
    dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
    transpose_kernel<<<grid, block, 0, st>>>((const uint16_t*)in, (uint16_t*)out, rows, cols);
    O1_LAUNCH_CHECK("transpose");
    return true;
}

}  // namespace o1

extern "C" float o1_hash_normal_host(uint64_t seed, uint64_t index) { return o1::hash_normal(seed, index); }
