// Qwen3-VL vision tower of the edit / reference-image modes: the producer of the `image_embeds` and
// DeepStack tensors that hd_forward scatters into the <image_pad> rows.  Same entry points, structs and
// results as o1.c's src/model/vision.c:98-650 and src/cuda/vision_kernels.cu:14-340, re-composed for the
// tensor-core kernels of this library:
//
//   patch_embed            hd_linear-style GEMM + bias (K = 1536)
//   + interpolated pos     one kernel: 4-corner gather, bf16 round, add            (vision.c:436-439)
//   rotary table           one kernel: bf16(inv_freq * coord) -> cos|sin [n,72]     (vision.c:444-446)
//   27 x block             LayerNorm -> qkv GEMM+bias -> split + fp32 rotary into 128-wide zero-padded heads
//                          -> flash attention (head_dim 72 runs as 128: the pad columns add 0 to every
//                          score and produce 0 output columns) -> compact -> proj GEMM+bias+residual
//                          -> LayerNorm -> fc1 GEMM+bias+GELU(tanh) (N = 4304, ragged tile edge)
//                          -> fc2 GEMM+bias+residual (K = 4304, ragged last K block)
//   DeepStack mergers      after blocks 8 / 16 / 24: LayerNorm over 4608 -> GEMM+bias+GELU(erf) -> GEMM+bias
//   final merger           LayerNorm over 1152 -> view [n/4, 4608] -> GEMM+bias+GELU(erf) -> GEMM+bias
//
// No S x S score, probability or mask buffer exists (the reference workspace holds 2*16*n*n + n*n bf16
// elements for them); the workspace is O(n).  Nothing allocates or synchronises inside the forward.
#include "common.cuh"
#include "kernels.h"
#include "../../include/o1_b200.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

namespace o1 {

#define O1_VLAUNCH_CHECK(name)                                                       \
    do {                                                                             \
        cudaError_t e__ = cudaGetLastError();                                        \
        if (e__ != cudaSuccess) { set_error(name ": %s", cudaGetErrorString(e__)); return false; } \
    } while (0)

static constexpr int V_DEPTH = 27, V_H = 1152, V_HEADS = 16, V_D = 72, V_I = 4304, V_OUT = 4096;
static constexpr int V_PATCH = 1536, V_NPOS_SIDE = 48, V_MERGED = 4608, V_DP = 128 /* padded head */;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// LayerNorm over the last dimension, bf16 in / out, fp32 statistics as vision_kernels.cu:50-87:
// mean = sum/cols, var = sum(x^2)/cols - mean^2, y = bf16((x - mean) * rsqrt(var + eps) * w + b).
// One warp per row (rows are 2.3 - 9 KB: shuffles only, no block barrier); the second pass re-reads the row
// from L1.  cols % 8 == 0 takes 128-bit accesses.
static constexpr int LN_WARPS = 4;
__global__ void __launch_bounds__(LN_WARPS * 32)
layernorm_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w, const uint16_t* __restrict__ b,
                 uint16_t* __restrict__ y, int rows, int cols, float eps, int vec) {
    const int row = blockIdx.x * LN_WARPS + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const uint16_t* xr = x + (size_t)row * cols;
    uint16_t* yr = y + (size_t)row * cols;
    float s = 0.f, ss = 0.f;
    if (vec) {
        for (int i = lane * 8; i < cols; i += 256) {
            const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
            const float f[8] = {bf16lo(v.x), bf16hi(v.x), bf16lo(v.y), bf16hi(v.y),
                                bf16lo(v.z), bf16hi(v.z), bf16lo(v.w), bf16hi(v.w)};
#pragma unroll
            for (int j = 0; j < 8; ++j) { s += f[j]; ss += f[j] * f[j]; }
        }
    } else {
        for (int i = lane; i < cols; i += 32) { const float f = bf16_to_f32(xr[i]); s += f; ss += f * f; }
    }
    s = warp_sum(s);
    ss = warp_sum(ss);
    const float inv = 1.0f / (float)cols;
    const float mean = s * inv;
    const float var = ss * inv - mean * mean;
    const float inv_std = rsqrtf(var + eps);
    if (vec) {
        for (int i = lane * 8; i < cols; i += 256) {
            const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
            const uint4 wv = *reinterpret_cast<const uint4*>(w + i);
            uint4 bv = make_uint4(0, 0, 0, 0);
            if (b) bv = *reinterpret_cast<const uint4*>(b + i);
            const float f[8] = {bf16lo(v.x), bf16hi(v.x), bf16lo(v.y), bf16hi(v.y),
                                bf16lo(v.z), bf16hi(v.z), bf16lo(v.w), bf16hi(v.w)};
            const float g[8] = {bf16lo(wv.x), bf16hi(wv.x), bf16lo(wv.y), bf16hi(wv.y),
                                bf16lo(wv.z), bf16hi(wv.z), bf16lo(wv.w), bf16hi(wv.w)};
            const float c[8] = {bf16lo(bv.x), bf16hi(bv.x), bf16lo(bv.y), bf16hi(bv.y),
                                bf16lo(bv.z), bf16hi(bv.z), bf16lo(bv.w), bf16hi(bv.w)};
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = (f[j] - mean) * inv_std * g[j] + c[j];
            uint4 ov;
            ov.x = pack_bf16x2(o[0], o[1]); ov.y = pack_bf16x2(o[2], o[3]);
            ov.z = pack_bf16x2(o[4], o[5]); ov.w = pack_bf16x2(o[6], o[7]);
            *reinterpret_cast<uint4*>(yr + i) = ov;
        }
    } else {
        for (int i = lane; i < cols; i += 32) {
            const float f = (bf16_to_f32(xr[i]) - mean) * inv_std;
            yr[i] = f32_to_bf16(f * bf16_to_f32(w[i]) + (b ? bf16_to_f32(b[i]) : 0.0f));
        }
    }
}

// The same arithmetic with the row held in registers (rows of at most NV * 256 elements: the tower's 1152 and
// the mergers' 4608): every element is read from memory once, all NV loads of a lane are in flight together, and
// the sums run over the lane's elements in the same order as in layernorm_kernel, so the two agree bit for bit.
template <int NV>
__global__ void __launch_bounds__(LN_WARPS * 32)
layernorm_reg_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w, const uint16_t* __restrict__ b,
                     uint16_t* __restrict__ y, int rows, int cols, float eps) {
    const int row = blockIdx.x * LN_WARPS + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const uint16_t* xr = x + (size_t)row * cols;
    uint16_t* yr = y + (size_t)row * cols;
    uint4 v[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = lane * 8 + k * 256;
        v[k] = i < cols ? *reinterpret_cast<const uint4*>(xr + i) : make_uint4(0, 0, 0, 0);
    }
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        if (lane * 8 + k * 256 < cols) {
            const float f[8] = {bf16lo(v[k].x), bf16hi(v[k].x), bf16lo(v[k].y), bf16hi(v[k].y),
                                bf16lo(v[k].z), bf16hi(v[k].z), bf16lo(v[k].w), bf16hi(v[k].w)};
#pragma unroll
            for (int j = 0; j < 8; ++j) { s += f[j]; ss += f[j] * f[j]; }
        }
    }
    s = warp_sum(s);
    ss = warp_sum(ss);
    const float inv = 1.0f / (float)cols;
    const float mean = s * inv;
    const float var = ss * inv - mean * mean;
    const float inv_std = rsqrtf(var + eps);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = lane * 8 + k * 256;
        if (i < cols) {
            const uint4 wv = *reinterpret_cast<const uint4*>(w + i);
            uint4 bv = make_uint4(0, 0, 0, 0);
            if (b) bv = *reinterpret_cast<const uint4*>(b + i);
            const float f[8] = {bf16lo(v[k].x), bf16hi(v[k].x), bf16lo(v[k].y), bf16hi(v[k].y),
                                bf16lo(v[k].z), bf16hi(v[k].z), bf16lo(v[k].w), bf16hi(v[k].w)};
            const float g[8] = {bf16lo(wv.x), bf16hi(wv.x), bf16lo(wv.y), bf16hi(wv.y),
                                bf16lo(wv.z), bf16hi(wv.z), bf16lo(wv.w), bf16hi(wv.w)};
            const float c[8] = {bf16lo(bv.x), bf16hi(bv.x), bf16lo(bv.y), bf16hi(bv.y),
                                bf16lo(bv.z), bf16hi(bv.z), bf16lo(bv.w), bf16hi(bv.w)};
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = (f[j] - mean) * inv_std * g[j] + c[j];
            uint4 ov;
            ov.x = pack_bf16x2(o[0], o[1]); ov.y = pack_bf16x2(o[2], o[3]);
            ov.z = pack_bf16x2(o[4], o[5]); ov.w = pack_bf16x2(o[6], o[7]);
            *reinterpret_cast<uint4*>(yr + i) = ov;
        }
    }
}

bool vision_layernorm(const void* x, const void* w, const void* b, void* y, int rows, int cols, float eps,
                      cudaStream_t st) {
    if (!x || !w || !y || rows <= 0 || cols <= 0) { set_error("vision_layernorm: bad args"); return false; }
    const int vec = (cols % 8) == 0 && ((((uintptr_t)x) | ((uintptr_t)w) | ((uintptr_t)b) | ((uintptr_t)y)) & 15) == 0;
    const int grid = (rows + LN_WARPS - 1) / LN_WARPS;
    if (vec && cols <= 5 * 256) {
        layernorm_reg_kernel<5><<<grid, LN_WARPS * 32, 0, st>>>((const uint16_t*)x, (const uint16_t*)w, (const uint16_t*)b,
                                                               (uint16_t*)y, rows, cols, eps);
        O1_VLAUNCH_CHECK("vision_layernorm");
        return true;
    }
    if (vec && cols <= 18 * 256) {
        layernorm_reg_kernel<18><<<grid, LN_WARPS * 32, 0, st>>>((const uint16_t*)x, (const uint16_t*)w, (const uint16_t*)b,
                                                                (uint16_t*)y, rows, cols, eps);
        O1_VLAUNCH_CHECK("vision_layernorm");
        return true;
    }
    layernorm_kernel<<<(rows + LN_WARPS - 1) / LN_WARPS, LN_WARPS * 32, 0, st>>>(
        (const uint16_t*)x, (const uint16_t*)w, (const uint16_t*)b, (uint16_t*)y, rows, cols, eps, vec);
    O1_VLAUNCH_CHECK("vision_layernorm");
    return true;
}

// GELU, tanh form (block MLP) or erf form (mergers): vision_kernels.cu:100-133
__global__ void gelu_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ y, size_t n, int exact) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = bf16_to_f32(x[i]);
    float r;
    if (exact) {
        r = 0.5f * v * (1.0f + erff(v * 0.7071067811865476f));
    } else {
        const float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
        r = 0.5f * v * (1.0f + tanhf(u));
    }
    y[i] = f32_to_bf16(r);
}
bool vision_gelu(const void* x, void* y, size_t n, int exact, cudaStream_t st) {
    if (!x || !y || n == 0) { set_error("vision_gelu: bad args"); return false; }
    gelu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>((const uint16_t*)x, (uint16_t*)y, n, exact);
    O1_VLAUNCH_CHECK("vision_gelu");
    return true;
}

// Interpolated position embedding (vision_kernels.cu:148-168): row r of the output is the weighted sum of four
// rows of the [2304, hidden] table, rounded to bf16.  With `add` the patch embedding is added on top
// (vision.c:439: bf16(patch + pos)) in the same pass.
__global__ void pos_interp_kernel(const uint16_t* __restrict__ pe, const int* __restrict__ idx,
                                  const float* __restrict__ wgt, const uint16_t* __restrict__ add,
                                  uint16_t* __restrict__ y, int n, int hidden) {
    const int row = blockIdx.x;
    int i4[4];
    float w4[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) { i4[k] = idx[(size_t)k * n + row]; w4[k] = wgt[(size_t)k * n + row]; }
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float acc = 0.0f;
#pragma unroll
        for (int k = 0; k < 4; ++k) acc += w4[k] * bf16_to_f32(pe[(size_t)i4[k] * hidden + c]);
        float v = bf16_round(acc);
        if (add) v = bf16_to_f32(add[(size_t)row * hidden + c]) + v;
        y[(size_t)row * hidden + c] = f32_to_bf16(v);
    }
}
bool vision_pos_interp(const void* pe, const int* idx, const float* wgt, const void* add, void* y, int n,
                       int hidden, cudaStream_t st) {
    if (!pe || !idx || !wgt || !y || n <= 0 || hidden <= 0) { set_error("vision_pos_interp: bad args"); return false; }
    pos_interp_kernel<<<n, 256, 0, st>>>((const uint16_t*)pe, idx, wgt, (const uint16_t*)add, (uint16_t*)y, n, hidden);
    O1_VLAUNCH_CHECK("vision_pos_interp");
    return true;
}

// Rotary angles (vision_kernels.cu:183-231): rot[r, k] = bf16(inv_freq[k] * row(r)), rot[r, half + k] =
// bf16(inv_freq[k] * col(r)); cos / sin of [rot | rot] in fp32, [n, 4*half].  rot_out (optional) keeps the bf16
// angles, cosd / sind (optional) the tables.
__global__ void rot_table_kernel(const float* __restrict__ inv_freq, const int* __restrict__ coords,
                                 uint16_t* __restrict__ rot_out, float* __restrict__ cosd, float* __restrict__ sind,
                                 int n, int half) {
    const int row = blockIdx.x;
    const int r = coords[row], c = coords[n + row];
    const int rd = 2 * half;
    for (int k = threadIdx.x; k < rd; k += blockDim.x) {
        const float f = inv_freq[k < half ? k : k - half];
        const uint16_t a16 = f32_to_bf16(f * (float)(k < half ? r : c));
        if (rot_out) rot_out[(size_t)row * rd + k] = a16;
        if (cosd) {
            const float a = bf16_to_f32(a16);
            const float cs = cosf(a), sn = sinf(a);
            cosd[(size_t)row * 2 * rd + k] = cs; cosd[(size_t)row * 2 * rd + rd + k] = cs;
            sind[(size_t)row * 2 * rd + k] = sn; sind[(size_t)row * 2 * rd + rd + k] = sn;
        }
    }
}
__global__ void rot_cos_sin_kernel(const uint16_t* __restrict__ rot, float* __restrict__ cosd,
                                   float* __restrict__ sind, int rd) {
    const int row = blockIdx.x;
    for (int k = threadIdx.x; k < rd; k += blockDim.x) {
        const float a = bf16_to_f32(rot[(size_t)row * rd + k]);
        const float cs = cosf(a), sn = sinf(a);
        cosd[(size_t)row * 2 * rd + k] = cs; cosd[(size_t)row * 2 * rd + rd + k] = cs;
        sind[(size_t)row * 2 * rd + k] = sn; sind[(size_t)row * 2 * rd + rd + k] = sn;
    }
}
bool vision_rot_table(const float* inv_freq, const int* coords, void* rot_out, float* cosd, float* sind, int n,
                      int half, cudaStream_t st) {
    if (!inv_freq || !coords || n <= 0 || half <= 0 || (!rot_out && !cosd) || (!cosd != !sind)) {
        set_error("vision_rot: bad args");
        return false;
    }
    rot_table_kernel<<<n, 64, 0, st>>>(inv_freq, coords, (uint16_t*)rot_out, cosd, sind, n, half);
    O1_VLAUNCH_CHECK("vision_rot");
    return true;
}
bool vision_rot_cos_sin(const void* rot, float* cosd, float* sind, int n, int half, cudaStream_t st) {
    if (!rot || !cosd || !sind || n <= 0 || half <= 0) { set_error("vision_rot_cos_sin: bad args"); return false; }
    rot_cos_sin_kernel<<<n, 64, 0, st>>>((const uint16_t*)rot, cosd, sind, 2 * half);
    O1_VLAUNCH_CHECK("vision_rot_cos_sin");
    return true;
}

// Layout kernels of the reference's stand-alone entry points (vision_kernels.cu:246-340): pure index maps.
//   mode 0: qkv [n, 3*H*D] -> q / k / v [H, n, D]          (qkv_split)
//   mode 1: [H, n, D] -> [n, H*D]                          (attn_merge)
__global__ void vision_perm_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ o0,
                                   uint16_t* __restrict__ o1p, uint16_t* __restrict__ o2, int n, int heads, int d,
                                   int mode) {
    const long total = (long)n * heads * d;
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int dd = (int)(i % d);
    const long sh = i / d;
    const int s = (int)(sh % n), h = (int)(sh / n);
    const long hm = ((long)h * n + s) * d + dd;
    if (mode == 0) {
        const long base = (long)s * 3 * heads * d + (long)h * d + dd;
        o0[hm] = in[base];
        o1p[hm] = in[base + (long)heads * d];
        o2[hm] = in[base + 2l * heads * d];
    } else {
        o0[((long)s * heads + h) * d + dd] = in[hm];
    }
}
bool vision_qkv_split(const void* qkv, void* q, void* k, void* v, int n, int heads, int d, cudaStream_t st) {
    if (!qkv || !q || !k || !v || n <= 0 || heads <= 0 || d <= 0) { set_error("vision_qkv_split: bad args"); return false; }
    const long total = (long)n * heads * d;
    vision_perm_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const uint16_t*)qkv, (uint16_t*)q, (uint16_t*)k,
                                                                       (uint16_t*)v, n, heads, d, 0);
    O1_VLAUNCH_CHECK("vision_qkv_split");
    return true;
}
bool vision_attn_merge(const void* hm, void* sm, int heads, int n, int d, cudaStream_t st) {
    if (!hm || !sm || n <= 0 || heads <= 0 || d <= 0) { set_error("vision_attn_merge: bad args"); return false; }
    const long total = (long)n * heads * d;
    vision_perm_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const uint16_t*)hm, (uint16_t*)sm, nullptr,
                                                                       nullptr, n, heads, d, 1);
    O1_VLAUNCH_CHECK("vision_attn_merge");
    return true;
}
// 2x2 unshuffle of a row-major [gh*gw, hidden] grid into [gh/2*gw/2, 4*hidden] (vision_kernels.cu:246-267)
__global__ void spatial_merge_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out, int gw, int hidden) {
    const int orow = blockIdx.x, mw = gw / 2;
    const int oh = orow / mw, ow = orow % mw;
    for (int c = threadIdx.x; c < 4 * hidden; c += blockDim.x) {
        const int slot = c / hidden, cc = c - slot * hidden;
        const int irow = (2 * oh + (slot >> 1)) * gw + 2 * ow + (slot & 1);
        out[(size_t)orow * 4 * hidden + c] = in[(size_t)irow * hidden + cc];
    }
}
bool vision_spatial_merge(const void* in, void* out, int gh, int gw, int hidden, cudaStream_t st) {
    if (!in || !out || gh <= 0 || gw <= 0 || hidden <= 0 || (gh % 2) || (gw % 2)) {
        set_error("vision_spatial_merge: bad args");
        return false;
    }
    spatial_merge_kernel<<<(gh / 2) * (gw / 2), 256, 0, st>>>((const uint16_t*)in, (uint16_t*)out, gw, hidden);
    O1_VLAUNCH_CHECK("vision_spatial_merge");
    return true;
}

// What the block loop uses instead of split + two rotary passes: one pass from qkv [n, 3*16*72] to
// q | k | v [n, 3*16*128] with every head zero-padded to 128 columns, q and k rotated in fp32 with a single
// bf16 rounding (hd_apply_rotary_f32, src/cuda/rope.cu:155-178: out = x*cos -+ x_partner*sin).
// One thread per (token, which, head, 8-column group of the padded head).
__global__ void split_rope_pad_kernel(const uint16_t* __restrict__ qkv, const float* __restrict__ cosd,
                                      const float* __restrict__ sind, uint16_t* __restrict__ out, int n) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const long total = (long)n * 3 * V_HEADS * (V_DP / 8);
    if (i >= total) return;
    const int g = (int)(i % (V_DP / 8));
    long r = i / (V_DP / 8);
    const int h = (int)(r % V_HEADS); r /= V_HEADS;
    const int which = (int)(r % 3);
    const int s = (int)(r / 3);
    uint4 o = make_uint4(0, 0, 0, 0);
    if (g * 8 < V_D) {
        const uint16_t* src = qkv + (size_t)s * 3 * V_H + (size_t)which * V_H + (size_t)h * V_D;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int d = g * 8 + j;
            const float x0 = bf16_to_f32(src[d]);
            if (which == 2) { v[j] = x0; continue; }
            const int half = V_D / 2;
            const float xh = bf16_to_f32(src[d < half ? d + half : d - half]);
            const float c = cosd[(size_t)s * V_D + d], sn = sind[(size_t)s * V_D + d];
            v[j] = (d < half) ? (x0 * c - xh * sn) : (x0 * c + xh * sn);
        }
        o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
        o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
    }
    *reinterpret_cast<uint4*>(out + (size_t)s * 3 * V_HEADS * V_DP + (size_t)which * V_HEADS * V_DP + (size_t)h * V_DP + g * 8) = o;
}
// attention output [n, 16*128] (padded heads) -> [n, 16*72]
__global__ void unpad_heads_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out, int n) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const long total = (long)n * V_HEADS * (V_D / 8);
    if (i >= total) return;
    const int g = (int)(i % (V_D / 8));
    const long r = i / (V_D / 8);
    const int h = (int)(r % V_HEADS);
    const long s = r / V_HEADS;
    *reinterpret_cast<uint4*>(out + (size_t)s * V_H + h * V_D + g * 8) =
        *reinterpret_cast<const uint4*>(in + (size_t)s * V_HEADS * V_DP + h * V_DP + g * 8);
}

// GEMM + bias (+ GELU) on the tensor-core kernel where its tiles apply, otherwise the SIMT GEMM and a GELU pass
static bool linear_act(const void* x, const void* w, const void* b, void* y, int M, int N, int K, int act /*0 none, 1 tanh, 2 erf*/,
                       cudaStream_t st, int* launches) {
    if (act && gemm_tc_supported(M, N, K, EPI_BIAS_GELU)) {
        ++*launches;
        return gemm_bf16(x, w, nullptr, y, M, N, K, EPI_BIAS_GELU, b, nullptr, act == 2 ? 1.0f : 0.0f, 0, st);
    }
    if (!gemm_bf16(x, w, nullptr, y, M, N, K, EPI_BIAS, b, nullptr, 0.f, 0, st)) return false;
    ++*launches;
    if (act) { if (!vision_gelu(y, y, (size_t)M * N, act == 2, st)) return false; ++*launches; }
    return true;
}

static inline int64_t up256(int64_t v) { return (v + 255) & ~(int64_t)255; }

}  // namespace o1

using namespace o1;

extern "C" {

// ------------------------------------------------------------ stand-alone kernels (vision_kernels.h:17-45)
void hd_vision_patch(const void* x, const void* w, const void* bias, void* y, int n, int in_dim, int out_dim) {
    if (!x || !w || !y || n <= 0 || in_dim <= 0 || out_dim <= 0) { set_error("vision_patch: bad args"); return; }
    // Conv3d over the patchified input = a linear layer (the reference's HD_VISION_PATCH_GEMM form)
    if (gemm_bf16(x, w, nullptr, y, n, out_dim, in_dim, bias ? EPI_BIAS : EPI_STORE, bias, nullptr, 0.f, 0, current_stream()))
        o1_launch_count_add(1);
}
void hd_vision_layernorm(const void* x, const void* w, const void* b, void* y, int rows, int cols, float eps) {
    if (vision_layernorm(x, w, b, y, rows, cols, eps, current_stream())) o1_launch_count_add(1);
}
void hd_vision_gelu(const void* x, void* y, size_t n) { if (vision_gelu(x, y, n, 0, current_stream())) o1_launch_count_add(1); }
void hd_vision_gelu_exact(const void* x, void* y, size_t n) { if (vision_gelu(x, y, n, 1, current_stream())) o1_launch_count_add(1); }
void hd_vision_pos_interp(const void* pe, const int* idx, const float* wgt, void* y, int n, int hidden) {
    if (vision_pos_interp(pe, idx, wgt, nullptr, y, n, hidden, current_stream())) o1_launch_count_add(1);
}
void hd_vision_rot(const float* inv_freq, const int* coords, void* y, int n, int half) {
    if (!y) { set_error("vision_rot: bad args"); return; }
    if (vision_rot_table(inv_freq, coords, y, nullptr, nullptr, n, half, current_stream())) o1_launch_count_add(1);
}
void hd_vision_rot_cos_sin(const void* rot, float* cosd, float* sind, int n, int half) {
    if (vision_rot_cos_sin(rot, cosd, sind, n, half, current_stream())) o1_launch_count_add(1);
}
void hd_vision_spatial_merge(const void* in, void* out, int gh, int gw, int hidden) {
    if (vision_spatial_merge(in, out, gh, gw, hidden, current_stream())) o1_launch_count_add(1);
}
void hd_vision_qkv_split(const void* qkv, void* q, void* k, void* v, int n, int heads, int d) {
    if (vision_qkv_split(qkv, q, k, v, n, heads, d, current_stream())) o1_launch_count_add(1);
}
void hd_vision_attn_merge(const void* hm, void* sm, int heads, int n, int d) {
    if (vision_attn_merge(hm, sm, heads, n, d, current_stream())) o1_launch_count_add(1);
}

// ------------------------------------------------------------ binding (vision.c:43-127)
static const void* vis_find(const hd_weight_store* ws, const char* name) {
    for (int64_t i = 0; i < ws->n_allocs; ++i)
        if (ws->allocs[i].name[0] && strcmp(ws->allocs[i].name, name) == 0) return ws->allocs[i].dev_ptr;
    return nullptr;
}
static bool vis_bind(const hd_weight_store* ws, const char* prefix, const char* const* suffix, const void** dst[], int count) {
    char name[256];
    for (int k = 0; k < count; ++k) {
        snprintf(name, sizeof(name), "%s.%s", prefix, suffix[k]);
        *dst[k] = vis_find(ws, name);
        if (!*dst[k]) { hd_set_error("vision: missing %s", name); return false; }
    }
    return true;
}
hd_status hd_vision_resolve(const hd_weight_store* wstore, hd_vision_binding* out) {
    if (!wstore || !out) { hd_set_error("vision: null argument in resolve"); return HD_ERR_MISSING; }
    memset(out, 0, sizeof(*out));
    out->patch_proj_w = vis_find(wstore, "model.visual.patch_embed.proj.weight");
    out->patch_proj_b = vis_find(wstore, "model.visual.patch_embed.proj.bias");
    out->pos_embed = vis_find(wstore, "model.visual.pos_embed.weight");
    if (!out->patch_proj_w || !out->patch_proj_b || !out->pos_embed) {
        hd_set_error("vision: missing patch_embed/pos_embed weights");
        return HD_ERR_MISSING;
    }
    static const char* const bsfx[12] = {"norm1.weight", "norm1.bias", "norm2.weight", "norm2.bias", "attn.qkv.weight",
                                         "attn.qkv.bias", "attn.proj.weight", "attn.proj.bias", "mlp.linear_fc1.weight",
                                         "mlp.linear_fc1.bias", "mlp.linear_fc2.weight", "mlp.linear_fc2.bias"};
    static const char* const msfx[6] = {"norm.weight", "norm.bias", "linear_fc1.weight", "linear_fc1.bias",
                                        "linear_fc2.weight", "linear_fc2.bias"};
    char prefix[128];
    for (int i = 0; i < V_DEPTH; ++i) {
        hd_vision_block_binding* b = &out->blocks[i];
        const void** dst[12] = {&b->norm1_w, &b->norm1_b, &b->norm2_w, &b->norm2_b, &b->qkv_w, &b->qkv_b,
                                &b->proj_w, &b->proj_b, &b->fc1_w, &b->fc1_b, &b->fc2_w, &b->fc2_b};
        snprintf(prefix, sizeof(prefix), "model.visual.blocks.%d", i);
        if (!vis_bind(wstore, prefix, bsfx, dst, 12)) return HD_ERR_MISSING;
    }
    for (int j = -1; j < HD_VISION_NUM_DS; ++j) {
        hd_vision_merger_binding* m = j < 0 ? &out->merger : &out->deepstack[j];
        const void** dst[6] = {&m->norm_w, &m->norm_b, &m->fc1_w, &m->fc1_b, &m->fc2_w, &m->fc2_b};
        if (j < 0) snprintf(prefix, sizeof(prefix), "model.visual.merger");
        else snprintf(prefix, sizeof(prefix), "model.visual.deepstack_merger_list.%d", j);
        if (!vis_bind(wstore, prefix, msfx, dst, 6)) return HD_ERR_MISSING;
    }
    return HD_OK;
}

// ------------------------------------------------------------ workspace (O(n); vision.c:135-194 is O(n^2))
void hd_vision_layout(int64_t n, int64_t m, hd_vision_offsets* o) {
    if (!o) return;
    int64_t b = 0;
    auto take = [&](int64_t bytes) { const int64_t at = b; b += up256(bytes); return at; };
    const int64_t nH = n * V_H * 2;
    o->patch_out = take(nH);
    o->pos_emb = -1; o->rot = -1;
    o->h_a = take(nH); o->h_b = take(nH); o->ln1 = take(nH); o->attn_resid = take(nH); o->ln2 = take(nH);
    o->fc2 = take(nH);
    o->mlp_resid = o->h_b;
    o->q = take(n * 3 * V_HEADS * V_DP * 2);
    o->k = o->q + V_HEADS * V_DP * 2;
    o->v = o->k + V_HEADS * V_DP * 2;
    o->qr = o->q; o->kr = o->k;
    o->qkv = take(n * 3 * V_H * 2);
    o->scores = take(n * V_HEADS * V_DP * 2);
    o->probs = -1; o->mask = -1;
    o->attn_out = take(nH);
    o->fc1 = take(n * V_I * 2);
    o->cosf = take(n * V_D * 4);
    o->sinf = take(n * V_D * 4);
    o->merged = -1;
    o->merge_norm = take(nH);
    o->merge_fc1 = take(m * V_MERGED * 2);
    o->merge_fc2 = -1;
    o->ds_merged = take(m * V_MERGED * 2);
    o->ds_fc1 = take(m * V_MERGED * 2);
    o->ds_fc2 = -1;
    o->total_bytes = b;
}
int64_t hd_vision_workspace_bytes(int64_t n) {
    int64_t m = n / 4;
    if (m < 1) m = 1;
    hd_vision_offsets o;
    hd_vision_layout(n, m, &o);
    return o.total_bytes;
}
int64_t hd_vision_tables_bytes(int64_t n) { return n * 4 * 4 + n * 4 * 4 + n * 2 * 4 + 18 * 4; }

hd_status hd_vision_prepare_tables(hd_vision_workspace* ws, int n, int grid_h, int grid_w) {
    if (!ws || n <= 0 || grid_h <= 0 || grid_w <= 0 || (grid_h % 2) || (grid_w % 2) || n != grid_h * grid_w) {
        hd_set_error("vision: bad prepare_tables args");
        return HD_ERR_MISSING;
    }
    if (ws->tables_n == n && ws->tables_gh == grid_h && ws->tables_gw == grid_w && ws->pos_idx) return HD_OK;
    if (!ws->tables) { hd_set_error("vision: table region not bound"); return HD_ERR_MISSING; }
    int* idx = (int*)malloc((size_t)n * 4 * sizeof(int));
    float* wgt = (float*)malloc((size_t)n * 4 * sizeof(float));
    int* coords = (int*)malloc((size_t)n * 2 * sizeof(int));
    if (!idx || !wgt || !coords) { free(idx); free(wgt); free(coords); hd_set_error("vision: table build oom"); return HD_ERR_OOM; }
    // Token r is patch (h, w) in 2x2 block-major order (the processor's order, vision.c:209-213).  Its position
    // embedding is the bilinear mix of the 48 x 48 learned grid at (h*47/(gh-1), w*47/(gw-1)), fp32 (vision.c:229-244).
    const int side = V_NPOS_SIDE, mw = grid_w / 2;
    for (int r = 0; r < n; ++r) {
        const int blk = r >> 2, h = (blk / mw) * 2 + ((r >> 1) & 1), w = (blk % mw) * 2 + (r & 1);
        const float hf = (float)h * (float)(side - 1) / (float)(grid_h - 1);
        const float wf = (float)w * (float)(side - 1) / (float)(grid_w - 1);
        const int h0 = (int)hf, w0 = (int)wf;
        const int h1 = h0 + 1 < side ? h0 + 1 : side - 1, w1 = w0 + 1 < side ? w0 + 1 : side - 1;
        const float dh = hf - (float)h0, dw = wf - (float)w0;
        idx[r] = h0 * side + w0;          wgt[r] = (1.0f - dh) * (1.0f - dw);
        idx[n + r] = h0 * side + w1;      wgt[n + r] = (1.0f - dh) * dw;
        idx[2 * n + r] = h1 * side + w0;  wgt[2 * n + r] = dh * (1.0f - dw);
        idx[3 * n + r] = h1 * side + w1;  wgt[3 * n + r] = dh * dw;
        coords[r] = h;
        coords[n + r] = w;
    }
    float inv_freq[18];
    for (int k = 0; k < 18; ++k) inv_freq[k] = 1.0f / powf(10000.0f, (float)(2 * k) / 36.0f);   // vision.c:324-328
    uint8_t* t = (uint8_t*)ws->tables;
    int* d_idx = (int*)t;            t += (size_t)n * 16;
    float* d_wgt = (float*)t;        t += (size_t)n * 16;
    int* d_coords = (int*)t;         t += (size_t)n * 8;
    float* d_inv = (float*)t;
    cudaError_t e = cudaMemcpy(d_idx, idx, (size_t)n * 16, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(d_wgt, wgt, (size_t)n * 16, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(d_coords, coords, (size_t)n * 8, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(d_inv, inv_freq, sizeof(inv_freq), cudaMemcpyHostToDevice);
    free(idx); free(wgt); free(coords);
    if (e != cudaSuccess) { hd_set_error("vision: table upload: %s", cudaGetErrorString(e)); return HD_ERR_RUNTIME; }
    ws->pos_idx = d_idx; ws->pos_wgt = d_wgt; ws->rot_coords = d_coords; ws->rot_inv = d_inv;
    ws->tables_n = n; ws->tables_gh = grid_h; ws->tables_gw = grid_w;
    return HD_OK;
}

// ------------------------------------------------------------ forward (vision.c:345-650)
static bool snap(void* dst, const void* src, size_t bytes, cudaStream_t st) {
    if (!dst) return true;
    return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, st) == cudaSuccess;
}

hd_status hd_vision_forward(const hd_vision_binding* bw, hd_vision_workspace* ws, const void* pixel_values, int n,
                            int grid_h, int grid_w, void* image_embeds_out, void* deepstack_out[HD_VISION_NUM_DS]) {
    if (!bw || !ws || !pixel_values || n <= 0 || grid_h <= 0 || grid_w <= 0 || !image_embeds_out || !ws->patch_out) {
        hd_set_error("vision: null argument");
        return HD_ERR_MISSING;
    }
    if ((grid_h % 2) || (grid_w % 2) || n != grid_h * grid_w) {
        hd_set_error("vision: grid %dx%d (n = %d) not a whole number of 2x2 merge blocks", grid_h, grid_w, n);
        return HD_ERR_MISSING;
    }
    if (!ws->pos_idx || !ws->pos_wgt || !ws->rot_coords || !ws->rot_inv || ws->tables_n != n ||
        ws->tables_gh != grid_h || ws->tables_gw != grid_w) {
        hd_set_error("vision: persistent tables not prepared for this shape");
        return HD_ERR_MISSING;
    }
    const int m = n / 4;
    const float eps = 1e-6f;
    const float scaling = (float)(1.0 / sqrt((double)V_D));
    cudaStream_t st = current_stream();
    hd_vision_offsets o;
    hd_vision_layout(n, m, &o);
    uint8_t* base = (uint8_t*)ws->patch_out;
    uint16_t* patch_out = (uint16_t*)(base + o.patch_out);
    uint16_t* h_a = (uint16_t*)(base + o.h_a);
    uint16_t* h_b = (uint16_t*)(base + o.h_b);
    uint16_t* ln1 = (uint16_t*)(base + o.ln1);
    uint16_t* attn_resid = (uint16_t*)(base + o.attn_resid);
    uint16_t* ln2 = (uint16_t*)(base + o.ln2);
    uint16_t* fc2 = (uint16_t*)(base + o.fc2);
    uint16_t* qkvp = (uint16_t*)(base + o.q);
    uint16_t* qkv = (uint16_t*)(base + o.qkv);
    uint16_t* attn_pad = (uint16_t*)(base + o.scores);
    uint16_t* attn_out = (uint16_t*)(base + o.attn_out);
    uint16_t* fc1 = (uint16_t*)(base + o.fc1);
    float* cosf_t = (float*)(base + o.cosf);
    float* sinf_t = (float*)(base + o.sinf);
    uint16_t* merge_norm = (uint16_t*)(base + o.merge_norm);
    uint16_t* merge_fc1 = (uint16_t*)(base + o.merge_fc1);
    uint16_t* ds_fc1out = (uint16_t*)(base + o.ds_merged);
    uint16_t* ds_norm = (uint16_t*)(base + o.ds_fc1);
    int launches = 0;
    const size_t nH = (size_t)n * V_H * 2;
#define VIS_TRY(call)                                                                              \
    do {                                                                                           \
        if (!(call)) { hd_set_error("vision: %s", hd_cuda_last_error()); o1_launch_count_add(launches); return HD_ERR_RUNTIME; } \
    } while (0)

    // patch embedding + interpolated position embedding -> h_a
    VIS_TRY(linear_act(pixel_values, bw->patch_proj_w, bw->patch_proj_b, patch_out, n, V_H, V_PATCH, 0, st, &launches));
    VIS_TRY(vision_pos_interp(bw->pos_embed, (const int*)ws->pos_idx, (const float*)ws->pos_wgt, patch_out, h_a, n, V_H, st));
    // rotary cos | sin [n, 72]
    VIS_TRY(vision_rot_table((const float*)ws->rot_inv, (const int*)ws->rot_coords, nullptr, cosf_t, sinf_t, n, 18, st));
    launches += 2;

    const uint16_t* cur_in = h_a;
    uint16_t* cur_out = h_b;
    for (int i = 0; i < V_DEPTH; ++i) {
        const hd_vision_block_binding* blk = &bw->blocks[i];
        void** s0 = i == 0 ? ws->block0_snaps : nullptr;
        VIS_TRY(vision_layernorm(cur_in, blk->norm1_w, blk->norm1_b, ln1, n, V_H, eps, st));
        VIS_TRY(linear_act(ln1, blk->qkv_w, blk->qkv_b, qkv, n, 3 * V_H, V_H, 0, st, &launches));
        {
            const long total = (long)n * 3 * V_HEADS * (V_DP / 8);
            split_rope_pad_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(qkv, cosf_t, sinf_t, qkvp, n);
        }
        VIS_TRY(flash_attention(qkvp, 3 * V_HEADS * V_DP, qkvp + V_HEADS * V_DP, 3 * V_HEADS * V_DP,
                                qkvp + 2 * V_HEADS * V_DP, 3 * V_HEADS * V_DP, attn_pad, V_HEADS * V_DP, n, V_HEADS,
                                V_HEADS, 0, scaling, st));
        {
            const long total = (long)n * V_HEADS * (V_D / 8);
            unpad_heads_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(attn_pad, attn_out, n);
        }
        VIS_TRY(cudaGetLastError() == cudaSuccess);
        // the two residual adds ride in the projections' epilogues unless a snapshot asks for the bare projection
        // (or the row count is below the tensor-core tile minimum)
        const bool fuse = gemm_tc_supported(n, V_H, V_H, EPI_BIAS_RESID) && !(s0 && (s0[HD_B0_PROJ] || s0[HD_B0_FC2]));
        if (fuse) {
            VIS_TRY(gemm_bf16(attn_out, blk->proj_w, nullptr, attn_resid, n, V_H, V_H, EPI_BIAS_RESID, blk->proj_b, cur_in, 0.f, 0, st));
        } else {
            VIS_TRY(linear_act(attn_out, blk->proj_w, blk->proj_b, attn_resid, n, V_H, V_H, 0, st, &launches));
            if (s0) VIS_TRY(snap(s0[HD_B0_PROJ], attn_resid, nH, st));
            VIS_TRY(residual_add(cur_in, attn_resid, attn_resid, (size_t)n * V_H, st));
        }
        VIS_TRY(vision_layernorm(attn_resid, blk->norm2_w, blk->norm2_b, ln2, n, V_H, eps, st));
        VIS_TRY(linear_act(ln2, blk->fc1_w, blk->fc1_b, fc1, n, V_I, V_H, 1, st, &launches));
        if (fuse) {
            VIS_TRY(gemm_bf16(fc1, blk->fc2_w, nullptr, cur_out, n, V_H, V_I, EPI_BIAS_RESID, blk->fc2_b, attn_resid, 0.f, 0, st));
        } else {
            VIS_TRY(linear_act(fc1, blk->fc2_w, blk->fc2_b, fc2, n, V_H, V_I, 0, st, &launches));
            VIS_TRY(residual_add(attn_resid, fc2, cur_out, (size_t)n * V_H, st));
        }
        launches += 7;

        if (s0) {
            VIS_TRY(snap(s0[HD_B0_INPUT], cur_in, nH, st) && snap(s0[HD_B0_NORM1], ln1, nH, st) &&
                    snap(s0[HD_B0_QKV], qkv, (size_t)n * 3 * V_H * 2, st) && snap(s0[HD_B0_ATTN_MERGED], attn_out, nH, st) &&
                    snap(s0[HD_B0_ATTN_RESID], attn_resid, nH, st) && snap(s0[HD_B0_NORM2], ln2, nH, st) &&
                    (fuse || snap(s0[HD_B0_FC2], fc2, nH, st)) && snap(s0[HD_B0_OUTPUT], cur_out, nH, st));
            VIS_TRY(snap(ws->block0_snap, cur_out, nH, st));
        }
        VIS_TRY(snap(ws->block_out_snaps[i], cur_out, nH, st));

        // DeepStack mergers read the block output as [m, 4608] (tokens are 2x2 block-major already)
        if (deepstack_out && (i == 8 || i == 16 || i == 24)) {
            const int j = i / 8 - 1;
            const hd_vision_merger_binding* ds = &bw->deepstack[j];
            if (!deepstack_out[j]) { hd_set_error("vision: deepstack_out[%d] is null", j); return HD_ERR_MISSING; }
            VIS_TRY(vision_layernorm(cur_out, ds->norm_w, ds->norm_b, ds_norm, m, V_MERGED, eps, st));
            VIS_TRY(linear_act(ds_norm, ds->fc1_w, ds->fc1_b, ds_fc1out, m, V_MERGED, V_MERGED, 2, st, &launches));
            VIS_TRY(linear_act(ds_fc1out, ds->fc2_w, ds->fc2_b, deepstack_out[j], m, V_OUT, V_MERGED, 0, st, &launches));
            ++launches;
        }
        uint16_t* t = cur_out;
        cur_out = const_cast<uint16_t*>(cur_in);
        cur_in = t;
    }

    // final merger: LayerNorm over 1152, then four consecutive rows form one 4608-wide row
    const hd_vision_merger_binding* mg = &bw->merger;
    VIS_TRY(vision_layernorm(cur_in, mg->norm_w, mg->norm_b, merge_norm, n, V_H, eps, st));
    ++launches;
    VIS_TRY(snap(ws->merger_snaps[0], merge_norm, nH, st));
    VIS_TRY(linear_act(merge_norm, mg->fc1_w, mg->fc1_b, merge_fc1, m, V_MERGED, V_MERGED, 2, st, &launches));
    VIS_TRY(linear_act(merge_fc1, mg->fc2_w, mg->fc2_b, image_embeds_out, m, V_OUT, V_MERGED, 0, st, &launches));
    VIS_TRY(snap(ws->merger_snaps[4], image_embeds_out, (size_t)m * V_OUT * 2, st));
#undef VIS_TRY
    o1_launch_count_add(launches);
    return HD_OK;
}

}  // extern "C"
