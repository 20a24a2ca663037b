// Host-side pieces of the step loop that must match the reference bit for bit, and the final
// latent -> RGB conversion on the device.
//  * torch-compatible MT19937 float randn (o1.c src/runtime/torch_rng.c:34-121), initial latent =
//    randn(1,3,H,W; seed+1) pixel-unshuffled to [token, c*p*p + p1*p + p2] times the noise scale
//    (src/runtime/generate.c:78-104, :1266)
//  * sigma schedules (src/model/scheduler.c:26-64, 117-195), noise scale ramp (:197-208) and the
//    per-step noise clamp of the flash path (generate.c:1423-1438)
//  * decode (src/runtime/decode.c:5-27) fused with the NaN / range gate (generate.c:1474-1496)
//  * the per-step noise of the flash scheduler as a pipeline: a host thread draws step i+1 into
//    pinned memory while the device runs step i; mean / unbiased std / clamp run on the device
//    (generate.c:1419-1439 does all of it on the host, serially, inside the step)
#include "common.cuh"
#include "../../include/o1_b200.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <condition_variable>
#include <mutex>
#include <thread>
#include <vector>

namespace {

struct Mt {
    uint32_t state[624];
    int left, next;
};
void mt_seed(Mt* r, uint64_t seed) {
    r->state[0] = (uint32_t)(seed & 0xffffffffu);
    for (int j = 1; j < 624; ++j) r->state[j] = 1812433253u * (r->state[j - 1] ^ (r->state[j - 1] >> 30)) + (uint32_t)j;
    r->left = 1;
    r->next = 0;
}
inline uint32_t mix(uint32_t u, uint32_t v) {
    return (((u & 0x80000000u) | (v & 0x7fffffffu)) >> 1) ^ ((v & 1u) ? 0x9908b0dfu : 0u);
}
void mt_refill(Mt* r) {
    uint32_t* p = r->state;
    for (int j = 0; j < 227; ++j) p[j] = p[j + 397] ^ mix(p[j], p[j + 1]);
    for (int j = 227; j < 623; ++j) p[j] = p[j - 227] ^ mix(p[j], p[j + 1]);
    p[623] = p[396] ^ mix(p[623], p[0]);
    r->left = 624;
    r->next = 0;
}
inline uint32_t mt_u32(Mt* r) {
    if (--r->left == 0) mt_refill(r);
    uint32_t y = r->state[r->next++];
    y ^= y >> 11;
    y ^= (y << 7) & 0x9d2c5680u;
    y ^= (y << 15) & 0xefc60000u;
    y ^= y >> 18;
    return y;
}
inline float mt_uniform(Mt* r) { return (float)((mt_u32(r) & 0xFFFFFFu) * (1.0f / 16777216.0f)); }
// n uniforms at once: same draws as n calls of mt_uniform, tempered straight out of the state
// array in loops the compiler can vectorise.  left + next == 625 holds after every scalar draw
// (624 + 1 after a refill), so left - 1 entries are ready at state[next].
void mt_uniform_fill(Mt* r, float* out, int64_t n) {
    while (n > 0) {
        if (r->left <= 1) { mt_refill(r); r->left = 625; }
        const int64_t k = n < (int64_t)(r->left - 1) ? n : (int64_t)(r->left - 1);
        const uint32_t* src = r->state + r->next;
        for (int64_t i = 0; i < k; ++i) {
            uint32_t y = src[i];
            y ^= y >> 11;
            y ^= (y << 7) & 0x9d2c5680u;
            y ^= (y << 15) & 0xefc60000u;
            y ^= y >> 18;
            out[i] = (float)((y & 0xFFFFFFu) * (1.0f / 16777216.0f));
        }
        r->next += (int)k;
        r->left -= (int)k;
        out += k;
        n -= k;
    }
}
void box_muller_16(float* d) {
    for (int j = 0; j < 8; ++j) {
        const float u1 = 1.0f - d[j], u2 = d[j + 8];
        const float rad = sqrtf(-2.0f * logf(u1));
        const float th = (float)(6.283185307179586 * (double)u2);
        d[j] = rad * cosf(th);
        d[j + 8] = rad * sinf(th);
    }
}
// The uniform draws are one sequential stream; the Box-Muller transform of the groups of 16 is
// independent per group and is spread over `threads` host threads.
void mt_randn(Mt* r, float* out, int64_t n, int threads = 1) {
    if (n >= 16) {
        mt_uniform_fill(r, out, n);
        const int64_t groups = (n - 15 + 15) / 16;     // groups starting at 0, 16, ... < n - 15
        if (threads > 1 && groups >= 4096) {
            std::vector<std::thread> pool;
            const int64_t per = (groups + threads - 1) / threads;
            for (int t = 0; t < threads; ++t) {
                const int64_t g0 = t * per, g1 = g0 + per < groups ? g0 + per : groups;
                if (g0 >= g1) break;
                pool.emplace_back([=] { for (int64_t g = g0; g < g1; ++g) box_muller_16(out + g * 16); });
            }
            for (auto& th : pool) th.join();
        } else {
            for (int64_t i = 0; i < n - 15; i += 16) box_muller_16(out + i);
        }
        if (n % 16 != 0) {
            float* d = out + (n - 16);
            mt_uniform_fill(r, d, 16);
            box_muller_16(d);
        }
        return;
    }
    bool cached = false;
    double cache = 0.0;
    for (int64_t i = 0; i < n; ++i) {
        double ret;
        if (cached) { ret = cache; cached = false; }
        else {
            const uint64_t v1 = ((uint64_t)mt_u32(r) << 32) | mt_u32(r);
            const uint64_t v2 = ((uint64_t)mt_u32(r) << 32) | mt_u32(r);
            const double u1 = (double)(v1 & ((1ULL << 53) - 1)) * (1.0 / 9007199254740992.0);
            const double u2 = (double)(v2 & ((1ULL << 53) - 1)) * (1.0 / 9007199254740992.0);
            const double rad = sqrt(-2.0 * log1p(-u2));
            const double theta = 2.0 * 3.14159265358979323846 * u1;
            cache = rad * sin(theta);
            cached = true;
            ret = rad * cos(theta);
        }
        out[i] = (float)ret;
    }
}

// stats: [0] = number of non-finite values, [1] = float bits of min, [2] = float bits of max
__global__ void decode_rgb_kernel(const uint16_t* __restrict__ z, int grid_h, int grid_w, int patch, int channels,
                                  unsigned char* __restrict__ rgb, unsigned int* __restrict__ stats) {
    const long feats = (long)channels * patch * patch;
    const long n = (long)grid_h * grid_w * feats;
    const int w = grid_w * patch;
    int bad = 0;
    float mn = INFINITY, mx = -INFINITY;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const float v = o1::bf16_to_f32(z[i]);
        if (isnan(v) || isinf(v)) { ++bad; continue; }
        mn = fminf(mn, v);
        mx = fmaxf(mx, v);
        const long tok = i / feats;
        const int f = (int)(i - tok * feats);
        const int c = f / (patch * patch), p1 = (f / patch) % patch, p2 = f % patch;
        const int tr = (int)(tok / grid_w), tc = (int)(tok % grid_w);
        float px = roundf((v + 1.0f) / 2.0f * 255.0f);
        px = px < 0.f ? 0.f : (px > 255.f ? 255.f : px);
        rgb[((size_t)(tr * patch + p1) * w + (size_t)(tc * patch + p2)) * channels + c] = (unsigned char)px;
    }
    // order-preserving integer images of the floats make atomicMin / atomicMax usable
    auto key = [](float f) { unsigned u = __float_as_uint(f); return (u & 0x80000000u) ? ~u : (u | 0x80000000u); };
    if (bad) atomicAdd(&stats[0], (unsigned)bad);
    if (mn <= mx) { atomicMin(&stats[1], key(mn)); atomicMax(&stats[2], key(mx)); }
}

// ---- noise statistics on the device: deterministic fp64 sums (fixed grid, partials added in block order)
constexpr int STAT_BLOCKS = 1024, STAT_THREADS = 256;
// partial[b] = sum over this block's elements of (x - *shift)^pw, pw = 1 or 2; shift may be null (0)
template <int PW>
__global__ void noise_partial_kernel(const float* __restrict__ x, size_t n, const double* __restrict__ shift,
                                     double* __restrict__ partial) {
    __shared__ double sh[STAT_THREADS];
    const double m = shift ? *shift : 0.0;
    double acc = 0.0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const double d = (double)x[i] - m;
        acc += PW == 1 ? d : d * d;
    }
    sh[threadIdx.x] = acc;
    __syncthreads();
    for (int s = STAT_THREADS / 2; s > 0; s >>= 1) {
        if ((int)threadIdx.x < s) sh[threadIdx.x] += sh[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) partial[blockIdx.x] = sh[0];
}
// stage 0: res[0] = mean.  stage 1: res[1] = clip = clip_std * (float)sqrt(ss / (n - 1))
__global__ void noise_final_kernel(const double* __restrict__ partial, size_t n, float clip_std, int stage,
                                   double* __restrict__ res) {
    double s = 0.0;
    for (int b = 0; b < STAT_BLOCKS; ++b) s += partial[b];
    if (stage == 0) res[0] = s / (double)n;
    else res[1] = (double)(clip_std * (float)sqrt(s / (double)(n - 1)));
}
__global__ void noise_clamp_kernel(float* __restrict__ x, size_t n, const double* __restrict__ res) {
    const float clip = (float)res[1];
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = x[i];
        x[i] = v > clip ? clip : (v < -clip ? -clip : v);
    }
}

struct NoisePipe {
    Mt rng;
    size_t n = 0;
    float clip_std = 0.f;
    int threads = 1;
    float* pinned[2] = {nullptr, nullptr};
    cudaEvent_t copied[2] = {nullptr, nullptr};   // H2D of the buffer has finished: the worker may overwrite it
    bool copy_pending[2] = {false, false};
    double* dev_scratch = nullptr;                // STAT_BLOCKS partials + 2 results
    std::thread worker;
    std::mutex mu;
    std::condition_variable cv;
    int produced = 0;       // steps fully drawn by the worker
    int requested = 1;      // steps the worker may draw (one ahead of the consumer)
    int consumed = 0;
    bool stop = false;
    int device = 0;
};

void noise_worker(NoisePipe* p) {
    cudaSetDevice(p->device);
    for (;;) {
        int step;
        {
            std::unique_lock<std::mutex> lk(p->mu);
            p->cv.wait(lk, [&] { return p->stop || p->produced < p->requested; });
            if (p->stop) return;
            step = p->produced;
        }
        const int b = step & 1;
        if (p->copy_pending[b]) { cudaEventSynchronize(p->copied[b]); p->copy_pending[b] = false; }
        mt_randn(&p->rng, p->pinned[b], (int64_t)p->n, p->threads);
        {
            std::lock_guard<std::mutex> lk(p->mu);
            p->produced = step + 1;
        }
        p->cv.notify_all();
    }
}

}  // namespace

extern "C" {

// ------------------------------------------------------------------ RNG + initial latent (host)
void* o1_torch_rng_create(uint64_t seed) {
    Mt* r = (Mt*)malloc(sizeof(Mt));
    if (r) mt_seed(r, seed);
    return r;
}
void o1_torch_rng_randn(void* rng, float* out_host, int64_t n) { if (rng && out_host && n > 0) mt_randn((Mt*)rng, out_host, n); }
void o1_torch_rng_randn_mt(void* rng, float* out_host, int64_t n, int threads) {
    if (rng && out_host && n > 0) mt_randn((Mt*)rng, out_host, n, threads < 1 ? 1 : threads);
}
uint32_t o1_torch_rng_u32(void* rng) { return rng ? mt_u32((Mt*)rng) : 0; }
void o1_torch_rng_free(void* rng) { free(rng); }

hd_status o1_initial_latent_host(uint64_t seed, int height, int width, int patch, float noise_scale, void* z_host) {
    if (!z_host || height <= 0 || width <= 0 || patch <= 0 || height % patch || width % patch) {
        hd_set_error("initial_latent: bad dimensions");
        return HD_ERR_MISSING;
    }
    const int64_t n = (int64_t)3 * height * width;
    float* noise = (float*)malloc((size_t)n * sizeof(float));
    if (!noise) { hd_set_error("initial_latent: out of host memory"); return HD_ERR_OOM; }
    Mt r;
    mt_seed(&r, seed + 1);
    mt_randn(&r, noise, n);
    const int gw = width / patch, feats = 3 * patch * patch;
    uint16_t* z = (uint16_t*)z_host;
    for (int c = 0; c < 3; ++c)
        for (int y = 0; y < height; ++y) {
            const int th = y / patch, p1 = y % patch;
            const float* row = noise + ((size_t)c * height + y) * width;
            for (int x = 0; x < width; ++x)
                z[(size_t)(th * gw + x / patch) * feats + c * patch * patch + p1 * patch + x % patch] =
                    o1::f32_to_bf16(row[x] * noise_scale);
        }
    free(noise);
    return HD_OK;
}

// ------------------------------------------------------------------ schedules (host)
int o1_sigmas_dev(float* sigmas) {
    static const int ts[28] = {999, 987, 974, 960, 945, 929, 913, 895, 877, 857, 836, 814, 790, 764,
                               737, 707, 675, 640, 602, 560, 515, 464, 409, 347, 278, 199, 110, 8};
    if (!sigmas) return 0;
    for (int i = 0; i < 28; ++i) sigmas[i] = (float)ts[i] / 1000.0f;
    sigmas[28] = 0.0f;
    return 29;
}
int o1_sigmas_flash(int steps, float shift, float* sigmas) {
    if (!sigmas || steps < 2) return 0;
    const double sh = (double)shift, raw_min = 0.0010000000474974513;
    const double sigma_min = sh * raw_min / (1.0 + (sh - 1.0) * raw_min);
    const double lo = 1000.0, hi = sigma_min * 1000.0, d = (hi - lo) / (double)(steps - 1);
    for (int i = 0; i < steps; ++i) {
        const double sig = (lo + d * (double)i) / 1000.0;
        sigmas[i] = (float)(sh * sig / (1.0 + (sh - 1.0) * sig));
    }
    sigmas[steps] = 0.0f;
    return steps + 1;
}
int o1_sigmas_default(int steps, float shift, float* sigmas) {
    if (!sigmas || steps < 1) return 0;
    const double sigma_max = 0.9996664524078369, sh = (double)shift, d = -sigma_max / (double)steps;
    for (int i = 0; i < steps; ++i) {
        const double sig = sigma_max + d * (double)i;
        sigmas[i] = (float)(sh * sig / (1.0 + (sh - 1.0) * sig));
    }
    sigmas[steps] = 0.0f;
    return steps + 1;
}
float o1_noise_scale(int n_sigmas, int step_index, float start, float end) {
    if (step_index < 0) step_index = 0;
    const int num_steps = n_sigmas > 1 ? n_sigmas - 1 : 1;
    if (num_steps <= 1) return start;
    if (step_index >= num_steps) step_index = num_steps - 1;
    return start + (end - start) * (float)step_index / (float)(num_steps - 1);
}
void o1_noise_clamp_host(float* noise, size_t n, float clip_std) {
    if (!noise || clip_std <= 0.0f || n < 2) return;
    double m = 0.0, ss = 0.0;
    for (size_t i = 0; i < n; ++i) m += (double)noise[i];
    m /= (double)n;
    for (size_t i = 0; i < n; ++i) { const double d = (double)noise[i] - m; ss += d * d; }
    const float clip = clip_std * (float)sqrt(ss / (double)(n - 1));
    for (size_t i = 0; i < n; ++i) noise[i] = noise[i] > clip ? clip : (noise[i] < -clip ? -clip : noise[i]);
}

// ------------------------------------------------------------------ per-step noise pipeline (flash scheduler)
// Stream of draws: the generator is seeded once (the reference seeds it with request seed + 1,
// generate.c:1296) and every step takes the next n normals from it, so step i of the pipe equals the
// i-th hd_torch_randn_f32(&step_rng, ., n) of the reference loop.
int o1_noise_pipe_create(o1_noise_pipe** out, uint64_t seed, size_t n, float clip_std, int host_threads) {
    if (!out || n < 2) { hd_set_error("noise pipe: bad arguments"); return -1; }
    NoisePipe* p = new NoisePipe();
    mt_seed(&p->rng, seed);
    p->n = n;
    p->clip_std = clip_std;
    p->threads = host_threads < 1 ? 1 : host_threads;
    cudaGetDevice(&p->device);
    cudaError_t e = cudaSuccess;
    for (int b = 0; b < 2 && e == cudaSuccess; ++b) {
        e = cudaHostAlloc((void**)&p->pinned[b], n * sizeof(float), cudaHostAllocDefault);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&p->copied[b], cudaEventDisableTiming);
    }
    if (e == cudaSuccess) e = cudaMalloc((void**)&p->dev_scratch, (STAT_BLOCKS + 2) * sizeof(double));
    if (e != cudaSuccess) {
        hd_set_error("noise pipe: %s", cudaGetErrorString(e));
        for (int b = 0; b < 2; ++b) { if (p->pinned[b]) cudaFreeHost(p->pinned[b]); if (p->copied[b]) cudaEventDestroy(p->copied[b]); }
        if (p->dev_scratch) cudaFree(p->dev_scratch);
        delete p;
        return -1;
    }
    p->worker = std::thread(noise_worker, p);   // starts on step 0 at once
    *out = reinterpret_cast<o1_noise_pipe*>(p);
    return 0;
}

hd_status o1_noise_pipe_next(o1_noise_pipe* pipe, float* noise_dev, void* stream) {
    NoisePipe* p = reinterpret_cast<NoisePipe*>(pipe);
    if (!p || !noise_dev) { hd_set_error("noise pipe: bad arguments"); return HD_ERR_MISSING; }
    cudaStream_t st = stream ? (cudaStream_t)stream : o1::current_stream();
    int step;
    {
        std::unique_lock<std::mutex> lk(p->mu);
        step = p->consumed;
        p->cv.wait(lk, [&] { return p->produced > step; });
    }
    const int b = step & 1;
    cudaError_t e = cudaMemcpyAsync(noise_dev, p->pinned[b], p->n * sizeof(float), cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaEventRecord(p->copied[b], st);
    if (e != cudaSuccess) { hd_set_error("noise pipe: %s", cudaGetErrorString(e)); return HD_ERR_RUNTIME; }
    {
        // the worker touches copy_pending[b] again only after `requested` lets it reach step + 2
        std::lock_guard<std::mutex> lk(p->mu);
        p->copy_pending[b] = true;
        p->consumed = step + 1;
        p->requested = step + 2;     // draw the next step while the device works on this one
    }
    p->cv.notify_all();
    if (p->clip_std > 0.0f) {
        double* part = p->dev_scratch;
        double* res = p->dev_scratch + STAT_BLOCKS;
        noise_partial_kernel<1><<<STAT_BLOCKS, STAT_THREADS, 0, st>>>(noise_dev, p->n, nullptr, part);
        noise_final_kernel<<<1, 1, 0, st>>>(part, p->n, p->clip_std, 0, res);
        noise_partial_kernel<2><<<STAT_BLOCKS, STAT_THREADS, 0, st>>>(noise_dev, p->n, res, part);
        noise_final_kernel<<<1, 1, 0, st>>>(part, p->n, p->clip_std, 1, res);
        long blocks = (long)((p->n + 255) / 256);
        if (blocks > (long)o1::sm_count() * 16) blocks = (long)o1::sm_count() * 16;
        noise_clamp_kernel<<<(unsigned)blocks, 256, 0, st>>>(noise_dev, p->n, res);
        o1_launch_count_add(5);
        e = cudaGetLastError();
        if (e != cudaSuccess) { hd_set_error("noise pipe: %s", cudaGetErrorString(e)); return HD_ERR_RUNTIME; }
    }
    return HD_OK;
}

void o1_noise_pipe_free(o1_noise_pipe* pipe) {
    NoisePipe* p = reinterpret_cast<NoisePipe*>(pipe);
    if (!p) return;
    {
        std::lock_guard<std::mutex> lk(p->mu);
        p->stop = true;
    }
    p->cv.notify_all();
    if (p->worker.joinable()) p->worker.join();
    for (int b = 0; b < 2; ++b) {
        if (p->copy_pending[b]) cudaEventSynchronize(p->copied[b]);
        cudaFreeHost(p->pinned[b]);
        cudaEventDestroy(p->copied[b]);
    }
    cudaFree(p->dev_scratch);
    delete p;
}

// ------------------------------------------------------------------ decode + gate (device)
// z_dev [grid_h*grid_w, channels*patch*patch] bf16 -> rgb_dev [H, W, channels] uint8.  stats_dev: 3 uint32 of
// scratch.  Returns HD_OK and fills n_bad / min / max; the caller applies the reference's gate
// (fail if n_bad > 0 or the range leaves [-2, 2]).  Synchronises the current stream.
hd_status o1_decode_to_rgb(const void* z_dev, int grid_h, int grid_w, int patch, int channels, void* rgb_dev,
                           void* stats_dev, int* n_bad, float* vmin, float* vmax) {
    if (!z_dev || !rgb_dev || !stats_dev || grid_h <= 0 || grid_w <= 0 || patch <= 0 || channels <= 0) {
        hd_set_error("decode: bad arguments");
        return HD_ERR_MISSING;
    }
    cudaStream_t st = o1::current_stream();
    const unsigned init[3] = {0u, 0xFFFFFFFFu, 0u};
    cudaError_t e = cudaMemcpyAsync(stats_dev, init, sizeof(init), cudaMemcpyHostToDevice, st);
    const long n = (long)grid_h * grid_w * channels * patch * patch;
    long blocks = (n + 255) / 256;
    if (blocks > (long)o1::sm_count() * 16) blocks = (long)o1::sm_count() * 16;
    if (e == cudaSuccess) {
        decode_rgb_kernel<<<(unsigned)blocks, 256, 0, st>>>((const uint16_t*)z_dev, grid_h, grid_w, patch, channels,
                                                            (unsigned char*)rgb_dev, (unsigned*)stats_dev);
        o1_launch_count_add(1);
        e = cudaGetLastError();
    }
    unsigned out[3];
    if (e == cudaSuccess) e = cudaMemcpyAsync(out, stats_dev, sizeof(out), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) { hd_set_error("decode: %s", cudaGetErrorString(e)); return HD_ERR_RUNTIME; }
    auto unkey = [](unsigned k) { unsigned u = (k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k; float f; memcpy(&f, &u, 4); return f; };
    if (n_bad) *n_bad = (int)out[0];
    if (vmin) *vmin = out[1] == 0xFFFFFFFFu ? NAN : unkey(out[1]);
    if (vmax) *vmax = out[2] == 0u ? NAN : unkey(out[2]);
    return HD_OK;
}

}  // extern "C"
