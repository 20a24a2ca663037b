// Host engine + C ABI of libo1b200.so.
//
//  * process state: current stream, error buffers, device error word
//  * hd_* primitive wrappers (o1.c src/cuda/hd_cuda.h:34-198)
//  * hd_sdpa_* plan shim (include/hd_cudnn_sdpa.h:30-94)
//  * hd_decoder_block (src/model/block.c:137-385), re-composed as
//      rmsnorm -> q/k/v GEMMs into one [S,6144] buffer -> fused q/k norm+rope
//      -> flash attention (seq-major in/out) -> o_proj GEMM (+residual)
//      -> rmsnorm -> gate|up GEMM (+SwiGLU) -> down GEMM (+residual)
//  * hd_forward (src/model/forward.c:190-405)
//  * o1_denoise_step_cfg (src/runtime/generate.c:1314-1360 + :900-905)
//  * hd_lora_merge_gpu (src/model/lora_merge.cu:35-109)
// Nothing here allocates device memory on the forward path; the only
// allocations are the per-device error word and LoRA staging.
#include "common.cuh"
#include "kernels.h"
#include "../../include/o1_b200.h"

#include <math.h>
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <map>
#include <mutex>
#include <vector>

// ===================================================================== state
namespace o1 {

static cudaStream_t g_stream = nullptr;
static char g_cuda_err[512] = {0};
static char g_model_err[512] = {0};
static char g_lora_err[512] = {0};
static std::atomic<int64_t> g_launches{0};

cudaStream_t current_stream() { return g_stream; }
char* errbuf() { return g_cuda_err; }
void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_cuda_err, sizeof(g_cuda_err), fmt, ap);
    va_end(ap);
}
static void set_model_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_model_err, sizeof(g_model_err), fmt, ap);
    va_end(ap);
}

struct DevState {
    int* err_word = nullptr;   // [0] error word of the bounded waits, [1] result slot of the mask probe
    int sms = 0;
};
static DevState& dev_state() {
    static std::map<int, DevState> states;
    static std::mutex mu;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lk(mu);
    DevState& s = states[dev];
    if (!s.err_word) {
        if (cudaMalloc(&s.err_word, 2 * sizeof(int)) == cudaSuccess) cudaMemset(s.err_word, 0, 2 * sizeof(int));
        cudaDeviceGetAttribute(&s.sms, cudaDevAttrMultiProcessorCount, dev);
        if (s.sms <= 0) s.sms = 148;
    }
    return s;
}
int* device_error_word() { return dev_state().err_word; }
int sm_count() { return dev_state().sms; }

static inline void count(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// ---- per-launch event timing (off by default)
struct ProfRec { int kind; double work; cudaEvent_t a, b; };
static bool g_prof_on = false;
static std::vector<ProfRec> g_prof;
static size_t g_prof_used = 0;
static int g_prof_open = -1;
void prof_before(int kind, double work, cudaStream_t st) {
    g_prof_open = -1;
    if (!g_prof_on) return;
    if (g_prof_used == g_prof.size()) {
        ProfRec r;
        if (cudaEventCreate(&r.a) != cudaSuccess || cudaEventCreate(&r.b) != cudaSuccess) return;
        g_prof.push_back(r);
    }
    ProfRec& r = g_prof[g_prof_used];
    r.kind = kind; r.work = work;
    cudaEventRecord(r.a, st);
    g_prof_open = (int)g_prof_used++;
}
void prof_after(cudaStream_t st) {
    if (g_prof_open >= 0) cudaEventRecord(g_prof[g_prof_open].b, st);
    g_prof_open = -1;
}

}  // namespace o1

using namespace o1;

struct hd_gemm_runtime {
    int device_id;
    size_t workspace_bytes;
};
struct hd_sdpa_plan {
    int q_heads, kv_heads, seq, ar_len, head_dim;
    float scale;
};

extern "C" {

// ============================================================ error reporting
const char* hd_last_error(void) { return g_model_err; }
void hd_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_model_err, sizeof(g_model_err), fmt, ap);
    va_end(ap);
}
const char* hd_cuda_last_error(void) { return g_cuda_err; }
void hd_cuda_clear_error(void) { g_cuda_err[0] = 0; }
char* hd_cuda_errbuf(void) { return g_cuda_err; }
const char* hd_lora_last_error(void) { return g_lora_err; }

void o1_set_stream(void* stream) { g_stream = (cudaStream_t)stream; }
void* o1_get_stream(void) { return (void*)g_stream; }
int o1_sm_count(void) { return sm_count(); }
void o1_launch_count_add(int n) { count(n); }
int64_t o1_launch_count(int reset) {
    int64_t v = g_launches.load();
    if (reset) g_launches.store(0);
    return v;
}
// Event timing of the tensor-core launches: enable (1) resets the records, disable (0) stops recording.
void o1_profile_enable(int on) {
    g_prof_on = on != 0;
    if (on) g_prof_used = 0;
}
// Sums the records of one kind (0..4 GEMM by epilogue, 5 attention) after synchronising the device:
// total milliseconds, launches and algorithmic work (FLOP).  Returns 0 on success.
int o1_profile_summary(int kind, double* total_ms, int64_t* launches, double* work) {
    if (cudaDeviceSynchronize() != cudaSuccess) return 1;
    double ms = 0, w = 0;
    int64_t n = 0;
    for (size_t i = 0; i < g_prof_used; ++i) {
        if (g_prof[i].kind != kind) continue;
        float t = 0.f;
        if (cudaEventElapsedTime(&t, g_prof[i].a, g_prof[i].b) != cudaSuccess) continue;
        ms += t; w += g_prof[i].work; ++n;
    }
    if (total_ms) *total_ms = ms;
    if (launches) *launches = n;
    if (work) *work = w;
    return 0;
}
int o1_device_error(void) {
    int* w = device_error_word();
    if (!w) return -1;
    int v = 0;
    cudaError_t e = cudaMemcpyAsync(&v, w, sizeof(int), cudaMemcpyDeviceToHost, g_stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(g_stream);
    if (e != cudaSuccess) { set_error("device_error: %s", cudaGetErrorString(e)); return -1; }
    if (v != 0) cudaMemsetAsync(w, 0, sizeof(int), g_stream);
    return v;
}

// ================================================================ bf16 helpers
float hd_bf16_to_f32(uint16_t b) { return bf16_to_f32(b); }
uint16_t hd_f32_to_bf16(float f) { return f32_to_bf16(f); }
void hd_bf16_buf_to_f32(const void* src, float* dst, size_t n) {
    const uint16_t* s = (const uint16_t*)src;
    for (size_t i = 0; i < n; ++i) dst[i] = bf16_to_f32(s[i]);
}
void hd_f32_buf_to_bf16(const float* src, void* dst, size_t n) {
    uint16_t* d = (uint16_t*)dst;
    for (size_t i = 0; i < n; ++i) d[i] = f32_to_bf16(src[i]);
}

// ============================================================ primitive level
void hd_rmsnorm(const void* x, const void* w, void* y, int rows, int cols, float eps) {
    if (rmsnorm(x, w, y, rows, cols, eps, g_stream)) count();
}
void hd_silu(const void* x, void* y, size_t n) { if (silu(x, y, n, g_stream)) count(); }
void hd_swiglu(const void* g, const void* u, void* y, size_t n) { if (swiglu(g, u, y, n, g_stream)) count(); }
void hd_residual_add(const void* x, const void* a, void* y, size_t n) {
    if (residual_add(x, a, y, n, g_stream)) count();
}
void hd_linear(const void* x, const void* w, const void* bias, void* y, int M, int N, int K,
               int transpose_w) {
    if (!x || !w || !y || M <= 0 || N <= 0 || K <= 0) { set_error("linear: bad args"); return; }
    if (!transpose_w) { set_error("linear: transpose_w=0 unsupported"); return; }
    if (gemm_bf16(x, w, nullptr, y, M, N, K, bias ? EPI_BIAS : EPI_STORE, bias, nullptr, 0.f, 0, g_stream))
        count();
}
void hd_linear_reference(const void* x, const void* w, const void* bias, void* y, int M, int N,
                         int K, int transpose_w) {
    hd_linear(x, w, bias, y, M, N, K, transpose_w);
}
void hd_timestep_embed(const float* t, float* y, int N, int dim) {
    if (timestep_embed(t, y, N, dim, g_stream)) count();
}
// true when the GPU cannot dereference p: plain (unregistered) host memory on a machine without unified addressing
// of pageable memory.  o1.c is developed on a unified-memory part, where its own tests hand malloc'd arrays to
// kernels (tests/unit/test_primitives.c:366-372); here such a pointer would fault the kernel.
static bool is_plain_host_pointer(const void* p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
    if (a.type != cudaMemoryTypeUnregistered) return false;
    int dev = 0, pageable = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&pageable, cudaDevAttrPageableMemoryAccess, dev);
    return pageable == 0;
}
void hd_mrope_cos_sin(const float* pos, int bs, int seq, const int64_t* section, int n_section,
                      int head_dim, float theta, float attention_scaling, int interleaved,
                      float* cosd, float* sind) {
    if (cosd && sind && seq > 0 && head_dim > 0 && bs > 0 && (is_plain_host_pointer(cosd) || is_plain_host_pointer(sind))) {
        // host output arrays: compute into a device buffer and copy back (this entry point is not on the forward's
        // path, which builds its own table once per forward)
        const size_t n = (size_t)bs * seq * head_dim;
        float* tmp = nullptr;
        if (cudaMalloc(&tmp, 2 * n * sizeof(float)) != cudaSuccess) { set_error("mrope: staging allocation failed"); return; }
        if (mrope_cos_sin(pos, bs, seq, section, n_section, head_dim, theta, attention_scaling, interleaved, tmp, tmp + n,
                          g_stream)) {
            count();
            cudaMemcpyAsync(cosd, tmp, n * sizeof(float), cudaMemcpyDeviceToHost, g_stream);
            cudaMemcpyAsync(sind, tmp + n, n * sizeof(float), cudaMemcpyDeviceToHost, g_stream);
            cudaStreamSynchronize(g_stream);
        }
        cudaFree(tmp);
        return;
    }
    if (mrope_cos_sin(pos, bs, seq, section, n_section, head_dim, theta, attention_scaling,
                      interleaved, cosd, sind, g_stream))
        count();
}
void hd_apply_rotary(const void* x, const float* c, const float* s, void* y, int heads, int seq, int dim) {
    if (apply_rotary(x, c, s, y, heads, seq, dim, 0, g_stream)) count();
}
void hd_apply_rotary_f32(const void* x, const float* c, const float* s, void* y, int heads, int seq,
                         int dim) {
    if (apply_rotary(x, c, s, y, heads, seq, dim, 1, g_stream)) count();
}
void hd_head_split(const void* in, void* out, int seq, int heads, int dim) {
    if (head_split(in, out, seq, heads, dim, g_stream)) count();
}
void hd_head_merge(const void* in, void* out, int seq, int heads, int dim) {
    if (head_merge(in, out, seq, heads, dim, g_stream)) count();
}
void hd_gather_rows(const void* table, const void* idx, void* out, int M, int cols, int64_t nrows) {
    if (gather_rows(table, idx, out, M, cols, nrows, g_stream)) count();
}
void hd_apply_tms_condition(const void* idx, const void* emb, const void* t_emb, void* out, int M,
                            int H, int64_t tms_id) {
    if (tms_condition(idx, emb, t_emb, out, M, H, tms_id, g_stream)) count();
}
void hd_scale_f32(const float* in, float* out, float s, int n) { if (scale_f32(in, out, s, n, g_stream)) count(); }
void hd_f32_convert_bf16(const float* in, void* out, int n) { if (f32_to_bf16_buf(in, out, n, g_stream)) count(); }
void hd_sched_bf16_upcast(const void* in, float* out, int n) { if (sched_bf16_upcast(in, out, n, g_stream)) count(); }
void hd_sched_denoised(const float* z, const float* mo, float sigma, float* den, int n) {
    if (sched_denoised(z, mo, sigma, den, n, g_stream)) count();
}
void hd_sched_z_next(const float* noise, const float* den, float sigma_next, float s_noise,
                     float* z_next, int n) {
    if (sched_z_next(noise, den, sigma_next, s_noise, z_next, n, g_stream)) count();
}
void hd_sched_vcond(const void* z, const void* xp, float sigma, float* mo, int n) {
    if (sched_vcond(z, xp, sigma, mo, n, g_stream)) count();
}
void hd_sched_flow_match_step(const void* z, const float* mo, float sigma, float sigma_next,
                              void* z_next, int n) {
    if (sched_flow_match_step(z, mo, sigma, sigma_next, z_next, n, g_stream)) count();
}
void hd_sched_cfg_guided(const float* mc, const float* mu, float g, float* mo, int n) {
    if (sched_cfg_guided(mc, mu, g, mo, n, g_stream)) count();
}
void hd_unipc_convert(const float* sample, const float* mo, float sigma_cur, float* conv, int n) {
    if (unipc_convert(sample, mo, sigma_cur, conv, n, g_stream)) count();
}
void hd_unipc_correct(const float* last, const float* mo0, const float* mo_old, const float* conv,
                      float sig_t, float sig_s0, float alpha_t, float h_phi_1, float B_h,
                      float rhos_c0, float rhos_c1, float inv_rks0, int order_c, float* out, int n) {
    if (unipc_correct(last, mo0, mo_old, conv, sig_t, sig_s0, alpha_t, h_phi_1, B_h, rhos_c0, rhos_c1,
                      inv_rks0, order_c, out, n, g_stream))
        count();
}
void hd_unipc_predict(const float* sample, const float* mo0, const float* mo_old, float sig_t,
                      float sig_s0, float alpha_t, float h_phi_1, float B_h, float rhos_p,
                      float inv_rks0, int order_p, float* out, int n) {
    if (unipc_predict(sample, mo0, mo_old, sig_t, sig_s0, alpha_t, h_phi_1, B_h, rhos_p, inv_rks0,
                      order_p, out, n, g_stream))
        count();
}
void hd_vision_masked_scatter(const void* dst, const uint8_t* mask, const void* src, void* out,
                              int rows, int cols) {
    if (masked_scatter(dst, mask, src, out, rows, cols, g_stream)) count();
}
void hd_vision_deepstack_inject(const void* in, const uint8_t* mask, const void* emb, void* out,
                                int rows, int cols) {
    if (deepstack_inject(in, mask, emb, out, rows, cols, g_stream)) count();
}

hd_gemm_runtime* hd_gemm_runtime_init(int device_id, size_t workspace_bytes) {
    hd_gemm_runtime* rt = (hd_gemm_runtime*)calloc(1, sizeof(*rt));
    if (rt) { rt->device_id = device_id; rt->workspace_bytes = workspace_bytes; }
    return rt;
}
void hd_gemm_runtime_destroy(hd_gemm_runtime* rt) { free(rt); }
void* hd_gemm_workspace(hd_gemm_runtime*) { return nullptr; }
size_t hd_gemm_workspace_bytes(hd_gemm_runtime*) { return 0; }
void hd_gemm_set_backend(int) {}
void hd_gemm_set_prod_backend(int) {}

}  // extern "C"

// ====================================================== prefix-causal mask probe
// The reference passes attention structure as a bf16 [S,S] additive tensor
// (0 / 0xFF7F).  This path only needs ar_len; it is recovered with O(S)
// reads: row r is causal iff its last column is masked, and for a
// prefix-causal mask the causal rows are exactly [0, ar_len).  Each row is
// also checked at its diagonal (must be open) and just right of it (must be
// closed for causal rows, open otherwise); a mismatch reports -1.
__global__ void mask_probe_kernel(const uint16_t* __restrict__ mask, int S, int* __restrict__ out) {
    __shared__ int s_cnt, s_bad, s_last_causal;
    if (threadIdx.x == 0) { s_cnt = 0; s_bad = 0; s_last_causal = -1; }
    __syncthreads();
    for (int r = threadIdx.x; r < S; r += blockDim.x) {
        const uint16_t* row = mask + (size_t)r * S;
        const bool causal = (r < S - 1) && (row[S - 1] != 0) && (row[S - 1] != 0x8000);
        if (causal) { atomicAdd(&s_cnt, 1); atomicMax(&s_last_causal, r); }
        const bool diag_open = (row[r] == 0) || (row[r] == 0x8000);
        bool right_ok = true;
        if (r + 1 < S) {
            const bool right_open = (row[r + 1] == 0) || (row[r + 1] == 0x8000);
            right_ok = causal ? !right_open : right_open;
        }
        if (!diag_open || !right_ok) atomicAdd(&s_bad, 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // causal rows must form the prefix [0, cnt)
        const bool prefix = (s_cnt == 0) || (s_last_causal == s_cnt - 1);
        out[0] = (s_bad == 0 && prefix) ? s_cnt : -1;
    }
}

// Probed on every call: a caller may free and re-allocate, or rewrite in place, a mask at the same address
// with another causal prefix (o1.c allocates its mask per request, src/runtime/generate.c:1202-1209), so
// nothing about a mask pointer may be remembered.  Costs O(S) reads and one stream synchronisation; callers
// that pass an hd_sdpa_plan created with ar_len never come here.
static int probe_ar_len(const void* mask_dev, int S, cudaStream_t st) {
    int* w = device_error_word();
    if (!w) return -1;
    int* slot = w + 1;
    mask_probe_kernel<<<1, 1024, 0, st>>>((const uint16_t*)mask_dev, S, slot);
    count();
    int v = -1;
    if (cudaMemcpyAsync(&v, slot, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess) return -1;
    if (cudaStreamSynchronize(st) != cudaSuccess) return -1;
    return v;
}

extern "C" {

// ================================================================== sdpa shim
static int sdpa_new(hd_sdpa_plan** out, int batch, int qh, int kvh, int seq, int ar_len, int hd,
                    float scale) {
    if (!out || batch != 1 || hd != 128 || qh <= 0 || kvh <= 0 || (qh % kvh) != 0 || seq <= 0) {
        set_error("sdpa: unsupported shape (batch must be 1, head_dim 128)");
        return 1;
    }
    hd_sdpa_plan* p = (hd_sdpa_plan*)calloc(1, sizeof(*p));
    if (!p) { set_error("sdpa: out of host memory"); return 1; }
    p->q_heads = qh; p->kv_heads = kvh; p->seq = seq; p->ar_len = ar_len; p->head_dim = hd;
    p->scale = scale;
    *out = p;
    return 0;
}
int hd_sdpa_create(hd_sdpa_plan** out, int batch, int qh, int kvh, int seq_q, int seq_kv, int hd,
                   float scale) {
    if (seq_q != seq_kv) { set_error("sdpa: seq_q != seq_kv unsupported"); return 1; }
    return sdpa_new(out, batch, qh, kvh, seq_q, -1, hd, scale);
}
int hd_sdpa_create_split(hd_sdpa_plan** out, int batch, int qh, int kvh, int seq, int ar_len, int hd,
                         float scale) {
    if (ar_len < 0 || ar_len > seq) { set_error("sdpa: bad ar_len"); return 1; }
    return sdpa_new(out, batch, qh, kvh, seq, ar_len, hd, scale);
}
int hd_sdpa_create_prod(hd_sdpa_plan** out, int batch, int qh, int kvh, int seq, int ar_len, int hd,
                        float scale) {
    if (ar_len < 0 || ar_len >= seq) ar_len = -1;  // reference falls back to the masked plan
    return sdpa_new(out, batch, qh, kvh, seq, ar_len, hd, scale);
}
static int sdpa_ar_len(hd_sdpa_plan* p, const void* mask, cudaStream_t st) {
    if (p->ar_len >= 0) return p->ar_len;
    if (!mask) return 0;
    const int ar = probe_ar_len(mask, p->seq, st);
    if (ar < 0) set_error("sdpa: mask is not prefix-causal");
    return ar;
}
int hd_sdpa_execute(hd_sdpa_plan* plan, const void* q, const void* k, const void* v,
                    const void* mask, void* out, void* stream) {
    if (!plan || !q || !k || !v || !out) { set_error("sdpa: null argument"); return 1; }
    cudaStream_t st = stream ? (cudaStream_t)stream : g_stream;
    const int ar = sdpa_ar_len(plan, mask, st);
    if (ar < 0) return 1;
    if (!flash_attention_hm(q, k, v, out, plan->seq, plan->q_heads, plan->kv_heads, ar, plan->scale,
                            true, st))
        return 1;
    count();
    return 0;
}
int hd_sdpa_execute_split(hd_sdpa_plan* plan, const void* q, const void* k, const void* v, void* out,
                          void* stream) {
    if (!plan || plan->ar_len < 0) { set_error("sdpa: not a split plan"); return 1; }
    return hd_sdpa_execute(plan, q, k, v, nullptr, out, stream);
}
int hd_sdpa_execute_split_pass(hd_sdpa_plan* plan, int which, const void* q, const void* k,
                               const void* v, void* out, void* stream) {
    // pass 0 = the causal rows [0, ar_len), pass 1 = the rows [ar_len, seq) that see every key
    // (include/hd_cudnn_sdpa.h:77-82); the same kernel, restricted to that pass's query rows
    if (!plan || plan->ar_len < 0) { set_error("sdpa: not a split plan"); return 1; }
    if (!q || !k || !v || !out || (which != 0 && which != 1)) { set_error("sdpa: bad argument"); return 1; }
    const int lo = which == 0 ? 0 : plan->ar_len, hi = which == 0 ? plan->ar_len : plan->seq;
    if (lo >= hi) return 0;
    cudaStream_t st = stream ? (cudaStream_t)stream : g_stream;
    if (!flash_attention_hm(q, k, v, out, plan->seq, plan->q_heads, plan->kv_heads, plan->ar_len, plan->scale, true,
                            st, lo, hi))
        return 1;
    count();
    return 0;
}
void hd_sdpa_destroy(hd_sdpa_plan* plan) { free(plan); }

void hd_attention_eager(const void* q, const void* k, const void* v, const void* mask, void* scores,
                        void* probs, void* out, int heads, int kv_heads, int seq, int dim,
                        float scaling) {
    // head_dim 128 with a prefix-causal (or no) mask runs the flash kernel and leaves scores / probs untouched
    // (they are O(S^2) buffers this path exists to avoid).  Anything else -- another head_dim, an arbitrary
    // additive mask -- runs the materialising kernels, which need and fill both buffers as the reference does.
    if (!q || !k || !v || !out) { set_error("attention: bad args"); return; }
    int ar = 0;
    if (mask && dim == 128) ar = probe_ar_len(mask, seq, g_stream);
    if (dim != 128 || ar < 0) {
        if (!mask || !scores || !probs) {
            set_error(dim != 128 ? "attention: head_dim != 128 needs the mask, scores and probs buffers"
                                 : "attention: mask is not prefix-causal (the general path needs scores and probs buffers)");
            return;
        }
        if (attention_materialised(q, k, v, mask, scores, probs, out, heads, kv_heads, seq, dim, scaling, g_stream)) count();
        return;
    }
    if (flash_attention_hm(q, k, v, out, seq, heads, kv_heads, ar, scaling, false, g_stream)) count();
}

// =============================================================== decoder block
// scratch layout (bf16 unless noted), every region 256-byte aligned
struct BlockScratch {
    uint16_t *ln, *qkv, *attn, *ar, *post, *swi, *tmp;
    float* cs;   // [S,128] cos|sin table when the block is called stand-alone
    int64_t bytes;
};
static BlockScratch carve_block(void* base, int64_t S, int heads, int kv_heads, int hidden, int ff,
                                int hd) {
    BlockScratch b;
    int64_t o = 0;
    auto take = [&](int64_t nbytes) { int64_t r = o; o += (nbytes + 255) & ~(int64_t)255; return r; };
    const int64_t qkv_cols = (int64_t)(heads + 2 * kv_heads) * hd;
    const int64_t o_ln = take(S * hidden * 2);
    const int64_t o_qkv = take(S * qkv_cols * 2);
    const int64_t o_attn = take(S * heads * hd * 2);
    const int64_t o_ar = take(S * hidden * 2);
    const int64_t o_post = take(S * hidden * 2);
    const int64_t o_swi = take(S * ff * 2);
    const int64_t o_tmp = take(S * hidden * 2);
    const int64_t o_cs = take(S * 128 * 4);
    uint8_t* p = (uint8_t*)base;
    b.ln = (uint16_t*)(p + o_ln); b.qkv = (uint16_t*)(p + o_qkv); b.attn = (uint16_t*)(p + o_attn);
    b.ar = (uint16_t*)(p + o_ar); b.post = (uint16_t*)(p + o_post); b.swi = (uint16_t*)(p + o_swi);
    b.tmp = (uint16_t*)(p + o_tmp); b.cs = (float*)(p + o_cs);
    b.bytes = o;
    return b;
}

int64_t hd_decoder_block_scratch_bytes(int64_t seq, int heads, int kv_heads, int hidden, int ff_hidden,
                                       int head_dim) {
    return carve_block(nullptr, seq, heads, kv_heads, hidden, ff_hidden, head_dim).bytes + 256;
}

}  // extern "C"

#define BLK_TRY(expr, what)                                                   \
    do {                                                                      \
        if (!(expr)) { set_model_error("block: %s: %s", what, g_cuda_err); return HD_ERR_RUNTIME; } \
        count();                                                              \
    } while (0)

static hd_status copy_dd(void* dst, const void* src, size_t bytes, cudaStream_t st) {
    cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) { set_model_error("device copy: %s", cudaGetErrorString(e)); return HD_ERR_IO; }
    return HD_OK;
}

// cs: [S,128] cos|sin table for this sequence (built once per forward).
// mod: NULL (o1.c's block) or the six adaLN vectors [shift_msa | scale_msa | gate_msa | shift_mlp | scale_mlp |
// gate_mlp], each [hidden] bf16: norm * (1 + scale) + shift before a branch, x + gate * branch after it.
static hd_status block_forward(const void* in, const float* cs, int ar_len, const hd_block_binding* bw,
                               void* scratch, hd_block_internals* ints, void* out, int64_t S64,
                               int heads, int kv_heads, int hidden, int ff, int hd, cudaStream_t st,
                               const uint16_t* mod = nullptr) {
    const int S = (int)S64;
    BlockScratch b = carve_block((void*)(((uintptr_t)scratch + 255) & ~(uintptr_t)255), S, heads,
                                 kv_heads, hidden, ff, hd);
    const float eps = 1e-6f;
    const float scaling = (float)(1.0 / sqrt((double)hd));
    const int qc = heads * hd, kc = kv_heads * hd, ld = qc + 2 * kc;

    // 1. input RMSNorm
    BLK_TRY(rmsnorm_mod(in, bw->input_ln, mod ? mod + hidden : nullptr, mod, b.ln, S, hidden, eps, st), "input_norm");
    // 2-6. q/k/v projections into one seq-major buffer [S, qc | kc | kc]; the per-head RMSNorm + MRoPE of q and k
    // (block.c:266-289) run inside the projections' epilogues where the tensor-core tiles cover the shape,
    // otherwise as one in-place kernel per tensor (no head split either way)
    if (gemm_tc_supported(S, qc, hidden, EPI_QKNORM) && gemm_tc_supported(S, kc, hidden, EPI_QKNORM)) {
        // one launch over the three weight tensors (three launches each end in a partly filled wave of tiles)
        BLK_TRY(gemm_qkv(b.ln, hidden, bw->q_proj, bw->k_proj, bw->v_proj, b.qkv, ld, S, qc, kc, hidden, bw->q_norm,
                         bw->k_norm, cs, eps, 0, nullptr, nullptr, nullptr, st), "qkv_proj+norm+rope");
    } else {
        BLK_TRY(gemm_bf16_ld(b.ln, hidden, bw->q_proj, nullptr, b.qkv, ld, S, qc, hidden, EPI_STORE,
                             nullptr, nullptr, 0, 0.f, 0, st), "q_proj");
        BLK_TRY(gemm_bf16_ld(b.ln, hidden, bw->k_proj, nullptr, b.qkv + qc, ld, S, kc, hidden, EPI_STORE,
                             nullptr, nullptr, 0, 0.f, 0, st), "k_proj");
        BLK_TRY(gemm_bf16_ld(b.ln, hidden, bw->v_proj, nullptr, b.qkv + qc + kc, ld, S, kc, hidden,
                             EPI_STORE, nullptr, nullptr, 0, 0.f, 0, st), "v_proj");
        BLK_TRY(qk_norm_rope(b.qkv, ld, S, heads, bw->q_norm, cs, eps, st), "q_norm_rope");
        BLK_TRY(qk_norm_rope(b.qkv + qc, ld, S, kv_heads, bw->k_norm, cs, eps, st), "k_norm_rope");
    }
    // 7. attention, output already seq-major [S, heads*hd]
    // (the SwiGLU buffer is idle until step 11: it holds the partial results of key-split tail items)
    BLK_TRY(flash_attention(b.qkv, ld, b.qkv + qc, ld, b.qkv + qc + kc, ld, b.attn, qc, S, heads,
                            kv_heads, ar_len, scaling, st, b.swi, (size_t)S * ff * 2), "attention");
    // 8-9. o_proj (+ residual)
    if (mod) {
        if (ints && ints->attn_hidden)
            BLK_TRY(gemm_bf16(b.attn, bw->o_proj, nullptr, ints->attn_hidden, S, hidden, qc, EPI_STORE, nullptr,
                              nullptr, 0.f, 0, st), "o_proj");
        BLK_TRY(gemm_bf16_ld(b.attn, qc, bw->o_proj, nullptr, b.ar, hidden, S, hidden, qc, EPI_GATE_RESID,
                             mod + 2 * hidden, in, hidden, 0.f, 0, st), "o_proj+gate+resid");
    } else if (ints && ints->attn_hidden) {
        BLK_TRY(gemm_bf16(b.attn, bw->o_proj, nullptr, b.tmp, S, hidden, qc, EPI_STORE, nullptr,
                          nullptr, 0.f, 0, st), "o_proj");
        BLK_TRY(residual_add(in, b.tmp, b.ar, (size_t)S * hidden, st), "attn_resid");
        if (copy_dd(ints->attn_hidden, b.tmp, (size_t)S * hidden * 2, st) != HD_OK) return HD_ERR_IO;
    } else {
        BLK_TRY(gemm_bf16_ld(b.attn, qc, bw->o_proj, nullptr, b.ar, hidden, S, hidden, qc, EPI_RESID,
                             nullptr, in, hidden, 0.f, 0, st), "o_proj+resid");
    }
    // 10. post-attention RMSNorm
    BLK_TRY(rmsnorm_mod(b.ar, bw->post_ln, mod ? mod + 4 * hidden : nullptr, mod ? mod + 3 * hidden : nullptr, b.post, S,
                        hidden, eps, st), "post_norm");
    // 11. gate|up GEMM with SwiGLU epilogue, then down (+ residual) straight into out
    BLK_TRY(gemm_bf16(b.post, bw->gate_proj, bw->up_proj, b.swi, S, ff, hidden, EPI_SWIGLU, nullptr,
                      nullptr, 0.f, 0, st), "gate_up_swiglu");
    if (mod) {
        if (ints && ints->mlp_out)
            BLK_TRY(gemm_bf16(b.swi, bw->down_proj, nullptr, ints->mlp_out, S, hidden, ff, EPI_STORE, nullptr,
                              nullptr, 0.f, 0, st), "down_proj");
        BLK_TRY(gemm_bf16_ld(b.swi, ff, bw->down_proj, nullptr, out, hidden, S, hidden, ff, EPI_GATE_RESID,
                             mod + 5 * hidden, b.ar, hidden, 0.f, 0, st), "down_proj+gate+resid");
    } else if (ints && ints->mlp_out) {
        BLK_TRY(gemm_bf16(b.swi, bw->down_proj, nullptr, b.tmp, S, hidden, ff, EPI_STORE, nullptr,
                          nullptr, 0.f, 0, st), "down_proj");
        BLK_TRY(residual_add(b.ar, b.tmp, out, (size_t)S * hidden, st), "mlp_resid");
        if (copy_dd(ints->mlp_out, b.tmp, (size_t)S * hidden * 2, st) != HD_OK) return HD_ERR_IO;
    } else {
        BLK_TRY(gemm_bf16_ld(b.swi, ff, bw->down_proj, nullptr, out, hidden, S, hidden, ff, EPI_RESID,
                             nullptr, b.ar, hidden, 0.f, 0, st), "down_proj+resid");
    }
    if (ints) {
        if (ints->ln0 && copy_dd(ints->ln0, b.ln, (size_t)S * hidden * 2, st) != HD_OK) return HD_ERR_IO;
        if (ints->attn_resid && copy_dd(ints->attn_resid, b.ar, (size_t)S * hidden * 2, st) != HD_OK) return HD_ERR_IO;
        if (ints->post_ln && copy_dd(ints->post_ln, b.post, (size_t)S * hidden * 2, st) != HD_OK) return HD_ERR_IO;
    }
    return HD_OK;
}

static bool dims_supported(int heads, int kv_heads, int hidden, int ff, int hd) {
    return hd == 128 && heads > 0 && kv_heads > 0 && (heads % kv_heads) == 0 && (hidden % 256) == 0 &&
           (ff % 128) == 0 && hidden > 0 && ff > 0;
}

extern "C" {

static hd_status decoder_block_entry(const void* in_dev, const float* pos_dev, const void* mask_dev,
                           const hd_block_binding* bw, const int64_t* sec_dev, void* scratch,
                           int64_t scratch_bytes, hd_block_internals* ints, void* out_dev,
                           int64_t seq, int heads, int kv_heads, int hidden, int ff_hidden,
                           int head_dim, hd_sdpa_plan* sdpa, const uint16_t* mod) {
    (void)sec_dev;
    if (!in_dev || !pos_dev || !bw || !scratch || !out_dev || (!mask_dev && !sdpa)) {
        hd_set_error("block: null argument");
        return HD_ERR_MISSING;
    }
    if (!dims_supported(heads, kv_heads, hidden, ff_hidden, head_dim)) {
        hd_set_error("block: unsupported dims (head_dim must be 128)");
        return HD_ERR_UNSUPPORTED;
    }
    if (scratch_bytes < hd_decoder_block_scratch_bytes(seq, heads, kv_heads, hidden, ff_hidden, head_dim)) {
        hd_set_error("block: scratch too small");
        return HD_ERR_OOM;
    }
    int ar_len;
    if (sdpa && sdpa->ar_len >= 0) ar_len = sdpa->ar_len;
    else {
        ar_len = mask_dev ? probe_ar_len(mask_dev, (int)seq, g_stream) : 0;
        if (ar_len < 0) { hd_set_error("block: mask is not prefix-causal"); return HD_ERR_UNSUPPORTED; }
    }
    BlockScratch b = carve_block((void*)(((uintptr_t)scratch + 255) & ~(uintptr_t)255), seq, heads,
                                 kv_heads, hidden, ff_hidden, head_dim);
    if (!mrope_table64(pos_dev, (int)seq, 5000000.0f, b.cs, g_stream)) {
        hd_set_error("block: mrope: %s", g_cuda_err);
        return HD_ERR_RUNTIME;
    }
    count();
    return block_forward(in_dev, b.cs, ar_len, bw, scratch, ints, out_dev, seq, heads, kv_heads, hidden,
                         ff_hidden, head_dim, g_stream, mod);
}

hd_status hd_decoder_block(const void* in_dev, const float* pos_dev, const void* mask_dev,
                           const hd_block_binding* bw, const int64_t* sec_dev, void* scratch,
                           int64_t scratch_bytes, hd_block_internals* ints, void* out_dev,
                           int64_t seq, int heads, int kv_heads, int hidden, int ff_hidden,
                           int head_dim, hd_sdpa_plan* sdpa) {
    return decoder_block_entry(in_dev, pos_dev, mask_dev, bw, sec_dev, scratch, scratch_bytes, ints, out_dev, seq,
                               heads, kv_heads, hidden, ff_hidden, head_dim, sdpa, nullptr);
}

// adaLN variant of the block (six modulation vectors from the timestep embedding); o1.c has no such block
hd_status o1_decoder_block_adaln(const void* in_dev, const float* pos_dev, const void* mask_dev,
                                 const hd_block_binding* bw, const void* mod6_dev, void* scratch,
                                 int64_t scratch_bytes, hd_block_internals* ints, void* out_dev, int64_t seq,
                                 int heads, int kv_heads, int hidden, int ff_hidden, int head_dim,
                                 hd_sdpa_plan* sdpa) {
    if (!mod6_dev || (((uintptr_t)mod6_dev) & 15)) { hd_set_error("block: modulation vectors missing or unaligned"); return HD_ERR_MISSING; }
    return decoder_block_entry(in_dev, pos_dev, mask_dev, bw, nullptr, scratch, scratch_bytes, ints, out_dev, seq,
                               heads, kv_heads, hidden, ff_hidden, head_dim, sdpa, (const uint16_t*)mod6_dev);
}

// mod6 [6*hidden] = Linear(SiLU(t_emb)): w [6*hidden, hidden], b [6*hidden], tmp [hidden] scratch
hd_status o1_adaln_modulation(const void* t_emb_dev, const void* w_dev, const void* b_dev, void* tmp_dev,
                              void* mod6_dev, int hidden) {
    if (!t_emb_dev || !w_dev || !b_dev || !tmp_dev || !mod6_dev || hidden <= 0) { hd_set_error("adaln: null argument"); return HD_ERR_MISSING; }
    if (!silu(t_emb_dev, tmp_dev, (size_t)hidden, g_stream) ||
        !gemm_bf16(tmp_dev, w_dev, nullptr, mod6_dev, 1, 6 * hidden, hidden, EPI_BIAS, b_dev, nullptr, 0.f, 0, g_stream)) {
        hd_set_error("adaln: %s", g_cuda_err);
        return HD_ERR_RUNTIME;
    }
    count(2);
    return HD_OK;
}

// ==================================================================== forward
// workspace layout; names as in src/model/forward.c:117-134 plus "rope_table"
enum { WS_HIDDEN_A, WS_HIDDEN_B, WS_H_TEXT, WS_NORM_OUT, WS_HEAD_OUT, WS_T_EMB, WS_TE_HIDDEN, WS_FREQ,
       WS_FREQ_BF16, WS_T_SCALED, WS_XE_STAGE, WS_XE_OUT, WS_BLOCK_SCRATCH, WS_ROPE, WS_COUNT };

static int64_t forward_layout(int64_t seq, int text_len, int img, int hidden, int heads, int kv_heads,
                              int ff, int hd, int64_t off[WS_COUNT], int64_t* block_bytes) {
    int64_t o = 0;
    auto take = [&](int idx, int64_t nbytes) { off[idx] = o; o += (nbytes + 255) & ~(int64_t)255; };
    take(WS_HIDDEN_A, seq * hidden * 2);
    take(WS_HIDDEN_B, seq * hidden * 2);
    take(WS_H_TEXT, (int64_t)text_len * hidden * 2);
    take(WS_NORM_OUT, seq * hidden * 2);
    take(WS_HEAD_OUT, seq * 3072 * 2);
    take(WS_T_EMB, hidden * 2);
    take(WS_TE_HIDDEN, hidden * 2);
    take(WS_FREQ, 256 * 4);
    take(WS_FREQ_BF16, 256 * 2);
    take(WS_T_SCALED, 4);
    take(WS_XE_STAGE, (int64_t)img * 1024 * 2);
    take(WS_XE_OUT, (int64_t)img * hidden * 2);
    take(WS_ROPE, seq * 128 * 4);
    const int64_t bs = hd_decoder_block_scratch_bytes(seq, heads, kv_heads, hidden, ff, hd);
    if (block_bytes) *block_bytes = bs;
    take(WS_BLOCK_SCRATCH, bs);
    return o;
}

int64_t hd_forward_workspace_bytes(int64_t seq, int img_tokens, int heads, int kv_heads, int hidden,
                                   int ff_hidden, int head_dim, int64_t* block_scratch_bytes) {
    int64_t off[WS_COUNT];
    int64_t text = seq - img_tokens;
    if (text < 0) text = 0;
    return forward_layout(seq, (int)text, img_tokens, hidden, heads, kv_heads, ff_hidden, head_dim, off,
                          block_scratch_bytes);
}

int64_t hd_forward_ws_offset(const char* name, int64_t seq, int text_len, int img_tokens, int heads,
                             int kv_heads, int hidden, int ff_hidden, int head_dim,
                             int64_t* block_scratch_bytes) {
    if (!name) return -1;
    int64_t off[WS_COUNT];
    forward_layout(seq, text_len, img_tokens, hidden, heads, kv_heads, ff_hidden, head_dim, off,
                   block_scratch_bytes);
    static const struct { const char* n; int idx; } map[] = {
        {"hidden_a", WS_HIDDEN_A}, {"hidden_b", WS_HIDDEN_B}, {"h_text", WS_H_TEXT},
        {"norm_out", WS_NORM_OUT}, {"head_out", WS_HEAD_OUT}, {"t_emb", WS_T_EMB},
        {"te_hidden", WS_TE_HIDDEN}, {"freq", WS_FREQ}, {"freq_bf16", WS_FREQ_BF16},
        {"t_scaled", WS_T_SCALED}, {"xe_stage", WS_XE_STAGE}, {"xe_out", WS_XE_OUT},
        {"block_scratch", WS_BLOCK_SCRATCH}, {"rope_table", WS_ROPE},
    };
    for (size_t i = 0; i < sizeof(map) / sizeof(map[0]); ++i)
        if (strcmp(map[i].n, name) == 0) return off[map[i].idx];
    return -1;
}

int hd_forward_num_layers(const hd_forward_binding* bw) { return bw ? bw->n_layers : 0; }

}  // extern "C"

#define FWD_TRY(expr, what)                                                     \
    do {                                                                        \
        if (!(expr)) { set_model_error("forward: %s: %s", what, g_cuda_err); return HD_ERR_RUNTIME; } \
        count();                                                                \
    } while (0)
#define FWD_COPY(dst, src, bytes)                                               \
    do {                                                                        \
        if ((dst) && copy_dd((dst), (src), (bytes), st) != HD_OK) return HD_ERR_IO; \
    } while (0)

static hd_status forward_impl(const hd_forward_binding* bw, hd_forward_workspace* ws,
                              const int64_t* input_ids, int T, const float* pos_f32, int ar_len,
                              const void* vinputs, int I, const hd_visual_cond* visual,
                              const float* timestep, int S, int heads, int kv_heads, int H, int ff,
                              int hd, int tms_id, hd_forward_diagnostics* diag, void* out_dev,
                              cudaStream_t st) {
    uint8_t* base = (uint8_t*)ws->hidden_a;
    int64_t off[WS_COUNT], bs_bytes;
    forward_layout(S, T, I, H, heads, kv_heads, ff, hd, off, &bs_bytes);
    uint16_t* hidden_a = (uint16_t*)(base + off[WS_HIDDEN_A]);
    uint16_t* hidden_b = (uint16_t*)(base + off[WS_HIDDEN_B]);
    uint16_t* h_text = (uint16_t*)(base + off[WS_H_TEXT]);
    uint16_t* norm_out = (uint16_t*)(base + off[WS_NORM_OUT]);
    uint16_t* t_emb = (uint16_t*)(base + off[WS_T_EMB]);
    uint16_t* te_hidden = (uint16_t*)(base + off[WS_TE_HIDDEN]);
    float* freq = (float*)(base + off[WS_FREQ]);
    uint16_t* freq_bf16 = (uint16_t*)(base + off[WS_FREQ_BF16]);
    float* t_scaled = (float*)(base + off[WS_T_SCALED]);
    uint16_t* xe_stage = (uint16_t*)(base + off[WS_XE_STAGE]);
    float* rope = (float*)(base + off[WS_ROPE]);
    void* scratch = base + off[WS_BLOCK_SCRATCH];
    const float eps = 1e-6f;

    // step 2: t_emb = t_embedder1(timestep)   (forward.c:253-265)
    FWD_TRY(scale_f32(timestep, t_scaled, 1000.0f, 1, st), "t_scale");
    FWD_TRY(timestep_embed(t_scaled, freq, 1, 256, st), "t_sinusoid");
    FWD_TRY(f32_to_bf16_buf(freq, freq_bf16, 256, st), "t_cast");
    FWD_TRY(gemm_bf16(freq_bf16, bw->te0_w, nullptr, te_hidden, 1, H, 256, EPI_BIAS, bw->te0_b, nullptr,
                      0.f, 0, st), "t_mlp0");
    FWD_TRY(silu(te_hidden, t_emb, (size_t)H, st), "t_silu");
    FWD_TRY(gemm_bf16(t_emb, bw->te2_w, nullptr, te_hidden, 1, H, H, EPI_BIAS, bw->te2_b, nullptr, 0.f,
                      0, st), "t_mlp2");
    // t_emb now lives in te_hidden (the reference copies it back; no need here)
    const uint16_t* t_vec = te_hidden;

    // steps 1+3: text rows, with the tms row(s) replaced by t_emb
    if (visual || (diag && diag->after_embedding)) {
        FWD_TRY(gather_rows(bw->embed_tokens, input_ids, h_text, T, H, 151936, st), "embed");
        if (diag) FWD_COPY(diag->after_embedding, h_text, (size_t)T * H * 2);
        if (visual) {
            FWD_TRY(masked_scatter(h_text, visual->visual_mask, visual->image_embeds, hidden_a, T, H, st),
                    "masked_scatter");
            FWD_TRY(tms_condition(input_ids, hidden_a, t_vec, hidden_a, T, H, tms_id, st), "tms");
        } else {
            FWD_TRY(tms_condition(input_ids, h_text, t_vec, hidden_a, T, H, tms_id, st), "tms");
        }
    } else {
        FWD_TRY(embed_text(bw->embed_tokens, input_ids, t_vec, hidden_a, T, H, 151936, tms_id, st),
                "embed+tms");
    }
    if (diag) FWD_COPY(diag->after_timestep_conditioning, hidden_a, (size_t)T * H * 2);

    // steps 4+5: x_embedder over the image rows, written straight behind the text rows
    uint16_t* img_rows = hidden_a + (size_t)T * H;
    int I_live = I;
    if (ws->xe_ref && ws->n_ref > 0 && ws->n_ref < I) I_live = I - ws->n_ref;
    FWD_TRY(gemm_bf16(vinputs, bw->xe1_w, nullptr, xe_stage, I_live, 1024, 3072, EPI_STORE, nullptr,
                      nullptr, 0.f, 0, st), "x_embed1");
    FWD_TRY(gemm_bf16(xe_stage, bw->xe2_w, nullptr, img_rows, I_live, H, 1024, EPI_BIAS, bw->xe2_b,
                      nullptr, 0.f, 0, st), "x_embed2");
    if (I_live < I) FWD_COPY(img_rows + (size_t)I_live * H, ws->xe_ref, (size_t)ws->n_ref * H * 2);
    if (diag) {
        FWD_COPY(diag->after_target_embedding, img_rows, (size_t)I * H * 2);
        FWD_COPY(diag->after_block_0_input, hidden_a, (size_t)S * H * 2);
    }

    // rotary table once per forward (the reference rebuilds it in every block)
    FWD_TRY(mrope_table64(pos_f32, S, 5000000.0f, rope, st), "mrope_table");

    // step 6: decoder blocks, ping-pong
    const void* cur_in = hidden_a;
    void* cur_out = hidden_b;
    const int n = bw->n_layers;
    for (int i = 0; i < n; ++i) {
        hd_status s = block_forward(cur_in, rope, ar_len, &bw->blocks[i], scratch, nullptr, cur_out, S,
                                    heads, kv_heads, H, ff, hd, st);
        if (s != HD_OK) return s;
        if (diag) {
            void* dst = nullptr;
            if (i == 0) dst = diag->after_block_0;
            else if (i == n / 2) dst = diag->after_block_mid;
            else if (i == n - 1) dst = diag->after_block_last;
            FWD_COPY(dst, cur_out, (size_t)S * H * 2);
        }
        if (visual && i < 3) {
            FWD_TRY(deepstack_inject(cur_out, visual->visual_mask, visual->deepstack[i], (void*)cur_in, S,
                                     H, st), "deepstack");
        } else {
            void* t = cur_out; cur_out = (void*)cur_in; cur_in = t;
        }
    }
    const void* final_hidden = cur_in;
    if (diag) FWD_COPY(diag->before_final_norm, final_hidden, (size_t)S * H * 2);

    // steps 7+8: final norm, head (+bias) straight into out_dev
    FWD_TRY(rmsnorm(final_hidden, bw->fnorm_w, norm_out, S, H, eps, st), "final_norm");
    if (diag) FWD_COPY(diag->after_final_norm, norm_out, (size_t)S * H * 2);
    FWD_TRY(gemm_bf16(norm_out, bw->fl_w, nullptr, out_dev, S, 3072, H, EPI_BIAS, bw->fl_b, nullptr, 0.f,
                      0, st), "head");
    if (diag) FWD_COPY(diag->after_final_head, out_dev, (size_t)S * 3072 * 2);
    return HD_OK;
}

extern "C" {

hd_status hd_forward(const hd_forward_binding* bw, hd_forward_workspace* ws, const int64_t* input_ids,
                     int text_len, const float* pos_f32, const void* mask_dev, const void* vinputs,
                     int img_tokens, const hd_visual_cond* visual, const float* timestep,
                     const int64_t* sec_dev, int seq, int heads, int kv_heads, int hidden, int ff_hidden,
                     int head_dim, int tms_token_id, hd_forward_diagnostics* diag, void* out_dev,
                     void* stream) {
    (void)sec_dev;
    if (!bw || !ws || !input_ids || !pos_f32 || !vinputs || !timestep || !out_dev ||
        (!mask_dev && !(ws && ws->sdpa))) {
        hd_set_error("forward: null argument");
        return HD_ERR_MISSING;
    }
    if (text_len + img_tokens != seq) { hd_set_error("forward: text+img != seq"); return HD_ERR_MISSING; }
    if (!ws->hidden_a) { hd_set_error("forward: workspace buffer not allocated"); return HD_ERR_MISSING; }
    if (!dims_supported(heads, kv_heads, hidden, ff_hidden, head_dim)) {
        hd_set_error("forward: unsupported dims");
        return HD_ERR_UNSUPPORTED;
    }
    cudaStream_t st = stream ? (cudaStream_t)stream : g_stream;
    int ar_len;
    if (ws->sdpa && ws->sdpa->ar_len >= 0) ar_len = ws->sdpa->ar_len;
    else {
        ar_len = mask_dev ? probe_ar_len(mask_dev, seq, st) : 0;
        if (ar_len < 0) { hd_set_error("forward: mask is not prefix-causal"); return HD_ERR_UNSUPPORTED; }
    }
    return forward_impl(bw, ws, input_ids, text_len, pos_f32, ar_len, vinputs, img_tokens, visual,
                        timestep, seq, heads, kv_heads, hidden, ff_hidden, head_dim, tms_token_id, diag,
                        out_dev, st);
}

// ============================================================ added entry points
int o1_gemm(const void* x, int ldx, const void* w, const void* w2, void* y, int ldy, int M, int N, int K,
            int epi, const void* bias, const void* resid, int ldr, float scale, int force_bn) {
    if (!gemm_bf16_ld(x, ldx, w, w2, y, ldy, M, N, K, epi, bias, resid, ldr, scale, force_bn, g_stream))
        return 1;
    count();
    return 0;
}
int o1_gemm_qkv(const void* x, int ldx, const void* wq, const void* wk, const void* wv, void* y, int ldy, int M, int qc,
                int kc, int K, const void* q_norm, const void* k_norm, const float* cs, float eps) {
    if (!gemm_qkv(x, ldx, wq, wk, wv, y, ldy, M, qc, kc, K, q_norm, k_norm, cs, eps, 0, nullptr, nullptr, nullptr, g_stream))
        return 1;
    count();
    return 0;
}
int o1_flash_attention(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, void* out,
                       int ldo, int S, int heads, int kv_heads, int ar_len, float scale) {
    if (!flash_attention(q, ldq, k, ldk, v, ldv, out, ldo, S, heads, kv_heads, ar_len, scale, g_stream))
        return 1;
    count();
    return 0;
}
int o1_flash_attention_ws(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, void* out,
                          int ldo, int S, int heads, int kv_heads, int ar_len, float scale, void* scratch,
                          size_t scratch_bytes) {
    if (!flash_attention(q, ldq, k, ldk, v, ldv, out, ldo, S, heads, kv_heads, ar_len, scale, g_stream, scratch,
                         scratch_bytes))
        return 1;
    count();
    return 0;
}
void o1_attention_tail_ways(int ways) { attention_tail_ways(ways); }
void o1_attention_tile_mode(int mode) { attention_tile_mode(mode); }
void o1_gemm_pair_mode(int mode) { gemm_pair_mode(mode); }
int o1_gemm_pair_capacity(void) { return gemm_pair_capacity(); }
int o1_mrope_table(const float* pos, int seq, float theta, float* cs) {
    if (!mrope_table64(pos, seq, theta, cs, g_stream)) return 1;
    count();
    return 0;
}
int o1_qk_norm_rope(void* x, int ld, int S, int heads, const void* w, const float* cs, float eps) {
    if (!qk_norm_rope(x, ld, S, heads, w, cs, eps, g_stream)) return 1;
    count();
    return 0;
}
int o1_sched_cfg_flow_step(const void* z, const void* xc, const void* xu, float sigma, float sigma_next,
                           float g, void* z_next, size_t n) {
    if (!sched_cfg_flow_step(z, xc, xu, sigma, sigma_next, g, z_next, n, g_stream)) return 1;
    count();
    return 0;
}
int o1_fill_normal_bf16(void* dst, size_t n, uint64_t seed, float mean, float std) {
    if (!fill_normal_bf16(dst, n, seed, mean, std, g_stream)) return 1;
    count();
    return 0;
}
int o1_fill_normal_f32(float* dst, size_t n, uint64_t seed, float mean, float std) {
    if (!fill_normal_f32(dst, n, seed, mean, std, g_stream)) return 1;
    count();
    return 0;
}

// Both branches with the same text length, positions and causal prefix (BASELINE's CFG definition).
hd_status o1_denoise_step_cfg(const hd_forward_binding* bw, hd_forward_workspace* ws,
                              const int64_t* ids_cond, const int64_t* ids_uncond, int text_len,
                              const float* pos_f32, int ar_len, const void* z, int img_tokens,
                              const float* timestep_dev, float sigma, float sigma_next, float guidance,
                              void* xp_scratch, void* z_next, int heads, int kv_heads, int hidden,
                              int ff_hidden, int head_dim, int tms_token_id) {
    return o1_denoise_step_cfg_ref(bw, ws, ids_cond, ids_uncond, text_len, pos_f32, ar_len, z, img_tokens,
                                   img_tokens, nullptr, timestep_dev, sigma, sigma_next, guidance, xp_scratch,
                                   z_next, heads, kv_heads, hidden, ff_hidden, head_dim, tms_token_id);
}

hd_status o1_denoise_step_cfg_ref(const hd_forward_binding* bw, hd_forward_workspace* ws,
                                  const int64_t* ids_cond, const int64_t* ids_uncond, int text_len,
                                  const float* pos_f32, int ar_len, const void* z, int img_tokens,
                                  int target_tokens, const hd_visual_cond* visual, const float* timestep_dev,
                                  float sigma, float sigma_next, float guidance, void* xp_scratch, void* z_next,
                                  int heads, int kv_heads, int hidden, int ff_hidden, int head_dim,
                                  int tms_token_id) {
    o1_cfg_branch c = {ids_cond, text_len, pos_f32, ar_len, visual};
    o1_cfg_branch u = {ids_uncond, text_len, pos_f32, ar_len, visual};
    return o1_denoise_step_cfg_branches(bw, ws, &c, &u, z, img_tokens, target_tokens, timestep_dev, sigma,
                                        sigma_next, guidance, xp_scratch, z_next, heads, kv_heads, hidden,
                                        ff_hidden, head_dim, tms_token_id);
}

// Each branch brings its own token ids, text length, positions and causal prefix, as o1.c's CFG loop does
// (src/runtime/generate.c:1111-1206 builds a second, normally shorter, sequence for the unconditional prompt;
// :1340-1356 runs it with seq_text_len[1], posd[1], seq_S_uncond and slices its prediction at its own text
// length).  ws must be sized for the longer sequence; xp_scratch holds (S_cond + S_uncond) * 3072 bf16.
hd_status o1_denoise_step_cfg_branches(const hd_forward_binding* bw, hd_forward_workspace* ws,
                                       const o1_cfg_branch* cond, const o1_cfg_branch* uncond, const void* z,
                                       int img_tokens, int target_tokens, const float* timestep_dev, float sigma,
                                       float sigma_next, float guidance, void* xp_scratch, void* z_next, int heads,
                                       int kv_heads, int hidden, int ff_hidden, int head_dim, int tms_token_id) {
    if (target_tokens <= 0 || target_tokens > img_tokens) {
        hd_set_error("denoise_step: target_tokens out of range");
        return HD_ERR_MISSING;
    }
    if (!bw || !ws || !ws->hidden_a || !cond || !uncond || !cond->ids || !uncond->ids || !cond->pos_f32 ||
        !uncond->pos_f32 || cond->text_len <= 0 || uncond->text_len <= 0 || !z || !timestep_dev || !xp_scratch ||
        !z_next) {
        hd_set_error("denoise_step: null argument");
        return HD_ERR_MISSING;
    }
    if (!dims_supported(heads, kv_heads, hidden, ff_hidden, head_dim)) {
        hd_set_error("denoise_step: unsupported dims");
        return HD_ERR_UNSUPPORTED;
    }
    const int Sc = cond->text_len + img_tokens, Su = uncond->text_len + img_tokens;
    uint16_t* xc = (uint16_t*)xp_scratch;
    uint16_t* xu = xc + (size_t)Sc * 3072;
    hd_status s = forward_impl(bw, ws, cond->ids, cond->text_len, cond->pos_f32, cond->ar_len, z, img_tokens,
                               cond->visual, timestep_dev, Sc, heads, kv_heads, hidden, ff_hidden, head_dim,
                               tms_token_id, nullptr, xc, g_stream);
    if (s != HD_OK) return s;
    s = forward_impl(bw, ws, uncond->ids, uncond->text_len, uncond->pos_f32, uncond->ar_len, z, img_tokens,
                     uncond->visual, timestep_dev, Su, heads, kv_heads, hidden, ff_hidden, head_dim, tms_token_id,
                     nullptr, xu, g_stream);
    if (s != HD_OK) return s;
    // target rows start at row text_len of each prediction (generate.c:1330, :1352 slice them by a copy);
    // reference rows that follow the target in z are inputs only and are not stepped
    const size_t n = (size_t)target_tokens * 3072;
    if (!sched_cfg_flow_step(z, xc + (size_t)cond->text_len * 3072, xu + (size_t)uncond->text_len * 3072, sigma,
                             sigma_next, guidance, z_next, n, g_stream)) {
        hd_set_error("denoise_step: scheduler: %s", g_cuda_err);
        return HD_ERR_RUNTIME;
    }
    count();
    return HD_OK;
}

hd_status o1_denoise_step_cfg_host(const hd_forward_binding* bw, hd_forward_workspace* ws,
                                   const int64_t* ids_cond, const int64_t* ids_uncond, int text_len,
                                   const float* pos_f32, int ar_len, const void* z_host, void* z_dev,
                                   int img_tokens, float sigma, float sigma_next, float guidance,
                                   float* timestep_dev, void* xp_scratch, void* z_next_dev,
                                   void* z_next_host, int heads, int kv_heads, int hidden, int ff_hidden,
                                   int head_dim, int tms_token_id) {
    if (!z_host || !z_dev || !z_next_dev || !z_next_host || !timestep_dev) {
        hd_set_error("denoise_step_host: null argument");
        return HD_ERR_MISSING;
    }
    const size_t bytes = (size_t)img_tokens * 3072 * 2;
    const float t = 1.0f - sigma;   // generate.c:1315
    cudaError_t e = cudaMemcpyAsync(z_dev, z_host, bytes, cudaMemcpyHostToDevice, g_stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(timestep_dev, &t, sizeof(float), cudaMemcpyHostToDevice, g_stream);
    if (e != cudaSuccess) { hd_set_error("denoise_step_host: H2D: %s", cudaGetErrorString(e)); return HD_ERR_IO; }
    hd_status s = o1_denoise_step_cfg(bw, ws, ids_cond, ids_uncond, text_len, pos_f32, ar_len, z_dev,
                                      img_tokens, timestep_dev, sigma, sigma_next, guidance, xp_scratch,
                                      z_next_dev, heads, kv_heads, hidden, ff_hidden, head_dim,
                                      tms_token_id);
    if (s != HD_OK) return s;
    e = cudaMemcpyAsync(z_next_host, z_next_dev, bytes, cudaMemcpyDeviceToHost, g_stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(g_stream);
    if (e != cudaSuccess) { hd_set_error("denoise_step_host: D2H: %s", cudaGetErrorString(e)); return HD_ERR_IO; }
    return HD_OK;
}

}  // extern "C"
