/*
 * o1_oracle.c -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * Plain C / OpenMP restatement, on the CPU, of the arithmetic o1.c performs on
 * its denoising hot path.  It exists to check the CUDA library and to be
 * timed as the host baseline; nothing the library ships calls into it.
 * Every function names the o1.c file:line whose arithmetic it follows,
 * including the places where that code rounds to bf16.
 *
 * Pinning: the pieces below are checked (tests/test_oracle_cpu.py) against
 * the reference's own in-tree vectors -- scheduler/sigma dumps
 * (tests/unit/oracle_dump.txt, oracle_dump_matrix.txt), the analytic cases of
 * tests/unit/test_primitives.c, the position rules of tests/unit/test_seq_ref.c
 * and docs/M1_NUMERICAL_CONTRACT.md -- through fixtures under tests/golden/,
 * against outputs of the reference's own CPU code (torch_rng.c, sequence.c,
 * scheduler.c compiled into oracle/_ref), and on the GPU box against the
 * reference's CUDA build (oracle/_ref/libo1ref.so) on identical inputs.
 *
 * Build: make -C oracle oracle   ->  oracle/libo1oracle.so
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ bf16 */
/* src/cuda/cuda_internal.h:21-40, src/cuda/support.cu:21-28: RNE by integer
 * add, NaN not special-cased. */
static inline float bf2f(uint16_t b) {
    uint32_t u = ((uint32_t)b) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static inline uint16_t f2bf(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
static inline float bfr(float f) { return bf2f(f2bf(f)); }

ORC_API float orc_bf16_to_f32(uint16_t b) { return bf2f(b); }
ORC_API uint16_t orc_f32_to_bf16(float f) { return f2bf(f); }
ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------ seeded init
 * The same counter-based generator as the library's o1_fill_normal_* (integer
 * hash -> Irwin-Hall(8) -> one exact int->float conversion, one multiply, one
 * fused-free multiply-add pair), so host and device weights agree bit for bit. */
static inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
ORC_API float orc_hash_normal(uint64_t seed, uint64_t i) {
    const uint64_t a = splitmix64(seed ^ (i * 2 + 0) * 0xD1B54A32D192ED03ull);
    const uint64_t b = splitmix64(seed ^ (i * 2 + 1) * 0xD1B54A32D192ED03ull);
    int sum = 0;
    for (int k = 0; k < 4; ++k) {
        sum += (int)((a >> (16 * k)) & 0xFFFF);
        sum += (int)((b >> (16 * k)) & 0xFFFF);
    }
    return ((float)(sum - 262140)) * (1.0f / 53509.9f);
}
static inline float normal_val(uint64_t seed, uint64_t i, float mean, float std) {
    volatile float prod = std * orc_hash_normal(seed, i); /* no contraction into an fma */
    return mean + prod;
}
ORC_API void orc_fill_normal_bf16(uint16_t *dst, size_t n, uint64_t seed, float mean, float std) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) dst[i] = f2bf(normal_val(seed, i, mean, std));
}
ORC_API void orc_fill_normal_f32(float *dst, size_t n, uint64_t seed, float mean, float std) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) dst[i] = normal_val(seed, i, mean, std);
}
/* rows [row0, row0+nrows) of a [*, cols] tensor whose element (r,c) has counter r*cols+c */
ORC_API void orc_fill_normal_rows_bf16(uint16_t *dst, int64_t row0, int64_t nrows, int64_t cols,
                                       uint64_t seed, float mean, float std) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < nrows; ++r)
        for (int64_t c = 0; c < cols; ++c)
            dst[r * cols + c] = f2bf(normal_val(seed, (uint64_t)((row0 + r) * cols + c), mean, std));
}

/* ------------------------------------------------------------------ RMSNorm
 * src/cuda/norm.cu:12-48: fp32 sum of squares, inv = rsqrt(mean + eps),
 * y = bf16((w * x) * inv). */
ORC_API void orc_rmsnorm(const uint16_t *x, const uint16_t *w, uint16_t *y, int rows, int cols,
                         float eps) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        const uint16_t *xr = x + (size_t)r * cols;
        uint16_t *yr = y + (size_t)r * cols;
        float sq = 0.f;
        for (int i = 0; i < cols; ++i) {
            const float v = bf2f(xr[i]);
            sq += v * v;
        }
        const float inv = 1.0f / sqrtf(sq / (float)cols + eps);
        for (int i = 0; i < cols; ++i) yr[i] = f2bf(bf2f(w[i]) * bf2f(xr[i]) * inv);
    }
}

/* ------------------------------------------------------------------ activations
 * src/cuda/act.cu:13-34, residual.cu:14-23 */
ORC_API void orc_silu(const uint16_t *x, uint16_t *y, size_t n) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        const float v = bf2f(x[i]);
        y[i] = f2bf(v * (1.0f / (1.0f + expf(-v))));
    }
}
ORC_API void orc_swiglu(const uint16_t *g, const uint16_t *u, uint16_t *y, size_t n) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        const float gv = bf2f(g[i]);
        const float sg = 1.0f / (1.0f + expf(-gv));
        y[i] = f2bf(bfr(gv * sg) * bf2f(u[i]));
    }
}
ORC_API void orc_residual_add(const uint16_t *x, const uint16_t *a, uint16_t *y, size_t n) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) y[i] = f2bf(bf2f(x[i]) + bf2f(a[i]));
}

/* ------------------------------------------------------------------ linear
 * y[M,N] = x[M,K] . w[N,K]^T, fp32 accumulate, one bf16 rounding
 * (src/cuda/gemm.cu:35-71, 302-321); a bias is added in a second pass with a
 * second rounding, as the production path does (gemm.cu:226-236, 456-460). */
ORC_API void orc_linear(const uint16_t *x, const uint16_t *w, const uint16_t *bias, uint16_t *y, int M,
                        int N, int K) {
    float *xf = (float *)malloc((size_t)M * K * sizeof(float));
    float *wf = (float *)malloc((size_t)N * K * sizeof(float));
    if (!xf || !wf) { free(xf); free(wf); return; }
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < (size_t)M * K; ++i) xf[i] = bf2f(x[i]);
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < (size_t)N * K; ++i) wf[i] = bf2f(w[i]);
    const int MB = 8;
#pragma omp parallel for collapse(2) schedule(dynamic, 4)
    for (int m0 = 0; m0 < M; m0 += MB) {
        for (int n = 0; n < N; ++n) {
            const float *wr = wf + (size_t)n * K;
            const int mend = m0 + MB < M ? m0 + MB : M;
            for (int m = m0; m < mend; ++m) {
                const float *xr = xf + (size_t)m * K;
                float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                int k = 0;
                for (; k + 8 <= K; k += 8)
                    for (int j = 0; j < 8; ++j) acc[j] += xr[k + j] * wr[k + j];
                float s = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
                for (; k < K; ++k) s += xr[k] * wr[k];
                float v = s;
                if (bias) v = bfr(v) + bf2f(bias[n]);
                y[(size_t)m * N + n] = f2bf(v);
            }
        }
    }
    free(xf);
    free(wf);
}

/* ------------------------------------------------------------------ timestep embed
 * src/cuda/gemm.cu:531-545 */
ORC_API void orc_timestep_embed(const float *t, float *y, int N, int dim) {
    const int half = dim / 2;
    for (int n = 0; n < N; ++n)
        for (int d = 0; d < dim; ++d) {
            const int p = d < half ? d : d - half;
            const float freq = expf(-logf(10000.0f) * (float)p / (float)half);
            const float arg = t[n] * freq;
            float v = (d < half) ? cosf(arg) : sinf(arg);
            if ((dim % 2) && d == dim - 1) v = 0.0f;
            y[n * dim + d] = v;
        }
}

/* ------------------------------------------------------------------ MRoPE
 * src/cuda/rope.cu:28-71: interleaved 3-axis selection; cos/sin fp32 [bs,seq,dim] */
ORC_API void orc_mrope_cos_sin(const float *pos, int bs, int seq, const int64_t *section, int n_section,
                               int dim, float theta, float scaling, int interleaved, float *cosd,
                               float *sind) {
    const int half = dim / 2;
    for (int b = 0; b < bs; ++b)
#pragma omp parallel for schedule(static)
        for (int s = 0; s < seq; ++s)
            for (int k = 0; k < dim; ++k) {
                const int kk = k < half ? k : k - half;
                int axis = 0;
                if (interleaved) {
                    const int chunk = kk / 3, slot = kk % 3;
                    if ((slot == 1 || slot == 2) && slot <= n_section - 1 && chunk < (int)section[slot])
                        axis = slot;
                } else {
                    int acc = 0;
                    for (int t = 0; t < n_section && t < 3; ++t) {
                        if (kk < acc + (int)section[t]) { axis = t; break; }
                        acc += (int)section[t];
                    }
                }
                const float p = pos[(size_t)axis * bs * seq + (size_t)b * seq + s];
                const float base = expf(-logf(theta) * (2.0f * (float)kk) / (float)dim);
                const float ang = base * p;
                cosd[((size_t)b * seq + s) * dim + k] = cosf(ang) * scaling;
                sind[((size_t)b * seq + s) * dim + k] = sinf(ang) * scaling;
            }
}
/* src/cuda/rope.cu:97-134: rotate-half on head-major [heads,seq,dim], three bf16 roundings */
ORC_API void orc_apply_rotary(const uint16_t *x, const float *cosd, const float *sind, uint16_t *y,
                              int heads, int seq, int dim) {
    const int half = dim / 2;
#pragma omp parallel for collapse(2) schedule(static)
    for (int h = 0; h < heads; ++h)
        for (int s = 0; s < seq; ++s) {
            const uint16_t *xr = x + ((size_t)h * seq + s) * dim;
            uint16_t *yr = y + ((size_t)h * seq + s) * dim;
            for (int d = 0; d < dim; ++d) {
                const float x0 = bf2f(xr[d]);
                const float xh = bf2f(xr[d < half ? d + half : d - half]);
                const float a = bfr(x0 * cosd[(size_t)s * dim + d]);
                const float b = bfr(xh * sind[(size_t)s * dim + d]);
                yr[d] = f2bf(bfr(d < half ? a - b : a + b));
            }
        }
}

/* ------------------------------------------------------------------ attention
 * src/cuda/attn.cu:22-113 (eager): fp32 scores = dot * scale + mask, fp32
 * softmax with max subtraction, probs rounded to bf16, fp32 PV, bf16 out;
 * GQA kh = h / (heads/kv_heads).  q [heads,seq,d], k/v [kv,seq,d] head-major,
 * out [seq,heads,d].  The mask is the prefix-causal one of
 * src/runtime/sequence.c:120-142 expressed by ar_len: rows < ar_len see keys
 * <= row (the bf16-min additive entries underflow the others to exactly 0). */
ORC_API void orc_attention(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint16_t *out,
                           int heads, int kv_heads, int seq, int d, float scaling, int ar_len) {
    const int grp = heads / kv_heads;
#pragma omp parallel
    {
        float *sc = (float *)malloc((size_t)seq * sizeof(float));
        float *acc = (float *)malloc((size_t)d * sizeof(float));
#pragma omp for collapse(2) schedule(dynamic, 8)
        for (int h = 0; h < heads; ++h)
            for (int s = 0; s < seq; ++s) {
                const int kh = h / grp;
                const uint16_t *qr = q + ((size_t)h * seq + s) * d;
                const int nk = (s < ar_len) ? s + 1 : seq;
                float mx = -INFINITY;
                for (int t = 0; t < nk; ++t) {
                    const uint16_t *kr = k + ((size_t)kh * seq + t) * d;
                    float a = 0.f;
                    for (int i = 0; i < d; ++i) a += bf2f(qr[i]) * bf2f(kr[i]);
                    a *= scaling;
                    sc[t] = a;
                    if (a > mx) mx = a;
                }
                float sum = 0.f;
                for (int t = 0; t < nk; ++t) sum += expf(sc[t] - mx);
                const float inv = 1.0f / sum;
                for (int i = 0; i < d; ++i) acc[i] = 0.f;
                for (int t = 0; t < nk; ++t) {
                    const float p = bfr(expf(sc[t] - mx) * inv);
                    const uint16_t *vr = v + ((size_t)kh * seq + t) * d;
                    for (int i = 0; i < d; ++i) acc[i] += p * bf2f(vr[i]);
                }
                uint16_t *o = out + ((size_t)s * heads + h) * d;
                for (int i = 0; i < d; ++i) o[i] = f2bf(acc[i]);
            }
        free(sc);
        free(acc);
    }
}

/* Same arithmetic on seq-major operands (q [S,ldq], k [S,ldk], v [S,ldv], out [S,ldo], head h at
 * columns [h*d, h*d+d)), optionally only for the listed query rows (rows == NULL: all), so that a
 * sample of a full-size problem can be checked in seconds. out rows not listed are left untouched. */
ORC_API void orc_attention_rows(const uint16_t *q, int ldq, const uint16_t *k, int ldk, const uint16_t *v,
                                int ldv, uint16_t *out, int ldo, int heads, int kv_heads, int seq, int d,
                                float scaling, int ar_len, const int *rows, int nrows) {
    const int grp = heads / kv_heads;
    const int nr = rows ? nrows : seq;
#pragma omp parallel
    {
        float *sc = (float *)malloc((size_t)seq * sizeof(float));
        float *acc = (float *)malloc((size_t)d * sizeof(float));
#pragma omp for collapse(2) schedule(dynamic, 4)
        for (int h = 0; h < heads; ++h)
            for (int ri = 0; ri < nr; ++ri) {
                const int s = rows ? rows[ri] : ri;
                const int kh = h / grp;
                const uint16_t *qr = q + (size_t)s * ldq + (size_t)h * d;
                const int nk = (s < ar_len) ? s + 1 : seq;
                float mx = -INFINITY;
                for (int t = 0; t < nk; ++t) {
                    const uint16_t *kr = k + (size_t)t * ldk + (size_t)kh * d;
                    float a = 0.f;
                    for (int i = 0; i < d; ++i) a += bf2f(qr[i]) * bf2f(kr[i]);
                    a *= scaling;
                    sc[t] = a;
                    if (a > mx) mx = a;
                }
                float sum = 0.f;
                for (int t = 0; t < nk; ++t) sum += expf(sc[t] - mx);
                const float inv = 1.0f / sum;
                for (int i = 0; i < d; ++i) acc[i] = 0.f;
                for (int t = 0; t < nk; ++t) {
                    const float p = bfr(expf(sc[t] - mx) * inv);
                    const uint16_t *vr = v + (size_t)t * ldv + (size_t)kh * d;
                    for (int i = 0; i < d; ++i) acc[i] += p * bf2f(vr[i]);
                }
                uint16_t *o = out + (size_t)s * ldo + (size_t)h * d;
                for (int i = 0; i < d; ++i) o[i] = f2bf(acc[i]);
            }
        free(sc);
        free(acc);
    }
}

/* src/cuda/attn.cu:180-218 */
ORC_API void orc_head_split(const uint16_t *in, uint16_t *out, int seq, int heads, int dim) {
    for (int s = 0; s < seq; ++s)
        for (int h = 0; h < heads; ++h)
            memcpy(out + ((size_t)h * seq + s) * dim, in + ((size_t)s * heads + h) * dim, (size_t)dim * 2);
}
ORC_API void orc_head_merge(const uint16_t *in, uint16_t *out, int seq, int heads, int dim) {
    for (int s = 0; s < seq; ++s)
        for (int h = 0; h < heads; ++h)
            memcpy(out + ((size_t)s * heads + h) * dim, in + ((size_t)h * seq + s) * dim, (size_t)dim * 2);
}

/* ------------------------------------------------------------------ decoder block
 * src/model/block.c:247-356, op for op, each intermediate stored as bf16
 * exactly where the reference stores it.  weights: 11 pointers in the order of
 * hd_block_binding (block.h:48-62).  ints: 5 optional [S,hidden] outputs in
 * the order of hd_block_internals (block.h:34-40), entries may be NULL. */
typedef struct {
    const uint16_t *q_proj, *k_proj, *v_proj, *o_proj, *input_ln, *post_ln, *gate_proj, *up_proj,
        *down_proj, *q_norm, *k_norm;
} orc_block_weights;

/* adaLN pieces of the modulated block variant (no counterpart in o1.c, whose blocks are
 * unmodulated -- "parity unpinned": these define the arithmetic the CUDA variant is checked against).
 * mod = [shift_msa | scale_msa | gate_msa | shift_mlp | scale_mlp | gate_mlp], each [hidden] bf16. */
static void orc_modulate(uint16_t *x, const uint16_t *shift, const uint16_t *scale, int rows, int cols) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < cols; ++c) {
            uint16_t *p = x + (size_t)r * cols + c;
            *p = f2bf(bf2f(*p) * (1.0f + bf2f(scale[c])) + bf2f(shift[c]));
        }
}
static void orc_gated_residual(const uint16_t *x, const uint16_t *branch, const uint16_t *gate, uint16_t *y,
                               int rows, int cols) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < cols; ++c) {
            const size_t i = (size_t)r * cols + c;
            y[i] = f2bf(bf2f(x[i]) + bfr(bf2f(gate[c]) * bf2f(branch[i])));
        }
}
/* mod[6*hidden] = Linear(SiLU(t_emb)): w [6*hidden, hidden], b [6*hidden] */
ORC_API void orc_adaln_modulation(const uint16_t *t_emb, const uint16_t *w, const uint16_t *b, uint16_t *mod,
                                  int hidden) {
    uint16_t *act = (uint16_t *)malloc((size_t)hidden * 2);
    if (!act) return;
    orc_silu(t_emb, act, (size_t)hidden);
    orc_linear(act, w, b, mod, 1, 6 * hidden, hidden);
    free(act);
}

static int decoder_block_impl(const uint16_t *in, const float *pos /* [3,S] */, int ar_len,
                              const orc_block_weights *w, uint16_t *out, uint16_t **ints, int S,
                              int heads, int kv_heads, int hidden, int ff, int hd, const uint16_t *mod);
ORC_API int orc_decoder_block(const uint16_t *in, const float *pos /* [3,S] */, int ar_len,
                              const orc_block_weights *w, uint16_t *out, uint16_t **ints, int S,
                              int heads, int kv_heads, int hidden, int ff, int hd) {
    return decoder_block_impl(in, pos, ar_len, w, out, ints, S, heads, kv_heads, hidden, ff, hd, NULL);
}
/* the same block with adaLN: norm * (1 + scale) + shift before each branch, x + gate * branch after it */
ORC_API int orc_decoder_block_adaln(const uint16_t *in, const float *pos, int ar_len, const orc_block_weights *w,
                                    const uint16_t *mod, uint16_t *out, uint16_t **ints, int S, int heads,
                                    int kv_heads, int hidden, int ff, int hd) {
    if (!mod) return 1;
    return decoder_block_impl(in, pos, ar_len, w, out, ints, S, heads, kv_heads, hidden, ff, hd, mod);
}
static int decoder_block_impl(const uint16_t *in, const float *pos /* [3,S] */, int ar_len,
                              const orc_block_weights *w, uint16_t *out, uint16_t **ints, int S,
                              int heads, int kv_heads, int hidden, int ff, int hd, const uint16_t *mod) {
    const float eps = 1e-6f, theta = 5000000.0f;
    const float scaling = (float)(1.0 / sqrt((double)hd));
    const size_t SH = (size_t)S * heads * hd, SK = (size_t)S * kv_heads * hd, SHID = (size_t)S * hidden,
                 SI = (size_t)S * ff;
    uint16_t *ln = malloc(SHID * 2), *qp = malloc(SH * 2), *q = malloc(SH * 2), *qr = malloc(SH * 2),
             *kp = malloc(SK * 2), *k = malloc(SK * 2), *kr = malloc(SK * 2), *vp = malloc(SK * 2),
             *v = malloc(SK * 2), *as = malloc(SH * 2), *ah = malloc(SHID * 2), *ar = malloc(SHID * 2),
             *post = malloc(SHID * 2), *gate = malloc(SI * 2), *up = malloc(SI * 2), *swi = malloc(SI * 2),
             *mlp = malloc(SHID * 2);
    float *cs = malloc((size_t)S * hd * 4), *sn = malloc((size_t)S * hd * 4);
    int rc = 0;
    if (!ln || !qp || !q || !qr || !kp || !k || !kr || !vp || !v || !as || !ah || !ar || !post || !gate ||
        !up || !swi || !mlp || !cs || !sn) { rc = 1; goto done; }
    const int64_t section[3] = {24, 20, 20};
    orc_rmsnorm(in, w->input_ln, ln, S, hidden, eps);                          /* :248 */
    if (mod) orc_modulate(ln, mod, mod + hidden, S, hidden);
    orc_linear(ln, w->q_proj, NULL, qp, S, heads * hd, hidden);                /* :253 */
    orc_linear(ln, w->k_proj, NULL, kp, S, kv_heads * hd, hidden);
    orc_linear(ln, w->v_proj, NULL, vp, S, kv_heads * hd, hidden);
    orc_head_split(qp, q, S, heads, hd);                                       /* :260 */
    orc_head_split(kp, k, S, kv_heads, hd);
    orc_head_split(vp, v, S, kv_heads, hd);
    orc_rmsnorm(q, w->q_norm, qr, S * heads, hd, eps);                         /* :267 */
    orc_rmsnorm(k, w->k_norm, kr, S * kv_heads, hd, eps);
    orc_mrope_cos_sin(pos, 1, S, section, 3, hd, theta, 1.0f, 1, cs, sn);      /* :275 */
    orc_apply_rotary(qr, cs, sn, q, heads, S, hd);                             /* :281 */
    orc_apply_rotary(kr, cs, sn, k, kv_heads, S, hd);
    orc_attention(q, k, v, as, heads, kv_heads, S, hd, scaling, ar_len);       /* :296-312 */
    orc_linear(as, w->o_proj, NULL, ah, S, hidden, heads * hd);                /* :321 */
    if (mod) orc_gated_residual(in, ah, mod + 2 * hidden, ar, S, hidden);
    else orc_residual_add(in, ah, ar, SHID);                                   /* :326 */
    orc_rmsnorm(ar, w->post_ln, post, S, hidden, eps);                         /* :331 */
    if (mod) orc_modulate(post, mod + 3 * hidden, mod + 4 * hidden, S, hidden);
    orc_linear(post, w->gate_proj, NULL, gate, S, ff, hidden);                 /* :336 */
    orc_linear(post, w->up_proj, NULL, up, S, ff, hidden);
    orc_swiglu(gate, up, swi, SI);                                             /* :340 */
    orc_linear(swi, w->down_proj, NULL, mlp, S, hidden, ff);                   /* :343 */
    if (mod) orc_gated_residual(ar, mlp, mod + 5 * hidden, out, S, hidden);
    else orc_residual_add(ar, mlp, out, SHID);                                 /* :348 */
    if (ints) {
        if (ints[0]) memcpy(ints[0], ln, SHID * 2);
        if (ints[1]) memcpy(ints[1], ah, SHID * 2);
        if (ints[2]) memcpy(ints[2], ar, SHID * 2);
        if (ints[3]) memcpy(ints[3], post, SHID * 2);
        if (ints[4]) memcpy(ints[4], mlp, SHID * 2);
    }
done:
    free(ln); free(qp); free(q); free(qr); free(kp); free(k); free(kr); free(vp); free(v); free(as);
    free(ah); free(ar); free(post); free(gate); free(up); free(swi); free(mlp); free(cs); free(sn);
    return rc;
}

/* ------------------------------------------------------------------ forward
 * src/model/forward.c:249-397.  embed_rows: the T embedding rows already
 * gathered for input_ids (row i = table[ids[i]], OOB ids -> row 0, embed.cu:15-29);
 * globals in the order of hd_forward_binding (forward.h:40-52) without the
 * table.  timestep is the model timestep t = 1 - sigma.  out [S,3072]. */
typedef struct {
    const uint16_t *te0_w, *te0_b, *te2_w, *te2_b, *xe1_w, *xe2_w, *xe2_b, *fl_w, *fl_b, *fnorm_w;
} orc_forward_globals;

/* visual conditioning (forward.c:277-285, 363-369; vision_kernels.cu:344-401): rows of the text block
 * whose vmask byte is set receive the next row of image_embeds before the tms substitution, and after
 * each of the first three blocks the same rows get deepstack[i] added (bf16 add).  vmask NULL = plain T2I. */
ORC_API int orc_forward_visual(const orc_forward_globals *g, const orc_block_weights *blocks, int n_layers,
                               const int64_t *ids, const uint16_t *embed_rows, int T, const float *pos,
                               int ar_len, const uint16_t *vinputs, int I, float timestep, int64_t tms_id,
                               uint16_t *out, uint16_t *hidden_dump, int heads, int kv_heads, int H, int ff,
                               int hd, const uint8_t *vmask /* [S] */, const uint16_t *image_embeds,
                               const uint16_t *const *deepstack /* [3] */);
ORC_API int orc_forward(const orc_forward_globals *g, const orc_block_weights *blocks, int n_layers,
                        const int64_t *ids, const uint16_t *embed_rows, int T, const float *pos,
                        int ar_len, const uint16_t *vinputs, int I, float timestep, int64_t tms_id,
                        uint16_t *out, uint16_t *hidden_dump /* [n_layers+1][S,hidden] or NULL */,
                        int heads, int kv_heads, int H, int ff, int hd) {
    return orc_forward_visual(g, blocks, n_layers, ids, embed_rows, T, pos, ar_len, vinputs, I, timestep, tms_id, out,
                              hidden_dump, heads, kv_heads, H, ff, hd, NULL, NULL, NULL);
}
ORC_API int orc_forward_visual(const orc_forward_globals *g, const orc_block_weights *blocks, int n_layers,
                               const int64_t *ids, const uint16_t *embed_rows, int T, const float *pos,
                               int ar_len, const uint16_t *vinputs, int I, float timestep, int64_t tms_id,
                               uint16_t *out, uint16_t *hidden_dump, int heads, int kv_heads, int H, int ff,
                               int hd, const uint8_t *vmask, const uint16_t *image_embeds,
                               const uint16_t *const *deepstack) {
    const int S = T + I;
    const float eps = 1e-6f;
    uint16_t *ha = malloc((size_t)S * H * 2), *hb = malloc((size_t)S * H * 2);
    uint16_t *xs = malloc((size_t)I * 1024 * 2), *no = malloc((size_t)S * H * 2);
    uint16_t t_emb[16384], te_hidden[16384], freq_bf[256];
    float freq[256];
    if (!ha || !hb || !xs || !no || H > 16384) { free(ha); free(hb); free(xs); free(no); return 1; }
    /* step 2 (:253-265): t*1000 -> sinusoid(256) -> bf16 -> linear+bias -> silu -> linear+bias */
    float ts = timestep * 1000.0f;
    orc_timestep_embed(&ts, freq, 1, 256);
    for (int i = 0; i < 256; ++i) freq_bf[i] = f2bf(freq[i]);
    orc_linear(freq_bf, g->te0_w, g->te0_b, te_hidden, 1, H, 256);
    orc_silu(te_hidden, t_emb, (size_t)H);
    orc_linear(t_emb, g->te2_w, g->te2_b, te_hidden, 1, H, H);
    memcpy(t_emb, te_hidden, (size_t)H * 2);
    /* steps 1+3 (:272-292): text rows, tms rows replaced by t_emb (embed.cu:44-58) */
    for (int i = 0, vr = 0; i < T; ++i) {
        const uint16_t *src = embed_rows + (size_t)i * H;
        if (vmask && vmask[i]) src = image_embeds + (size_t)(vr++) * H;   /* masked scatter first ... */
        if (ids[i] == tms_id) src = t_emb;                                /* ... then the tms substitution */
        memcpy(ha + (size_t)i * H, src, (size_t)H * 2);
    }
    /* steps 4+5 (:301-325): x_embedder proj1 (no bias), proj2 (+bias), concatenated after the text */
    orc_linear(vinputs, g->xe1_w, NULL, xs, I, 1024, 3072);
    orc_linear(xs, g->xe2_w, g->xe2_b, ha + (size_t)T * H, I, H, 1024);
    if (hidden_dump) memcpy(hidden_dump, ha, (size_t)S * H * 2);
    /* step 6 (:341-375) */
    uint16_t *cur_in = ha, *cur_out = hb;
    int rc = 0;
    for (int l = 0; l < n_layers && rc == 0; ++l) {
        rc = orc_decoder_block(cur_in, pos, ar_len, &blocks[l], cur_out, NULL, S, heads, kv_heads, H, ff, hd);
        if (vmask && l < 3 && rc == 0) {                                  /* DeepStack add on the pad rows */
            for (int i = 0, vr = 0; i < S; ++i) {
                if (!vmask[i]) continue;
                const uint16_t *d = deepstack[l] + (size_t)(vr++) * H;
                uint16_t *row = cur_out + (size_t)i * H;
                for (int c = 0; c < H; ++c) row[c] = f2bf(bf2f(row[c]) + bf2f(d[c]));
            }
        }
        if (hidden_dump) memcpy(hidden_dump + (size_t)(l + 1) * S * H, cur_out, (size_t)S * H * 2);
        uint16_t *t = cur_in; cur_in = cur_out; cur_out = t;
    }
    /* steps 7+8 (:388-397) */
    if (rc == 0) {
        orc_rmsnorm(cur_in, g->fnorm_w, no, S, H, eps);
        orc_linear(no, g->fl_w, g->fl_b, out, S, 3072, H);
    }
    free(ha); free(hb); free(xs); free(no);
    return rc;
}

/* ------------------------------------------------------------------ scheduler
 * src/cuda/sched.cu:23-72, 137-144, 164-229: fp32, torch left-to-right order.
 * nvcc contracts a*b+c into an fma in those kernels (default -fmad=true; for p*q + r*s it
 * fuses the first product and rounds the second), so the same contraction is written out
 * here and this file is built with -ffp-contract=off. */
ORC_API void orc_sched_vcond(const uint16_t *z, const uint16_t *xp, float sigma, float *mo, size_t n) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) mo[i] = (bf2f(z[i]) - bf2f(xp[i])) / sigma;
}
ORC_API void orc_sched_cfg_guided(const float *mc, const float *mu, float g, float *mo, size_t n) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) mo[i] = fmaf(1.0f - g, mu[i], g * mc[i]);
}
ORC_API void orc_sched_flow_match_step(const uint16_t *z, const float *mo, float sigma, float sigma_next,
                                       uint16_t *z_next, size_t n) {
    const float dt = sigma_next - sigma;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) z_next[i] = f2bf(fmaf(dt, mo[i], bf2f(z[i])));
}
ORC_API void orc_sched_denoised(const float *z, const float *mo, float sigma, float *den, size_t n) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) den[i] = fmaf(-mo[i], sigma, z[i]);
}
ORC_API void orc_sched_z_next(const float *noise, const float *den, float sigma_next, float s_noise,
                              float *z_next, size_t n) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i)
        z_next[i] = fmaf(sigma_next * noise[i], s_noise, (1.0f - sigma_next) * den[i]);
}
/* vcond x2 -> cfg -> flow-match step, the composition of generate.c:1334,1356-1359 with :900-905 */
ORC_API void orc_sched_cfg_flow_step(const uint16_t *z, const uint16_t *xc, const uint16_t *xu, float sigma,
                                     float sigma_next, float g, uint16_t *z_next, size_t n) {
    const float dt = sigma_next - sigma;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        const float zf = bf2f(z[i]);
        const float mc = (zf - bf2f(xc[i])) / sigma;
        const float mu = (zf - bf2f(xu[i])) / sigma;
        const float mo = fmaf(1.0f - g, mu, g * mc);
        z_next[i] = f2bf(fmaf(dt, mo, zf));
    }
}
ORC_API void orc_unipc_convert(const float *sample, const float *mo, float sigma_cur, float *conv, size_t n) {
    for (size_t i = 0; i < n; ++i) conv[i] = fmaf(-sigma_cur, mo[i], sample[i]);
}
ORC_API void orc_unipc_correct(const float *last, const float *mo0, const float *mo_old, const float *conv,
                               float sig_t, float sig_s0, float alpha_t, float h_phi_1, float B_h,
                               float rhos_c0, float rhos_c1, float inv_rks0, int order_c, float *out,
                               size_t n) {
    for (size_t i = 0; i < n; ++i) {
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
}
ORC_API void orc_unipc_predict(const float *sample, const float *mo0, const float *mo_old, float sig_t,
                               float sig_s0, float alpha_t, float h_phi_1, float B_h, float rhos_p,
                               float inv_rks0, int order_p, float *out, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        float x_t = (sig_t / sig_s0) * sample[i] - alpha_t * h_phi_1 * mo0[i];
        if (order_p == 2) {
            const float D1s = (mo_old[i] - mo0[i]) * inv_rks0;
            x_t -= alpha_t * B_h * (rhos_p * D1s);
        }
        out[i] = x_t;
    }
}

/* sigma schedules, src/model/scheduler.c:26-64 (Dev frozen list) and :117-158
 * (flash / flow_match ramp with shift): fp64 ramp, fp32 result. */
static const int ORC_DEV_TIMESTEPS[28] = {999, 987, 974, 960, 945, 929, 913, 895, 877, 857, 836, 814, 790,
                                          764, 737, 707, 675, 640, 602, 560, 515, 464, 409, 347, 278, 199,
                                          110, 8};
ORC_API int orc_sigmas_dev(float *sigmas /* [29] */) {
    for (int i = 0; i < 28; ++i) sigmas[i] = (float)ORC_DEV_TIMESTEPS[i] / 1000.0f;
    sigmas[28] = 0.0f;
    return 29;
}

/* src/model/scheduler.c:117-158: flash / flow_match ramp in timestep space, shift applied, fp64 -> fp32 */
ORC_API int orc_sigmas_flash(int steps, float shift, float *sigmas /* [steps+1] */) {
    if (steps < 2) return 0;
    const double sh = (double)shift, sigma_max = 1.0, raw_min = 0.0010000000474974513;
    const double sigma_min = sh * raw_min / (1.0 + (sh - 1.0) * raw_min);
    const double lo = sigma_max * 1000.0, hi = sigma_min * 1000.0, d = (hi - lo) / (double)(steps - 1);
    for (int i = 0; i < steps; ++i) {
        const double sig = (lo + d * (double)i) / 1000.0;
        sigmas[i] = (float)(sh * sig / (1.0 + (sh - 1.0) * sig));
    }
    sigmas[steps] = 0.0f;
    return steps + 1;
}
/* src/model/scheduler.c:173-195: default (UniPC) ramp, linear in sigma space */
ORC_API int orc_sigmas_default(int steps, float shift, float *sigmas /* [steps+1] */) {
    if (steps < 1) return 0;
    const double sigma_max = 0.9996664524078369, sh = (double)shift, d = (0.0 - sigma_max) / (double)steps;
    for (int i = 0; i < steps; ++i) {
        const double sig = sigma_max + d * (double)i;
        sigmas[i] = (float)(sh * sig / (1.0 + (sh - 1.0) * sig));
    }
    sigmas[steps] = 0.0f;
    return steps + 1;
}
/* src/model/scheduler.c:197-208 */
ORC_API float orc_noise_scale(int n_sigmas, int step_index, float start, float end) {
    if (step_index < 0) step_index = 0;
    const int num_steps = n_sigmas > 1 ? n_sigmas - 1 : 1;
    if (num_steps <= 1) return start;
    if (step_index >= num_steps) step_index = num_steps - 1;
    return start + (end - start) * (float)step_index / (float)(num_steps - 1);
}
/* per-step noise clamp of the flash path (src/runtime/generate.c:1423-1438): fp64 mean and
 * unbiased std, clip = clip_std * std, clamp in place */
ORC_API void orc_noise_clamp(float *noise, size_t n, float clip_std) {
    if (clip_std <= 0.0f || n < 2) return;
    double m = 0.0;
    for (size_t i = 0; i < n; ++i) m += (double)noise[i];
    m /= (double)n;
    double ss = 0.0;
    for (size_t i = 0; i < n; ++i) { const double d = (double)noise[i] - m; ss += d * d; }
    const float clip = clip_std * (float)sqrt(ss / (double)(n - 1));
    for (size_t i = 0; i < n; ++i) {
        if (noise[i] > clip) noise[i] = clip;
        else if (noise[i] < -clip) noise[i] = -clip;
    }
}

/* ------------------------------------------------------------------ LoRA
 * include/hd_lora.h:10-14, src/model/lora_merge.cu:26-33,86-93: FP32 delta,
 * W = bf16(f32(W) + scale*delta), scale = multiplier*alpha/rank. */
ORC_API void orc_lora_merge(uint16_t *w, const float *up /* [N,R] */, const float *down /* [R,K] */, int N,
                            int K, int R, float scale) {
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) {
        float *acc = (float *)calloc((size_t)K, sizeof(float));
        for (int r = 0; r < R; ++r) {
            const float a = up[(size_t)n * R + r];
            const float *dr = down + (size_t)r * K;
            for (int k = 0; k < K; ++k) acc[k] += a * dr[k];
        }
        for (int k = 0; k < K; ++k) {
            volatile float sd = scale * acc[k];
            w[(size_t)n * K + k] = f2bf(bf2f(w[(size_t)n * K + k]) + sd);
        }
        free(acc);
    }
}

/* ------------------------------------------------------------------ torch RNG
 * src/runtime/torch_rng.c:34-121: mt19937 (torch CPU generator) + the float
 * randn path: uniform fill then Box-Muller in blocks of 16, tail block redrawn. */
typedef struct {
    uint32_t state[624];
    int left, next;
} orc_mt;
static void mt_seed(orc_mt *r, uint64_t seed) {
    r->state[0] = (uint32_t)(seed & 0xffffffffu);
    for (int j = 1; j < 624; ++j)
        r->state[j] = 1812433253u * (r->state[j - 1] ^ (r->state[j - 1] >> 30)) + (uint32_t)j;
    r->left = 1;
    r->next = 0;
}
static inline uint32_t mt_mix(uint32_t u, uint32_t v) {
    return (((u & 0x80000000u) | (v & 0x7fffffffu)) >> 1) ^ ((v & 1u) ? 0x9908b0dfu : 0u);
}
static void mt_refill(orc_mt *r) {
    uint32_t *p = r->state;
    for (int j = 0; j < 624 - 397; ++j) p[j] = p[j + 397] ^ mt_mix(p[j], p[j + 1]);
    for (int j = 624 - 397; j < 623; ++j) p[j] = p[j + 397 - 624] ^ mt_mix(p[j], p[j + 1]);
    p[623] = p[396] ^ mt_mix(p[623], p[0]);
    r->left = 624;
    r->next = 0;
}
static inline uint32_t mt_u32(orc_mt *r) {
    if (--r->left == 0) mt_refill(r);
    uint32_t y = r->state[r->next++];
    y ^= y >> 11;
    y ^= (y << 7) & 0x9d2c5680u;
    y ^= (y << 15) & 0xefc60000u;
    y ^= y >> 18;
    return y;
}
static inline float mt_uniform(orc_mt *r) {
    return (float)((mt_u32(r) & ((1u << 24) - 1u)) * (1.0f / 16777216.0f));
}
static void box_muller_16(float *d) {
    for (int j = 0; j < 8; ++j) {
        const float u1 = 1.0f - d[j];
        const float u2 = d[j + 8];
        const float rad = sqrtf(-2.0f * logf(u1));
        const float th = (float)(6.283185307179586 * (double)u2);
        d[j] = rad * cosf(th);
        d[j + 8] = rad * sinf(th);
    }
}
static void mt_randn(orc_mt *rp, float *out, int64_t n);
ORC_API void orc_torch_randn(uint64_t seed, float *out, int64_t n) {
    orc_mt r;
    mt_seed(&r, seed);
    mt_randn(&r, out, n);
}
/* a generator that keeps its state across calls, as hd_torch_rng does (torch_rng.h) */
ORC_API void *orc_rng_create(uint64_t seed) {
    orc_mt *r = (orc_mt *)malloc(sizeof(orc_mt));
    if (r) mt_seed(r, seed);
    return r;
}
ORC_API void orc_rng_randn(void *r, float *out, int64_t n) { mt_randn((orc_mt *)r, out, n); }
ORC_API void orc_rng_free(void *r) { free(r); }
static void mt_randn(orc_mt *rp, float *out, int64_t n) {
    orc_mt r = *rp;
    if (n >= 16) {
        for (int64_t i = 0; i < n; ++i) out[i] = mt_uniform(&r);
        for (int64_t i = 0; i < n - 15; i += 16) box_muller_16(out + i);
        if (n % 16 != 0) {
            float *d = out + (n - 16);
            for (int j = 0; j < 16; ++j) d[j] = mt_uniform(&r);
            box_muller_16(d);
        }
    } else {
        int cached = 0;
        double cache = 0.0;
        for (int64_t i = 0; i < n; ++i) {
            double ret;
            if (cached) { ret = cache; cached = 0; }
            else {
                const uint64_t v1 = ((uint64_t)mt_u32(&r) << 32) | mt_u32(&r);
                const uint64_t v2 = ((uint64_t)mt_u32(&r) << 32) | mt_u32(&r);
                const double u1 = (double)(v1 & ((1ULL << 53) - 1)) * (1.0 / 9007199254740992.0);
                const double u2 = (double)(v2 & ((1ULL << 53) - 1)) * (1.0 / 9007199254740992.0);
                const double rad = sqrt(-2.0 * log1p(-u2));
                const double theta = 2.0 * 3.14159265358979323846 * u1;
                cache = rad * sin(theta);
                cached = 1;
                ret = rad * cos(theta);
            }
            out[i] = (float)ret;
        }
    }
    *rp = r;
}
ORC_API void orc_torch_rng_u32(uint64_t seed, uint32_t *out, int64_t n) {
    orc_mt r;
    mt_seed(&r, seed);
    for (int64_t i = 0; i < n; ++i) out[i] = mt_u32(&r);
}

/* initial latent: randn(1,3,Hpx,Wpx) with seed+1 (generate.c:78-83), pixel_unshuffle into
 * [tok, c*p*p + p1*p + p2] (generate.c:87-104), times noise_scale (generate.c:1266), bf16 */
ORC_API int orc_initial_latent(uint64_t seed, int height, int width, int patch, float noise_scale,
                               uint16_t *z /* [(H/p)*(W/p), 3*p*p] */) {
    const int gh = height / patch, gw = width / patch;
    const int64_t n = (int64_t)3 * height * width;
    float *noise = (float *)malloc((size_t)n * sizeof(float));
    if (!noise) return 1;
    orc_torch_randn(seed + 1, noise, n);
    const int C = 3 * patch * patch;
    for (int c = 0; c < 3; ++c)
        for (int y = 0; y < height; ++y)
            for (int x = 0; x < width; ++x) {
                const int h = y / patch, p1 = y % patch, w = x / patch, p2 = x % patch;
                const float v = noise[((size_t)c * height + y) * width + x] * noise_scale;
                z[(size_t)(h * gw + w) * C + c * patch * patch + p1 * patch + p2] = f2bf(v);
            }
    (void)gh;
    free(noise);
    return 0;
}

/* ------------------------------------------------------------------ sequence
 * src/runtime/sequence.c:88-118: T2I position ids fp32 [3,S]; ar_len = text_len-1 (:120-142) */
ORC_API int orc_seq_t2i(int text_len, int grid_h, int grid_w, int fix_point, float *pos /* [3,S] */) {
    const int S = text_len + grid_h * grid_w;
    for (int i = 0; i < text_len; ++i) pos[i] = pos[S + i] = pos[2 * S + i] = (float)i;
    for (int h = 0; h < grid_h; ++h)
        for (int w = 0; w < grid_w; ++w) {
            const int idx = text_len + h * grid_w + w;
            pos[idx] = (float)fix_point;
            pos[S + idx] = (float)(fix_point + h);
            pos[2 * S + idx] = (float)(fix_point + w);
        }
    return text_len - 1;
}
/* src/runtime/sequence.c:232-363: K-reference layout.  text_ids [text_len] is the expanded template
 * (K runs of <|vision_start|> + cond_h*cond_w <|image_pad|>) + boi + tms.  Sequence = text | target
 * grid | K reference grids.  Vision blocks in order: K template blocks (positions continue the text,
 * grid at text position), the target (grid at fix_point), K reference blocks (grid at max_pos+1 on all
 * three axes).  geom[r] = {tokens, grid_h, grid_w, cond_h, cond_w}.  Writes ids [S], pos [3,S];
 * returns ar_len = text_len - 1 (rows from the tms token on attend to everything, :375-410), or -1. */
ORC_API int orc_seq_ref(const int64_t *text_ids, int text_len, int K, const int *geom /* [K][5] */, int grid_h,
                        int grid_w, int fix_point, int64_t vision_start_id, int64_t image_pad_id,
                        int64_t *ids, float *pos, int S) {
    const int image_len = grid_h * grid_w;
    int total = text_len + image_len;
    for (int r = 0; r < K; ++r) total += geom[r * 5 + 0];
    if (total != S || K < 0 || K > 20) return -1;
    memcpy(ids, text_ids, (size_t)text_len * sizeof(int64_t));
    int off = text_len;
    ids[off++] = vision_start_id;
    for (int i = 1; i < image_len; ++i) ids[off++] = image_pad_id;
    for (int r = 0; r < K; ++r) {
        ids[off++] = vision_start_id;
        for (int i = 1; i < geom[r * 5 + 0]; ++i) ids[off++] = image_pad_id;
    }
    int vs_pos[41], vs_n = 0;
    for (int i = 0; i < S && vs_n < 41; ++i)
        if (ids[i] == vision_start_id) vs_pos[vs_n++] = i;
    if (vs_n != 2 * K + 1) return -1;
    int max_pos = -1, fp = fix_point, st_pos = 0;
    for (int v = 0; v < 2 * K + 1; ++v) {
        const int ed = vs_pos[v] + 1;
        const int skip = (v < K) ? 0 : 1;
        int tlen = ed - st_pos - (skip ? 1 : 0);
        if (tlen < 0) tlen = 0;
        const int st_idx = (max_pos >= 0) ? max_pos + 1 : 0;
        for (int i = 0; i < tlen; ++i)
            pos[st_pos + i] = pos[S + st_pos + i] = pos[2 * S + st_pos + i] = (float)(st_idx + i);
        max_pos = st_idx + tlen - 1;
        int gh, gw;
        if (v < K) { gh = geom[v * 5 + 3]; gw = geom[v * 5 + 4]; }
        else if (v == K) { gh = grid_h; gw = grid_w; }
        else { gh = geom[(v - K - 1) * 5 + 1]; gw = geom[(v - K - 1) * 5 + 2]; }
        if (gh <= 0 || gw <= 0) return -1;
        int base;
        if (skip) {
            if (fp > 0) fp -= st_idx;
            base = fp + st_idx;
            fp = 0;
        } else {
            base = tlen + st_idx;
        }
        for (int h = 0; h < gh; ++h)
            for (int w = 0; w < gw; ++w) {
                const int idx = st_pos + tlen + h * gw + w;
                pos[idx] = (float)base;
                pos[S + idx] = (float)(base + h);
                pos[2 * S + idx] = (float)(base + w);
            }
        const int gmax = base + ((gh > gw ? gh : gw) - 1);
        if (gmax > max_pos) max_pos = gmax;
        st_pos += tlen + gh * gw;
    }
    for (int i = st_pos; i < S; ++i) {
        const float p = (float)(max_pos + 1 + (i - st_pos));
        pos[i] = pos[S + i] = pos[2 * S + i] = p;
    }
    return text_len - 1;
}
/* the bf16 additive mask itself (0 / 0xFF7F), for checking the mask probe */
ORC_API void orc_prefix_causal_mask(int S, int ar_len, uint16_t *mask /* [S,S] */) {
    for (int r = 0; r < S; ++r)
        for (int c = 0; c < S; ++c) mask[(size_t)r * S + c] = (r < ar_len && c > r) ? 0xFF7Fu : 0u;
}

/* ====================================================================== vision tower
 * Qwen3-VL ViT of the edit modes, src/model/vision.c:345-650 with the kernels of
 * src/cuda/vision_kernels.cu.  Tokens are in the processor's 2x2 block-major order. */

/* vision_kernels.cu:50-87: fp32 sum and sum of squares, var = E[x^2] - mean^2,
 * y = bf16((x - mean) * rsqrt(var + eps) * w + b) */
ORC_API void orc_layernorm(const uint16_t *x, const uint16_t *w, const uint16_t *b, uint16_t *y, int rows,
                           int cols, float eps) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        const uint16_t *xr = x + (size_t)r * cols;
        uint16_t *yr = y + (size_t)r * cols;
        float s = 0.f, ss = 0.f;
        for (int i = 0; i < cols; ++i) {
            const float v = bf2f(xr[i]);
            s += v;
            ss += v * v;
        }
        const float inv = 1.0f / (float)cols;
        const float mean = s * inv;
        const float var = ss * inv - mean * mean;
        const float inv_std = 1.0f / sqrtf(var + eps);
        for (int i = 0; i < cols; ++i) {
            const float v = (bf2f(xr[i]) - mean) * inv_std;
            yr[i] = f2bf(v * bf2f(w[i]) + (b ? bf2f(b[i]) : 0.0f));
        }
    }
}

/* vision_kernels.cu:100-133: exact = 0 tanh form (block MLP), 1 erf form (mergers) */
ORC_API void orc_gelu(const uint16_t *x, uint16_t *y, size_t n, int exact) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        const float v = bf2f(x[i]);
        float r;
        if (exact) {
            r = 0.5f * v * (1.0f + erff(v * 0.7071067811865476f));
        } else {
            const float g = 0.7978845608028654f * (v + 0.044715f * v * v * v);
            r = 0.5f * v * (1.0f + tanhf(g));
        }
        y[i] = f2bf(r);
    }
}

/* src/cuda/rope.cu:155-178 (hd_apply_rotary_f32): fp32 rotation, one bf16 rounding.
 * x, y [heads, seq, dim]; cos / sin [seq, dim]. */
ORC_API void orc_apply_rotary_f32(const uint16_t *x, const float *cosd, const float *sind, uint16_t *y, int heads,
                                  int seq, int dim) {
    const int half = dim / 2;
#pragma omp parallel for collapse(2) schedule(static)
    for (int h = 0; h < heads; ++h)
        for (int s = 0; s < seq; ++s) {
            const uint16_t *xr = x + ((size_t)h * seq + s) * dim;
            uint16_t *yr = y + ((size_t)h * seq + s) * dim;
            for (int d = 0; d < dim; ++d) {
                const float x0 = bf2f(xr[d]);
                const float xh = bf2f(xr[d < half ? d + half : d - half]);
                const float c = cosd[(size_t)s * dim + d], sn = sind[(size_t)s * dim + d];
                yr[d] = f2bf(d < half ? x0 * c - xh * sn : x0 * c + xh * sn);
            }
        }
}

/* Host tables of vision.c:215-280 and :324-328 for an image of grid_h x grid_w patches:
 * idx / wgt [4, n] (bilinear corners in the 48 x 48 learned grid), coords [2, n] (row, col), inv_freq [18]. */
ORC_API void orc_vision_tables(int grid_h, int grid_w, int *idx, float *wgt, int *coords, float *inv_freq) {
    const int side = 48, mw = grid_w / 2, n = grid_h * grid_w;
    for (int r = 0; r < n; ++r) {
        const int blk = r / 4, in = r % 4;
        const int h = (blk / mw) * 2 + in / 2, w = (blk % mw) * 2 + in % 2;
        const float hf = (float)h * (float)(side - 1) / (float)(grid_h - 1);
        const float wf = (float)w * (float)(side - 1) / (float)(grid_w - 1);
        const int h0 = (int)hf, w0 = (int)wf;
        const int h1 = h0 + 1 < side ? h0 + 1 : side - 1, w1 = w0 + 1 < side ? w0 + 1 : side - 1;
        const float dh = hf - (float)h0, dw = wf - (float)w0;
        idx[r] = h0 * side + w0;
        idx[n + r] = h0 * side + w1;
        idx[2 * n + r] = h1 * side + w0;
        idx[3 * n + r] = h1 * side + w1;
        wgt[r] = (1.0f - dh) * (1.0f - dw);
        wgt[n + r] = (1.0f - dh) * dw;
        wgt[2 * n + r] = dh * (1.0f - dw);
        wgt[3 * n + r] = dh * dw;
        coords[r] = h;
        coords[n + r] = w;
    }
    for (int k = 0; k < 18; ++k) inv_freq[k] = 1.0f / powf(10000.0f, (float)(2 * k) / 36.0f);
}

/* Whole tower.  w: the 351 tensors in the order of hd_vision_binding (vision.h:102-109): patch_proj w, b,
 * pos_embed, 27 x {norm1 w b, norm2 w b, qkv w b, proj w b, fc1 w b, fc2 w b}, merger {norm w b, fc1 w b,
 * fc2 w b}, 3 x DeepStack merger.  pixels [n,1536]; image_embeds [n/4,4096]; deepstack NULL or [3][n/4,4096];
 * block_out NULL or [27][n,1152] (every block's output).  Returns 0, or -1 on bad arguments / allocation. */
ORC_API int orc_vision_forward(const uint16_t *const *w, const uint16_t *pixels, int grid_h, int grid_w,
                               uint16_t *image_embeds, uint16_t *deepstack, uint16_t *block_out) {
    enum { H = 1152, HD = 16, D = 72, I = 4304, O = 4096, PD = 1536, MG = 4608, DEPTH = 27 };
    if (!w || !pixels || !image_embeds || grid_h <= 0 || grid_w <= 0 || grid_h % 2 || grid_w % 2) return -1;
    const int n = grid_h * grid_w, m = n / 4;
    const float eps = 1e-6f, scaling = (float)(1.0 / sqrt((double)D));
    const size_t nH = (size_t)n * H;
    int *idx = (int *)malloc((size_t)n * 4 * sizeof(int)), *coords = (int *)malloc((size_t)n * 2 * sizeof(int));
    float *wgt = (float *)malloc((size_t)n * 4 * sizeof(float)), inv_freq[18];
    float *cs = (float *)malloc((size_t)n * D * sizeof(float)), *sn = (float *)malloc((size_t)n * D * sizeof(float));
    uint16_t *buf = (uint16_t *)malloc((nH * 8 + (size_t)n * 3 * H + nH * 5 + (size_t)n * I + (size_t)m * MG * 2) * 2);
    if (!idx || !coords || !wgt || !cs || !sn || !buf) { free(idx); free(coords); free(wgt); free(cs); free(sn); free(buf); return -1; }
    uint16_t *p = buf;
    uint16_t *cur = p; p += nH;
    uint16_t *pos = p; p += nH;
    uint16_t *ln = p; p += nH;
    uint16_t *att = p; p += nH;
    uint16_t *ares = p; p += nH;
    uint16_t *ln2 = p; p += nH;
    uint16_t *f2 = p; p += nH;
    uint16_t *tmp = p; p += nH;
    uint16_t *qkv = p; p += (size_t)n * 3 * H;
    uint16_t *q = p; p += nH;
    uint16_t *k = p; p += nH;
    uint16_t *v = p; p += nH;
    uint16_t *qr = p; p += nH;
    uint16_t *kr = p; p += nH;
    uint16_t *f1 = p; p += (size_t)n * I;
    uint16_t *mn = p; p += (size_t)m * MG;
    uint16_t *mf = p; p += (size_t)m * MG;
    orc_vision_tables(grid_h, grid_w, idx, wgt, coords, inv_freq);

    /* patch embedding, vision_kernels.cu:16-31 (default path): bf16(acc + bias), one rounding */
#pragma omp parallel for schedule(static)
    for (int r = 0; r < n; ++r)
        for (int c = 0; c < H; ++c) {
            float acc = 0.f;
            for (int kk = 0; kk < PD; ++kk) acc += bf2f(pixels[(size_t)r * PD + kk]) * bf2f(w[0][(size_t)c * PD + kk]);
            tmp[(size_t)r * H + c] = f2bf(acc + bf2f(w[1][c]));
        }
    /* interpolated position embedding :148-168, then hidden = bf16(patch + pos) (vision.c:439) */
    for (int r = 0; r < n; ++r)
        for (int c = 0; c < H; ++c) {
            float acc = 0.f;
            for (int kk = 0; kk < 4; ++kk) acc += wgt[(size_t)kk * n + r] * bf2f(w[2][(size_t)idx[(size_t)kk * n + r] * H + c]);
            pos[(size_t)r * H + c] = f2bf(acc);
        }
    orc_residual_add(tmp, pos, cur, nH);
    /* rotary tables :183-231: angle = bf16(inv_freq * coord), emb = [rowf | colf | rowf | colf] */
    for (int r = 0; r < n; ++r)
        for (int kk = 0; kk < 36; ++kk) {
            const float a = bfr(inv_freq[kk % 18] * (float)(kk < 18 ? coords[r] : coords[n + r]));
            cs[(size_t)r * D + kk] = cs[(size_t)r * D + 36 + kk] = cosf(a);
            sn[(size_t)r * D + kk] = sn[(size_t)r * D + 36 + kk] = sinf(a);
        }

    const uint16_t *const *bw = w + 3;
    for (int i = 0; i < DEPTH; ++i, bw += 12) {
        orc_layernorm(cur, bw[0], bw[1], ln, n, H, eps);                       /* vision.c:465 */
        orc_linear(ln, bw[4], bw[5], qkv, n, 3 * H, H);                        /* :469 */
        for (int h = 0; h < HD; ++h)                                           /* :473, vision_kernels.cu:283-302 */
            for (int s = 0; s < n; ++s)
                for (int d = 0; d < D; ++d) {
                    const size_t dst = ((size_t)h * n + s) * D + d, src = (size_t)s * 3 * H + (size_t)h * D + d;
                    q[dst] = qkv[src];
                    k[dst] = qkv[src + H];
                    v[dst] = qkv[src + 2 * H];
                }
        orc_apply_rotary_f32(q, cs, sn, qr, HD, n, D);                         /* :475-476 */
        orc_apply_rotary_f32(k, cs, sn, kr, HD, n, D);
        orc_attention(qr, kr, v, att, HD, HD, n, D, scaling, 0);               /* :500 (zero mask: full attention) */
        orc_linear(att, bw[6], bw[7], tmp, n, H, H);                           /* :506 */
        orc_residual_add(cur, tmp, ares, nH);                                  /* :508 */
        orc_layernorm(ares, bw[2], bw[3], ln2, n, H, eps);                     /* :512 */
        orc_linear(ln2, bw[8], bw[9], f1, n, I, H);                            /* :516 */
        orc_gelu(f1, f1, (size_t)n * I, 0);                                    /* :522 */
        orc_linear(f1, bw[10], bw[11], f2, n, H, I);                           /* :525 */
        orc_residual_add(ares, f2, cur, nH);                                   /* :527 */
        if (block_out) memcpy(block_out + (size_t)i * nH, cur, nH * 2);
        if (deepstack && (i == 8 || i == 16 || i == 24)) {                     /* :562-596 */
            const uint16_t *const *ds = w + 3 + 12 * DEPTH + 6 + 6 * (i / 8 - 1);
            orc_layernorm(cur, ds[0], ds[1], mn, m, MG, eps);
            orc_linear(mn, ds[2], ds[3], mf, m, MG, MG);
            orc_gelu(mf, mf, (size_t)m * MG, 1);
            orc_linear(mf, ds[4], ds[5], deepstack + (size_t)(i / 8 - 1) * m * O, m, O, MG);
        }
    }
    const uint16_t *const *mg = w + 3 + 12 * DEPTH;                            /* :617-645 */
    orc_layernorm(cur, mg[0], mg[1], mn, n, H, eps);
    orc_linear(mn, mg[2], mg[3], mf, m, MG, MG);
    orc_gelu(mf, mf, (size_t)m * MG, 1);
    orc_linear(mf, mg[4], mg[5], image_embeds, m, O, MG);
    free(idx); free(coords); free(wgt); free(cs); free(sn); free(buf);
    return 0;
}
