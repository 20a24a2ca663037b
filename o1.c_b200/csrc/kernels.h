// Internal (C++) interface between the kernel files and the host engine.
// Everything here launches on the stream passed in and allocates nothing.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <atomic>

namespace o1 {

// EPI_QKNORM: per-head RMSNorm + rotary of a q / k projection inside the GEMM epilogue (every 128 output columns
// are one head; `bias` carries the norm weight [128], `resid` the fp32 cos|sin table [M,128], `scale` the epsilon)
// EPI_BIAS_GELU: bf16(gelu(bf16(bf16(acc) + bias))), tanh form when `scale` == 0, erf form otherwise (vision tower)
// EPI_BIAS_RESID: bf16(resid + bf16(bf16(acc) + bias)): a biased projection followed by the residual add
// EPI_GATE_RESID: bf16(resid + bf16(gate[col] * bf16(acc))), the gate vector passed as `bias` (adaLN block variant)
// EPI_QKV: q | k | v projections in one launch (gemm_qkv): EPI_QKNORM on the q and k column tiles, EPI_STORE on the v tiles
enum Epi { EPI_STORE = 0, EPI_BIAS = 1, EPI_RESID = 2, EPI_SWIGLU = 3, EPI_LORA = 4, EPI_QKNORM = 6, EPI_BIAS_GELU = 7,
           EPI_BIAS_RESID = 8, EPI_GATE_RESID = 9, EPI_QKV = 10 };

// ---- engine.cu: optional per-launch event timing of the tensor-core kernels.
// kind: 0..4 = GEMM by epilogue (Epi), 5 = flash attention.  Costs two event
// records per launch when enabled, nothing when disabled.
enum { PROF_ATTN = 5, PROF_KINDS = 6 };
void prof_before(int kind, double work, cudaStream_t st);
void prof_after(cudaStream_t st);

// ---- gemm_tc.cu
bool gemm_bf16(const void* x, const void* w, const void* w2, void* y, int M, int N, int K, int epi,
               const void* bias, const void* resid, float scale, int force_bn, cudaStream_t st);
// Same, with explicit row pitches (elements) for x and y so that a GEMM can
// read / write a column slice of a wider buffer.
bool gemm_bf16_ld(const void* x, int ldx, const void* w, const void* w2, void* y, int ldy, int M,
                  int N, int K, int epi, const void* bias, const void* resid, int ldr, float scale,
                  int force_bn, cudaStream_t st);
// Same, plus blocked operand layouts for sequence-parallel exchanges:
//  o_cb / o_cb_stride: output column c is stored at y + (c / o_cb) * o_cb_stride + row * ldy + c % o_cb
//  a_kblk / a_rows   : input column k of row r is read from x[((k / a_kblk) * a_rows + r) * ldx + k % a_kblk]
bool gemm_bf16_ex(const void* x, int ldx, const void* w, const void* w2, void* y, int ldy, int M, int N,
                  int K, int epi, const void* bias, const void* resid, int ldr, float scale, int force_bn,
                  int o_cb, long o_cb_stride, int a_kblk, int a_rows, cudaStream_t st, void* const* o_tab = nullptr);
bool gemm_tc_supported(int M, int N, int K, int epi);
// q | k | v projections + per-head norm + rotary of q and k as one launch; see gemm_tc.cu
bool gemm_qkv(const void* x, int ldx, const void* wq, const void* wk, const void* wv, void* y, int ldy, int M, int qc,
              int kc, int K, const void* q_norm, const void* k_norm, const float* cs, float eps, int n_dst,
              void* const* tq, void* const* tk, void* const* tv, cudaStream_t st);
// copies the (cached) tensor map of a row-major bf16 matrix into *out; false + error text on failure
bool cached_tmap(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_rows);
// sets a kernel's dynamic shared-memory limit once per device (`done`: one bit per device ordinal)
bool func_attr_once(std::atomic<uint64_t>& done, const void* func, int smem_bytes, const char* what);

// ---- attn_tc.cu
// q [S, ldq] (heads*128 columns used), k/v [S, ldk]/[S, ldv] (kv_heads*128),
// out [S, ldo] seq-major; rows < ar_len are causal, rows >= ar_len see all keys.
// scratch (optional, 16-byte aligned): room for the partial results of key-split tail items; without it
// every (256 query rows, head) item is one CTA and the last wave of CTAs may be mostly empty
bool flash_attention(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv,
                     void* out, int ldo, int S, int heads, int kv_heads, int ar_len, float scale,
                     cudaStream_t st, void* scratch = nullptr, size_t scratch_bytes = 0);

// [row_lo, row_hi): the query rows to compute and write (row_hi < 0: all rows)
bool flash_attention_hm(const void* q, const void* k, const void* v, void* out, int S, int heads,
                        int kv_heads, int ar_len, float scale, bool out_head_major, cudaStream_t st,
                        int row_lo = 0, int row_hi = -1);
// tail split policy of flash_attention*: 0 = automatic, 1 = never, n = n key-range parts when they fit
void attention_tail_ways(int ways);
void attention_tile_mode(int mode);   // 0: by sequence length; 1: two query tiles per CTA; 2: one query tile per CTA
int gemm_pair_capacity();
void gemm_pair_mode(int mode);   // 0: single-CTA GEMM tiles only; 1: CTA pairs (cta_group::2) for the large-M families
// seq-major operands; output rows [b*out_rows, (b+1)*out_rows) go to out_tab[b] (row-major, leading
// dimension ldo), which may be peer-mapped memory of another GPU
bool flash_attention_tab(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv,
                         void* const* out_tab, int out_rows, int ldo, int S, int heads, int kv_heads,
                         int ar_len, float scale, cudaStream_t st, void* scratch = nullptr, size_t scratch_bytes = 0);

// ---- elementwise.cu
// O(seq^2) attention that stores bf16 scores and probabilities: any head_dim, any additive bf16 mask [seq,seq]
// (q [heads,seq,dim], k/v [kv_heads,seq,dim] head-major; out [seq,heads,dim])
bool attention_materialised(const void* q, const void* k, const void* v, const void* mask, void* scores, void* probs,
                            void* out, int heads, int kv_heads, int seq, int dim, float scaling, cudaStream_t st);
bool rmsnorm(const void* x, const void* w, void* y, int rows, int cols, float eps, cudaStream_t st);
bool rmsnorm_mod(const void* x, const void* w, const void* scale, const void* shift, void* y, int rows, int cols,
                 float eps, cudaStream_t st);
bool silu(const void* x, void* y, size_t n, cudaStream_t st);
bool swiglu(const void* gate, const void* up, void* y, size_t n, cudaStream_t st);
bool residual_add(const void* x, const void* a, void* y, size_t n, cudaStream_t st);
bool mrope_cos_sin(const float* pos, int bs, int seq, const int64_t* section, int n_section,
                   int head_dim, float theta, float scaling, int interleaved, float* cosd,
                   float* sind, cudaStream_t st);
// compact table: cs[s][0..63] = cos, cs[s][64..127] = sin of the 64 distinct angles
bool mrope_table64(const float* pos, int seq, float theta, float* cs, cudaStream_t st);
// rows [row0, row0+rows) of a sequence whose position ids are pos[3, pos_stride]
bool mrope_table64_rows(const float* pos, int pos_stride, int row0, int rows, float theta, float* cs,
                        cudaStream_t st);
bool apply_rotary(const void* x, const float* cosd, const float* sind, void* y, int heads, int seq,
                  int dim, int f32_mode, cudaStream_t st);
// fused per-head RMSNorm + rotary, in place on a seq-major [S, ld] buffer
// holding `heads` heads of 128 starting at column 0 (weights w[128]).
bool qk_norm_rope(void* x, int ld, int S, int heads, const void* w, const float* cs_table,
                  float eps, cudaStream_t st);
// same with heads grouped in slabs: head h sits at x + (h / hpb) * blk_stride + s * ld + (h % hpb) * 128
bool qk_norm_rope_blocked(void* x, int ld, int S, int heads, int hpb, long blk_stride, const void* w,
                          const float* cs_table, float eps, cudaStream_t st);
bool head_split(const void* in, void* out, int seq, int heads, int dim, cudaStream_t st);
bool head_merge(const void* in, void* out, int seq, int heads, int dim, cudaStream_t st);
bool gather_rows(const void* table, const void* idx, void* out, int M, int cols, int64_t nrows,
                 cudaStream_t st);
bool tms_condition(const void* idx, const void* emb, const void* t_emb, void* out, int M, int H,
                   int64_t tms_id, cudaStream_t st);
// gather + tms substitution in one pass: out[row] = (id==tms) ? t_emb : table[id]
bool embed_text(const void* table, const void* idx, const void* t_emb, void* out, int M, int H,
                int64_t nrows, int64_t tms_id, cudaStream_t st);
bool scale_f32(const float* in, float* out, float s, int n, cudaStream_t st);
bool f32_to_bf16_buf(const float* in, void* out, int n, cudaStream_t st);
bool timestep_embed(const float* t, float* y, int N, int dim, cudaStream_t st);
bool masked_scatter(const void* h_text, const uint8_t* mask, const void* embeds, void* out, int T,
                    int H, cudaStream_t st);
bool deepstack_inject(const void* in, const uint8_t* mask, const void* ds, void* out, int S, int H,
                      cudaStream_t st);
bool fill_normal_bf16(void* dst, size_t n, uint64_t seed, float mean, float std, cudaStream_t st);
bool fill_normal_f32(float* dst, size_t n, uint64_t seed, float mean, float std, cudaStream_t st);
bool transpose_bf16(const void* in, void* out, int rows, int cols, cudaStream_t st);

// ---- sched.cu
bool sched_bf16_upcast(const void* in, float* out, int n, cudaStream_t st);
bool sched_denoised(const float* z, const float* mo, float sigma, float* den, int n, cudaStream_t st);
bool sched_z_next(const float* noise, const float* den, float sigma_next, float s_noise,
                  float* z_next, int n, cudaStream_t st);
bool sched_vcond(const void* z, const void* xp, float sigma, float* mo, int n, cudaStream_t st);
bool sched_flow_match_step(const void* z, const float* mo, float sigma, float sigma_next,
                           void* z_next, int n, cudaStream_t st);
bool sched_cfg_guided(const float* mo_c, const float* mo_u, float g, float* mo, int n, cudaStream_t st);
// fused vcond x2 + cfg + flow-match step (8 bytes / element instead of 40)
bool sched_cfg_flow_step(const void* z, const void* xp_cond, const void* xp_uncond, float sigma,
                         float sigma_next, float g, void* z_next, size_t n, cudaStream_t st);
bool unipc_convert(const float* sample, const float* mo, float sigma_cur, float* conv, int n,
                   cudaStream_t st);
bool unipc_correct(const float* last, const float* mo0, const float* mo_old, const float* conv,
                   float sig_t, float sig_s0, float alpha_t, float h_phi_1, float B_h, float rhos_c0,
                   float rhos_c1, float inv_rks0, int order_c, float* out, int n, cudaStream_t st);
bool unipc_predict(const float* sample, const float* mo0, const float* mo_old, float sig_t,
                   float sig_s0, float alpha_t, float h_phi_1, float B_h, float rhos_p,
                   float inv_rks0, int order_p, float* out, int n, cudaStream_t st);

}  // namespace o1
