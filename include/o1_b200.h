/*
 * o1_b200.h -- C ABI of libo1b200.so: the HiDream-O1 denoising hot path of
 * o1.c (decoder blocks, full forward, flow-matching scheduler / CFG update,
 * load-time LoRA merge) re-implemented for NVIDIA B200 (sm_100a).
 *
 * Three groups of entry points:
 *   1. hd_*  primitive level: same names, argument order and error behaviour as
 *      o1.c's src/cuda/hd_cuda.h:34-198 and src/cuda/gemm.h:35-68 (void
 *      functions on device pointers, errors through hd_cuda_last_error()).
 *   2. hd_*  model level: hd_decoder_block / hd_forward / hd_sdpa_* /
 *      hd_lora_merge_gpu with the signatures of src/model/block.h:26-98,
 *      src/model/forward.h:40-181, include/hd_cudnn_sdpa.h:30-94 and
 *      include/hd_lora.h:32-79, returning hd_status (include/hidream.h:24-35).
 *   3. o1_*  explicit entry points added by this library (stream selection,
 *      fused kernels, the CFG denoise step, seeded initialisers, multi-GPU).
 *
 * All pointers are CUDA device pointers unless a name ends in _host.  No
 * entry point takes or returns a PyTorch type.  Work is enqueued on the
 * library's current stream (o1_set_stream; default: the legacy default
 * stream, as in o1.c).  The library is not re-entrant: one thread at a time,
 * as o1.c's engine (src/server/o1_server.c:926-940 guarantees this).
 */
#ifndef O1_B200_H
#define O1_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ status */
/* include/hidream.h:24-35 */
typedef enum {
    HD_OK = 0,
    HD_ERR_IO = 1,
    HD_ERR_PARSE = 2,
    HD_ERR_PROFILE = 3,
    HD_ERR_MANIFEST = 4,
    HD_ERR_MISMATCH = 5,
    HD_ERR_MISSING = 6,
    HD_ERR_OOM = 7,
    HD_ERR_RUNTIME = 8,
    HD_ERR_UNSUPPORTED = 9
} hd_status;

/* include/hidream.h:37-40 (model-level message buffer) */
const char *hd_last_error(void);
void hd_set_error(const char *fmt, ...);
/* src/cuda/hd_cuda.h:46-47, src/cuda/cuda_internal.h:16 (primitive-level buffer) */
const char *hd_cuda_last_error(void);
void hd_cuda_clear_error(void);
char *hd_cuda_errbuf(void);

/* --------------------------------------------------- 1. primitive level */
/* src/cuda/hd_cuda.h:30-41 -- host bf16 helpers (RNE, no NaN special case) */
float hd_bf16_to_f32(uint16_t b);
uint16_t hd_f32_to_bf16(float f);
void hd_bf16_buf_to_f32(const void *src, float *dst, size_t n);
void hd_f32_buf_to_bf16(const float *src, void *dst, size_t n);

/* src/cuda/hd_cuda.h:58-59 */
void hd_rmsnorm(const void *x_dev, const void *w_dev, void *y_dev, int rows, int cols, float eps);
/* src/cuda/hd_cuda.h:62-68 */
void hd_silu(const void *x_dev, void *y_dev, size_t n);
void hd_swiglu(const void *gate_dev, const void *up_dev, void *y_dev, size_t n);
void hd_residual_add(const void *x_dev, const void *a_dev, void *y_dev, size_t n);
/* src/cuda/hd_cuda.h:76-77, src/cuda/gemm.h:47-58.  y = x W^T (+bias); only
 * transpose_w == 1 is supported, as in the reference. */
void hd_linear(const void *x_dev, const void *w_dev, const void *bias_dev, void *y_dev, int M,
               int N, int K, int transpose_w);
void hd_linear_reference(const void *x_dev, const void *w_dev, const void *bias_dev, void *y_dev,
                         int M, int N, int K, int transpose_w);
/* src/cuda/hd_cuda.h:83 */
void hd_timestep_embed(const float *t_dev, float *y_dev, int N, int dim);
/* src/cuda/hd_cuda.h:90-93 */
void hd_mrope_cos_sin(const float *pos_dev, int bs, int seq, const int64_t *section_dev,
                      int n_section, int head_dim, float theta, float attention_scaling,
                      int interleaved, float *cos_dev, float *sin_dev);
/* src/cuda/hd_cuda.h:99-111 */
void hd_apply_rotary(const void *x_dev, const float *cos_dev, const float *sin_dev, void *y_dev,
                     int heads, int seq, int dim);
void hd_apply_rotary_f32(const void *x_dev, const float *cos_dev, const float *sin_dev,
                         void *y_dev, int heads, int seq, int dim);
/* src/cuda/hd_cuda.h:118-122.  q [heads,seq,dim], k/v [kv_heads,seq,dim],
 * mask [seq,seq] bf16 additive (must be prefix-causal, see hd_sdpa_execute),
 * out [seq,heads,dim].  scores_dev / probs_dev are accepted and left
 * untouched: this implementation never materialises S x S tensors. */
void hd_attention_eager(const void *q_dev, const void *k_dev, const void *v_dev,
                        const void *mask_dev, void *scores_dev, void *probs_dev, void *out_dev,
                        int heads, int kv_heads, int seq, int dim, float scaling);
/* src/cuda/hd_cuda.h:128-129 */
void hd_head_split(const void *in_dev, void *out_dev, int seq, int heads, int dim);
void hd_head_merge(const void *in_dev, void *out_dev, int seq, int heads, int dim);
/* src/cuda/hd_cuda.h:136-146 */
void hd_gather_rows(const void *table_dev, const void *idx_dev, void *out_dev, int M, int cols,
                    int64_t nrows);
void hd_apply_tms_condition(const void *idx_dev, const void *emb_dev, const void *t_emb_dev,
                            void *out_dev, int M, int H, int64_t tms_id);
/* src/cuda/hd_cuda.h:149-151 */
void hd_scale_f32(const float *in_dev, float *out_dev, float s, int n);
void hd_f32_convert_bf16(const float *in_dev, void *out_dev, int n);
/* src/cuda/hd_cuda.h:158-175 -- scheduler pointwise kernels */
void hd_sched_bf16_upcast(const void *in_dev, float *out_dev, int n);
void hd_sched_denoised(const float *z_dev, const float *mo_dev, float sigma, float *denoised_dev,
                       int n);
void hd_sched_z_next(const float *noise_dev, const float *denoised_dev, float sigma_next,
                     float s_noise, float *z_next_dev, int n);
void hd_sched_vcond(const void *z_dev, const void *xp_dev, float sigma, float *mo_dev, int n);
void hd_sched_flow_match_step(const void *z_dev, const float *mo_dev, float sigma,
                              float sigma_next, void *z_next_dev, int n);
/* src/cuda/hd_cuda.h:181-182 */
void hd_sched_cfg_guided(const float *mo_cond, const float *mo_uncond, float g, float *mo_guided,
                         int n);
/* src/cuda/hd_cuda.h:188-198 -- FlowUniPC bh2 pointwise updates */
void hd_unipc_convert(const float *sample_dev, const float *mo_dev, float sigma_cur,
                      float *conv_dev, int n);
void hd_unipc_correct(const float *last_dev, const float *mo0_dev, const float *mo_old_dev,
                      const float *conv_dev, float sig_t, float sig_s0, float alpha_t,
                      float h_phi_1, float B_h, float rhos_c0, float rhos_c1, float inv_rks0,
                      int order_c, float *out_dev, int n);
void hd_unipc_predict(const float *sample_dev, const float *mo0_dev, const float *mo_old_dev,
                      float sig_t, float sig_s0, float alpha_t, float h_phi_1, float B_h,
                      float rhos_p, float inv_rks0, int order_p, float *out_dev, int n);
/* src/cuda/vision_kernels.h:46-51 -- the two vision kernels hd_forward calls */
void hd_vision_masked_scatter(const void *dst, const uint8_t *mask, const void *src, void *out,
                              int rows, int cols);
void hd_vision_deepstack_inject(const void *in, const uint8_t *mask, const void *emb, void *out,
                                int rows, int cols);

/* src/cuda/gemm.h:23-68 -- runtime handle kept for source compatibility.  No
 * library handles exist here; init returns a small tag object. */
typedef struct hd_gemm_runtime hd_gemm_runtime;
hd_gemm_runtime *hd_gemm_runtime_init(int device_id, size_t workspace_bytes);
void hd_gemm_runtime_destroy(hd_gemm_runtime *rt);
void *hd_gemm_workspace(hd_gemm_runtime *rt);
size_t hd_gemm_workspace_bytes(hd_gemm_runtime *rt);
void hd_gemm_set_backend(int use_production);      /* accepted, no effect */
void hd_gemm_set_prod_backend(int backend);        /* accepted, no effect */

/* ------------------------------------------------------ 2. model level */
/* include/hd_cudnn_sdpa.h:30-94.  A plan only records (seq, heads, ar_len,
 * scale): there is nothing to build.  q/k/v/out are head-major [H,S,128]
 * as in the reference.  A plan made by hd_sdpa_create (no ar_len) takes
 * ar_len from the mask passed to hd_sdpa_execute: the mask must be the
 * prefix-causal one of src/runtime/sequence.c:120-142, anything else fails. */
typedef struct hd_sdpa_plan hd_sdpa_plan;
int hd_sdpa_create(hd_sdpa_plan **out, int batch, int q_heads, int kv_heads, int seq_q, int seq_kv,
                   int head_dim, float scale);
int hd_sdpa_create_split(hd_sdpa_plan **out, int batch, int q_heads, int kv_heads, int seq,
                         int ar_len, int head_dim, float scale);
int hd_sdpa_create_prod(hd_sdpa_plan **out, int batch, int q_heads, int kv_heads, int seq,
                        int ar_len, int head_dim, float scale);
int hd_sdpa_execute(hd_sdpa_plan *plan, const void *q, const void *k, const void *v,
                    const void *mask, void *out, void *stream);
int hd_sdpa_execute_split(hd_sdpa_plan *plan, const void *q, const void *k, const void *v,
                          void *out, void *stream);
int hd_sdpa_execute_split_pass(hd_sdpa_plan *plan, int which, const void *q, const void *k,
                               const void *v, void *out, void *stream);
void hd_sdpa_destroy(hd_sdpa_plan *plan);

/* src/model/block.h:34-40 */
typedef struct {
    void *ln0;
    void *attn_hidden;
    void *attn_resid;
    void *post_ln;
    void *mlp_out;
} hd_block_internals;

/* src/model/block.h:48-62 -- all bf16, [out,in] row-major */
typedef struct {
    int layer_idx;
    const void *q_proj;
    const void *k_proj;
    const void *v_proj;
    const void *o_proj;
    const void *input_ln;
    const void *post_ln;
    const void *gate_proj;
    const void *up_proj;
    const void *down_proj;
    const void *q_norm;
    const void *k_norm;
} hd_block_binding;

/* src/model/block.h:26-28.  Returns what THIS implementation needs, which is
 * O(seq): no heads*seq*seq score buffers (src/model/block.c:106-131 has two). */
int64_t hd_decoder_block_scratch_bytes(int64_t seq, int heads, int kv_heads, int hidden,
                                       int ff_hidden, int head_dim);
/* src/model/block.h:90-98.  mask_dev is only read when sdpa == NULL (to
 * recover ar_len); sec_dev is accepted for signature compatibility (the
 * section [24,20,20] is a compile-time constant of the path). */
hd_status hd_decoder_block(const void *in_dev, const float *pos_dev, const void *mask_dev,
                           const hd_block_binding *bw, const int64_t *sec_dev, void *scratch,
                           int64_t scratch_bytes, hd_block_internals *ints, void *out_dev,
                           int64_t seq, int heads, int kv_heads, int hidden, int ff_hidden,
                           int head_dim, hd_sdpa_plan *sdpa);

/* src/model/forward.h:40-59 */
typedef struct {
    const void *embed_tokens;
    const void *te0_w;
    const void *te0_b;
    const void *te2_w;
    const void *te2_b;
    const void *xe1_w;
    const void *xe2_w;
    const void *xe2_b;
    const void *fl_w;
    const void *fl_b;
    const void *fnorm_w;
    int n_layers;
    hd_block_binding *blocks;
} hd_forward_binding;

/* src/model/forward.h:66-93.  Only hidden_a (base of the caller's buffer),
 * xe_ref / n_ref, block_scratch_bytes and sdpa are read. */
typedef struct {
    void *hidden_a;
    void *hidden_b;
    void *h_text;
    void *norm_out;
    void *head_out;
    void *t_emb;
    void *te_hidden;
    void *freq;
    void *freq_bf16;
    void *t_scaled;
    void *xe_stage;
    void *xe_out;
    void *xe_ref;
    int n_ref;
    void *block_scratch;
    int64_t block_scratch_bytes;
    hd_sdpa_plan *sdpa;
} hd_forward_workspace;

/* src/model/forward.h:96-107 */
typedef struct {
    void *after_embedding;
    void *after_timestep_conditioning;
    void *after_target_embedding;
    void *after_block_0_input;
    void *after_block_0;
    void *after_block_mid;
    void *after_block_last;
    void *before_final_norm;
    void *after_final_norm;
    void *after_final_head;
} hd_forward_diagnostics;

/* src/model/forward.h:129-134 */
typedef struct {
    const void *image_embeds;
    const void *deepstack[3];
    const uint8_t *visual_mask;
    int v_tokens;
} hd_visual_cond;

/* src/model/weights.h:75-106: one tensor of the device store / the store itself (one arena) */
typedef struct {
    void *dev_ptr;
    int64_t nbytes;
    char name[256];
} hd_device_alloc;
typedef struct {
    int device_id;
    char device_name[256];
    int compute_major;
    int compute_minor;
    int64_t device_mem_bytes;
    int64_t host_bytes_loaded;
    int64_t device_bytes_allocated;
    int64_t n_allocations;
    int64_t largest_numel;
    char largest_name[256];
    hd_device_alloc *allocs;
    int64_t n_allocs;
    struct hd_gemm_runtime *gemm;
    void *arena_ptr;
    int64_t arena_bytes;
    void *upload_stream; /* cudaStream_t */
} hd_weight_store;
/* src/model/weights.h:125-131.  GGUF v3, tensors F32 / F16 / BF16 (io/gguf.c:196-206), all stored bf16. */
hd_status hd_weights_to_device_gguf(const char *gguf_path, int device_id, hd_weight_store *out);
/* Header only: the same store (arena allocated, tensor addresses fixed) with the payload left unwritten, for ranks
 * that receive the arena bytes from the rank that read the file (e.g. ncclBroadcast of arena_ptr / arena_bytes).
 * The layout depends only on the header and is identical on every rank.  (src/model/weights.c:519-669 reads the
 * whole file on every process.) */
hd_status o1_weights_gguf_layout(const char *gguf_path, int device_id, hd_weight_store *out);
void hd_weight_store_free(hd_weight_store *s);
const char *hd_weights_last_error(void);
/* header-only parse, no GPU needed: returns the tensor count (or -1) and describes tensor `index` */
int64_t o1_gguf_probe(const char *path, int64_t index, char *name_out, size_t name_cap, int64_t *numel, int *type,
                      int64_t *file_offset);
/* src/model/block.h:68-70, src/model/forward.h:115-118: bind tensors by their manifest names */
hd_status hd_block_resolve(const hd_weight_store *wstore, int layer_idx, hd_block_binding *out);

/* src/model/forward.h:122-124 */
int64_t hd_forward_workspace_bytes(int64_t seq, int img_tokens, int heads, int kv_heads, int hidden,
                                   int ff_hidden, int head_dim, int64_t *block_scratch_bytes);
/* src/model/forward.h:152-166.  `stream`, when non-NULL, is a cudaStream_t the
 * forward runs on (the reference ignores it); NULL = the library's current
 * stream. */
hd_status hd_forward(const hd_forward_binding *bw, hd_forward_workspace *ws,
                     const int64_t *input_ids, int text_len, const float *pos_f32,
                     const void *mask_dev, const void *vinputs, int img_tokens,
                     const hd_visual_cond *visual, const float *timestep, const int64_t *sec_dev,
                     int seq, int heads, int kv_heads, int hidden, int ff_hidden, int head_dim,
                     int tms_token_id, hd_forward_diagnostics *diag, void *out_dev, void *stream);
int hd_forward_num_layers(const hd_forward_binding *bw);
hd_status hd_forward_resolve(const hd_weight_store *wstore, int n_layers, hd_forward_binding *out);
void hd_forward_binding_free(hd_forward_binding *b);
/* src/model/forward.h:177-181 */
int64_t hd_forward_ws_offset(const char *name, int64_t seq, int text_len, int img_tokens, int heads,
                             int kv_heads, int hidden, int ff_hidden, int head_dim,
                             int64_t *block_scratch_bytes);

/* include/hd_lora.h:32-45 */
typedef struct {
    char lora_prefix[256];
    char base_tensor[256];
    uint32_t rank;
    uint32_t in_dim;
    uint32_t out_dim;
    float alpha;
    float multiplier;
    void *down_dev; /* [rank, in_dim]  fp32 */
    void *up_dev;   /* [out_dim, rank] fp32 */
    void *base_dev; /* [out_dim, in_dim] bf16, merged in place */
} hd_lora_entry;
/* include/hd_lora.h:75-76.  W = bf16(f32(W) + multiplier*alpha/rank * up@down). */
hd_status hd_lora_merge_gpu(hd_lora_entry *entries, size_t count, void *stream /* cudaStream_t */);
const char *hd_lora_last_error(void);

/* ------------------------------------------------ vision tower (edit / reference-image modes)
 * src/model/vision.h:39-230 and src/cuda/vision_kernels.h:17-51: the Qwen3-VL ViT that turns the patchified
 * conditioning image into `image_embeds` and the three DeepStack tensors consumed by hd_forward
 * (hd_visual_cond).  Frozen configuration: 27 blocks, hidden 1152, 16 heads x 72, MLP 4304, LayerNorm eps
 * 1e-6, GELU tanh in the blocks / erf in the mergers, 2x2 spatial merge into 4096-wide rows. */
#define HD_VISION_DEPTH 27
#define HD_VISION_HIDDEN 1152
#define HD_VISION_HEADS 16
#define HD_VISION_HEAD_DIM 72
#define HD_VISION_INTERMEDIATE 4304
#define HD_VISION_OUT_HIDDEN 4096
#define HD_VISION_MERGE_SIZE 2
#define HD_VISION_PATCH_DIM 1536
#define HD_VISION_NUM_POS 2304
#define HD_VISION_NUM_DS 3
enum {
    HD_B0_INPUT = 0, HD_B0_NORM1, HD_B0_QKV, HD_B0_Q, HD_B0_K, HD_B0_V, HD_B0_Q_ROT, HD_B0_K_ROT,
    HD_B0_ATTN_HEADS, HD_B0_ATTN_MERGED, HD_B0_PROJ, HD_B0_ATTN_RESID, HD_B0_NORM2, HD_B0_FC1, HD_B0_FC2,
    HD_B0_OUTPUT, HD_B0_SNAP_COUNT
};
/* src/model/vision.h:76-109: borrowed bf16 tensors [out, in] of the weight store */
typedef struct {
    const void *norm1_w, *norm1_b, *norm2_w, *norm2_b;   /* [1152] */
    const void *qkv_w, *qkv_b;                           /* [3456,1152], [3456] */
    const void *proj_w, *proj_b;                         /* [1152,1152], [1152] */
    const void *fc1_w, *fc1_b;                           /* [4304,1152], [4304] */
    const void *fc2_w, *fc2_b;                           /* [1152,4304], [1152] */
} hd_vision_block_binding;
typedef struct {
    const void *norm_w, *norm_b;                         /* [1152] (final) or [4608] (DeepStack) */
    const void *fc1_w, *fc1_b;                           /* [4608,4608], [4608] */
    const void *fc2_w, *fc2_b;                           /* [4096,4608], [4096] */
} hd_vision_merger_binding;
typedef struct {
    const void *patch_proj_w, *patch_proj_b;             /* [1152,1536], [1152] */
    const void *pos_embed;                               /* [2304,1152] */
    hd_vision_block_binding blocks[HD_VISION_DEPTH];
    hd_vision_merger_binding merger;
    hd_vision_merger_binding deepstack[HD_VISION_NUM_DS];
} hd_vision_binding;
/* src/model/vision.h:116-180, same fields in the same order.  On input only `patch_out` (= base of a
 * region of hd_vision_workspace_bytes(n) bytes), the table fields filled by hd_vision_prepare_tables and the
 * snapshot pointers are read; `sdpa` is accepted and ignored (attention is this library's flash kernel for
 * every n).  Snapshots that exist on this path: block0_snap, block_out_snaps[], block0_snaps[INPUT, NORM1,
 * QKV, ATTN_MERGED, PROJ, ATTN_RESID, NORM2, FC2, OUTPUT]; the others name tensors that are never
 * materialised here (head-major q/k/v, pre-GELU fc1, merger stages) and are left untouched. */
typedef struct {
    void *patch_out, *pos_emb, *rot, *cosf, *sinf, *h_a, *h_b, *ln1, *qkv, *q, *k, *v, *qr, *kr, *scores, *probs,
        *attn_out, *attn_resid, *ln2, *fc1, *fc2, *mlp_resid, *merged, *merge_norm, *merge_fc1, *merge_fc2,
        *ds_merged, *ds_fc1, *ds_fc2;
    void *pos_idx, *pos_wgt, *rot_coords, *rot_inv;      /* device tables inside `tables` */
    void *tables;                                        /* hd_vision_tables_bytes(n) bytes, caller-owned */
    int tables_n, tables_gh, tables_gw;                  /* what the tables were built for (-1 = nothing) */
    int64_t bytes;
    hd_sdpa_plan *sdpa;
    void *block0_snap;
    void *block0_snaps[HD_B0_SNAP_COUNT];
    void *block_out_snaps[HD_VISION_DEPTH];
    void *merger_snaps[5];
    void *ds_merger_snaps[HD_VISION_NUM_DS][4];
} hd_vision_workspace;
/* src/model/vision.h:184-191: byte offsets from the workspace base.  The workspace here is O(n): -1 marks a
 * tensor of the reference layout that this path never materialises (pos_emb, rot, probs, mask, merged,
 * merge_fc2, ds_fc2).  q, k, v are the three 2048-column slices of one [n, 6144] buffer: head h occupies
 * columns 128h .. 128h+71 of its slice, the remaining 56 are zero, q and k are already rotated (qr = q,
 * kr = k).  `scores` is the attention output in the same padded form [n, 2048]; cosf / sinf are [n, 72] fp32;
 * mlp_resid = h_b (where the 27th block leaves its output). */
typedef struct {
    int64_t patch_out, pos_emb, rot, h_a, h_b, ln1, attn_resid, ln2, fc2, mlp_resid, q, k, v, qr, kr, qkv,
        scores, probs, mask, attn_out, fc1, cosf, sinf, merged, merge_norm, merge_fc1, merge_fc2, ds_merged,
        ds_fc1, ds_fc2, total_bytes;
} hd_vision_offsets;
void hd_vision_layout(int64_t n, int64_t m, hd_vision_offsets *o);
/* src/model/vision.h:197-209 */
hd_status hd_vision_resolve(const hd_weight_store *wstore, hd_vision_binding *out);
int64_t hd_vision_workspace_bytes(int64_t n);
int64_t hd_vision_tables_bytes(int64_t n);
/* src/model/vision.c:288-339: interpolation corners / weights, rotary coordinates and inverse frequencies for
 * an (n = grid_h * grid_w) image, computed on the host and copied into ws->tables (blocking copies: set-up,
 * not forward).  A repeated shape returns at once. */
hd_status hd_vision_prepare_tables(hd_vision_workspace *ws, int n, int grid_h, int grid_w);
/* src/model/vision.h:225-230.  pixel_values [n,1536] bf16 in processor (2x2 block-major) order;
 * image_embeds_out [n/4,4096]; deepstack_out NULL or three [n/4,4096] buffers.  Enqueued on the library's
 * current stream. */
hd_status hd_vision_forward(const hd_vision_binding *bw, hd_vision_workspace *ws, const void *pixel_values, int n,
                            int grid_h, int grid_w, void *image_embeds_out, void *deepstack_out[HD_VISION_NUM_DS]);
/* src/cuda/vision_kernels.h:17-45: the tower's stand-alone kernels (void, errors via hd_cuda_last_error) */
void hd_vision_patch(const void *x, const void *w, const void *bias, void *y, int n, int in_dim, int out_dim);
void hd_vision_layernorm(const void *x, const void *w, const void *b, void *y, int rows, int cols, float eps);
void hd_vision_gelu(const void *x, void *y, size_t n);
void hd_vision_gelu_exact(const void *x, void *y, size_t n);
void hd_vision_pos_interp(const void *pos_embed, const int *idx, const float *wgt, void *y, int n, int hidden);
void hd_vision_rot(const float *inv_freq, const int *coords, void *y, int n, int half);
void hd_vision_rot_cos_sin(const void *rot, float *cosd, float *sind, int n, int half);
void hd_vision_spatial_merge(const void *in, void *out, int gh, int gw, int hidden);
void hd_vision_qkv_split(const void *qkv, void *q, void *k, void *v, int n, int heads, int d);
void hd_vision_attn_merge(const void *hm, void *sm, int heads, int n, int d);

/* ------------------------------------------------ 3. added entry points */
/* adaLN-modulated decoder block (the "6-way modulation from a timestep embedding" block shape).  No counterpart
 * in o1.c, whose blocks are unmodulated (src/model/block.c:247-356) and whose timestep enters as a token
 * (src/cuda/embed.cu:44-58): results are defined by the CPU oracle's orc_decoder_block_adaln only.
 * mod6 = [shift_msa | scale_msa | gate_msa | shift_mlp | scale_mlp | gate_mlp], each [hidden] bf16:
 *   h = bf16(bf16(rmsnorm(x)) * (1 + scale) + shift) before a branch, x = bf16(x + bf16(gate * branch)) after it
 * (the norm kernel and the o_proj / down_proj epilogues take the vectors; no extra pass over the activations).
 * Other arguments as hd_decoder_block.  o1_adaln_modulation: mod6 = Linear(SiLU(t_emb)), w [6*hidden, hidden]. */
hd_status o1_adaln_modulation(const void *t_emb_dev, const void *w_dev, const void *b_dev, void *tmp_dev,
                              void *mod6_dev, int hidden);
hd_status o1_decoder_block_adaln(const void *in_dev, const float *pos_dev, const void *mask_dev,
                                 const hd_block_binding *bw, const void *mod6_dev, void *scratch,
                                 int64_t scratch_bytes, hd_block_internals *ints, void *out_dev, int64_t seq,
                                 int heads, int kv_heads, int hidden, int ff_hidden, int head_dim,
                                 hd_sdpa_plan *sdpa);
/* Stream every later call enqueues on (a cudaStream_t; NULL = legacy default). */
void o1_set_stream(void *stream);
void *o1_get_stream(void);
/* Kernels whose bounded waits ran out record a code in a device word;
 * this reads and clears it (synchronises the current stream). 0 = clean. */
int o1_device_error(void);
int o1_sm_count(void);
/* Per-launch CUDA-event timing of the tensor-core kernels on their own stream (off by default;
 * two event records per launch when on).  kind 0..4 = GEMM by epilogue, 5 = flash attention. */
void o1_profile_enable(int on);
int o1_profile_summary(int kind, double *total_ms, int64_t *launches, double *work_flop);
/* Number of kernels this library launched since the last reset. */
int64_t o1_launch_count(int reset);

/* Tensor-core GEMM with a choice of fused epilogue and explicit row pitches.
 * epi: 0 store, 1 +bias, 2 +residual, 3 SwiGLU (w = gate, w2 = up, N = ff),
 * 4 LoRA read-modify-write, 7 +bias then GELU (tanh form when scale == 0, erf form otherwise), 8 +bias then
 * +residual (bf16(resid + bf16(bf16(acc) + bias))).
 * force_bn: 0 auto, 128 or 256.  Shapes: M >= 8 and K % 8 == 0 run on the tensor cores (a ragged last K block
 * is zero-filled); epilogues 0, 1, 7 accept any N % 8 == 0 (ragged right tile edge), the others N % 128 == 0;
 * anything else runs a SIMT kernel (epilogues 0 and 1 only).  Returns 0 on success. */
int o1_gemm(const void *x, int ldx, const void *w, const void *w2, void *y, int ldy, int M, int N,
            int K, int epi, const void *bias, const void *resid, int ldr, float scale, int force_bn);
/* The q, k and v projections of a decoder block (src/model/block.c:257-265) with the per-head RMSNorm + rotary of
 * q and k (:266-289) as ONE launch over the three weight tensors: y [M, qc | kc | kc] (row pitch ldy) =
 * norm_rope(x wq^T) | norm_rope(x wk^T) | x wv^T.  q_norm / k_norm [128] bf16, cs [M,128] fp32 (o1_mrope_table),
 * qc and kc multiples of 128, M >= 8.  Bit-identical to three o1_gemm calls (epilogues 6, 6, 0). */
int o1_gemm_qkv(const void *x, int ldx, const void *wq, const void *wk, const void *wv, void *y, int ldy, int M,
                int qc, int kc, int K, const void *q_norm, const void *k_norm, const float *cs, float eps);
/* Prefix-causal flash attention on seq-major operands: q [S, ldq], k [S, ldk],
 * v [S, ldv], out [S, ldo]; head h at columns [128h, 128h+128). */
int o1_flash_attention(const void *q, int ldq, const void *k, int ldk, const void *v, int ldv,
                       void *out, int ldo, int S, int heads, int kv_heads, int ar_len, float scale);
/* Same with device scratch (16-byte aligned) for key-split tail items: when the number of (256 query rows,
 * head) items is not a multiple of the SM count, the items of the last, partly filled wave are cut along the
 * keys into several CTAs whose fp32 partial results (133,120 bytes each) a merge kernel combines.  The forward
 * and the SP stages pass the idle SwiGLU buffer.  Too little scratch only reduces or disables the split. */
int o1_flash_attention_ws(const void *q, int ldq, const void *k, int ldk, const void *v, int ldv, void *out,
                          int ldo, int S, int heads, int kv_heads, int ar_len, float scale, void *scratch,
                          size_t scratch_bytes);
/* Policy of that split: 0 = automatic (default), 1 = never, n > 1 = n parts whenever scratch and key count allow. */
void o1_attention_tail_ways(int ways);
/* Which attention kernel: 0 = by sequence length (default: one query tile of 128 rows per CTA with triple-buffered
 * scores for S < 8192, two query tiles that share the K/V tiles above), 1 = always the two-tile kernel, 2 = always
 * the one-tile kernel (environment O1_ATTN_TILE_MODE sets the initial value).  Same arithmetic up to fp32 summation
 * order and the reference max of the lazy rescale. */
void o1_attention_tile_mode(int mode);
/* GEMM tile form for the large-M families (plain, bias, residual, SwiGLU, grouped q|k|v) when the problem has at least
 * two rounds of 256 x 256 tiles: 1 (default; environment O1_GEMM_PAIR=0 turns it off) = a cluster of two CTAs per
 * tile with cta_group::2 MMAs, each CTA holding 128 rows of A and of the accumulator and half of the B tile;
 * 0 = one CTA per 128 x 256 tile; 2 = pairs for the SwiGLU family as well (measured 1.6 % slower for that family in
 * the power-capped step, so not the default).  All forms add a row's K products in the same order: same bits.  No reference
 * counterpart (cuBLASLt picks its own kernels there, src/cuda/gemm.cu:413-461). */
void o1_gemm_pair_mode(int mode);
/* CTA pairs of the GEMM kernel the current device holds at once (the pair form never launches more); -1 on error. */
int o1_gemm_pair_capacity(void);
/* cos|sin table [S,128] fp32 for section [24,20,20], theta 5e6 (built once per forward). */
int o1_mrope_table(const float *pos_dev, int seq, float theta, float *cs_dev);
/* Per-head RMSNorm + rotary, in place on [S, ld] holding `heads` heads. */
int o1_qk_norm_rope(void *x, int ld, int S, int heads, const void *w, const float *cs_dev, float eps);
/* z' = bf16(z + (sigma_next-sigma) * ((1-g)*(z-xu)/sigma + g*(z-xc)/sigma)):
 * hd_sched_vcond x2 + hd_sched_cfg_guided + hd_sched_flow_match_step in one pass. */
int o1_sched_cfg_flow_step(const void *z, const void *xp_cond, const void *xp_uncond, float sigma,
                           float sigma_next, float g, void *z_next, size_t n);
/* Seeded counter-based N(mean, std) fill (integer hash, identical on host). */
int o1_fill_normal_bf16(void *dst, size_t n, uint64_t seed, float mean, float std);
int o1_fill_normal_f32(float *dst, size_t n, uint64_t seed, float mean, float std);
float o1_hash_normal_host(uint64_t seed, uint64_t index);

/* No counterpart in the reference.  Merges ONE LoRA target, W = bf16(f32(W) + scale * up@down), without
 * allocating device memory: its FP32 delta scratch is a fixed 16 MiB array inside the library (held by
 * every GPU that loads it).  For hosts that cannot call cudaMalloc: all HBM already owned by their own
 * pool, or other streams busy so that the device-wide stall of cudaMalloc/cudaFree is not acceptable.
 * base_dev [out_dim,in_dim] bf16 (in place), up_dev [out_dim,rank] fp32, down_dev [rank,in_dim] fp32,
 * scale = multiplier*alpha/rank.  Limits: in_dim <= 262144, rank <= 4096, else HD_ERR_UNSUPPORTED.
 * The first call on a device looks up the scratch address (cudaGetSymbolAddress): make that call
 * before any stream capture.  All calls share the scratch: calls that overlap on the GPU race. */
hd_status o1_lora_merge_static(void *base_dev, const float *up_dev, const float *down_dev, uint32_t out_dim,
                               uint32_t in_dim, uint32_t rank, float scale, void *stream);

/* One CFG denoise step on device-resident state: x_c = forward(ids_cond),
 * x_u = forward(ids_uncond), z' = cfg_flow_step(z, x_c, x_u).  Composition of
 * src/runtime/generate.c:1314-1360 with the flow-match update of :900-905.
 * timestep_dev holds t = 1 - sigma.  ws is used for both branches in turn;
 * xp_scratch holds 2 * seq * 3072 bf16. */
hd_status o1_denoise_step_cfg(const hd_forward_binding *bw, hd_forward_workspace *ws,
                              const int64_t *ids_cond, const int64_t *ids_uncond, int text_len,
                              const float *pos_f32, int ar_len, const void *z, int img_tokens,
                              const float *timestep_dev, float sigma, float sigma_next,
                              float guidance, void *xp_scratch, void *z_next, int heads,
                              int kv_heads, int hidden, int ff_hidden, int head_dim,
                              int tms_token_id);
/* Same step for reference / edit sequences (src/runtime/generate.c:858-941): z holds the target latent rows
 * followed by the static reference rows (img_tokens rows in all, the vinputs of hd_forward); only the first
 * target_tokens rows are stepped into z_next [target_tokens, 3072].  visual may be NULL. */
hd_status o1_denoise_step_cfg_ref(const hd_forward_binding *bw, hd_forward_workspace *ws,
                                  const int64_t *ids_cond, const int64_t *ids_uncond, int text_len,
                                  const float *pos_f32, int ar_len, const void *z, int img_tokens,
                                  int target_tokens, const hd_visual_cond *visual, const float *timestep_dev,
                                  float sigma, float sigma_next, float guidance, void *xp_scratch, void *z_next,
                                  int heads, int kv_heads, int hidden, int ff_hidden, int head_dim,
                                  int tms_token_id);
/* The same step with a sequence of its own per branch, as the reference's CFG loop has it: the unconditional
 * prompt is tokenised separately and is normally shorter (src/runtime/generate.c:1111-1206 seq_text_len[1],
 * posd[1], seq_S_uncond; :1340-1356 runs and slices that branch at its own text length).  Padding the shorter
 * prompt instead would let image rows attend to the pad rows.  Each branch: ids [text_len] int64, pos_f32
 * [3, text_len + img_tokens], ar_len (text_len - 1 for T2I), visual (may be NULL).  ws (one workspace, used by
 * both branches in turn) must come from hd_forward_workspace_bytes of the LONGER sequence; xp_scratch holds
 * (S_cond + S_uncond) * 3072 bf16.  The scheduler update is the flow-match Euler step; the reference's own
 * CFG path steps with FlowUniPC (generate.c:1362-1416), which a host composes from hd_forward, hd_sched_vcond,
 * hd_sched_cfg_guided and hd_unipc_* exactly as there. */
typedef struct {
    const int64_t *ids;
    int text_len;
    const float *pos_f32;
    int ar_len;
    const hd_visual_cond *visual;
} o1_cfg_branch;
hd_status o1_denoise_step_cfg_branches(const hd_forward_binding *bw, hd_forward_workspace *ws,
                                       const o1_cfg_branch *cond, const o1_cfg_branch *uncond, const void *z,
                                       int img_tokens, int target_tokens, const float *timestep_dev, float sigma,
                                       float sigma_next, float guidance, void *xp_scratch, void *z_next, int heads,
                                       int kv_heads, int hidden, int ff_hidden, int head_dim, int tms_token_id);
/* Same step with HOST latents: copies z_host -> device, runs the step, copies
 * z_next back and synchronises.  z_dev / z_next_dev are caller-owned staging. */
hd_status o1_denoise_step_cfg_host(const hd_forward_binding *bw, hd_forward_workspace *ws,
                                   const int64_t *ids_cond, const int64_t *ids_uncond,
                                   int text_len, const float *pos_f32, int ar_len,
                                   const void *z_host, void *z_dev, int img_tokens, float sigma,
                                   float sigma_next, float guidance, float *timestep_dev,
                                   void *xp_scratch, void *z_next_dev, void *z_next_host,
                                   int heads, int kv_heads, int hidden, int ff_hidden,
                                   int head_dim, int tms_token_id);

/* ------------------------------------------- host pieces of the step loop + final decode
 * torch-compatible MT19937 float randn: src/runtime/torch_rng.c:34-121 (hd_torch_rng_seed / _u32 / _randn_f32) */
void *o1_torch_rng_create(uint64_t seed);
void o1_torch_rng_randn(void *rng, float *out_host, int64_t n);
uint32_t o1_torch_rng_u32(void *rng);
void o1_torch_rng_free(void *rng);
/* randn(1,3,H,W; seed+1) -> pixel_unshuffle -> x noise_scale -> bf16 [tokens, 3*patch*patch]:
 * src/runtime/generate.c:78-104, :1264-1268 */
hd_status o1_initial_latent_host(uint64_t seed, int height, int width, int patch, float noise_scale,
                                 void *z_host);
/* src/model/scheduler.c:53-64 (Dev list), :117-158 (flash / flow_match), :173-195 (default); return count */
int o1_sigmas_dev(float *sigmas /* [29] */);
int o1_sigmas_flash(int steps, float shift, float *sigmas /* [steps+1] */);
int o1_sigmas_default(int steps, float shift, float *sigmas /* [steps+1] */);
/* src/model/scheduler.c:197-208; src/runtime/generate.c:1423-1438 */
float o1_noise_scale(int n_sigmas, int step_index, float start, float end);
void o1_noise_clamp_host(float *noise, size_t n, float clip_std);
/* Same draws as o1_torch_rng_randn with the Box-Muller transform spread over host threads. */
void o1_torch_rng_randn_mt(void *rng, float *out_host, int64_t n, int threads);
/* Per-step noise of the flash scheduler (src/runtime/generate.c:1296, :1419-1439) as a pipeline.  The
 * reference draws n normals on the host, computes mean / unbiased std in fp64, clamps at clip_std * std
 * and copies to the device, all inside the step.  Here a host thread draws step i+1 into pinned memory
 * while the device runs step i; o1_noise_pipe_next enqueues the copy of the current step's draw and the
 * statistics + clamp kernels on `stream` (NULL = current stream) and returns without synchronising.
 * The draws are bit-identical to the reference's; mean and std are fp64 sums in a different (fixed) order,
 * so the clip value can differ from the host's only if that changes the fp32 rounding of std.
 * create allocates 2 x n floats of pinned memory and 8 KB on the device; clip_std <= 0 disables the clamp. */
typedef struct o1_noise_pipe o1_noise_pipe;
int o1_noise_pipe_create(o1_noise_pipe **out, uint64_t seed, size_t n, float clip_std, int host_threads);
hd_status o1_noise_pipe_next(o1_noise_pipe *pipe, float *noise_dev, void *stream);
void o1_noise_pipe_free(o1_noise_pipe *pipe);
/* src/runtime/decode.c:5-27 fused with the NaN / range scan of src/runtime/generate.c:1474-1496, on the device */
hd_status o1_decode_to_rgb(const void *z_dev, int grid_h, int grid_w, int patch, int channels, void *rgb_dev,
                           void *stats_dev /* 12 bytes */, int *n_bad, float *vmin, float *vmax);

/* ------------------------------------------- sequence-parallel (Ulysses) form, added
 * No counterpart in the reference (it is single-GPU, src/main.c:242-243).  Token rows are sharded
 * over sp_size ranks: rank r owns rows [r*rows, (r+1)*rows), S = rows*sp_size.  Per block the caller
 * runs  o1_sp_block_pre -> exchange(send -> gath) -> o1_sp_block_attn -> exchange(attn -> recv) ->
 * o1_sp_block_post, where both exchanges are equal-split all-to-alls of contiguous slabs:
 *   send [sp_size][rows][C]   slab d = this rank's rows of q|k|v for the heads rank d owns,
 *   gath [S][C]               row block s = slab received from rank s   (C = (heads+2*kv_heads)*128/sp_size)
 *   attn [S][Hc]              row block d = slab sent to rank d          (Hc = heads*128/sp_size)
 *   recv [sp_size][rows][Hc]  slab s = this rank's rows of the heads rank s owns.
 * With sp_size == 1, send == gath and attn == recv may alias and no exchange is needed.
 * sp_size is at most O1_SP_MAX_RANKS (the peer tables below and the kernels' destination tables hold that many). */
#define O1_SP_MAX_RANKS 8
typedef struct {
    int sp_size, sp_rank;
    int S, T;          /* global token count, text token count */
    int row0, rows;    /* this rank's rows */
    int heads, kv_heads, hidden, ff, head_dim;
    int ar_len;
    void *send, *gath, *attn, *recv;
    void *ln, *ar, *post, *swi;    /* [rows,hidden] x3, [rows,ff] */
    float *rope;                   /* [rows,128] */
} o1_sp_ws;
void o1_launch_count_add(int n);
hd_status o1_sp_rope_table(const o1_sp_ws *w, const float *pos_global /* [3,S] */);
hd_status o1_sp_block_pre(const hd_block_binding *bw, const o1_sp_ws *w, const void *in);
hd_status o1_sp_block_attn(const o1_sp_ws *w);
hd_status o1_sp_block_post(const hd_block_binding *bw, const o1_sp_ws *w, const void *in, void *out);
hd_status o1_sp_forward_begin(const hd_forward_binding *bw, const o1_sp_ws *w, const int64_t *ids_global,
                              const void *vin_local, const float *timestep_dev, void *small, void *xe_stage,
                              int tms_token_id, void *hidden_out);
hd_status o1_sp_forward_end(const hd_forward_binding *bw, const o1_sp_ws *w, const void *hidden,
                            void *norm_scratch, void *out_local);
/* Visual conditioning of a sharded forward (src/model/forward.c:277-285 masked scatter of image_embeds into the
 * <image_pad> rows after the embedding, :363-369 DeepStack add after blocks 0..2), on this rank's rows.
 * mask_global [S] uint8 on the device; embed_row0 = marked rows before this rank's first row. */
hd_status o1_sp_visual_scatter(const o1_sp_ws *w, const uint8_t *mask_global, const void *image_embeds, int embed_row0,
                               const void *in, void *out);
hd_status o1_sp_deepstack(const o1_sp_ws *w, const uint8_t *mask_global, const void *deepstack_l, int embed_row0,
                          const void *in, void *out);

/* Direct form of the two exchanges: no collective call and no staging copy.  Each rank maps its peers' gath
 * [S][C] and recv [P][rows][Hc] buffers and a small flag array (CUDA IPC: o1_peer_*; in a C host
 * cudaIpcGetMemHandle / cudaIpcOpenMemHandle directly).  o1_sp_block_pre_direct's q/k/v GEMM epilogues apply the
 * per-head norm + rope to their own rows (cos|sin from o1_sp_rope_table) and store head group p straight into
 * rank p's gath; o1_sp_block_attn_direct's attention epilogue stores row block p straight into rank p's recv;
 * o1_sp_block_post is unchanged.
 * Results are bit-identical to the staged form.  Call order per block on every rank:
 *   pre_direct, barrier(e), attn_direct, barrier(e+1), post      (e grows by 2 per block, never reused)
 * The barrier is a kernel on the current stream that release-stores the epoch into every peer's flag array and
 * polls its own; its wait is bounded (device error code 30 after about two seconds).  Ranks must be on different
 * GPUs (two ranks' barrier kernels on one GPU would wait for each other without being co-scheduled). */
typedef struct {
    void *gath[O1_SP_MAX_RANKS];      /* rank p's gath buffer as mapped in this process ([sp_rank] = the local one)   */
    void *recv[O1_SP_MAX_RANKS];      /* rank p's recv buffer                                                         */
    void *flags[O1_SP_MAX_RANKS];     /* rank p's flag array: 8 x uint32, zero-initialised                            */
    void *rope_full;    /* optional: cos|sin table of all S rows (o1_sp_rope_table_full); the forward does not need it */
} o1_sp_peers;
int o1_peer_alloc(void **dev_ptr, size_t bytes);                 /* cudaMalloc + zero fill */
int o1_peer_free(void *dev_ptr);
int o1_peer_export(const void *dev_ptr, unsigned char handle[64]);
int o1_peer_open(const unsigned char handle[64], void **peer_ptr);
int o1_peer_close(void *peer_ptr);
hd_status o1_sp_rope_table_full(const o1_sp_ws *w, const o1_sp_peers *pt, const float *pos_global);
hd_status o1_sp_block_pre_direct(const hd_block_binding *bw, const o1_sp_ws *w, const o1_sp_peers *pt, const void *in);
hd_status o1_sp_block_attn_direct(const hd_block_binding *bw, const o1_sp_ws *w, const o1_sp_peers *pt);
hd_status o1_sp_barrier(const o1_sp_ws *w, const o1_sp_peers *pt, unsigned epoch);


/* The whole sharded forward of one rank in one call (direct form): what a C host would otherwise loop over the
 * stage functions above -- the counterpart, for a multi-GPU host, of the single hd_forward call in
 * src/runtime/generate.c:1323-1327.  ctx carries the workspace, the peer table, two [rows, hidden] buffers, the
 * scratch of o1_sp_forward_begin and the barrier epoch (start at 0; the library advances it).  Visual
 * conditioning: visual_mask [S] uint8 on the device, image_embeds / deepstack [V, hidden], embed_row0 = marked rows
 * before this rank's rows, visual_rows = marked rows among this rank's rows (0: nothing to do here). */
typedef struct {
    o1_sp_ws ws;
    o1_sp_peers peers;
    void *hid[2];
    void *small, *xe_stage;
    unsigned epoch;
    const uint8_t *visual_mask;
    const void *image_embeds;
    const void *deepstack[3];
    int embed_row0, visual_rows;
} o1_sp_ctx;
hd_status o1_sp_forward(const hd_forward_binding *bw, o1_sp_ctx *ctx, const int64_t *ids_global,
                        const float *pos_global, const void *vin_local, const float *timestep_dev, int tms_token_id,
                        void *out_local /* [rows, 3072] */);
/* One CFG step of a rank of a (CFG pair) x (SP group) layout: o1_sp_forward of this rank's branch, the partner's
 * prediction rows through peer copies + a two-rank flag barrier, the fused scheduler update
 * (src/runtime/generate.c:1340-1360 with the flow-match update of :900-905) on n_step_rows local target rows.
 * xp_local[p] / xp_partner[p] (p = step parity): [2][local image rows][3072] bf16 here and on the partner (mapped);
 * flags_*: 2 x uint32 each, zero-initialised; step starts at 0.  xp_scratch: [rows, 3072] bf16. */
typedef struct {
    int branch;                 /* 0 = conditional, 1 = unconditional */
    void *xp_local[2], *xp_partner[2];
    void *flags_local, *flags_partner;
    unsigned step;
} o1_cfg_pair;
hd_status o1_denoise_step_cfg_sp(const hd_forward_binding *bw, o1_sp_ctx *ctx, o1_cfg_pair *pair,
                                 const int64_t *ids_global, const float *pos_global, const void *z_local,
                                 int n_step_rows, const float *timestep_dev, float sigma, float sigma_next,
                                 float guidance, int tms_token_id, void *xp_scratch, void *z_next_local);
/* rank -> (image, CFG branch or -1, sp_rank) and sp_size for `world` GPUs; returns the number of images in flight,
 * -1 for an impossible combination.  O1_GPUS, O1_CFG_SPLIT, O1_SP_DEGREE in the environment override the defaults
 * (1 GPU: both branches; 2: CFG pair; 4: pair x SP2; 8: pair x SP4). */
int o1_parallel_layout(int world, int rank, int *image, int *branch, int *sp_rank, int *sp_size);

#ifdef __cplusplus
}
#endif
#endif /* O1_B200_H */
