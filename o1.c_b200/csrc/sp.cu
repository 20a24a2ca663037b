// Sequence-parallel (Ulysses) form of the forward: token rows are sharded across P ranks for every
// token-wise op (norms, all GEMMs, SwiGLU, residuals, embedding, head); around attention two all-to-all
// exchanges turn [S/P rows, all heads] into [all rows, heads/P] and back.  The reference has no
// multi-GPU code; this splits hd_decoder_block (o1.c src/model/block.c:247-356) at its two exchange
// points into three calls, and hd_forward (src/model/forward.c:249-397) into begin / end calls.
//
// No pack or unpack pass exists: the q/k/v projections write straight into the all-to-all send
// layout (one slab per destination rank), attention reads the received slabs as one [S, C] matrix and
// writes its output as [S, Hc] whose row blocks are the second exchange's send slabs, and o_proj reads
// the received slabs as K blocks of its A operand.  The exchanges themselves are the caller's
// (NCCL all-to-all with equal splits, or peer copies).
//
// Direct form (o1_sp_*_direct): the exchange is part of the producing kernel.  Every rank maps its
// peers' gath / recv buffers (CUDA IPC); the q/k/v GEMM epilogues store each destination's head group
// straight into that rank's gath rows, and attention stores each destination's row block straight into
// that rank's recv slab, so the NVLink transfer runs under the tensor-core work and no collective kernel
// or staging copy exists.  Per-head norm + rope then run on the receiving side (same arithmetic on the
// same values, so results are bit-identical to the staged form).  A flag barrier over peer memory
// (o1_sp_barrier) orders producers and consumers; its wait is bounded.
#include "common.cuh"
#include "kernels.h"
#include "../../include/o1_b200.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

using namespace o1;

#define SP_TRY(expr, what)                                                                  \
    do {                                                                                    \
        if (!(expr)) { hd_set_error("sp: %s: %s", what, hd_cuda_last_error()); return HD_ERR_RUNTIME; } \
        o1_launch_count_add(1);                                                             \
    } while (0)

extern "C" void o1_launch_count_add(int n);

static bool sp_ok(const o1_sp_ws* w) {
    return w && w->sp_size >= 1 && w->sp_size <= O1_SP_MAX_RANKS && w->sp_rank >= 0 && w->sp_rank < w->sp_size && w->head_dim == 128 &&
           w->heads % w->sp_size == 0 && w->kv_heads % w->sp_size == 0 && w->S == w->rows * w->sp_size &&
           w->row0 == w->sp_rank * w->rows && (w->hidden % 256) == 0 && (w->ff % 128) == 0 &&
           ((w->heads / w->sp_size) * 128) % 128 == 0;
}

// One thread per peer: release-store this rank's epoch into the peer's flag array, then poll this rank's
// own array for the peer's epoch.  Epochs only grow, so a late reader never misses one.  The wait is
// bounded (about two seconds of SM clock); on expiry the device error word gets code 30.
__global__ void sp_barrier_kernel(o1_sp_peers pt, int P, int rank, unsigned epoch, int* err) {
    const int p = threadIdx.x;
    if (p >= P || p == rank) return;
    unsigned* remote = (unsigned*)pt.flags[p] + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    const unsigned* mine = (const unsigned*)pt.flags[rank] + p;
    const long long t0 = clock64();
    for (;;) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if ((int)(v - epoch) >= 0) break;
        if (clock64() - t0 > 4000000000ll) { atomicExch(err, 30); break; }
    }
}

static bool peers_ok(const o1_sp_ws* w, const o1_sp_peers* pt) {
    if (!pt) return false;
    for (int p = 0; p < w->sp_size; ++p)
        if (!pt->gath[p] || !pt->recv[p] || !pt->flags[p]) return false;
    return true;
}

extern "C" {

// ------------------------------------------------------------------ peer-visible memory (CUDA IPC)
int o1_peer_alloc(void** dev_ptr, size_t bytes) {
    if (!dev_ptr || !bytes) return -1;
    cudaError_t e = cudaMalloc(dev_ptr, bytes);
    if (e == cudaSuccess) e = cudaMemset(*dev_ptr, 0, bytes);
    if (e != cudaSuccess) { hd_set_error("peer alloc: %s", cudaGetErrorString(e)); return -1; }
    return 0;
}
int o1_peer_free(void* dev_ptr) { return cudaFree(dev_ptr) == cudaSuccess ? 0 : -1; }
int o1_peer_export(const void* dev_ptr, unsigned char handle[64]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void*>(dev_ptr));
    if (e != cudaSuccess) { hd_set_error("peer export: %s", cudaGetErrorString(e)); return -1; }
    memcpy(handle, &h, 64);
    return 0;
}
int o1_peer_open(const unsigned char handle[64], void** peer_ptr) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    cudaError_t e = cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) { hd_set_error("peer open: %s", cudaGetErrorString(e)); return -1; }
    return 0;
}
int o1_peer_close(void* peer_ptr) { return cudaIpcCloseMemHandle(peer_ptr) == cudaSuccess ? 0 : -1; }

hd_status o1_sp_barrier(const o1_sp_ws* w, const o1_sp_peers* pt, unsigned epoch) {
    if (!sp_ok(w) || !peers_ok(w, pt)) { hd_set_error("sp: bad peer table"); return HD_ERR_MISSING; }
    if (w->sp_size == 1) return HD_OK;
    sp_barrier_kernel<<<1, 32, 0, current_stream()>>>(*pt, w->sp_size, w->sp_rank, epoch, device_error_word());
    o1_launch_count_add(1);
    if (cudaGetLastError() != cudaSuccess) { hd_set_error("sp: barrier launch failed"); return HD_ERR_RUNTIME; }
    return HD_OK;
}

// cos|sin table of ALL S rows (the direct form applies rope on the receiving side)
hd_status o1_sp_rope_table_full(const o1_sp_ws* w, const o1_sp_peers* pt, const float* pos_global) {
    if (!sp_ok(w) || !pt || !pt->rope_full || !pos_global) { hd_set_error("sp: bad workspace"); return HD_ERR_MISSING; }
    SP_TRY(mrope_table64_rows(pos_global, w->S, 0, w->S, 5000000.0f, (float*)pt->rope_full, current_stream()),
           "rope table");
    return HD_OK;
}

// in [rows, hidden] -> every rank's gath rows [rank*rows, (rank+1)*rows): RMSNorm, then q/k/v projections whose
// epilogues store head group p of the output into rank p's gath.  The per-head RMSNorm + rotary of q and k
// (block.c:266-289) run in the SENDER's epilogue, on its own rows' cos|sin table (w->rope, o1_sp_rope_table): what
// arrives is ready for attention, exactly as on one GPU.
hd_status o1_sp_block_pre_direct(const hd_block_binding* bw, const o1_sp_ws* w, const o1_sp_peers* pt, const void* in) {
    if (!sp_ok(w) || !peers_ok(w, pt) || !bw || !in || !w->rope) { hd_set_error("sp: bad arguments"); return HD_ERR_MISSING; }
    cudaStream_t st = current_stream();
    const int P = w->sp_size, R = w->rows, H = w->hidden;
    const int qc = w->heads * 128, kc = w->kv_heads * 128;
    const int qcp = qc / P, kcp = kc / P, C = qcp + 2 * kcp;
    void* tq[O1_SP_MAX_RANKS]; void* tk[O1_SP_MAX_RANKS]; void* tv[O1_SP_MAX_RANKS];
    for (int p = 0; p < P; ++p) {
        uint16_t* base = (uint16_t*)pt->gath[p] + (size_t)w->sp_rank * R * C;
        tq[p] = base; tk[p] = base + qcp; tv[p] = base + qcp + kcp;
    }
    SP_TRY(rmsnorm(in, bw->input_ln, w->ln, R, H, 1e-6f, st), "input_norm");
    SP_TRY(gemm_qkv(w->ln, H, bw->q_proj, bw->k_proj, bw->v_proj, nullptr, C, R, qc, kc, H, bw->q_norm, bw->k_norm, w->rope,
                    1e-6f, P, tq, tk, tv, st), "qkv_proj+norm+rope");
    return HD_OK;
}

// own gath [S][C] (all rows, this rank's heads, normed and rotated by their senders; complete after the barrier) ->
// attention whose epilogue stores row block p into rank p's recv slab [rank]
hd_status o1_sp_block_attn_direct(const hd_block_binding* bw, const o1_sp_ws* w, const o1_sp_peers* pt) {
    if (!sp_ok(w) || !peers_ok(w, pt) || !bw) { hd_set_error("sp: bad arguments"); return HD_ERR_MISSING; }
    cudaStream_t st = current_stream();
    const int P = w->sp_size, R = w->rows;
    const int qcp = w->heads * 128 / P, kcp = w->kv_heads * 128 / P, C = qcp + 2 * kcp;
    uint16_t* g = (uint16_t*)pt->gath[w->sp_rank];
    void* to[O1_SP_MAX_RANKS];
    for (int p = 0; p < P; ++p) to[p] = (uint16_t*)pt->recv[p] + (size_t)w->sp_rank * R * qcp;
    SP_TRY(flash_attention_tab(g, C, g + qcp, C, g + qcp + kcp, C, to, R, qcp, w->S, w->heads / P, w->kv_heads / P,
                               w->ar_len, (float)(1.0 / sqrt(128.0)), st, w->swi, (size_t)w->rows * w->ff * 2),
           "attention");
    return HD_OK;
}

hd_status o1_sp_rope_table(const o1_sp_ws* w, const float* pos_global) {
    if (!sp_ok(w) || !pos_global || !w->rope) { hd_set_error("sp: bad workspace"); return HD_ERR_MISSING; }
    SP_TRY(mrope_table64_rows(pos_global, w->S, w->row0, w->rows, 5000000.0f, w->rope, current_stream()),
           "rope table");
    return HD_OK;
}

// in [rows, hidden] -> send [P][rows][C]: RMSNorm, q/k/v projections, per-head norm + rope
hd_status o1_sp_block_pre(const hd_block_binding* bw, const o1_sp_ws* w, const void* in) {
    if (!sp_ok(w) || !bw || !in) { hd_set_error("sp: bad arguments"); return HD_ERR_MISSING; }
    cudaStream_t st = current_stream();
    const int P = w->sp_size, R = w->rows, H = w->hidden;
    const int qc = w->heads * 128, kc = w->kv_heads * 128;
    const int qcp = qc / P, kcp = kc / P, C = qcp + 2 * kcp;
    const long slab = (long)R * C;
    uint16_t* send = (uint16_t*)w->send;
    SP_TRY(rmsnorm(in, bw->input_ln, w->ln, R, H, 1e-6f, st), "input_norm");
    SP_TRY(gemm_bf16_ex(w->ln, H, bw->q_proj, nullptr, send, C, R, qc, H, EPI_STORE, nullptr, nullptr, 0, 0.f, 0,
                        qcp, slab, 0, 0, st), "q_proj");
    SP_TRY(gemm_bf16_ex(w->ln, H, bw->k_proj, nullptr, send + qcp, C, R, kc, H, EPI_STORE, nullptr, nullptr, 0, 0.f,
                        0, kcp, slab, 0, 0, st), "k_proj");
    SP_TRY(gemm_bf16_ex(w->ln, H, bw->v_proj, nullptr, send + qcp + kcp, C, R, kc, H, EPI_STORE, nullptr, nullptr, 0,
                        0.f, 0, kcp, slab, 0, 0, st), "v_proj");
    SP_TRY(qk_norm_rope_blocked(send, C, R, w->heads, w->heads / P, slab, bw->q_norm, w->rope, 1e-6f, st), "q_norm_rope");
    SP_TRY(qk_norm_rope_blocked(send + qcp, C, R, w->kv_heads, w->kv_heads / P, slab, bw->k_norm, w->rope, 1e-6f, st),
           "k_norm_rope");
    return HD_OK;
}

// gath [S][C] (all rows, this rank's heads) -> attn [S][Hc]
hd_status o1_sp_block_attn(const o1_sp_ws* w) {
    if (!sp_ok(w)) { hd_set_error("sp: bad workspace"); return HD_ERR_MISSING; }
    const int P = w->sp_size;
    const int qcp = w->heads * 128 / P, kcp = w->kv_heads * 128 / P, C = qcp + 2 * kcp;
    const uint16_t* g = (const uint16_t*)w->gath;
    SP_TRY(flash_attention(g, C, g + qcp, C, g + qcp + kcp, C, w->attn, qcp, w->S, w->heads / P, w->kv_heads / P,
                           w->ar_len, (float)(1.0 / sqrt(128.0)), current_stream(), w->swi,
                           (size_t)w->rows * w->ff * 2), "attention");
    return HD_OK;
}

// recv [P][rows][Hc] + in [rows, hidden] -> out [rows, hidden]: o_proj(+residual), RMSNorm, SwiGLU MLP(+residual)
hd_status o1_sp_block_post(const hd_block_binding* bw, const o1_sp_ws* w, const void* in, void* out) {
    if (!sp_ok(w) || !bw || !in || !out) { hd_set_error("sp: bad arguments"); return HD_ERR_MISSING; }
    cudaStream_t st = current_stream();
    const int P = w->sp_size, R = w->rows, H = w->hidden, qc = w->heads * 128, hc = qc / P;
    SP_TRY(gemm_bf16_ex(w->recv, hc, bw->o_proj, nullptr, w->ar, H, R, H, qc, EPI_RESID, nullptr, in, H, 0.f, 0, 0, 0,
                        P > 1 ? hc : 0, R, st), "o_proj+resid");
    SP_TRY(rmsnorm(w->ar, bw->post_ln, w->post, R, H, 1e-6f, st), "post_norm");
    SP_TRY(gemm_bf16(w->post, bw->gate_proj, bw->up_proj, w->swi, R, w->ff, H, EPI_SWIGLU, nullptr, nullptr, 0.f, 0,
                     st), "gate_up_swiglu");
    SP_TRY(gemm_bf16_ld(w->swi, w->ff, bw->down_proj, nullptr, out, H, R, H, w->ff, EPI_RESID, nullptr, w->ar, H,
                        0.f, 0, st), "down_proj+resid");
    return HD_OK;
}

// Embedding of this rank's rows: timestep MLP (replicated), text rows from the table with the tms row
// replaced, image rows through x_embedder.  ids_global [T] int64; vin_local: the latent rows of this
// rank's image tokens.  small: >= 4*hidden*2 + 4096 bytes of scratch; xe_stage [img_local, 1024] bf16.
hd_status o1_sp_forward_begin(const hd_forward_binding* bw, const o1_sp_ws* w, const int64_t* ids_global,
                              const void* vin_local, const float* timestep_dev, void* small, void* xe_stage,
                              int tms_token_id, void* hidden_out) {
    if (!sp_ok(w) || !bw || !ids_global || !timestep_dev || !small || !hidden_out) {
        hd_set_error("sp: bad arguments");
        return HD_ERR_MISSING;
    }
    cudaStream_t st = current_stream();
    const int H = w->hidden, T = w->T;
    uint8_t* sm = (uint8_t*)small;
    uint16_t* t_emb = (uint16_t*)sm;
    uint16_t* te_hidden = (uint16_t*)(sm + (size_t)H * 2);
    float* freq = (float*)(sm + (size_t)H * 4);
    uint16_t* freq_bf16 = (uint16_t*)(sm + (size_t)H * 4 + 1024);
    float* t_scaled = (float*)(sm + (size_t)H * 4 + 2048);
    SP_TRY(scale_f32(timestep_dev, t_scaled, 1000.0f, 1, st), "t_scale");
    SP_TRY(timestep_embed(t_scaled, freq, 1, 256, st), "t_sinusoid");
    SP_TRY(f32_to_bf16_buf(freq, freq_bf16, 256, st), "t_cast");
    SP_TRY(gemm_bf16(freq_bf16, bw->te0_w, nullptr, te_hidden, 1, H, 256, EPI_BIAS, bw->te0_b, nullptr, 0.f, 0, st), "t_mlp0");
    SP_TRY(silu(te_hidden, t_emb, (size_t)H, st), "t_silu");
    SP_TRY(gemm_bf16(t_emb, bw->te2_w, nullptr, te_hidden, 1, H, H, EPI_BIAS, bw->te2_b, nullptr, 0.f, 0, st), "t_mlp2");
    const int t0 = w->row0 < T ? w->row0 : T;
    const int t1 = (w->row0 + w->rows) < T ? (w->row0 + w->rows) : T;
    const int n_text = t1 - t0, n_img = w->rows - n_text;
    uint16_t* hid = (uint16_t*)hidden_out;
    if (n_text > 0)
        SP_TRY(embed_text(bw->embed_tokens, ids_global + t0, te_hidden, hid, n_text, H, 151936, tms_token_id, st),
               "embed+tms");
    if (n_img > 0) {
        if (!vin_local || !xe_stage) { hd_set_error("sp: image rows without latents"); return HD_ERR_MISSING; }
        SP_TRY(gemm_bf16(vin_local, bw->xe1_w, nullptr, xe_stage, n_img, 1024, 3072, EPI_STORE, nullptr, nullptr, 0.f,
                         0, st), "x_embed1");
        SP_TRY(gemm_bf16(xe_stage, bw->xe2_w, nullptr, hid + (size_t)n_text * H, n_img, H, 1024, EPI_BIAS, bw->xe2_b,
                         nullptr, 0.f, 0, st), "x_embed2");
    }
    return HD_OK;
}

// Visual conditioning on this rank's rows (src/model/forward.c:277-285, :363-369).  mask_global [S] uint8 marks the
// <image_pad> rows; embed_row0 = number of marked rows before this rank's first row (the caller counts them once
// per request), so that the k-th marked row of the whole sequence still receives row k.  Out of place: in -> out.
hd_status o1_sp_visual_scatter(const o1_sp_ws* w, const uint8_t* mask_global, const void* image_embeds, int embed_row0,
                               const void* in, void* out) {
    if (!sp_ok(w) || !mask_global || !image_embeds || !in || !out || embed_row0 < 0) { hd_set_error("sp: bad arguments"); return HD_ERR_MISSING; }
    SP_TRY(masked_scatter(in, mask_global + w->row0, (const uint16_t*)image_embeds + (size_t)embed_row0 * w->hidden, out,
                          w->rows, w->hidden, current_stream()), "masked_scatter");
    return HD_OK;
}
hd_status o1_sp_deepstack(const o1_sp_ws* w, const uint8_t* mask_global, const void* deepstack_l, int embed_row0,
                          const void* in, void* out) {
    if (!sp_ok(w) || !mask_global || !deepstack_l || !in || !out || embed_row0 < 0) { hd_set_error("sp: bad arguments"); return HD_ERR_MISSING; }
    SP_TRY(deepstack_inject(in, mask_global + w->row0, (const uint16_t*)deepstack_l + (size_t)embed_row0 * w->hidden, out,
                            w->rows, w->hidden, current_stream()), "deepstack");
    return HD_OK;
}

// final RMSNorm + head on this rank's rows: hidden [rows, hidden] -> out_local [rows, 3072]
hd_status o1_sp_forward_end(const hd_forward_binding* bw, const o1_sp_ws* w, const void* hidden, void* norm_scratch,
                            void* out_local) {
    if (!sp_ok(w) || !bw || !hidden || !norm_scratch || !out_local) { hd_set_error("sp: bad arguments"); return HD_ERR_MISSING; }
    cudaStream_t st = current_stream();
    SP_TRY(rmsnorm(hidden, bw->fnorm_w, norm_scratch, w->rows, w->hidden, 1e-6f, st), "final_norm");
    SP_TRY(gemm_bf16(norm_scratch, bw->fl_w, nullptr, out_local, w->rows, 3072, w->hidden, EPI_BIAS, bw->fl_b, nullptr,
                     0.f, 0, st), "head");
    return HD_OK;
}

// ------------------------------------------------------------------ whole sharded forward / CFG step in one call
// The loop a C host would otherwise write around the stage functions (direct form):
//   rope table of own rows, embedding, then per block  pre_direct, barrier, attn_direct, barrier, post
//   (DeepStack add after blocks 0..2 on ranks that own <image_pad> rows), final norm + head.
// Everything is enqueued on the current stream; nothing synchronises or allocates.
hd_status o1_sp_forward(const hd_forward_binding* bw, o1_sp_ctx* c, const int64_t* ids_global, const float* pos_global,
                        const void* vin_local, const float* timestep_dev, int tms_token_id, void* out_local) {
    if (!c || !bw || !ids_global || !pos_global || !timestep_dev || !out_local || !c->hid[0] || !c->hid[1] || !c->small) {
        hd_set_error("sp_forward: null argument");
        return HD_ERR_MISSING;
    }
    const o1_sp_ws* w = &c->ws;
    if (!sp_ok(w) || !peers_ok(w, &c->peers)) { hd_set_error("sp_forward: bad workspace or peer table"); return HD_ERR_MISSING; }
    hd_status s = o1_sp_rope_table(w, pos_global);
    if (s != HD_OK) return s;
    s = o1_sp_forward_begin(bw, w, ids_global, vin_local, timestep_dev, c->small, c->xe_stage, tms_token_id, c->hid[0]);
    if (s != HD_OK) return s;
    void* cur = c->hid[0];
    void* nxt = c->hid[1];
    const bool visual = c->visual_mask && c->image_embeds && c->visual_rows > 0;
    if (visual) {
        s = o1_sp_visual_scatter(w, c->visual_mask, c->image_embeds, c->embed_row0, cur, nxt);
        if (s != HD_OK) return s;
        void* t = cur; cur = nxt; nxt = t;
    }
    for (int l = 0; l < bw->n_layers; ++l) {
        const hd_block_binding* bb = &bw->blocks[l];
        if ((s = o1_sp_block_pre_direct(bb, w, &c->peers, cur)) != HD_OK) return s;
        if ((s = o1_sp_barrier(w, &c->peers, ++c->epoch)) != HD_OK) return s;
        if ((s = o1_sp_block_attn_direct(bb, w, &c->peers)) != HD_OK) return s;
        if ((s = o1_sp_barrier(w, &c->peers, ++c->epoch)) != HD_OK) return s;
        if ((s = o1_sp_block_post(bb, w, cur, nxt)) != HD_OK) return s;
        if (visual && l < 3 && c->deepstack[l]) {
            // the block's output is in nxt; the sum goes back into cur, which stays the next block's input
            if ((s = o1_sp_deepstack(w, c->visual_mask, c->deepstack[l], c->embed_row0, nxt, cur)) != HD_OK) return s;
        } else {
            void* t = cur; cur = nxt; nxt = t;
        }
    }
    return o1_sp_forward_end(bw, w, cur, w->ln, out_local);
}

// One CFG denoise step of a rank of a (CFG pair) x (SP group) layout: this rank's branch forward, exchange of the
// predictions with the CFG partner (same sp_rank, other branch) by plain device-to-device copies into the partner's
// mapped buffer + a two-rank flag barrier, then the fused scheduler update on this rank's target rows.  Both
// partners apply the identical kernel to identical inputs, so their latents stay bit-identical.  Prediction
// buffers are double-buffered by step parity: the partner's previous read of a slot precedes its arrival at the
// barrier this rank has already passed.
hd_status o1_denoise_step_cfg_sp(const hd_forward_binding* bw, o1_sp_ctx* c, o1_cfg_pair* pr, const int64_t* ids_global,
                                 const float* pos_global, const void* z_local, int n_step_rows, const float* timestep_dev,
                                 float sigma, float sigma_next, float guidance, int tms_token_id, void* xp_local,
                                 void* z_next_local) {
    if (!c || !pr || !xp_local || (pr->branch != 0 && pr->branch != 1) || !pr->xp_local[0] || !pr->xp_local[1] ||
        !pr->xp_partner[0] || !pr->xp_partner[1] || !pr->flags_local || !pr->flags_partner) {
        hd_set_error("denoise_step_sp: null argument");
        return HD_ERR_MISSING;
    }
    const o1_sp_ws* w = &c->ws;
    hd_status s = o1_sp_forward(bw, c, ids_global, pos_global, z_local, timestep_dev, tms_token_id, xp_local);
    if (s != HD_OK) return s;
    cudaStream_t st = current_stream();
    // this rank's image rows of the prediction (text rows come first on the ranks that own any)
    const int t0 = w->row0 < w->T ? w->row0 : w->T;
    const int t1 = (w->row0 + w->rows) < w->T ? (w->row0 + w->rows) : w->T;
    const int n_text = t1 - t0, n_img = w->rows - n_text;
    const int par = (int)(pr->step & 1u);
    const size_t bytes = (size_t)n_img * 3072 * 2, slot = (size_t)pr->branch * n_img * 3072;
    const uint16_t* mine = (const uint16_t*)xp_local + (size_t)n_text * 3072;
    if (bytes) {
        cudaError_t e = cudaMemcpyAsync((uint16_t*)pr->xp_local[par] + slot, mine, bytes, cudaMemcpyDeviceToDevice, st);
        if (e == cudaSuccess)
            e = cudaMemcpyAsync((uint16_t*)pr->xp_partner[par] + slot, mine, bytes, cudaMemcpyDeviceToDevice, st);
        if (e != cudaSuccess) { hd_set_error("denoise_step_sp: prediction exchange: %s", cudaGetErrorString(e)); return HD_ERR_IO; }
        o1_launch_count_add(2);
    }
    // two-rank barrier with the partner: rank index = branch
    o1_sp_peers pt;
    memset(&pt, 0, sizeof(pt));
    pt.flags[pr->branch] = pr->flags_local;
    pt.flags[pr->branch ^ 1] = pr->flags_partner;
    sp_barrier_kernel<<<1, 32, 0, st>>>(pt, 2, pr->branch, ++pr->step, device_error_word());
    o1_launch_count_add(1);
    if (cudaGetLastError() != cudaSuccess) { hd_set_error("denoise_step_sp: barrier launch failed"); return HD_ERR_RUNTIME; }
    if (n_step_rows > 0) {
        const uint16_t* xc = (const uint16_t*)pr->xp_local[par];
        const uint16_t* xu = xc + (size_t)n_img * 3072;
        if (!sched_cfg_flow_step(z_local, xc, xu, sigma, sigma_next, guidance, z_next_local, (size_t)n_step_rows * 3072, st)) {
            hd_set_error("denoise_step_sp: scheduler: %s", hd_cuda_last_error());
            return HD_ERR_RUNTIME;
        }
        o1_launch_count_add(1);
    }
    return HD_OK;
}

// Layout of `world` GPUs over images, CFG branches and sequence-parallel ranks:
//   1 GPU: both branches in turn; 2: CFG pair; 4: pair x SP2; 8: pair x SP4; more: several images.
// Environment overrides (read on every call): O1_GPUS (world), O1_CFG_SPLIT (0: both branches on every GPU,
// 1: split the pair), O1_SP_DEGREE (ranks per forward; must divide the 8 KV heads).
int o1_parallel_layout(int world, int rank, int* image, int* branch, int* sp_rank, int* sp_size) {
    const char* e;
    if ((e = getenv("O1_GPUS")) && atoi(e) > 0) world = atoi(e);
    if (world <= 0 || rank < 0 || rank >= world) return -1;
    int cfg_split = world >= 2 ? 1 : 0;
    if ((e = getenv("O1_CFG_SPLIT"))) cfg_split = atoi(e) != 0 && world >= 2;
    int sp = cfg_split ? world / 2 : world;
    if (sp > O1_SP_MAX_RANKS) sp = O1_SP_MAX_RANKS;
    if ((e = getenv("O1_SP_DEGREE")) && atoi(e) > 0) sp = atoi(e);
    if (sp < 1 || (8 % sp) != 0) return -1;                    // must divide the KV heads
    const int per_image = (cfg_split ? 2 : 1) * sp;
    if (per_image > world || (world % per_image) != 0) return -1;
    if (image) *image = rank / per_image;
    if (branch) *branch = cfg_split ? (rank % per_image) / sp : -1;
    if (sp_rank) *sp_rank = rank % sp;
    if (sp_size) *sp_size = sp;
    return world / per_image;                                  // images in flight
}

}  // extern "C"
