// Prefix-causal flash attention on the sm_100a tensor cores.  Replaces the
// cuDNN SDPA graphs (o1.c src/cuda/hd_cudnn_sdpa.cu:114-441) and the eager
// S x S path (src/cuda/attn.cu:22-174): scores are never written to HBM.
//
//   out[s, h, :] = softmax_t( q[s,h,:] . k[t,kh,:] / sqrt(128) + mask[s,t] ) v[t,kh,:]
//   kh = h / (heads / kv_heads); mask: rows s < ar_len see keys t <= s,
//   rows s >= ar_len see every key (o1.c src/runtime/sequence.c:120-142).
//
// Two kernels.  Long sequences (the benchmark's 16640 rows), flash_attn_kernel:
// one CTA = 256 query rows of one head: two query tiles of 128 rows that share every K/V tile
// brought into shared memory (half the K/V fill per query row of a one-tile CTA, and the two tiles'
// softmax and MMA phases overlap each other).  Operands stay seq-major ([S, heads*128]); head split /
// merge (attn.cu:180-218) disappear into the TMA coordinates and the output addressing.
//   warp 0     : TMA producer (two Q tiles once, then K tiles (2 stages) and V tiles (3 stages))
//   warp 1     : tcgen05.mma issuer: S_g = Q_g K_j^T into TMEM, O_g += P_g V_j with P_g read from
//                tensor memory and V as an MN-major operand, alternating between the groups
//   warps 2..17: two softmax groups of eight warps, one group per query tile, two threads per query
//                row (TMEM lane == row; the warps w and w+4 of a group own the same 32 lanes and
//                take 64 score columns each): fp32 scores -> running max (halves exchanged through
//                shared memory) / sum in the exp2 domain -> bf16 P written back into tensor memory
//                over the scores.  The softmax -> PV -> next-scores round trip of a group is the
//                critical path of the kernel, which is why a row is split over two threads.
// An accumulator is only rescaled when its running max grows by more than 2^8 (sum and
// accumulator share the same stale max, so the final division is still exact).
// Short sequences, flash_attn1_kernel: one query tile per CTA with triple-buffered scores (described at the kernel).
#include <cstdlib>
#include "common.cuh"
#include "ptx.cuh"
#include "kernels.h"

namespace o1 {

static constexpr int AQ = 128;      // query rows per softmax group
static constexpr int AQ2 = 256;     // query rows per CTA (two groups)
static constexpr int AKV = 128;     // keys per tile
static constexpr int AD = 128;      // head dim
static constexpr int TILE_BYTES = 128 * 128 * 2;   // 32 KB: two 64-column panels of 16 KB
static constexpr int PANEL_BYTES = 128 * 64 * 2;
static constexpr int K_STAGES = 2;
static constexpr int V_STAGES = 3;
static constexpr int ATTN_THREADS = 576;   // TMA warp, MMA warp, two softmax groups of eight warps
// Q x2 | K x2 | V x3 (P lives in tensor memory) + 192 B of barriers / slots + row-max exchange
static constexpr int ATTN_XCH = 2 * 2 * 128 * 4;   // [group][column half][row] floats
static constexpr int ATTN_SMEM = TILE_BYTES * (2 + K_STAGES + V_STAGES) + 192 + ATTN_XCH;

struct AttnArgs {
    uint16_t* out;
    int ldo;
    int S, heads, kv_heads, ar_len;
    int row_lo, row_hi; // only query rows in [row_lo, row_hi) are computed and written (whole range: 0, S)
    float scale_log2;   // scale * log2(e)
    // head h of q sits at TMA coordinates (h*q_hc + d, h*q_hr + s); same for k/v with
    // the kv head.  seq-major [S, H*128]: hc = 128, hr = 0; head-major [H,S,128]: hc = 0, hr = S.
    int q_hc, q_hr, kv_hc, kv_hr;
    long out_hoff;      // element offset of head h in the output: h * out_hoff
    int* err;
    // out_rows > 0: output rows [b*out_rows, (b+1)*out_rows) are written to out_tab[b] (possibly another
    // GPU's memory) instead of out
    int out_rows;
    uint16_t* out_tab[8];
    // Work items: item = head * nqb + query block.  The first n_plain items are one CTA each.  Each of the
    // remaining (tail) items is cut along the keys into `ways` CTAs that leave unnormalised partial results
    // (accumulator, running max, row sum) in part_o / part_ml for attn_merge_kernel, so that the last,
    // partly filled wave of CTAs is short.  ways == 1: no tail.
    int nqb, n_plain, ways;
    float* part_o;      // [slot][256 rows][128] fp32, slot = (item - n_plain) * ways + part
    float* part_ml;     // [slot][256 rows][2]: max (exp2 domain) the partial is relative to, row sum
};

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Packed fp32 pairs (one issue slot for two lanes' worth of FMA / ADD): the softmax warps are bound by
// instruction issue and latency, not by a pipe, so halving the FMA and ADD count of the exp2 loop is time saved.
__device__ __forceinline__ uint64_t pack_f32x2(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint32_t cvt_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// P = exp2(s * scale - m) for this thread's 64 scores, rounded to bf16 pairs and written to 32 tensor-memory
// columns at t_p; returns the fp32 sum of the unrounded values.
__device__ __forceinline__ float softmax_exp_store(const uint32_t (&r)[2][32], uint64_t scale2, uint64_t negm2, uint32_t t_p) {
    uint64_t lsa = pack_f32x2(0.f, 0.f), lsb = lsa;     // two independent chains of pair sums
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint64_t x2 = fma_f32x2(pack_f32x2(__uint_as_float(r[c][2 * i]), __uint_as_float(r[c][2 * i + 1])),
                                          scale2, negm2);
            float x0, x1;
            unpack_f32x2(x2, x0, x1);
            const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
            if (i & 1) lsb = add_f32x2(lsb, pack_f32x2(p0, p1));
            else lsa = add_f32x2(lsa, pack_f32x2(p0, p1));
            pk[i] = cvt_bf16x2(p0, p1);
        }
        tmem_st16(t_p + c * 16, pk);
    }
    tmem_st_wait();
    float s0, s1;
    unpack_f32x2(add_f32x2(lsa, lsb), s0, s1);
    return s0 + s1;
}

__global__ void __launch_bounds__(ATTN_THREADS, 1)
flash_attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const AttnArgs a) {
    // 7 tiles of 32 KB fill the SM's shared memory, so there is no room for an alignment pad or
    // static arrays: the dynamic window itself is declared 1024-byte aligned (checked below).
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* q_s = smem;                               // two query tiles
    uint8_t* k_s = q_s + 2 * TILE_BYTES;
    uint8_t* v_s = k_s + K_STAGES * TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + V_STAGES * TILE_BYTES);
    uint64_t* q_full = bars;                // 1
    uint64_t* k_full = bars + 1;            // K_STAGES
    uint64_t* k_empty = k_full + K_STAGES;
    uint64_t* v_full = k_empty + K_STAGES;  // V_STAGES
    uint64_t* v_empty = v_full + V_STAGES;
    uint64_t* s_full = v_empty + V_STAGES;  // 2 (one per group)
    uint64_t* p_ready = s_full + 2;         // 2
    uint64_t* o_done = p_ready + 2;         // 1
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 1);
    int* s_abort = reinterpret_cast<int*>(tmem_slot + 1);
    float* xch = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 192);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    int item = blockIdx.x, part = 0, ways = 1;
    if (item >= a.n_plain) {
        const int t = item - a.n_plain;
        item = a.n_plain + t / a.ways;
        part = t - (t / a.ways) * a.ways;
        ways = a.ways;
    }
    const int h = item / a.nqb;
    const int q0 = (item - h * a.nqb) * AQ2;
    const int kh = h / (a.heads / a.kv_heads);
    if (q0 + AQ2 <= a.row_lo || q0 >= a.row_hi) return;   // no row of this block is wanted (whole CTA, before any set-up)

    // keys this pair of query tiles can see (the second tile's range covers the first's)
    int kv_end = a.S;
    if (q0 + AQ2 - 1 < a.ar_len) kv_end = q0 + AQ2;   // all rows causal: keys <= last row
    if (kv_end > a.S) kv_end = a.S;
    const int tiles_all = (kv_end + AKV - 1) / AKV;
    const int j0 = (int)((long)part * tiles_all / ways);                  // first key tile of this CTA
    const int n_tiles = (int)((long)(part + 1) * tiles_all / ways) - j0;  // and how many it covers
    if (n_tiles <= 0) {
        // a part of a tail item that has fewer key tiles than parts: an empty partial (max -inf, sum 0), nothing else
        if (threadIdx.x < AQ2) {
            const int slot = (item - a.n_plain) * ways + part;
            *reinterpret_cast<float2*>(a.part_ml + ((size_t)slot * AQ2 + threadIdx.x) * 2) = make_float2(-INFINITY, 0.f);
        }
        return;
    }

    // a kernel that already failed on this device leaves its code in *err: do nothing then
    if (threadIdx.x == 0) {
        int ab = *reinterpret_cast<volatile int*>(a.err);
        if (ab == 0 && (smem_u32(smem) & 1023u) != 0) { ab = 20; atomicExch(a.err, 20); }
        *s_abort = ab;
    }
    __syncthreads();
    if (*s_abort != 0) return;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < K_STAGES; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
        for (int s = 0; s < V_STAGES; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&s_full[s], 1); mbar_init(&p_ready[s], 8); }
        mbar_init(o_done, 1);
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_S = tmem_base;         // scores of the two groups: columns [0,128) and [128,256)
    const uint32_t tmem_O = tmem_base + 256;   // output accumulators of the two groups: [256,384), [384,512)

    if (warp == 0) {
        // -------------------------------------------------------- TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&tmQ);
            tma_prefetch_desc(&tmK);
            tma_prefetch_desc(&tmV);
            mbar_expect_tx(q_full, 2 * TILE_BYTES);
#pragma unroll
            for (int g = 0; g < 2; ++g) {
                tma_load_2d(q_s + g * TILE_BYTES, &tmQ, q_full, h * a.q_hc, h * a.q_hr + q0 + g * AQ);
                tma_load_2d(q_s + g * TILE_BYTES + PANEL_BYTES, &tmQ, q_full, h * a.q_hc + 64,
                            h * a.q_hr + q0 + g * AQ);
            }
            auto load_k = [&](int j) -> bool {
                const int st = j % K_STAGES;
                if (!mbar_wait(&k_empty[st], ((j / K_STAGES) & 1) ^ 1)) { atomicExch(a.err, 11); return false; }
                mbar_expect_tx(&k_full[st], TILE_BYTES);
                tma_load_2d(k_s + st * TILE_BYTES, &tmK, &k_full[st], kh * a.kv_hc, kh * a.kv_hr + (j0 + j) * AKV);
                tma_load_2d(k_s + st * TILE_BYTES + PANEL_BYTES, &tmK, &k_full[st], kh * a.kv_hc + 64,
                            kh * a.kv_hr + (j0 + j) * AKV);
                return true;
            };
            auto load_v = [&](int j) -> bool {
                const int st = j % V_STAGES;
                if (!mbar_wait(&v_empty[st], ((j / V_STAGES) & 1) ^ 1)) { atomicExch(a.err, 12); return false; }
                mbar_expect_tx(&v_full[st], TILE_BYTES);
                tma_load_2d(v_s + st * TILE_BYTES, &tmV, &v_full[st], kh * a.kv_hc, kh * a.kv_hr + (j0 + j) * AKV);
                tma_load_2d(v_s + st * TILE_BYTES + PANEL_BYTES, &tmV, &v_full[st], kh * a.kv_hc + 64,
                            kh * a.kv_hr + (j0 + j) * AKV);
                return true;
            };
            // load order follows the consumer: K0, then per tile V(j), K(j+1)
            bool ok = load_k(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                ok = load_v(j);
                if (ok && j + 1 < n_tiles) ok = load_k(j + 1);
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0, 0);
            constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128, 0, 1);  // V is MN-major
            bool ok = mbar_wait(q_full, 0);
            if (!ok) atomicExch(a.err, 13);
            // S_g = Q_g K_j^T; one descriptor per operand tile, the eight K steps only move its
            // 16-byte-unit address field
            auto issue_qk = [&](int g, uint64_t k_desc) {
                const uint64_t q_desc = umma_desc_sw128(smem_u32(q_s + g * TILE_BYTES), 16, 1024);
#pragma unroll
                for (int kk = 0; kk < AD / 16; ++kk) {
                    const uint64_t off = (uint64_t)(((kk >> 2) * PANEL_BYTES + (kk & 3) * 32) >> 4);
                    umma_ss(tmem_S + g * 128, q_desc + off, k_desc + off, idesc_qk, kk != 0);
                }
                umma_commit(&s_full[g]);
            };
            auto k_ready = [&](int j, uint64_t& k_desc) -> bool {
                const int st = j % K_STAGES;
                if (!mbar_wait(&k_full[st], (j / K_STAGES) & 1)) { atomicExch(a.err, 14); return false; }
                tc_fence_after();
                k_desc = umma_desc_sw128(smem_u32(k_s + st * TILE_BYTES), 16, 1024);
                return true;
            };
            uint64_t k_desc = 0;
            if (ok) ok = k_ready(0, k_desc);
            if (ok) {
                issue_qk(0, k_desc);
                issue_qk(1, k_desc);
                umma_commit(&k_empty[0]);
            }
            // Per key tile j and group g: O_g += P_g(j) V_j, then S_g = Q_g K_{j+1}^T.  P_g overlays S_g in
            // tensor memory: MMAs of one thread execute in issue order, so the next score product
            // overwrites it only after the PV product has consumed it.  While group g runs its softmax
            // the tensor pipe works on the other group.
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int vst = j % V_STAGES;
                if (!mbar_wait(&v_full[vst], (j / V_STAGES) & 1)) { atomicExch(a.err, 15); ok = false; break; }
                const uint64_t v_desc = umma_desc_sw128(smem_u32(v_s + vst * TILE_BYTES), PANEL_BYTES, 1024);
                const bool more = j + 1 < n_tiles;
                if (more && !k_ready(j + 1, k_desc)) { ok = false; break; }
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    if (!mbar_wait(&p_ready[g], j & 1)) { atomicExch(a.err, 16); ok = false; break; }
                    tc_fence_after();
                    const uint32_t p_tmem = tmem_S + g * 128;   // bf16 P in the first 64 score columns
#pragma unroll
                    for (int kk = 0; kk < AKV / 16; ++kk)       // 16 keys down per step, 128 B per key row
                        umma_ts(tmem_O + g * 128, p_tmem + kk * 8, v_desc + (uint64_t)((kk * 16 * 128) >> 4),
                                idesc_pv, (j | kk) != 0);
                    if (more) issue_qk(g, k_desc);
                }
                if (!ok) break;
                umma_commit(&v_empty[vst]);
                if (more) umma_commit(&k_empty[(j + 1) % K_STAGES]);
            }
            umma_commit(o_done);
        }
    } else {
        // -------------------------------------------------------- softmax groups + output
        const int grp = (warp - 2) >> 3;         // which of the CTA's two query tiles
        const int half = ((warp - 2) >> 2) & 1;  // which 64 score / output columns of the row
        const int qd = warp & 3;                 // TMEM lane quadrant this warp may access
        const int row = qd * 32 + lane;          // row within the query tile
        const int qg0 = q0 + grp * AQ;           // first row of this group's tile
        const int row_g = qg0 + row;             // global query index
        const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
        const bool tile_has_causal = qg0 < a.ar_len;
        const bool row_causal = row_g < a.ar_len;
        const uint32_t t_s = tmem_S + grp * 128 + lane_off;
        const uint32_t t_o = tmem_O + grp * 128 + half * 64 + lane_off;
        float* x_mine = xch + (grp * 2 + half) * 128 + row;
        const float* x_other = xch + (grp * 2 + (half ^ 1)) * 128 + row;
        const int bar_id = 1 + grp;              // named barrier of the group's 256 threads
        constexpr int BAR_THREADS = 256;
        float m_used = -INFINITY;                // max the stored P / l / O of this row are relative to
        float l = 0.f;                           // this thread's share of the row sum
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int kv0 = (j0 + j) * AKV + half * 64;
            if (!mbar_wait(&s_full[grp], j & 1)) { atomicExch(a.err, 17); ok = false; break; }
            tc_fence_after();
            const bool need_mask = (kv0 + 64 > a.S) || (tile_has_causal && kv0 + 63 > qg0);
            // this thread's 64 fp32 scores go to registers with one wait
            uint32_t r[2][32];
            tmem_ld32(t_s + half * 64, r[0]);
            tmem_ld32(t_s + half * 64 + 32, r[1]);
            tmem_ld_wait();
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < 2; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int key = kv0 + c * 32 + i;
                        const bool allow = key < a.S && (!row_causal || key <= row_g);
                        if (!allow) r[c][i] = 0xff800000u;   // -inf
                    }
            }
            float mx;
            {
                // three-input max: 64 scores in 32 instructions, four independent chains
                float mxa = -INFINITY, mxb = -INFINITY, mxc = -INFINITY, mxd = -INFINITY;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    mxa = max3(mxa, __uint_as_float(r[0][2 * i]), __uint_as_float(r[0][2 * i + 1]));
                    mxb = max3(mxb, __uint_as_float(r[0][16 + 2 * i]), __uint_as_float(r[0][16 + 2 * i + 1]));
                    mxc = max3(mxc, __uint_as_float(r[1][2 * i]), __uint_as_float(r[1][2 * i + 1]));
                    mxd = max3(mxd, __uint_as_float(r[1][16 + 2 * i]), __uint_as_float(r[1][16 + 2 * i + 1]));
                }
                mx = max3(mxa, mxb, fmaxf(mxc, mxd));
            }
            // row max over both halves: the partner thread's value comes through shared memory.  The slot
            // is rewritten one tile later, after the partner has arrived on p_ready and a new s_full
            // has come round, so one barrier per tile is enough.
            *x_mine = mx;
            asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(BAR_THREADS) : "memory");
            mx = fmaxf(mx, *x_other);
            const float m_tile = mx * a.scale_log2;
            const bool grow = (m_tile - m_used) > 8.0f;      // also true while m_used == -inf
            if (__any_sync(0xffffffffu, grow)) {
                float alpha = 1.0f;
                if (grow) {
                    alpha = ex2_approx(m_used - m_tile);         // 0 on the first tile
                    m_used = m_tile;
                    l *= alpha;
                }
                if (j >= 1) {
                    // PV_g(j-1) was issued before QK_g(j), whose completion s_full just reported: O is
                    // complete and idle until PV_g(j), which waits for p_ready.  Each thread scales its
                    // own 64 output columns.
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        uint32_t o[16];
                        tmem_ld16(t_o + c * 16, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st16(t_o + c * 16, o);
                    }
                    tmem_st_wait();
                }
            }
            // P = exp2(s * scale_log2 - m_used) as packed bf16 pairs, written over the score columns
            // (this half's 64 scores are in registers by now, and the partner only writes after the
            // barrier above, i.e. after both loads): 64 scores become 32 columns at [half*32, +32).
            // A causal row may have no visible key in this tile and none before: m_used is still -inf
            // then and every score is masked; 0 keeps exp2(-inf + 0) = 0 instead of exp2(-inf + inf)
            const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
            const uint64_t scale2 = pack_f32x2(a.scale_log2, a.scale_log2), negm2 = pack_f32x2(neg_m, neg_m);
            l += softmax_exp_store(r, scale2, negm2, t_s + half * 32);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[grp]);
        }
        // ---- output: O / l -> bf16 -> out[row_g, h*128 + half*64 ..]
        if (ok && n_tiles > 0) {
            if (!mbar_wait(o_done, 0)) { atomicExch(a.err, 19); ok = false; }
            tc_fence_after();
        }
        // the row sum is the two threads' shares together (same exchange slots; every thread of the
        // group reaches this barrier: a failed wait above fails for the whole group alike)
        *x_mine = l;
        asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(BAR_THREADS) : "memory");
        l += *x_other;
        if (ok && ways > 1) {
            // partial result of a key range: accumulator as it is (relative to m_used), max and row sum
            const int slot = (item - a.n_plain) * ways + part;
            const int prow = grp * AQ + row;
            float* po = a.part_o + ((size_t)slot * AQ2 + prow) * AD + half * 64;
            if (half == 0) {
                float2 ml = make_float2(m_used, l);
                *reinterpret_cast<float2*>(a.part_ml + ((size_t)slot * AQ2 + prow) * 2) = ml;
            }
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
                uint32_t o[32];
                tmem_ld32(t_o + c * 32, o);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    *reinterpret_cast<uint4*>(po + c * 32 + i * 4) = make_uint4(o[i * 4], o[i * 4 + 1], o[i * 4 + 2], o[i * 4 + 3]);
            }
        } else if (ok && a.out_rows > 0) {
            // Row blocks of the output live in other GPUs' memory: leave as full 128-byte row segments (4 rows
            // per store instruction) instead of 16-byte pieces of 32 rows.  The staging slice is this warp's
            // 4 KB of the Q tiles, which no MMA reads any more once o_done has completed.
            const float inv_l = 1.0f / l;
            uint8_t* stg = q_s + (warp - 2) * (32 * 128);
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
                uint32_t o[32];
                tmem_ld32(t_o + c * 32, o);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint4 pk;
                    pk.x = cvt_bf16x2(__uint_as_float(o[i * 8 + 0]) * inv_l, __uint_as_float(o[i * 8 + 1]) * inv_l);
                    pk.y = cvt_bf16x2(__uint_as_float(o[i * 8 + 2]) * inv_l, __uint_as_float(o[i * 8 + 3]) * inv_l);
                    pk.z = cvt_bf16x2(__uint_as_float(o[i * 8 + 4]) * inv_l, __uint_as_float(o[i * 8 + 5]) * inv_l);
                    pk.w = cvt_bf16x2(__uint_as_float(o[i * 8 + 6]) * inv_l, __uint_as_float(o[i * 8 + 7]) * inv_l);
                    const int j = c * 4 + i;
                    *reinterpret_cast<uint4*>(stg + lane * 128 + ((j ^ (lane & 7)) * 16)) = pk;
                }
            }
            __syncwarp();
            const int ch = lane & 7;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int rr = k * 4 + (lane >> 3);
                const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((ch ^ (rr & 7)) * 16));
                const int rg = qg0 + qd * 32 + rr;
                if (rg < a.row_hi && rg >= a.row_lo) {
                    const int blk = rg / a.out_rows;
                    uint16_t* dst = a.out_tab[blk] + (size_t)(rg - blk * a.out_rows) * a.ldo + (size_t)h * a.out_hoff +
                                    half * 64 + ch * 8;
                    *reinterpret_cast<uint4*>(dst) = v;
                }
            }
        } else if (ok) {
            const float inv_l = 1.0f / l;
            uint16_t* dst = a.out + (size_t)row_g * a.ldo + (size_t)h * a.out_hoff + half * 64;
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
                uint32_t o[32];
                tmem_ld32(t_o + c * 32, o);
                tmem_ld_wait();
                if (row_g < a.row_hi && row_g >= a.row_lo) {
                    uint4* d4 = reinterpret_cast<uint4*>(dst + c * 32);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint4 pk;
                        pk.x = cvt_bf16x2(__uint_as_float(o[i * 8 + 0]) * inv_l, __uint_as_float(o[i * 8 + 1]) * inv_l);
                        pk.y = cvt_bf16x2(__uint_as_float(o[i * 8 + 2]) * inv_l, __uint_as_float(o[i * 8 + 3]) * inv_l);
                        pk.z = cvt_bf16x2(__uint_as_float(o[i * 8 + 4]) * inv_l, __uint_as_float(o[i * 8 + 5]) * inv_l);
                        pk.w = cvt_bf16x2(__uint_as_float(o[i * 8 + 6]) * inv_l, __uint_as_float(o[i * 8 + 7]) * inv_l);
                        d4[i] = pk;
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ---------------------------------------------------------------------------------------------------------------
// One query tile per CTA, scores triple-buffered: the form used for short sequences (S < 8192), where work items of
// 256 rows are too few and too coarse for 148 SMs (S = 1280: 160 items) and the serial chain of the two-tile kernel
// has nothing to hide behind.  Tensor memory: three score buffers of 128 columns + one output accumulator.  The MMA
// thread issues S(j+3) = Q K^T right after PV(j), so the scores of the next two key tiles are always there or on their
// way and the softmax warps never wait for a score product that waits for them.  Warps 2..9 and 10..17 are two softmax
// sets that take alternate key tiles (two threads per row, as above); they agree on the running max through shared
// memory: the set that takes tile j waits for the other set's decision for tile j-1 (made early in its phase) before it
// decides for tile j.  Measured stand-alone against the two-tile kernel: S = 1280 0.048 vs 0.072 ms, S = 4352 0.312 vs
// 0.339 ms, S = 16640 3.97 vs 3.63 ms (twice the K/V fill per query row and half as long work items cost more there
// than the chain).
static constexpr int T1_ROWS = 128;       // query rows per CTA and work item
static constexpr int T1_K_STAGES = 3;
static constexpr int T1_V_STAGES = 3;
static constexpr int T1_S_BUFS = 3;       // score buffers in tensor memory
static constexpr int T1_XCH = 2048;       // row-max exchange ([set][use][half][row] bf16), at the end [quarter][row] float sums
static constexpr int T1_SMEM = TILE_BYTES * (1 + T1_K_STAGES + T1_V_STAGES) + 192 + T1_XCH + 512;

// bounded wait with one outcome for the whole warp (the code behind it issues warp-wide tensor-memory accesses)
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity));
}

__global__ void __launch_bounds__(ATTN_THREADS, 1)
flash_attn1_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const AttnArgs a) {
    // Q | K x3 | V x3: 7 tiles of 32 KB again, the window 1024-byte aligned (checked below)
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* q_s = smem;                               // the query tile
    uint8_t* k_s = q_s + TILE_BYTES;
    uint8_t* v_s = k_s + T1_K_STAGES * TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + T1_V_STAGES * TILE_BYTES);
    uint64_t* q_full = bars;                // 1
    uint64_t* k_full = bars + 1;            // T1_K_STAGES
    uint64_t* k_empty = k_full + T1_K_STAGES;
    uint64_t* v_full = k_empty + T1_K_STAGES;  // T1_V_STAGES
    uint64_t* v_empty = v_full + T1_V_STAGES;
    uint64_t* s_full = v_empty + T1_V_STAGES;  // T1_S_BUFS (one per score buffer)
    uint64_t* p_ready = s_full + T1_S_BUFS;    // T1_S_BUFS
    uint64_t* m_pub = p_ready + T1_S_BUFS;     // 2 (one per softmax set)
    uint64_t* o_done = m_pub + 2;           // 1
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 1);
    int* s_abort = reinterpret_cast<int*>(tmem_slot + 1);
    float* xch = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 192);
    float* m_sh = xch + T1_XCH / 4;       // [row]: the max every stored P, partial sum and O is relative to

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    int item = blockIdx.x, part = 0, ways = 1;
    if (item >= a.n_plain) {
        const int t = item - a.n_plain;
        item = a.n_plain + t / a.ways;
        part = t - (t / a.ways) * a.ways;
        ways = a.ways;
    }
    const int h = item / a.nqb;
    const int q0 = (item - h * a.nqb) * T1_ROWS;
    const int kh = h / (a.heads / a.kv_heads);
    if (q0 + T1_ROWS <= a.row_lo || q0 >= a.row_hi) return;   // no row of this block is wanted (whole CTA, before any set-up)

    // keys this query tile can see
    int kv_end = a.S;
    if (q0 + T1_ROWS - 1 < a.ar_len) kv_end = q0 + T1_ROWS;   // all rows causal: keys <= last row
    if (kv_end > a.S) kv_end = a.S;
    const int tiles_all = (kv_end + AKV - 1) / AKV;
    const int j0 = (int)((long)part * tiles_all / ways);                  // first key tile of this CTA
    const int n_tiles = (int)((long)(part + 1) * tiles_all / ways) - j0;  // and how many it covers
    if (n_tiles <= 0) {
        // a part of a tail item that has fewer key tiles than parts: an empty partial (max -inf, sum 0), nothing else
        if (threadIdx.x < T1_ROWS) {
            const int slot = (item - a.n_plain) * ways + part;
            *reinterpret_cast<float2*>(a.part_ml + ((size_t)slot * T1_ROWS + threadIdx.x) * 2) = make_float2(-INFINITY, 0.f);
        }
        return;
    }

    // a kernel that already failed on this device leaves its code in *err: do nothing then
    if (threadIdx.x == 0) {
        int ab = *reinterpret_cast<volatile int*>(a.err);
        if (ab == 0 && (smem_u32(smem) & 1023u) != 0) { ab = 20; atomicExch(a.err, 20); }
        *s_abort = ab;
    }
    __syncthreads();
    if (*s_abort != 0) return;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < T1_K_STAGES; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
        for (int s = 0; s < T1_V_STAGES; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
        for (int s = 0; s < T1_S_BUFS; ++s) { mbar_init(&s_full[s], 1); mbar_init(&p_ready[s], 8); }
        for (int s = 0; s < 2; ++s) mbar_init(&m_pub[s], 4);
        mbar_init(o_done, 1);
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_S = tmem_base;         // three score buffers: columns [0,128), [128,256), [256,384)
    const uint32_t tmem_O = tmem_base + 384;   // output accumulator: [384,512)

    if (warp == 0) {
        // -------------------------------------------------------- TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&tmQ);
            tma_prefetch_desc(&tmK);
            tma_prefetch_desc(&tmV);
            mbar_expect_tx(q_full, TILE_BYTES);
            tma_load_2d(q_s, &tmQ, q_full, h * a.q_hc, h * a.q_hr + q0);
            tma_load_2d(q_s + PANEL_BYTES, &tmQ, q_full, h * a.q_hc + 64, h * a.q_hr + q0);
            auto load_k = [&](int j) -> bool {
                const int st = j % T1_K_STAGES;
                if (!mbar_wait(&k_empty[st], ((j / T1_K_STAGES) & 1) ^ 1)) { atomicExch(a.err, 11); return false; }
                mbar_expect_tx(&k_full[st], TILE_BYTES);
                tma_load_2d(k_s + st * TILE_BYTES, &tmK, &k_full[st], kh * a.kv_hc, kh * a.kv_hr + (j0 + j) * AKV);
                tma_load_2d(k_s + st * TILE_BYTES + PANEL_BYTES, &tmK, &k_full[st], kh * a.kv_hc + 64,
                            kh * a.kv_hr + (j0 + j) * AKV);
                return true;
            };
            auto load_v = [&](int j) -> bool {
                const int st = j % T1_V_STAGES;
                if (!mbar_wait(&v_empty[st], ((j / T1_V_STAGES) & 1) ^ 1)) { atomicExch(a.err, 12); return false; }
                mbar_expect_tx(&v_full[st], TILE_BYTES);
                tma_load_2d(v_s + st * TILE_BYTES, &tmV, &v_full[st], kh * a.kv_hc, kh * a.kv_hr + (j0 + j) * AKV);
                tma_load_2d(v_s + st * TILE_BYTES + PANEL_BYTES, &tmV, &v_full[st], kh * a.kv_hc + 64,
                            kh * a.kv_hr + (j0 + j) * AKV);
                return true;
            };
            // load order follows the consumer: K0 .. K(T1_S_BUFS-1), then per tile V(j), K(j+T1_S_BUFS)
            bool ok = true;
            for (int j = 0; j < T1_S_BUFS && j < n_tiles && ok; ++j) ok = load_k(j);
            for (int j = 0; j < n_tiles && ok; ++j) {
                ok = load_v(j);
                if (ok && j + T1_S_BUFS < n_tiles) ok = load_k(j + T1_S_BUFS);
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0, 0);
            constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128, 0, 1);  // V is MN-major
            bool ok = mbar_wait(q_full, 0);
            if (!ok) atomicExch(a.err, 13);
            const uint64_t q_desc = umma_desc_sw128(smem_u32(q_s), 16, 1024);
            // S(j) = Q K_j^T into score buffer j % T1_S_BUFS; one descriptor per operand tile, the eight K steps
            // only move its 16-byte-unit address field
            auto issue_qk = [&](int j) -> bool {
                const int st = j % T1_K_STAGES;
                if (!mbar_wait(&k_full[st], (j / T1_K_STAGES) & 1)) { atomicExch(a.err, 14); return false; }
                tc_fence_after();
                const uint64_t k_desc = umma_desc_sw128(smem_u32(k_s + st * TILE_BYTES), 16, 1024);
                const int b = j % T1_S_BUFS;
#pragma unroll
                for (int kk = 0; kk < AD / 16; ++kk) {
                    const uint64_t off = (uint64_t)(((kk >> 2) * PANEL_BYTES + (kk & 3) * 32) >> 4);
                    umma_ss(tmem_S + b * 128, q_desc + off, k_desc + off, idesc_qk, kk != 0);
                }
                umma_commit(&s_full[b]);
                umma_commit(&k_empty[st]);
                return true;
            };
            for (int j = 0; j < T1_S_BUFS && j < n_tiles && ok; ++j) ok = issue_qk(j);
            // Per key tile j: O += P(j) V_j, then S(j + T1_S_BUFS) = Q K^T into the buffer P(j) leaves (MMAs of one
            // thread execute in issue order).  The scores of the next T1_S_BUFS - 1 tiles are already there or on
            // their way, so the softmax warps never wait for a score product that waits for them.
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int vst = j % T1_V_STAGES;
                const int b = j % T1_S_BUFS;
                if (!mbar_wait(&v_full[vst], (j / T1_V_STAGES) & 1)) { atomicExch(a.err, 15); ok = false; break; }
                const uint64_t v_desc = umma_desc_sw128(smem_u32(v_s + vst * TILE_BYTES), PANEL_BYTES, 1024);
                if (!mbar_wait(&p_ready[b], (j / T1_S_BUFS) & 1)) { atomicExch(a.err, 16); ok = false; break; }
                tc_fence_after();
                const uint32_t p_tmem = tmem_S + b * 128;   // bf16 P in the first 64 columns of the buffer
#pragma unroll
                for (int kk = 0; kk < AKV / 16; ++kk)       // 16 keys down per step, 128 B per key row
                    umma_ts(tmem_O, p_tmem + kk * 8, v_desc + (uint64_t)((kk * 16 * 128) >> 4), idesc_pv, (j | kk) != 0);
                umma_commit(&v_empty[vst]);
                if (j + T1_S_BUFS < n_tiles) ok = issue_qk(j + T1_S_BUFS);
            }
            umma_commit(o_done);
        }
    } else {
        // -------------------------------------------------------- softmax sets + output
        const int set = (warp - 2) >> 3;         // set 0 takes the even key tiles, set 1 the odd ones
        const int half = ((warp - 2) >> 2) & 1;  // which 64 score columns of the row
        const int part4 = (warp - 2) >> 2;       // which 32 output columns of the row (epilogue)
        const int qd = warp & 3;                 // TMEM lane quadrant this warp may access
        const int row = qd * 32 + lane;          // row within the query tile
        const int row_g = q0 + row;              // global query index
        const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
        const bool tile_has_causal = q0 < a.ar_len;
        const bool row_causal = row_g < a.ar_len;
        const uint32_t t_o = tmem_O + half * 64 + lane_off;
        // row-max exchange slots of the two threads of a row: [set][use parity][half][row] bf16
        uint16_t* x16 = reinterpret_cast<uint16_t*>(xch) + set * 512 + row;
        const int bar_id = 1 + set;              // named barrier of the set's 256 threads
        constexpr int BAR_THREADS = 256;
        float m_mine = -INFINITY;                // max this thread's partial sum is relative to
        float l = 0.f;                           // this thread's share of the row sum
        bool ok = true;
        for (int j = set; j < n_tiles; j += 2) {
            const int b = j % T1_S_BUFS;
            const int use = (j >> 1) & 1;
            const int kv0 = (j0 + j) * AKV + half * 64;
            const uint32_t t_s = tmem_S + b * 128 + lane_off;
            // A thread whose wait ran out keeps taking part in the set's named barrier (one per tile) and does
            // nothing else, so that no partner is left waiting at a barrier that has no time limit.
            uint32_t r[2][32];
            uint32_t mb = 0;
            if (ok && !mbar_wait_warp(&s_full[b], (j / T1_S_BUFS) & 1)) { atomicExch(a.err, 17); ok = false; }
            if (ok) {
            tc_fence_after();
            const bool need_mask = (kv0 + 64 > a.S) || (tile_has_causal && kv0 + 63 > q0);
            // this thread's 64 fp32 scores go to registers with one wait
            tmem_ld32(t_s + half * 64, r[0]);
            tmem_ld32(t_s + half * 64 + 32, r[1]);
            tmem_ld_wait();
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < 2; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int key = kv0 + c * 32 + i;
                        const bool allow = key < a.S && (!row_causal || key <= row_g);
                        if (!allow) r[c][i] = 0xff800000u;   // -inf
                    }
            }
            float mx;
            {
                // three-input max: 64 scores in 32 instructions, four independent chains
                float mxa = -INFINITY, mxb = -INFINITY, mxc = -INFINITY, mxd = -INFINITY;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    mxa = max3(mxa, __uint_as_float(r[0][2 * i]), __uint_as_float(r[0][2 * i + 1]));
                    mxb = max3(mxb, __uint_as_float(r[0][16 + 2 * i]), __uint_as_float(r[0][16 + 2 * i + 1]));
                    mxc = max3(mxc, __uint_as_float(r[1][2 * i]), __uint_as_float(r[1][2 * i + 1]));
                    mxd = max3(mxd, __uint_as_float(r[1][16 + 2 * i]), __uint_as_float(r[1][16 + 2 * i + 1]));
                }
                mx = max3(mxa, mxb, fmaxf(mxc, mxd));
            }
            // Row max over both halves: the partner thread's value comes through shared memory.  The reference
            // value only has to be the same for both threads and not below the true max, so it travels as a
            // bf16 rounded toward +inf.  A slot is rewritten two uses later, after a barrier the partner only
            // reaches once it has read this use's value.
            mb = __float_as_uint(mx);
            mb = ((int32_t)mb >= 0) ? (mb + 0xffffu) : mb;     // +inf / NaN cannot occur in a score
            x16[use * 256 + half * 128] = (uint16_t)(mb >> 16);
            }
            asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(BAR_THREADS) : "memory");
            if (!ok) continue;
            float mx = fmaxf(__uint_as_float(mb & 0xffff0000u), __uint_as_float((uint32_t)x16[use * 256 + (half ^ 1) * 128] << 16));
            const float m_tile = mx * a.scale_log2;
            // the max in force after the previous tile, which the other set decided
            float m_prev = -INFINITY;
            if (j >= 1) {
                if (!mbar_wait_warp(&m_pub[set ^ 1], ((j - 1) >> 1) & 1)) { atomicExch(a.err, 18); ok = false; continue; }
                m_prev = m_sh[row];
            }
            if (m_prev != m_mine) {        // the other set raised it: this thread's sum follows
                l *= ex2_approx(m_mine - m_prev);     // m_mine == -inf: l is 0 and stays 0
                m_mine = m_prev;
            }
            const bool grow = (m_tile - m_mine) > 8.0f;      // also true while m_mine == -inf
            float alpha = 1.0f;
            if (grow) {
                alpha = ex2_approx(m_mine - m_tile);         // 0 on the first tile
                m_mine = m_tile;
                l *= alpha;
            }
            if (half == 0) {
                m_sh[row] = m_mine;
                __syncwarp();
                if (lane == 0) mbar_arrive(&m_pub[set]);
            }
            if (j >= 1 && __any_sync(0xffffffffu, grow)) {
                // O must hold all of PV(j-1) and nothing of PV(j): the first is what v_empty of tile j-1 reports,
                // the second waits for this set's p_ready.  Each thread scales its own 64 output columns.
                if (!mbar_wait_warp(&v_empty[(j - 1) % T1_V_STAGES], ((j - 1) / T1_V_STAGES) & 1)) { atomicExch(a.err, 21); ok = false; continue; }
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t o[16];
                    tmem_ld16(t_o + c * 16, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st16(t_o + c * 16, o);
                }
                tmem_st_wait();
            }
            // P = exp2(s * scale_log2 - m) as packed bf16 pairs, written over the score columns (this half's 64
            // scores are in registers by now, and the partner only writes after the barrier above, i.e. after
            // both loads): 64 scores become 32 columns at [half*32, +32).  A causal row may have no visible key
            // in this tile and none before: m is still -inf then and every score is masked; 0 keeps
            // exp2(-inf + 0) = 0 instead of exp2(-inf + inf)
            const float neg_m = (m_mine == -INFINITY) ? 0.f : -m_mine;
            const uint64_t scale2 = pack_f32x2(a.scale_log2, a.scale_log2), negm2 = pack_f32x2(neg_m, neg_m);
            l += softmax_exp_store(r, scale2, negm2, t_s + half * 32);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[b]);
        }
        // ---- the sums of the set that did not take the last tile follow its max
        if (ok && ((n_tiles - 1) & 1) != set) {
            if (!mbar_wait_warp(&m_pub[set ^ 1], ((n_tiles - 1) >> 1) & 1)) { atomicExch(a.err, 18); ok = false; }
            if (ok) {
                const float m_fin = m_sh[row];
                if (m_fin != m_mine) { l *= ex2_approx(m_mine - m_fin); m_mine = m_fin; }
            }
        }
        // ---- output: O / l -> bf16 -> out[row_g, h*128 + part4*32 ..]
        if (ok) {
            if (!mbar_wait_warp(o_done, 0)) { atomicExch(a.err, 19); ok = false; }
            tc_fence_after();
        }
        // the row sum is the four threads' shares together (the exchange window as [quarter][row] floats; every
        // softmax thread reaches these barriers: a failed wait above fails for all of them alike)
        asm volatile("bar.sync 3, 512;" ::: "memory");
        xch[part4 * 128 + row] = l;
        asm volatile("bar.sync 3, 512;" ::: "memory");
        const float lsum = (xch[row] + xch[128 + row]) + (xch[256 + row] + xch[384 + row]);
        if (ok) {
            uint32_t o[32];
            tmem_ld32(tmem_O + part4 * 32 + lane_off, o);
            tmem_ld_wait();
            if (ways > 1) {
                // partial result of a key range: accumulator as it is (relative to the max), max and row sum
                const int slot = (item - a.n_plain) * ways + part;
                float* po = a.part_o + ((size_t)slot * T1_ROWS + row) * AD + part4 * 32;
                if (part4 == 0) {
                    float2 ml = make_float2(m_mine, lsum);
                    *reinterpret_cast<float2*>(a.part_ml + ((size_t)slot * T1_ROWS + row) * 2) = ml;
                }
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    *reinterpret_cast<uint4*>(po + i * 4) = make_uint4(o[i * 4], o[i * 4 + 1], o[i * 4 + 2], o[i * 4 + 3]);
            } else {
                const float inv_l = 1.0f / lsum;
                uint4 pk[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    pk[i].x = cvt_bf16x2(__uint_as_float(o[i * 8 + 0]) * inv_l, __uint_as_float(o[i * 8 + 1]) * inv_l);
                    pk[i].y = cvt_bf16x2(__uint_as_float(o[i * 8 + 2]) * inv_l, __uint_as_float(o[i * 8 + 3]) * inv_l);
                    pk[i].z = cvt_bf16x2(__uint_as_float(o[i * 8 + 4]) * inv_l, __uint_as_float(o[i * 8 + 5]) * inv_l);
                    pk[i].w = cvt_bf16x2(__uint_as_float(o[i * 8 + 6]) * inv_l, __uint_as_float(o[i * 8 + 7]) * inv_l);
                }
                if (a.out_rows > 0) {
                    // Row blocks of the output live in other GPUs' memory: leave as 64-byte row segments (8 rows
                    // per store instruction) instead of 16-byte pieces of 32 rows.  The staging slice is this
                    // warp's 2 KB of the Q tile, which no MMA reads any more once o_done has completed.
                    uint8_t* stg = q_s + (warp - 2) * (32 * 64);
#pragma unroll
                    for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(stg + lane * 64 + ((i ^ (lane & 3)) * 16)) = pk[i];
                    __syncwarp();
                    const int ch = lane & 3;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int rr = k * 8 + (lane >> 2);
                        const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * 64 + ((ch ^ (rr & 3)) * 16));
                        const int rg = q0 + qd * 32 + rr;
                        if (rg < a.row_hi && rg >= a.row_lo) {
                            const int blk = rg / a.out_rows;
                            uint16_t* dst = a.out_tab[blk] + (size_t)(rg - blk * a.out_rows) * a.ldo + (size_t)h * a.out_hoff +
                                            part4 * 32 + ch * 8;
                            *reinterpret_cast<uint4*>(dst) = v;
                        }
                    }
                } else if (row_g < a.row_hi && row_g >= a.row_lo) {
                    uint4* d4 = reinterpret_cast<uint4*>(a.out + (size_t)row_g * a.ldo + (size_t)h * a.out_hoff + part4 * 32);
#pragma unroll
                    for (int i = 0; i < 4; ++i) d4[i] = pk[i];
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// Combines the partial results of the tail items: out = sum_i O_i 2^(m_i - M) / sum_i l_i 2^(m_i - M).
// One block per query row, one thread per output column.
__global__ void __launch_bounds__(AD) attn_merge_kernel(const AttnArgs a, int n_tail, int AQ2 /* rows per item */) {
    const int ti = blockIdx.x / AQ2, r = blockIdx.x - ti * AQ2;
    if (ti >= n_tail) return;
    const int item = a.n_plain + ti;
    const int h = item / a.nqb;
    const int row_g = (item - h * a.nqb) * AQ2 + r;
    if (row_g >= a.S) return;
    const int col = threadIdx.x;
    float M = -INFINITY;
    for (int i = 0; i < a.ways; ++i) M = fmaxf(M, a.part_ml[((size_t)(ti * a.ways + i) * AQ2 + r) * 2]);
    float num = 0.f, den = 0.f;
    for (int i = 0; i < a.ways; ++i) {
        const size_t pr = (size_t)(ti * a.ways + i) * AQ2 + r;
        const float m = a.part_ml[pr * 2];
        if (m == -INFINITY) continue;           // this key range held no visible key for the row
        const float wgt = exp2f(m - M);
        num = fmaf(a.part_o[pr * AD + col], wgt, num);
        den = fmaf(a.part_ml[pr * 2 + 1], wgt, den);
    }
    const float v = num * (1.0f / den);
    uint16_t* dst = a.out + (size_t)row_g * a.ldo + (size_t)h * a.out_hoff;
    if (a.out_rows > 0) {
        const int blk = row_g / a.out_rows;
        dst = a.out_tab[blk] + (size_t)(row_g - blk * a.out_rows) * a.ldo + (size_t)h * a.out_hoff;
    }
    dst[col] = f32_to_bf16(v);
}

// Number of key-range parts for the tail items: the last (total % SMs) items would otherwise occupy a wave
// of CTAs alone.  Cost of the tail in item durations: rounds of CTAs it needs, ceil(rem * w / SMs), times the
// duration of a part, 1/w plus a fixed share for its prologue, Q load and fp32 epilogue (about four key
// tiles' worth).  Measured on B200: the split pays when the tail is a sizeable part of a wave (76 of 148 SMs
// at 8 heads and S = 16640: -13 %) or when at most one full wave precedes it (S = 1280: -20 %); after many
// full waves the SMs have drifted apart and a tail of a few items costs next to nothing (no gain measured
// with 4 or 8 tail items after 7 or 14 waves), so it is left alone.  Every part keeps at least two key tiles.
static int g_tail_ways = 0;   // 0: choose; 1: never split; n > 1: n parts whenever they fit
void attention_tail_ways(int ways) { g_tail_ways = ways < 0 ? 0 : ways; }
// Which kernel: 0 = by sequence length (one query tile per CTA below 8192 keys, two from there on), 1 = always the two-tile
// kernel, 2 = always the one-tile kernel
static int g_tile_mode = -1;    // -1: not yet read from the environment (O1_ATTN_TILE_MODE)
void attention_tile_mode(int mode) { g_tile_mode = (mode < 0 || mode > 2) ? 0 : mode; }
static int tile_mode() {
    if (g_tile_mode < 0) {
        const char* e = getenv("O1_ATTN_TILE_MODE");
        g_tile_mode = (e && (e[0] == '1' || e[0] == '2')) ? e[0] - '0' : 0;
    }
    return g_tile_mode;
}

static int choose_tail_ways(int total, int nsm, int min_tiles, size_t scratch_bytes, int rows_item) {
    const int rem = total % nsm;
    if (rem == 0) return 1;
    const size_t part_bytes = (size_t)rows_item * AD * 4 + (size_t)rows_item * 2 * 4;
    if (g_tail_ways >= 1) {
        const bool fits = g_tail_ways * 2 <= min_tiles && (size_t)rem * g_tail_ways * part_bytes <= scratch_bytes;
        return fits ? g_tail_ways : 1;
    }
    const double fixed = 4.0 / min_tiles;
    int best = 1;
    double best_cost = 1.0;
    for (int w = 2; w <= 32 && w * 2 <= min_tiles; ++w) {
        if ((size_t)rem * w * part_bytes > scratch_bytes) break;
        const double cost = (double)((rem * w + nsm - 1) / nsm) * (1.0 / w + fixed) + 0.02;
        if (cost < best_cost - 1e-9) { best_cost = cost; best = w; }
    }
    const bool worth = rem * 4 >= nsm || total / nsm <= 1;
    return (worth && best_cost < 0.9) ? best : 1;
}

static bool flash_attention_impl(const void* q, int ldq, const void* k, int ldk, const void* v,
                                 int ldv, void* out, int ldo, int S, int heads, int kv_heads,
                                 int ar_len, float scale, bool in_head_major, bool out_head_major,
                                 cudaStream_t st, void* const* out_tab = nullptr, int out_rows = 0,
                                 void* scratch = nullptr, size_t scratch_bytes = 0, int row_lo = 0, int row_hi = -1) {
    if (out_tab) {
        if (out_rows <= 0 || (S + out_rows - 1) / out_rows > 8 || out_head_major) { set_error("attention: bad output table"); return false; }
        for (int i = 0; i < (S + out_rows - 1) / out_rows; ++i)
            if (!out_tab[i] || (((uintptr_t)out_tab[i]) & 15)) { set_error("attention: output table entry %d unusable", i); return false; }
        out = out_tab[0];
    }
    if (!q || !k || !v || !out || S <= 0 || heads <= 0 || kv_heads <= 0 || (heads % kv_heads) != 0) {
        set_error("attention: bad args");
        return false;
    }
    if ((ldo % 8) != 0 || (((uintptr_t)out) & 15)) { set_error("attention: output not 16-byte aligned"); return false; }
    if (ar_len < 0) ar_len = 0;
    if (ar_len > S) ar_len = S;
    CUtensorMap mq, mk, mv;
    bool maps_ok;
    if (in_head_major) {
        maps_ok = cached_tmap(&mq, q, (uint64_t)heads * S, AD, AD, 128) &&
                  cached_tmap(&mk, k, (uint64_t)kv_heads * S, AD, AD, 128) &&
                  cached_tmap(&mv, v, (uint64_t)kv_heads * S, AD, AD, 128);
    } else {
        maps_ok = cached_tmap(&mq, q, S, (uint64_t)heads * AD, ldq, 128) &&
                  cached_tmap(&mk, k, S, (uint64_t)kv_heads * AD, ldk, 128) &&
                  cached_tmap(&mv, v, S, (uint64_t)kv_heads * AD, ldv, 128);
    }
    if (!maps_ok) return false;
    const CUtensorMap *tq = &mq, *tk = &mk, *tv = &mv;
    const bool one_tile = tile_mode() == 2 || (tile_mode() == 0 && S < 8192);
    const int rows_item = one_tile ? T1_ROWS : AQ2;
    static std::atomic<uint64_t> attr_done{0}, attr1_done{0};
    if (one_tile) {
        if (!func_attr_once(attr1_done, (const void*)flash_attn1_kernel, T1_SMEM, "attention (one tile)")) return false;
    } else if (!func_attr_once(attr_done, (const void*)flash_attn_kernel, ATTN_SMEM, "attention")) return false;
    AttnArgs a;
    a.out = (uint16_t*)out; a.ldo = ldo;
    a.S = S; a.heads = heads; a.kv_heads = kv_heads; a.ar_len = ar_len;
    a.row_lo = row_lo < 0 ? 0 : row_lo;
    a.row_hi = (row_hi < 0 || row_hi > S) ? S : row_hi;
    if (a.row_lo != 0 || a.row_hi != S) { scratch = nullptr; scratch_bytes = 0; }   // a row range never splits its tail items
    a.scale_log2 = scale * 1.4426950408889634f;
    a.q_hc = in_head_major ? 0 : AD;  a.q_hr = in_head_major ? S : 0;
    a.kv_hc = a.q_hc;                 a.kv_hr = a.q_hr;
    a.out_hoff = out_head_major ? (long)S * AD : AD;
    if (out_head_major) a.ldo = AD;
    a.err = device_error_word();
    a.out_rows = out_tab ? out_rows : 0;
    for (int i = 0; i < 8; ++i) a.out_tab[i] = nullptr;
    if (out_tab) for (int i = 0; i < (S + out_rows - 1) / out_rows; ++i) a.out_tab[i] = (uint16_t*)out_tab[i];
    a.nqb = (S + rows_item - 1) / rows_item;
    const int total = a.nqb * heads;
    a.n_plain = total; a.ways = 1; a.part_o = nullptr; a.part_ml = nullptr;
    int n_tail = 0;
    if (scratch && scratch_bytes && (((uintptr_t)scratch) & 15) == 0) {
        const int nsm = sm_count();
        const int rem = total % nsm;
        // fewest key tiles among the tail items (all-causal query blocks stop at the diagonal)
        int min_tiles = 1 << 30;
        for (int it = total - rem; it < total; ++it) {
            const int q0 = (it % a.nqb) * rows_item;
            int kv_end = (q0 + rows_item - 1 < ar_len) ? q0 + rows_item : S;
            if (kv_end > S) kv_end = S;
            const int t = (kv_end + AKV - 1) / AKV;
            // (items of a few key tiles, the fully causal first query tiles, are short anyway: they do not limit
            // the number of parts, and parts of theirs that get no key tile leave an empty partial)
            if (t >= 4 && t < min_tiles) min_tiles = t;
        }
        const int w = (rem && min_tiles < (1 << 30)) ? choose_tail_ways(total, nsm, min_tiles, scratch_bytes, rows_item) : 1;
        if (w > 1) {
            n_tail = rem;
            a.n_plain = total - rem;
            a.ways = w;
            a.part_o = (float*)scratch;
            a.part_ml = a.part_o + (size_t)rem * w * rows_item * AD;
        }
    }
    dim3 grid(a.n_plain + n_tail * a.ways);
    {
        // QK^T + PV over the keys each row can see: 4*heads*128*(ar(ar+1)/2 + (S-ar)*S)
        const double keys = 0.5 * ar_len * (ar_len + 1.0) + (double)(S - ar_len) * S;
        prof_before(PROF_ATTN, 4.0 * heads * 128.0 * keys, st);
    }
    if (one_tile) flash_attn1_kernel<<<grid, ATTN_THREADS, T1_SMEM, st>>>(*tq, *tk, *tv, a);
    else flash_attn_kernel<<<grid, ATTN_THREADS, ATTN_SMEM, st>>>(*tq, *tk, *tv, a);
    if (n_tail) attn_merge_kernel<<<n_tail * rows_item, AD, 0, st>>>(a, n_tail, rows_item);
    prof_after(st);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_error("attention: launch: %s", cudaGetErrorString(e)); return false; }
    return true;
}

bool flash_attention(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv,
                     void* out, int ldo, int S, int heads, int kv_heads, int ar_len, float scale,
                     cudaStream_t st, void* scratch, size_t scratch_bytes) {
    return flash_attention_impl(q, ldq, k, ldk, v, ldv, out, ldo, S, heads, kv_heads, ar_len, scale,
                                false, false, st, nullptr, 0, scratch, scratch_bytes);
}
bool flash_attention_tab(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv,
                         void* const* out_tab, int out_rows, int ldo, int S, int heads, int kv_heads,
                         int ar_len, float scale, cudaStream_t st, void* scratch, size_t scratch_bytes) {
    return flash_attention_impl(q, ldq, k, ldk, v, ldv, nullptr, ldo, S, heads, kv_heads, ar_len, scale,
                                false, false, st, out_tab, out_rows, scratch, scratch_bytes);
}
// q [heads,S,128], k/v [kv_heads,S,128]; out head-major [heads,S,128] or seq-major [S, heads*128]
bool flash_attention_hm(const void* q, const void* k, const void* v, void* out, int S, int heads,
                        int kv_heads, int ar_len, float scale, bool out_head_major, cudaStream_t st,
                        int row_lo, int row_hi) {
    return flash_attention_impl(q, AD, k, AD, v, AD, out, heads * AD, S, heads, kv_heads, ar_len,
                                scale, true, out_head_major, st, nullptr, 0, nullptr, 0, row_lo, row_hi);
}

}  // namespace o1
