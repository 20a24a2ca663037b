// Dense linear layer  Y[M,N] = X[M,K] * W[N,K]^T  (bf16 in, fp32 accumulate,
// bf16 out) on the sm_100a tensor cores.  Replaces the cuBLASLt path of
// o1.c's hd_linear (src/cuda/gemm.cu:413-461, 506-525).
//
// Structure: persistent CTAs (one per SM), 128 x BN x 64 tiles.
//   warp 0      : TMA producer  (global -> 128B-swizzled shared, 4-6 stages)
//   warp 1      : tcgen05.mma issuer, accumulators in TMEM, double buffered
//   warps 2..5  : epilogue (tcgen05.ld -> registers -> fused op -> global)
// The epilogue of tile i overlaps the main loop of tile i+1.
//
// Fused epilogues keep the reference's bf16 rounding points:
//   BIAS   : bf16(bf16(acc) + bias)            (gemm.cu:226-236 second pass)
//   RESID  : bf16(bf16(acc) + resid)           (residual.cu:14-23)
//   SWIGLU : B tile = 128 gate rows + 128 up rows of the same columns;
//            bf16(bf16(silu(bf16 g)) * bf16 u) (act.cu:22-34)
//   LORA   : W = bf16(f32(W) + scale*acc)      (lora_merge.cu:26-33)
#include <cstdlib>
#include "common.cuh"
#include "ptx.cuh"
#include "kernels.h"

#include <atomic>
#include <map>
#include <mutex>
#include <tuple>

namespace o1 {

static constexpr int BM = 128;
static constexpr int BK = 64;
static constexpr int GEMM_THREADS = 192;

struct GemmArgs {
    int M, N, K;
    uint16_t* out;
    int ldo;
    const uint16_t* bias;
    const uint16_t* resid;
    int ldr;
    const float* rope;     // EPI_QKNORM: cos|sin table [M,128] fp32
    float scale;
    int num_m, num_n, group_m;
    // Output column blocks: column c lives at out + (c / o_cb) * o_cb_stride + row * ldo + c % o_cb
    // (o_cb == 0: plain row-major).  Lets a projection write its head groups into per-destination
    // slabs of an all-to-all send buffer.  o_cb must be a multiple of the tile width.
    int o_cb;
    long o_cb_stride;
    // With o_tab_n > 0 block b starts at o_tab[b] instead of out + b * o_cb_stride: the blocks may then
    // live in other GPUs' memory (peer-mapped), which turns the epilogue's stores into the transfer.
    int o_tab_n;
    uint16_t* o_tab[8];
    // Input K blocks: K columns [b*a_kblk, (b+1)*a_kblk) of row r live at x[(b*a_rows + r) * ldx + ...]
    // (a_kblk == 0: plain).  Lets a projection read the slabs an all-to-all received, one per source.
    int a_kblk, a_rows;
    // EPI_QKV: the output columns are three segments [q | k | v] with a weight tensor each (tensor maps B, B2, B3);
    // q and k tiles take the per-head norm + rotary epilogue (norm weights seg_norm[0], [1]), v tiles are stored as
    // they are.  seg_n = columns of q and of k (= v).  With output tables, segment s uses o_tab[8*s ...] and its own
    // block width seg_cb[s].
    int seg_n[2];
    const uint16_t* seg_norm[2];
    int seg_cb[3];
    uint16_t* seg_tab[16];    // tables of segments 1 and 2 (segment 0 uses o_tab)
    int* err;
};

// PAIR: two CTAs (a cluster) work on one 256 x BN tile with cta_group::2 MMAs; each holds its own 128 rows of A and
// of the accumulator and HALF of the B tile, so a stage is a third smaller and a B element is fetched into shared
// memory once per 256 output rows instead of once per 128.
template <int BN, bool PAIR = false>
struct GemmCfg {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = (PAIR ? BN / 2 : BN) * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = PAIR ? 6 : ((BN == 256) ? 4 : 6);
    static constexpr int STORE_STAGE_BYTES = 4 * 2 * 32 * 128;   // per epilogue warp two slices of 32 rows x 128 B (peer stores)
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/ + STORE_STAGE_BYTES;
    static constexpr int TMEM_COLS = 2 * BN;
};

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int group_m, int& mb, int& nb) {
    const int per_group = group_m * num_n;
    const int grp = tile / per_group;
    const int r = tile - grp * per_group;
    const int m_first = grp * group_m;
    int gm = num_m - m_first;
    if (gm > group_m) gm = group_m;
    mb = m_first + r % gm;
    nb = r / gm;
}

// GELU of a bf16-valued activation, as o1.c's vision kernels compute it (src/cuda/vision_kernels.cu:100-133):
// the tanh form of the ViT block MLP or the erf form of the patch mergers, fp32 throughout, rounded by the caller
__device__ __forceinline__ float gelu_of(float v, bool exact) {
    if (exact) return 0.5f * v * (1.0f + erff(v * 0.7071067811865476f));
    const float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    return 0.5f * v * (1.0f + tanhf(u));
}
__device__ __forceinline__ void store32_bf16(uint16_t* dst, const float (&v)[32]) {
    uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint4 o;
        o.x = pack_bf16x2(v[i * 8 + 0], v[i * 8 + 1]);
        o.y = pack_bf16x2(v[i * 8 + 2], v[i * 8 + 3]);
        o.z = pack_bf16x2(v[i * 8 + 4], v[i * 8 + 5]);
        o.w = pack_bf16x2(v[i * 8 + 6], v[i * 8 + 7]);
        d4[i] = o;
    }
}
__device__ __forceinline__ void load32_bf16(const uint16_t* src, float (&v)[32]) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint4 o = s4[i];
        v[i * 8 + 0] = bf16lo(o.x); v[i * 8 + 1] = bf16hi(o.x);
        v[i * 8 + 2] = bf16lo(o.y); v[i * 8 + 3] = bf16hi(o.y);
        v[i * 8 + 4] = bf16lo(o.z); v[i * 8 + 5] = bf16hi(o.z);
        v[i * 8 + 6] = bf16lo(o.w); v[i * 8 + 7] = bf16hi(o.w);
    }
}

template <int EPI, int BN, bool PAIR>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ CUtensorMap tmB3, const GemmArgs g) {
    using Cfg = GemmCfg<BN, PAIR>;
    static_assert(!PAIR || BN == 256, "the pair form splits a 256-wide B tile");
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* tfull = empty + STAGES;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    uint8_t* store_stage = smem + STAGES * Cfg::STAGE_BYTES + 256;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // a kernel that already failed on this device leaves its code in *err: do nothing then
    __shared__ int s_abort;
    if (threadIdx.x == 0) s_abort = *reinterpret_cast<volatile int*>(g.err);
    __syncthreads();
    if (!PAIR && s_abort != 0) return;      // (a pair decides together, after its first cluster barrier)
    const uint32_t rank = PAIR ? cluster_rank() : 0u;    // 0: the CTA that issues the pair's MMAs

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&tfull[s], 1);
            mbar_init(&tempty[s], PAIR ? 8 : 4);    // the epilogue warps of both CTAs arrive on the first CTA's
        }
        fence_mbar_init();
    }
    if (warp == 1) {
        if (PAIR) { tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish_pair(); }
        else { tmem_alloc(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish(); }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();           // both CTAs' barriers exist before either signals the other's
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool live = true;
    if (PAIR) live = (s_abort | ld_cluster_s32(map_to_rank(smem_u32(&s_abort), rank ^ 1u))) == 0;

    // the pair form walks tiles of 256 rows: row tile 2 * mb2 + rank of each belongs to this CTA
    const int sched_m = PAIR ? (g.num_m + 1) / 2 : g.num_m;
    const int sched_group = PAIR ? (g.group_m + 1) / 2 : g.group_m;
    const int num_tiles = sched_m * g.num_n;
    const int tile0 = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int tile_step = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const int kblocks = (g.K + BK - 1) / BK;   // a ragged last K block is zero-filled by TMA in both operands

    if (!live) {
        // nothing to do: straight to the common teardown
    } else if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&tmA);
            tma_prefetch_desc(&tmB);
            if (EPI == EPI_SWIGLU || EPI == EPI_QKV) tma_prefetch_desc(&tmB2);
            if (EPI == EPI_QKV) tma_prefetch_desc(&tmB3);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = tile0; tile < num_tiles && ok; tile += tile_step) {
                int mb, nb;
                tile_coords(tile, sched_m, g.num_n, sched_group, mb, nb);
                if (PAIR) mb = mb * 2 + (int)rank;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(&empty[stage], phase ^ 1)) { ok = false; atomicExch(g.err, 1); break; }
                    uint8_t* a_s = smem + stage * Cfg::STAGE_BYTES;
                    uint8_t* b_s = a_s + Cfg::A_BYTES;
                    if (!PAIR) mbar_expect_tx(&full[stage], Cfg::STAGE_BYTES);
                    else if (rank == 0) mbar_expect_tx(&full[stage], 2 * Cfg::STAGE_BYTES);   // both CTAs' halves
                    int a_c0 = kb * BK, a_c1 = mb * BM;
                    if (g.a_kblk > 0) {
                        const int blk = a_c0 / g.a_kblk;
                        a_c0 -= blk * g.a_kblk;
                        a_c1 += blk * g.a_rows;
                    }
                    if (PAIR) {
                        // this CTA's 128 rows of A and its 128 of the tile's 256 B rows (second half for the second CTA)
                        tma_load_2d_pair(a_s, &tmA, &full[stage], a_c0, a_c1);
                        if (EPI == EPI_SWIGLU) {
                            tma_load_2d_pair(b_s, rank == 0 ? &tmB : &tmB2, &full[stage], kb * BK, nb * 128);
                        } else if (EPI == EPI_QKV) {
                            const int col0 = nb * BN;
                            const int seg = col0 >= g.seg_n[0] + g.seg_n[1] ? 2 : (col0 >= g.seg_n[0] ? 1 : 0);
                            const int lrow = col0 - (seg == 2 ? g.seg_n[0] + g.seg_n[1] : (seg == 1 ? g.seg_n[0] : 0));
                            const CUtensorMap* mB = seg == 0 ? &tmB : (seg == 1 ? &tmB2 : &tmB3);
                            tma_load_2d_pair(b_s, mB, &full[stage], kb * BK, lrow + (int)rank * 128);
                        } else {
                            tma_load_2d_pair(b_s, &tmB, &full[stage], kb * BK, nb * BN + (int)rank * 128);
                        }
                        if (++stage == STAGES) { stage = 0; phase ^= 1; }
                        continue;
                    }
                    tma_load_2d(a_s, &tmA, &full[stage], a_c0, a_c1);
                    if (EPI == EPI_SWIGLU) {
                        // 128 gate rows then 128 up rows of the same output columns
                        tma_load_2d(b_s, &tmB, &full[stage], kb * BK, nb * 128);
                        tma_load_2d(b_s + 128 * BK * 2, &tmB2, &full[stage], kb * BK, nb * 128);
                    } else if (EPI == EPI_QKV) {
                        // the weight tensor of the segment this column tile lies in, at the segment's own row
                        const int col0 = nb * BN;
                        const int seg = col0 >= g.seg_n[0] + g.seg_n[1] ? 2 : (col0 >= g.seg_n[0] ? 1 : 0);
                        const int lrow = col0 - (seg == 2 ? g.seg_n[0] + g.seg_n[1] : (seg == 1 ? g.seg_n[0] : 0));
                        const CUtensorMap* mB = seg == 0 ? &tmB : (seg == 1 ? &tmB2 : &tmB3);
#pragma unroll
                        for (int h = 0; h < BN / 128; ++h)
                            tma_load_2d(b_s + h * 128 * BK * 2, mB, &full[stage], kb * BK, lrow + h * 128);
                    } else {
#pragma unroll
                        for (int h = 0; h < BN / 128; ++h)
                            tma_load_2d(b_s + h * 128 * BK * 2, &tmB, &full[stage], kb * BK,
                                        nb * BN + h * 128);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------ MMA issuer
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(PAIR ? 2 * BM : BM, BN, 0, 0);
            int stage = 0;
            uint32_t phase = 0;
            int as = 0;
            uint32_t aphase = 0;
            bool ok = true;
            for (int tile = tile0; tile < num_tiles && ok; tile += tile_step) {
                if (!mbar_wait(&tempty[as], aphase ^ 1)) { atomicExch(g.err, 2); break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + as * BN;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(&full[stage], phase)) { ok = false; atomicExch(g.err, 3); break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + stage * Cfg::STAGE_BYTES);
                    const uint64_t ad = umma_desc_sw128(a_addr, 16, 1024);
                    const uint64_t bd = umma_desc_sw128(a_addr + Cfg::A_BYTES, 16, 1024);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {  // 32 bytes per K step = 2 units of the address field
                        if (PAIR) umma_ss_pair(d_tmem, ad + 2 * k, bd + 2 * k, idesc, (kb | k) != 0);
                        else umma_ss(d_tmem, ad + 2 * k, bd + 2 * k, idesc, (kb | k) != 0);
                    }
                    if (PAIR) umma_commit_pair(&empty[stage]);
                    else umma_commit(&empty[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (PAIR) umma_commit_pair(&tfull[as]);
                else umma_commit(&tfull[as]);
                if (++as == 2) { as = 0; aphase ^= 1; }
            }
        }
    } else {
        // ------------------------------------------------------ epilogue
        const int q = warp & 3;  // TMEM lane quadrant this warp may access
        int as = 0;
        uint32_t aphase = 0;
        for (int tile = tile0; tile < num_tiles; tile += tile_step) {
            int mb, nb;
            tile_coords(tile, sched_m, g.num_n, sched_group, mb, nb);
            if (PAIR) mb = mb * 2 + (int)rank;
            if (!mbar_wait(&tfull[as], aphase)) { atomicExch(g.err, 4); break; }
            tc_fence_after();
            const int row = mb * BM + q * 32 + lane;
            const bool row_ok = row < g.M;
            const uint32_t t_row = tmem_base + as * BN + ((uint32_t)(q * 32) << 16);
            // EPI_QKV: which segment this column tile lies in decides the epilogue (warp-uniform); everything
            // below addresses the output through (seg_col0 + column inside the segment) or the segment's tables
            int seg = 0, seg_col0 = 0, lcol0 = nb * BN, cb = g.o_cb;
            uint16_t* const* tab = g.o_tab;
            const uint16_t* norm_w = g.bias;
            if (EPI == EPI_QKV) {
                seg = lcol0 >= g.seg_n[0] + g.seg_n[1] ? 2 : (lcol0 >= g.seg_n[0] ? 1 : 0);
                seg_col0 = seg == 2 ? g.seg_n[0] + g.seg_n[1] : (seg == 1 ? g.seg_n[0] : 0);
                lcol0 -= seg_col0;
                cb = g.seg_cb[seg];
                if (seg > 0) tab = g.seg_tab + (seg - 1) * 8;
                norm_w = g.seg_norm[seg == 1 ? 1 : 0];
            }
            const int epi_eff = (EPI == EPI_QKV) ? (seg < 2 ? (int)EPI_QKNORM : (int)EPI_STORE) : EPI;
            if (EPI == EPI_SWIGLU) {
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t rg[32], ru[32];
                    tmem_ld32(t_row + c * 32, rg);
                    tmem_ld32(t_row + 128 + c * 32, ru);
                    tmem_ld_wait();
                    if (row_ok) {
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float gg = bf16_round(__uint_as_float(rg[j]));
                            const float uu = bf16_round(__uint_as_float(ru[j]));
                            const float sg = 1.0f / (1.0f + expf(-gg));
                            v[j] = bf16_round(gg * sg) * uu;
                        }
                        store32_bf16(g.out + (size_t)row * g.ldo + nb * 128 + c * 32, v);
                    }
                }
            } else if (epi_eff == EPI_STORE && g.o_tab_n) {
                // Blocks of the output live in other GPUs' memory.  One thread per row would put 16-byte
                // pieces of 32 different rows into every store instruction; over NVLink each piece is a
                // packet of its own.  So 64 columns at a time go through a swizzled shared-memory slice of
                // this warp and leave as full 128-byte row segments (4 rows per instruction).
                uint8_t* stg = store_stage + q * (2 * 32 * 128);
#pragma unroll 1
                for (int c2 = 0; c2 < BN / 64; ++c2) {
                    uint32_t r0[32], r1[32];
                    tmem_ld32(t_row + c2 * 64, r0);
                    tmem_ld32(t_row + c2 * 64 + 32, r1);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint32_t* src = j < 4 ? &r0[(j & 3) * 8] : &r1[(j & 3) * 8];
                        uint4 o;
                        o.x = pack_bf16x2(__uint_as_float(src[0]), __uint_as_float(src[1]));
                        o.y = pack_bf16x2(__uint_as_float(src[2]), __uint_as_float(src[3]));
                        o.z = pack_bf16x2(__uint_as_float(src[4]), __uint_as_float(src[5]));
                        o.w = pack_bf16x2(__uint_as_float(src[6]), __uint_as_float(src[7]));
                        *reinterpret_cast<uint4*>(stg + lane * 128 + ((j ^ (lane & 7)) * 16)) = o;
                    }
                    __syncwarp();
                    const int col = lcol0 + c2 * 64;        // a 64-column group never straddles a block (cb % 128 == 0)
                    uint16_t* obase = tab[col / cb] + (col % cb);
                    const int ch = lane & 7;
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const int rr = k * 4 + (lane >> 3);
                        const uint4 o = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((ch ^ (rr & 7)) * 16));
                        const int grow = mb * BM + q * 32 + rr;
                        if (grow < g.M) *reinterpret_cast<uint4*>(obase + (size_t)grow * g.ldo + ch * 8) = o;
                    }
                    __syncwarp();
                }
            } else if (epi_eff == EPI_QKNORM) {
                // Per-head RMSNorm + rotary on the projection's output row (o1.c src/model/block.c:266-289 runs
                // head split, hd_rmsnorm, hd_apply_rotary as separate passes).  This thread owns the whole row of
                // the tile, i.e. BN/128 complete heads: the 128 values of a head are rounded to bf16 (the
                // projection's stored result), summed in the order of qk_norm_rope_kernel (eight partial sums of
                // 8 + 8 elements, pairwise tree) so that both paths agree bit for bit, normalised, rotated with the
                // partner 64 columns away, and written once.
#pragma unroll 1
                for (int hb = 0; hb < BN / 128; ++hb) {
                    uint32_t r[4][32];
#pragma unroll
                    for (int c = 0; c < 4; ++c) tmem_ld32(t_row + hb * 128 + c * 32, r[c]);
                    tmem_ld_wait();
                    if (row_ok) {
                        float part[8];
#pragma unroll
                        for (int t = 0; t < 8; ++t) {
                            float acc = 0.f;
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const int e = 8 * t + j;
                                const float lo = bf16_round(__uint_as_float(r[e >> 5][e & 31]));
                                const float hi = bf16_round(__uint_as_float(r[2 + (e >> 5)][e & 31]));
                                r[e >> 5][e & 31] = __float_as_uint(lo);
                                r[2 + (e >> 5)][e & 31] = __float_as_uint(hi);
                                acc = __fadd_rn(acc, __fmaf_rn(hi, hi, __fmul_rn(lo, lo)));
                            }
                            part[t] = acc;
                        }
                        const float sq = __fadd_rn(__fadd_rn(__fadd_rn(part[0], part[1]), __fadd_rn(part[2], part[3])),
                                                   __fadd_rn(__fadd_rn(part[4], part[5]), __fadd_rn(part[6], part[7])));
                        const float inv = rsqrtf(sq / 128.0f + g.scale);
                        const int col = seg_col0 + lcol0 + hb * 128;
                        const size_t ocol = g.o_cb ? (size_t)(col / g.o_cb) * g.o_cb_stride + (col % g.o_cb) : (size_t)col;
                        uint16_t* orow = g.o_tab_n ? nullptr : g.out + (size_t)row * g.ldo + ocol;
                        uint8_t* stg_row = store_stage + q * (2 * 32 * 128) + lane * 128;
                        const float* cs = g.rope + (size_t)row * 128;
#pragma unroll
                        for (int t = 0; t < 8; ++t) {
                            const uint4 wl4 = *reinterpret_cast<const uint4*>(norm_w + 8 * t);
                            const uint4 wh4 = *reinterpret_cast<const uint4*>(norm_w + 64 + 8 * t);
                            const float wl[8] = {bf16lo(wl4.x), bf16hi(wl4.x), bf16lo(wl4.y), bf16hi(wl4.y),
                                                 bf16lo(wl4.z), bf16hi(wl4.z), bf16lo(wl4.w), bf16hi(wl4.w)};
                            const float wh[8] = {bf16lo(wh4.x), bf16hi(wh4.x), bf16lo(wh4.y), bf16hi(wh4.y),
                                                 bf16lo(wh4.z), bf16hi(wh4.z), bf16lo(wh4.w), bf16hi(wh4.w)};
                            const float4 ca = *reinterpret_cast<const float4*>(cs + 8 * t);
                            const float4 cb = *reinterpret_cast<const float4*>(cs + 8 * t + 4);
                            const float4 sa = *reinterpret_cast<const float4*>(cs + 64 + 8 * t);
                            const float4 sb = *reinterpret_cast<const float4*>(cs + 64 + 8 * t + 4);
                            const float cc[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
                            const float ss[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};
                            float ol[8], oh[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const int e = 8 * t + j;
                                const float lo = __uint_as_float(r[e >> 5][e & 31]);
                                const float hi = __uint_as_float(r[2 + (e >> 5)][e & 31]);
                                const float a = bf16_round(wl[j] * lo * inv);
                                const float b = bf16_round(wh[j] * hi * inv);
                                ol[j] = bf16_round(a * cc[j]) - bf16_round(b * ss[j]);
                                oh[j] = bf16_round(b * cc[j]) + bf16_round(a * ss[j]);
                            }
                            uint4 po, ph;
                            po.x = pack_bf16x2(ol[0], ol[1]); po.y = pack_bf16x2(ol[2], ol[3]);
                            po.z = pack_bf16x2(ol[4], ol[5]); po.w = pack_bf16x2(ol[6], ol[7]);
                            ph.x = pack_bf16x2(oh[0], oh[1]); ph.y = pack_bf16x2(oh[2], oh[3]);
                            ph.z = pack_bf16x2(oh[4], oh[5]); ph.w = pack_bf16x2(oh[6], oh[7]);
                            if (g.o_tab_n) {
                                // destination rows live in another GPU's memory: both 64-column halves of the
                                // head go through this warp's two swizzled shared-memory slices first
                                *reinterpret_cast<uint4*>(stg_row + ((t ^ (lane & 7)) * 16)) = po;
                                *reinterpret_cast<uint4*>(stg_row + 32 * 128 + ((t ^ (lane & 7)) * 16)) = ph;
                            } else {
                                *reinterpret_cast<uint4*>(orow + 8 * t) = po;
                                *reinterpret_cast<uint4*>(orow + 64 + 8 * t) = ph;
                            }
                        }
                    }
                    if (g.o_tab_n) {
                        // leave as full 128-byte row segments, 4 rows per store instruction (a head never straddles
                        // a destination block: o_cb % 128 == 0)
                        __syncwarp();
                        const int col = lcol0 + hb * 128;
                        uint16_t* obase = tab[col / cb] + (col % cb);
                        const uint8_t* stg = store_stage + q * (2 * 32 * 128);
                        const int ch = lane & 7;
#pragma unroll
                        for (int hf = 0; hf < 2; ++hf)
#pragma unroll
                            for (int k = 0; k < 8; ++k) {
                                const int rr = k * 4 + (lane >> 3);
                                const uint4 o = *reinterpret_cast<const uint4*>(stg + hf * (32 * 128) + rr * 128 + ((ch ^ (rr & 7)) * 16));
                                const int grow = mb * BM + q * 32 + rr;
                                if (grow < g.M) *reinterpret_cast<uint4*>(obase + (size_t)grow * g.ldo + hf * 64 + ch * 8) = o;
                            }
                        __syncwarp();
                    }
                }
            } else if (EPI == EPI_LORA) {
                // In-place update of W.  The contraction is short (9 x rank), so this epilogue's read-modify-
                // write of W bounds the kernel: all of the row's W values of four 32-column groups are requested
                // before the first is used, which keeps about 32 KB per SM in flight instead of one load per thread.
#pragma unroll 1
                for (int c4 = 0; c4 < BN / 128; ++c4) {
                    uint4 wv[4][4];
                    const uint16_t* wrow = g.out + (size_t)row * g.ldo + nb * BN + c4 * 128;
                    if (row_ok) {
#pragma unroll
                        for (int c = 0; c < 4; ++c)
#pragma unroll
                            for (int i = 0; i < 4; ++i) wv[c][i] = reinterpret_cast<const uint4*>(wrow + c * 32)[i];
                    }
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t r[32];
                        tmem_ld32(t_row + c4 * 128 + c * 32, r);
                        tmem_ld_wait();
                        if (row_ok) {
                            uint4* dst = reinterpret_cast<uint4*>(g.out + (size_t)row * g.ldo + nb * BN + c4 * 128 + c * 32);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const uint4 o = wv[c][i];
                                uint4 n;
                                n.x = pack_bf16x2(bf16lo(o.x) + g.scale * __uint_as_float(r[i * 8 + 0]),
                                                  bf16hi(o.x) + g.scale * __uint_as_float(r[i * 8 + 1]));
                                n.y = pack_bf16x2(bf16lo(o.y) + g.scale * __uint_as_float(r[i * 8 + 2]),
                                                  bf16hi(o.y) + g.scale * __uint_as_float(r[i * 8 + 3]));
                                n.z = pack_bf16x2(bf16lo(o.z) + g.scale * __uint_as_float(r[i * 8 + 4]),
                                                  bf16hi(o.z) + g.scale * __uint_as_float(r[i * 8 + 5]));
                                n.w = pack_bf16x2(bf16lo(o.w) + g.scale * __uint_as_float(r[i * 8 + 6]),
                                                  bf16hi(o.w) + g.scale * __uint_as_float(r[i * 8 + 7]));
                                dst[i] = n;
                            }
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(t_row + c * 32, r);
                    tmem_ld_wait();
                    const int col = nb * BN + c * 32;
                    if (row_ok && col + 32 > g.N) {
                        // ragged right edge (N % 32 != 0, N % 8 == 0; plain, bias and bias+GELU epilogues only):
                        // the same arithmetic, eight columns at a time, nothing read or written beyond column N
                        if (EPI == EPI_STORE || EPI == EPI_BIAS || EPI == EPI_BIAS_GELU) {
                            for (int c8 = 0; c8 < 4 && col + c8 * 8 < g.N; ++c8) {
                                float v8[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) v8[j] = __uint_as_float(r[c8 * 8 + j]);
                                if (EPI != EPI_STORE) {
                                    const uint4 b4 = *reinterpret_cast<const uint4*>(g.bias + col + c8 * 8);
                                    const float b8[8] = {bf16lo(b4.x), bf16hi(b4.x), bf16lo(b4.y), bf16hi(b4.y),
                                                         bf16lo(b4.z), bf16hi(b4.z), bf16lo(b4.w), bf16hi(b4.w)};
#pragma unroll
                                    for (int j = 0; j < 8; ++j) v8[j] = bf16_round(v8[j]) + b8[j];
                                    if (EPI == EPI_BIAS_GELU) {
#pragma unroll
                                        for (int j = 0; j < 8; ++j) v8[j] = gelu_of(bf16_round(v8[j]), g.scale != 0.f);
                                    }
                                }
                                uint4 o;
                                o.x = pack_bf16x2(v8[0], v8[1]); o.y = pack_bf16x2(v8[2], v8[3]);
                                o.z = pack_bf16x2(v8[4], v8[5]); o.w = pack_bf16x2(v8[6], v8[7]);
                                *reinterpret_cast<uint4*>(g.out + (size_t)row * g.ldo + col + c8 * 8) = o;
                            }
                        }
                    } else if (row_ok) {
                        const size_t ocol = g.o_cb ? (size_t)(col / g.o_cb) * g.o_cb_stride + (col % g.o_cb)
                                                   : (size_t)col;
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                        if (EPI == EPI_BIAS || EPI == EPI_BIAS_GELU) {
                            float b[32];
                            load32_bf16(g.bias + col, b);
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = bf16_round(v[j]) + b[j];
                            if (EPI == EPI_BIAS_GELU) {
#pragma unroll
                                for (int j = 0; j < 32; ++j) v[j] = gelu_of(bf16_round(v[j]), g.scale != 0.f);
                            }
                        } else if (EPI == EPI_BIAS_RESID) {
                            // linear + bias stored as bf16, then the residual add of src/cuda/residual.cu:14-23
                            float b[32], rs[32];
                            load32_bf16(g.bias + col, b);
                            load32_bf16(g.resid + (size_t)row * g.ldr + col, rs);
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = rs[j] + bf16_round(bf16_round(v[j]) + b[j]);
                        } else if (EPI == EPI_GATE_RESID) {
                            float gt[32], rs[32];
                            load32_bf16(g.bias + col, gt);
                            load32_bf16(g.resid + (size_t)row * g.ldr + col, rs);
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = rs[j] + bf16_round(gt[j] * bf16_round(v[j]));
                        } else if (EPI == EPI_RESID) {
                            float b[32];
                            load32_bf16(g.resid + (size_t)row * g.ldr + col, b);
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = bf16_round(v[j]) + b[j];
                        } else if (EPI == EPI_LORA) {
                            float b[32];
                            load32_bf16(g.out + (size_t)row * g.ldo + ocol, b);
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = b[j] + g.scale * v[j];
                        }
                        store32_bf16(g.out + (size_t)row * g.ldo + ocol, v);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (PAIR) mbar_arrive_cluster(map_to_rank(smem_u32(&tempty[as]), 0));
                else mbar_arrive(&tempty[as]);
            }
            if (++as == 2) { as = 0; aphase ^= 1; }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();   // neither CTA leaves (or frees tensor memory) while the other may still signal it or feed an MMA
    tc_fence_after();
    if (warp == 1) {
        if (PAIR) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
        else tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// ---------------------------------------------------------------- SIMT path
// One warp per output element; used for M < 8 (timestep MLP, M = 1) and
// for shapes the tensor-core tiles do not cover (N % 128 or K % 64 != 0).
__global__ void gemm_simt_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w,
                                 const uint16_t* __restrict__ bias, uint16_t* __restrict__ y, int M,
                                 int N, int K, int ldx, int ldy) {
    const int warps_per_block = blockDim.x >> 5;
    const int n = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int m = blockIdx.y;
    const int lane = threadIdx.x & 31;
    if (n >= N) return;
    const uint16_t* xr = x + (size_t)m * ldx;
    const uint16_t* wr = w + (size_t)n * K;
    float acc = 0.f;
    if ((K & 7) == 0 && ((((uintptr_t)xr) | ((uintptr_t)wr)) & 15) == 0) {
        for (int k = lane * 8; k < K; k += 256) {
            const uint4 a = *reinterpret_cast<const uint4*>(xr + k);
            const uint4 b = *reinterpret_cast<const uint4*>(wr + k);
            acc += bf16lo(a.x) * bf16lo(b.x); acc += bf16hi(a.x) * bf16hi(b.x);
            acc += bf16lo(a.y) * bf16lo(b.y); acc += bf16hi(a.y) * bf16hi(b.y);
            acc += bf16lo(a.z) * bf16lo(b.z); acc += bf16hi(a.z) * bf16hi(b.z);
            acc += bf16lo(a.w) * bf16lo(b.w); acc += bf16hi(a.w) * bf16hi(b.w);
        }
    } else {
        for (int k = lane; k < K; k += 32) acc += bf16_to_f32(xr[k]) * bf16_to_f32(wr[k]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
        float v = acc;
        if (bias) v = bf16_round(v) + bf16_to_f32(bias[n]);
        y[(size_t)m * ldy + n] = f32_to_bf16(v);
    }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
        if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = (EncodeTiledFn)p;
    });
    return fn;
}

// Row-major bf16 matrix [rows, cols] with row pitch ld (elements); box is
// 64 columns x box_rows rows, 128-byte swizzle.
bool make_tmap_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                    uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("tensor map: cuTensorMapEncodeTiled entry point unavailable"); return false; }
    if ((((uintptr_t)base) & 15) || ((ld * 2) & 15)) {
        set_error("tensor map: base/pitch not 16-byte aligned");
        return false;
    }
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("tensor map: encode failed (%d)", (int)r); return false; }
    return true;
}

struct TmapKey {
    const void* p; uint64_t rows, cols, ld; uint32_t box;
    bool operator<(const TmapKey& o) const {
        return std::tie(p, rows, cols, ld, box) < std::tie(o.p, o.rows, o.cols, o.ld, o.box);
    }
};
// Encoding a tensor map costs a few microseconds on the host; weights and
// workspace buffers repeat every block and step, so cache by (ptr, shape).
// The map is copied out under the lock: the cache may be emptied by a later
// call (or another thread) while the caller still holds its copy.
bool cached_tmap(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_rows) {
    static std::map<TmapKey, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lk(mu);
    TmapKey k{base, rows, cols, ld, box_rows};
    auto it = cache.find(k);
    if (it != cache.end()) { *out = it->second; return true; }
    if (cache.size() > 8192) cache.clear();
    if (!make_tmap_bf16(out, base, rows, cols, ld, box_rows)) return false;
    cache.emplace(k, *out);
    return true;
}

// cudaFuncSetAttribute is per device: remember, per kernel instantiation, on which devices it was done.
bool func_attr_once(std::atomic<uint64_t>& done, const void* func, int smem_bytes, const char* what) {
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t bit = 1ull << (dev & 63);
    if (done.load(std::memory_order_acquire) & bit) return true;
    cudaError_t e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) { set_error("%s: smem attribute: %s", what, cudaGetErrorString(e)); return false; }
    done.fetch_or(bit, std::memory_order_release);
    return true;
}

// 0: single-CTA tiles only; 1 (default): 256-wide tiles of the large-M families run on CTA pairs; 2: SwiGLU family too
static int g_pair_mode = -1;
void gemm_pair_mode(int mode) { g_pair_mode = mode; }
static bool pair_wanted() {
    if (g_pair_mode < 0) {
        const char* e = getenv("O1_GEMM_PAIR");
        g_pair_mode = (e && e[0] == '0') ? 0 : ((e && e[0] == '2') ? 2 : 1);
    }
    return g_pair_mode != 0;
}

template <int EPI>
static bool launch_tc_pair(const CUtensorMap* tA, const CUtensorMap* tB, const CUtensorMap* tB2, GemmArgs& g,
                           cudaStream_t st, const CUtensorMap* tB3) {
    using Cfg = GemmCfg<256, true>;
    static std::atomic<uint64_t> attr_done{0};
    auto kern = gemm_tc_kernel<EPI, 256, true>;
    if (!func_attr_once(attr_done, (const void*)kern, Cfg::SMEM_BYTES, "gemm (pair)")) return false;
    const int tiles = ((g.num_m + 1) / 2) * g.num_n;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    // A persistent grid must be co-resident: as many pairs as the device can hold at once (a GPC with an odd number
    // of SMs leaves one without a partner), asked once per device.
    static std::atomic<int> max_pairs[64];
    int dev = 0;
    cudaGetDevice(&dev);
    int pairs = max_pairs[dev & 63].load(std::memory_order_acquire);
    if (pairs == 0) {
        cfg.gridDim = dim3(2 * (sm_count() / 2));
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) { cudaGetLastError(); n = sm_count() / 2; }
        if (n > sm_count() / 2) n = sm_count() / 2;
        pairs = n;
        max_pairs[dev & 63].store(n, std::memory_order_release);
    }
    if (pairs > tiles) pairs = tiles;
    prof_before(EPI == EPI_QKV ? (int)EPI_STORE : EPI, 2.0 * g.M * (double)g.N * g.K * (EPI == EPI_SWIGLU ? 2.0 : 1.0), st);
    cfg.gridDim = dim3(2 * pairs);
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, *tA, *tB, *tB2, tB3 ? *tB3 : *tB2, g);
    prof_after(st);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) { set_error("gemm (pair): launch: %s", cudaGetErrorString(e)); return false; }
    return true;
}

// CTA pairs of the GEMM kernel the current device can hold at once (what the pair form's grid is clamped to)
int gemm_pair_capacity() {
    using Cfg = GemmCfg<256, true>;
    auto kern = gemm_tc_kernel<EPI_STORE, 256, true>;
    if (cudaFuncSetAttribute((const void*)kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); return -1; }
    return n;
}

template <int EPI, int BN>
static bool launch_tc(const CUtensorMap* tA, const CUtensorMap* tB, const CUtensorMap* tB2,
                      GemmArgs& g, cudaStream_t st, const CUtensorMap* tB3 = nullptr) {
    // CTA pairs for the families that carry the large-M work, when there are at least two rounds of pair tiles.
    // Measured at 16640 rows, stand-alone: o_proj 1306 -> 1384, down 1348 -> 1423, q|k|v 1315 -> 1391, head 1203 -> 1235
    // TFLOP/s; gate|up + SwiGLU 1438 -> 1358, so that family keeps one CTA per tile.
    if constexpr (BN == 256 && (EPI == EPI_STORE || EPI == EPI_BIAS || EPI == EPI_RESID || EPI == EPI_QKV)) {
        if (pair_wanted() && ((g.num_m + 1) / 2) * g.num_n >= sm_count()) return launch_tc_pair<EPI>(tA, tB, tB2, g, st, tB3);
    }
    // mode 2: gate|up + SwiGLU too (in the power-capped step 1403 -> 1380 TFLOP/s for that family, step time unchanged)
    if constexpr (BN == 256 && EPI == EPI_SWIGLU) {
        if (pair_wanted() && g_pair_mode == 2 && ((g.num_m + 1) / 2) * g.num_n >= sm_count()) return launch_tc_pair<EPI>(tA, tB, tB2, g, st, tB3);
    }
    using Cfg = GemmCfg<BN>;
    static std::atomic<uint64_t> attr_done{0};
    auto kern = gemm_tc_kernel<EPI, BN, false>;
    if (!func_attr_once(attr_done, (const void*)kern, Cfg::SMEM_BYTES, "gemm")) return false;
    const int tiles = g.num_m * g.num_n;
    int grid = sm_count();
    if (grid > tiles) grid = tiles;
    prof_before((EPI == EPI_QKNORM || EPI == EPI_QKV) ? (int)EPI_STORE : (EPI == EPI_BIAS_GELU ? (int)EPI_BIAS : ((EPI == EPI_BIAS_RESID || EPI == EPI_GATE_RESID) ? (int)EPI_RESID : EPI)), 2.0 * g.M * (double)g.N * g.K * (EPI == EPI_SWIGLU ? 2.0 : 1.0), st);
    kern<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, st>>>(*tA, *tB, *tB2, tB3 ? *tB3 : *tB2, g);
    prof_after(st);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_error("gemm: launch: %s", cudaGetErrorString(e)); return false; }
    return true;
}

bool gemm_tc_supported(int M, int N, int K, int epi) {
    // tiny M (timestep MLP, M = 1) is a GEMV: SIMT path.  K only has to keep the rows 16-byte aligned for TMA
    // (the last K block may be ragged: both operands are zero-filled beyond K).
    if (M < 8 || (K % 8) != 0) return false;
    // a ragged right edge (N % 128 != 0, e.g. the 4304-wide MLP of the vision tower) is covered by the plain,
    // bias and bias+GELU epilogues, in steps of eight columns
    if (epi == EPI_STORE || epi == EPI_BIAS || epi == EPI_BIAS_GELU) return (N % 8) == 0;
    return (N % 128) == 0;   // EPI_SWIGLU: N = ff columns of each of gate / up
}

// epi: see Epi.  For EPI_SWIGLU, w = gate weight, w2 = up weight, N = ff.
bool gemm_bf16(const void* x, const void* w, const void* w2, void* y, int M, int N, int K, int epi,
               const void* bias, const void* resid, float scale, int force_bn, cudaStream_t st) {
    return gemm_bf16_ld(x, K, w, w2, y, N, M, N, K, epi, bias, resid, N, scale, force_bn, st);
}

bool gemm_bf16_ld(const void* x, int ldx, const void* w, const void* w2, void* y, int ldy, int M,
                  int N, int K, int epi, const void* bias, const void* resid, int ldr, float scale,
                  int force_bn, cudaStream_t st) {
    return gemm_bf16_ex(x, ldx, w, w2, y, ldy, M, N, K, epi, bias, resid, ldr, scale, force_bn, 0, 0, 0, 0, st);
}

bool gemm_bf16_ex(const void* x, int ldx, const void* w, const void* w2, void* y, int ldy, int M, int N,
                  int K, int epi, const void* bias, const void* resid, int ldr, float scale, int force_bn,
                  int o_cb, long o_cb_stride, int a_kblk, int a_rows, cudaStream_t st, void* const* o_tab) {
    if (!x || !w || (!y && !o_tab) || M <= 0 || N <= 0 || K <= 0) { set_error("gemm: bad args"); return false; }
    if (o_tab && (!o_cb || N / o_cb > 8 || (epi != EPI_STORE && epi != EPI_QKNORM))) {
        set_error("gemm: an output table needs column blocks (at most 8) and the plain or per-head norm epilogue");
        return false;
    }
    if ((o_cb || a_kblk) && !gemm_tc_supported(M, N, K, epi)) {
        set_error("gemm: blocked operand layouts need a tensor-core shape");
        return false;
    }
    if (o_cb && ((o_cb % 128) != 0 || (N % o_cb) != 0 || epi == EPI_SWIGLU)) {
        set_error("gemm: bad output column block %d", o_cb);
        return false;
    }
    if (a_kblk && ((a_kblk % BK) != 0 || (K % a_kblk) != 0)) {
        set_error("gemm: bad input K block %d", a_kblk);
        return false;
    }
    if (!gemm_tc_supported(M, N, K, epi)) {
        if (epi != EPI_STORE && epi != EPI_BIAS) { set_error("gemm: shape unsupported for fused epilogue"); return false; }
        dim3 block(128);
        dim3 grid((N + 3) / 4, M);
        gemm_simt_kernel<<<grid, block, 0, st>>>((const uint16_t*)x, (const uint16_t*)w,
                                                 (const uint16_t*)(epi == EPI_BIAS ? bias : nullptr), (uint16_t*)y, M, N, K,
                                                 ldx, ldy);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) { set_error("gemm(simt): launch: %s", cudaGetErrorString(e)); return false; }
        return true;
    }
    if ((N % 128) != 0 && ((ldy % 8) != 0 || (((uintptr_t)y) & 15) || (bias && (((uintptr_t)bias) & 15)))) {
        set_error("gemm: a ragged N needs 16-byte aligned output rows and bias");
        return false;
    }
    if ((epi == EPI_BIAS_RESID || epi == EPI_GATE_RESID) && (!bias || !resid || (((uintptr_t)bias) & 15) || (((uintptr_t)resid) & 15) || (ldr % 8))) {
        set_error("gemm: the bias / gate + residual epilogues need both operands, 16-byte aligned");
        return false;
    }
    GemmArgs g;
    g.M = M; g.N = N; g.K = K;
    g.out = (uint16_t*)y; g.ldo = ldy;
    g.bias = (const uint16_t*)bias;
    g.resid = (const uint16_t*)resid; g.ldr = ldr;
    g.scale = scale;
    g.rope = nullptr;
    if (epi == EPI_QKNORM) {
        // resid carries the cos|sin table, bias the norm weight; every 128 output columns are one head
        if (!bias || !resid || (N % 128) != 0 || (o_cb && (o_cb % 128) != 0) || (((uintptr_t)bias) & 15) ||
            (((uintptr_t)resid) & 15)) {
            set_error("gemm: per-head norm epilogue needs norm weight, cos|sin table and whole heads");
            return false;
        }
        g.rope = (const float*)resid;
        g.resid = nullptr;
    }
    g.err = device_error_word();
    g.num_m = (M + BM - 1) / BM;
    // Row tiles are visited in groups whose activation slab (group_m x 128 rows x K) stays L2-resident
    // (about 48 MB of the 126 MB) while the weights stream past it.
    {
        long gm = (48l << 20) / ((long)BM * K * 2);
        g.group_m = (int)(gm < 4 ? 4 : (gm > 32 ? 32 : gm));
    }
    g.o_cb = o_cb; g.o_cb_stride = o_cb_stride;
    g.o_tab_n = 0;
    for (int i = 0; i < 8; ++i) g.o_tab[i] = nullptr;
    if (o_tab) {
        g.o_tab_n = N / o_cb;
        for (int i = 0; i < g.o_tab_n; ++i) {
            if (!o_tab[i] || (((uintptr_t)o_tab[i]) & 15)) { set_error("gemm: output table entry %d unusable", i); return false; }
            g.o_tab[i] = (uint16_t*)o_tab[i];
        }
    }
    g.a_kblk = a_kblk; g.a_rows = a_rows;
    g.seg_n[0] = g.seg_n[1] = 0;
    g.seg_norm[0] = g.seg_norm[1] = nullptr;
    g.seg_cb[0] = g.seg_cb[1] = g.seg_cb[2] = 0;
    for (int i = 0; i < 16; ++i) g.seg_tab[i] = nullptr;

    CUtensorMap mA, mB, mB2;
    if (!(a_kblk ? cached_tmap(&mA, x, (uint64_t)(K / a_kblk) * a_rows, a_kblk, ldx, 128)
                 : cached_tmap(&mA, x, M, K, ldx, 128)))
        return false;
    if (!cached_tmap(&mB, w, N, K, K, 128)) return false;
    if (epi == EPI_SWIGLU) { if (!cached_tmap(&mB2, w2, N, K, K, 128)) return false; }
    else mB2 = mB;
    const CUtensorMap *tA = &mA, *tB = &mB, *tB2 = &mB2;

    if (epi == EPI_SWIGLU) {
        g.num_n = N / 128;
        return launch_tc<EPI_SWIGLU, 256>(tA, tB, tB2, g, st);
    }
    int bn = 256;
    if ((N % 256) != 0 || (o_cb && (o_cb % 256) != 0)) bn = 128;
    else {
        // small problems: halve the tile to fill the SMs
        const int tiles256 = g.num_m * (N / 256);
        if (tiles256 < 2 * sm_count()) bn = 128;
    }
    if (force_bn == 128 || force_bn == 256) {
        if (force_bn == 256 && ((N % 256) != 0 || (o_cb && (o_cb % 256) != 0))) {
            set_error("gemm: BN=256 needs N (and the output column block) %% 256 == 0");
            return false;
        }
        bn = force_bn;
    }
    g.num_n = (N + bn - 1) / bn;
    if (bn == 256) {
        switch (epi) {
            case EPI_STORE: return launch_tc<EPI_STORE, 256>(tA, tB, tB2, g, st);
            case EPI_BIAS:  return launch_tc<EPI_BIAS, 256>(tA, tB, tB2, g, st);
            case EPI_RESID: return launch_tc<EPI_RESID, 256>(tA, tB, tB2, g, st);
            case EPI_LORA:  return launch_tc<EPI_LORA, 256>(tA, tB, tB2, g, st);
            case EPI_QKNORM: return launch_tc<EPI_QKNORM, 256>(tA, tB, tB2, g, st);
            case EPI_BIAS_GELU: return launch_tc<EPI_BIAS_GELU, 256>(tA, tB, tB2, g, st);
            case EPI_BIAS_RESID: return launch_tc<EPI_BIAS_RESID, 256>(tA, tB, tB2, g, st);
            case EPI_GATE_RESID: return launch_tc<EPI_GATE_RESID, 256>(tA, tB, tB2, g, st);
        }
    } else {
        switch (epi) {
            case EPI_STORE: return launch_tc<EPI_STORE, 128>(tA, tB, tB2, g, st);
            case EPI_BIAS:  return launch_tc<EPI_BIAS, 128>(tA, tB, tB2, g, st);
            case EPI_RESID: return launch_tc<EPI_RESID, 128>(tA, tB, tB2, g, st);
            case EPI_LORA:  return launch_tc<EPI_LORA, 128>(tA, tB, tB2, g, st);
            case EPI_QKNORM: return launch_tc<EPI_QKNORM, 128>(tA, tB, tB2, g, st);
            case EPI_BIAS_GELU: return launch_tc<EPI_BIAS_GELU, 128>(tA, tB, tB2, g, st);
            case EPI_BIAS_RESID: return launch_tc<EPI_BIAS_RESID, 128>(tA, tB, tB2, g, st);
            case EPI_GATE_RESID: return launch_tc<EPI_GATE_RESID, 128>(tA, tB, tB2, g, st);
        }
    }
    set_error("gemm: unknown epilogue %d", epi);
    return false;
}

// q | k | v projections of one activation matrix as ONE launch: y[M, qc | kc | kc] (row pitch ldy) = x wq^T | x wk^T |
// x wv^T, the per-head RMSNorm + rotary applied to the q and k columns in the epilogue (norm weights q_norm / k_norm
// [128], cos|sin table cs [M,128] fp32).  Three launches of 14.05 + 3.5 + 3.5 waves of tiles (at 16640 rows) become
// one of 21.1; in the sharded forward the gain is larger (fewer rows per rank, the same three partial last waves).
// tq / tk / tv (all or none): per destination rank the base of that rank's q / k / v columns (block widths
// qc/P, kc/P, kc/P); rows then go to the tables instead of y.
bool gemm_qkv(const void* x, int ldx, const void* wq, const void* wk, const void* wv, void* y, int ldy, int M, int qc,
              int kc, int K, const void* q_norm, const void* k_norm, const float* cs, float eps, int n_dst,
              void* const* tq, void* const* tk, void* const* tv, cudaStream_t st) {
    const int N = qc + 2 * kc;
    const bool tabs = n_dst > 0;
    if (!x || !wq || !wk || !wv || (!y && !tabs) || !q_norm || !k_norm || !cs || M < 8 || (K % 8) != 0 || (qc % 128) != 0 ||
        (kc % 128) != 0 || qc <= 0 || kc <= 0 || ((((uintptr_t)q_norm) | ((uintptr_t)k_norm) | ((uintptr_t)cs)) & 15)) {
        set_error("gemm_qkv: bad args");
        return false;
    }
    if (tabs && (n_dst > 8 || !tq || !tk || !tv || (qc % n_dst) != 0 || (kc % n_dst) != 0 || ((qc / n_dst) % 128) != 0 ||
                 ((kc / n_dst) % 128) != 0)) {
        set_error("gemm_qkv: bad destination tables");
        return false;
    }
    GemmArgs g;
    g.M = M; g.N = N; g.K = K;
    g.out = (uint16_t*)y; g.ldo = ldy;
    g.bias = (const uint16_t*)q_norm;
    g.resid = nullptr; g.ldr = 0;
    g.rope = cs;
    g.scale = eps;
    g.err = device_error_word();
    g.num_m = (M + BM - 1) / BM;
    {
        long gm = (48l << 20) / ((long)BM * K * 2);
        g.group_m = (int)(gm < 4 ? 4 : (gm > 32 ? 32 : gm));
    }
    g.o_cb = 0; g.o_cb_stride = 0;
    g.o_tab_n = tabs ? n_dst : 0;
    g.a_kblk = 0; g.a_rows = 0;
    g.seg_n[0] = qc; g.seg_n[1] = kc;
    g.seg_norm[0] = (const uint16_t*)q_norm; g.seg_norm[1] = (const uint16_t*)k_norm;
    g.seg_cb[0] = tabs ? qc / n_dst : 0; g.seg_cb[1] = g.seg_cb[2] = tabs ? kc / n_dst : 0;
    for (int i = 0; i < 8; ++i) g.o_tab[i] = nullptr;
    for (int i = 0; i < 16; ++i) g.seg_tab[i] = nullptr;
    for (int i = 0; i < (tabs ? n_dst : 0); ++i) {
        if (!tq[i] || !tk[i] || !tv[i] || ((((uintptr_t)tq[i]) | ((uintptr_t)tk[i]) | ((uintptr_t)tv[i])) & 15)) {
            set_error("gemm_qkv: destination table entry %d unusable", i);
            return false;
        }
        g.o_tab[i] = (uint16_t*)tq[i]; g.seg_tab[i] = (uint16_t*)tk[i]; g.seg_tab[8 + i] = (uint16_t*)tv[i];
    }
    CUtensorMap mA, mQ, mK, mV;
    if (!cached_tmap(&mA, x, M, K, ldx, 128) || !cached_tmap(&mQ, wq, qc, K, K, 128) ||
        !cached_tmap(&mK, wk, kc, K, K, 128) || !cached_tmap(&mV, wv, kc, K, K, 128))
        return false;
    // 256-wide tiles need every segment (and every destination block) to be a multiple of 256 columns
    bool wide = (qc % 256) == 0 && (kc % 256) == 0;
    if (tabs && (((qc / n_dst) % 256) != 0 || ((kc / n_dst) % 256) != 0)) wide = false;
    if (wide && g.num_m * (N / 256) < 2 * sm_count()) wide = false;
    const int bn = wide ? 256 : 128;
    g.num_n = N / bn;
    return wide ? launch_tc<EPI_QKV, 256>(&mA, &mQ, &mK, g, st, &mV) : launch_tc<EPI_QKV, 128>(&mA, &mQ, &mK, g, st, &mV);
}

}  // namespace o1
