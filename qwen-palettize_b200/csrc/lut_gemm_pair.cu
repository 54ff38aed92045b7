// lut_gemm_pair: the two large palettized products, y = x W^T and dX = dY W (+ the LoRA block), on CTA PAIRS
// (tcgen05.mma.cta_group::2, M = 256): two CTAs of a cluster share one 256 x 256 output tile.
//
//   CTA r of the pair (r = rank in the cluster, 0 = leader)
//     - loads by TMA the 128 rows [m0 + 128 r, +128) of A into ITS shared memory,
//     - decodes the 128 B columns [j0 + 128 r, +128) of the tile (half of the packed weights) into ITS shared memory,
//     - owns the accumulator rows [128 r, +128) x 256 columns in ITS tensor memory and writes them out.
//   The leader's one MMA thread issues a single 256 x 256 x 16 instruction per 16 reduction elements; the hardware reads A
//   from each CTA's own shared memory and each half of B from the CTA that holds it.
//
// Against one CTA per tile (lut_gemm.cu: two 128 x 256 x 16 instructions that both re-read the 8 KB of B) this
//   * cuts shared-memory operand reads per SM from 12 KB to 8 KB per 128 x 256 x 16 of work (the single-CTA kernel ran at
//     about 140 B/cycle of demand against 128 B/cycle of shared-memory bandwidth),
//   * halves each CTA's accumulator to 256 of the 512 tensor-memory columns, so TWO accumulators fit and the epilogue of
//     tile i overlaps the main loop of tile i + 1,
//   * lets a stage span 128 reduction elements (32 KB A + 32 KB B per CTA): eight MMAs per barrier round trip.
// The thread that issues the MMAs is kept lean (precomputed descriptor words, one wait and one commit per stage): a lone
// thread retires a dependent instruction every five or six cycles, an MMA lasts 128, so two dozen instructions per MMA
// are enough to starve the tensor pipe.
//
// Synchronisation (every barrier named here lives at the same shared-memory offset in both CTAs):
//   full[s]     leader's copy: the leader's producer announces both CTAs' TMA bytes (each CTA's copies complete on the
//               LEADER's barrier) and every decode warp of BOTH CTAs arrives once (remote arrive from the peer)
//   empty[s]    own copy in each CTA: tcgen05.commit of the leader, multicast to both CTAs
//   acc_full[b] own copy in each CTA: tcgen05.commit multicast after the last reduction block of a tile
//   acc_empty[b] leader's copy: one arrival per epilogue warp of BOTH CTAs
// No load uses cluster multicast: every CTA issues its own plain TMA copies.
//
// Replaces, in the reference: fused_lut_linear_fwd_tc_kernel (scripts/fused_lut_kernel.cu:309),
// fused_lut_linear_bwd_grad_x_tc_kernel (:551) and the cuBLAS calls of the soft path
// (scripts/fused_lut_linear_cuda.py:912, :944), as lut_gemm.cu does for the shapes this kernel does not take.
#include "plz_launch.h"

namespace plz {

int g_pair_gemm = 1;  // 0: never use the CTA-pair kernel (comparisons, tests of the single-CTA kernel)

namespace {

struct PairParams {
    int M, J, R;
    int n_extra;             // 0 or 1 extra 64-wide reduction block from (A2, B2)
    int tiles_m, tiles_j, n_tiles;
    const uint8_t* packed; long long packed_pitch;
    const __nv_bfloat16* palette;
    int gs_n, gs_k, n_kgroups, gs_n_shift;
    int Wn, Wk;
    float alpha;
    StatusWord* status;
    unsigned long long* prof;  // diagnostics build: [gridDim][8] cycle counters (MMA thread 0..4, one decode thread 5..6)
};

constexpr int kDecodeWarps = 16;
constexpr int kEpiWarps = 4;   // one per TMEM lane group; the epilogue of a tile overlaps the main loop of the next
constexpr int kFirstEpiWarp = 2 + kDecodeWarps;
constexpr int kThreads = (2 + kDecodeWarps + kEpiWarps) * 32;  // 704
constexpr int kStages = 3;
constexpr int kBK = 128;                      // reduction elements per stage: two 64-wide (128-byte) swizzle blocks
constexpr uint32_t kBlkBytes = 128 * 64 * 2;  // one 64-wide block of 128 rows
constexpr uint32_t kABytes = 2 * kBlkBytes;   // this CTA's 128 rows of A
constexpr uint32_t kBBytes = 2 * kBlkBytes;   // this CTA's 128 columns of B
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr uint32_t kEpiStageBytes = 32 * 64 * 2;
constexpr uint32_t kEpiOff = kStages * kStageBytes;
constexpr uint32_t kBarOff = kEpiOff + kEpiWarps * kEpiStageBytes;
constexpr uint32_t kSmemBytes = kBarOff + 1024 + 256;

template <int BMODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
lut_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA2,
                     const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ CUtensorMap tmD, const PairParams p) {
    constexpr bool kBMn = (BMODE == B_DECODE_MN);
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    const uint32_t bar_base = base + kBarOff;
    auto full = [&](int s) { return bar_base + 8u * s; };
    auto empty = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto acc_full = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
    auto acc_empty = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + kBarOff + 8 * (2 * kStages + 4));
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();   // 0 = leader
    const uint32_t lead_bar_base = leader_addr(bar_base);   // the leader's barrier block as a shared::cluster address
    auto lead_full = [&](int s) { return lead_bar_base + 8u * s; };
    auto lead_acc_empty = [&](int b) { return lead_bar_base + 8u * (2 * kStages + 2 + b); };
    const int pair = blockIdx.x >> 1;
    const int n_pairs = gridDim.x >> 1;
    const int nkb = (p.R + kBK - 1) / kBK;   // a last stage that is only half covered reads zeros (TMA fill, decode bounds)
    const int nkb_total = nkb + p.n_extra;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full(s), 1 + 2 * kDecodeWarps);
            mbar_init(empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 2 * kEpiWarps);
        }
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmD);
        if (p.n_extra) { tma_prefetch_desc(&tmA2); tma_prefetch_desc(&tmB2); }
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32((const void*)tmem_slot), 512);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();   // both CTAs' barriers are initialised before anyone arrives on the other's
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    auto tile_origin = [&](int t, int& m0, int& j0) {
        j0 = (t % p.tiles_j) * 256;
        m0 = (t / p.tiles_j) * 256;
    };

    if (warp == 0) {
        // ------------------------------------------------------------- TMA producer (one per CTA)
        if (lane == 0) {
            bool ok = true;
            int s = 0;
            uint32_t ph = 0;
            for (int t = pair; t < p.n_tiles && ok; t += n_pairs) {
                int m0, j0;
                tile_origin(t, m0, j0);
                const int mrow = m0 + 128 * (int)rank;
                const int jr = j0 + 128 * (int)rank;
                for (int it = 0; it < nkb_total; ++it) {
                    ok = mbar_wait(empty(s), ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_EMPTY, 0);
                    if (!ok) break;
                    const uint32_t sA = base + s * kStageBytes;
                    const uint32_t sB = sA + kABytes;
                    const bool extra = it >= nkb;
                    // the leader announces the bytes of BOTH CTAs for this stage
                    if (rank == 0) mbar_arrive_expect_tx(full(s), extra ? 4u * kBlkBytes : 2u * kABytes);
                    if (!extra) {
                        tma_load_2d_pair(sA, &tmA, lead_full(s), it * kBK, mrow);
                        tma_load_2d_pair(sA + kBlkBytes, &tmA, lead_full(s), it * kBK + 64, mrow);
                    } else {
                        // the LoRA block is one 64-wide block: A2 into block 0 of A, B2 by TMA into block 0 of B
                        tma_load_2d_pair(sA, &tmA2, lead_full(s), 0, mrow);
                        if (kBMn) {
                            tma_load_2d_pair(sB, &tmB2, lead_full(s), jr, 0);
                            tma_load_2d_pair(sB + kBlkBytes, &tmB2, lead_full(s), jr + 64, 0);
                        } else {
                            tma_load_2d_pair(sB, &tmB2, lead_full(s), 0, jr);
                        }
                    }
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------- MMA issuer (leader only)
        if (rank == 0 && lane == 0) {
            const uint32_t idesc = make_idesc(256, 256, 0, kBMn ? 1 : 0);
            // descriptor words of stage 0; a stage is kStageBytes >> 4 = 4096 further in the low word
            const uint64_t ad0 = make_sdesc(base, 16u, 1024u);
            const uint64_t bd0 = kBMn ? make_sdesc(base + kABytes, kBlkBytes, 1024u) : make_sdesc(base + kABytes, 16u, 1024u);
            const uint32_t a_hi = (uint32_t)(ad0 >> 32), b_hi = (uint32_t)(bd0 >> 32);
            uint32_t a_lo = (uint32_t)ad0, b_lo = (uint32_t)bd0;
            const uint32_t a_lo0 = a_lo, b_lo0 = b_lo;
            bool ok = true;
            int s = 0, lt = 0;
            uint32_t ph = 0;
            long long wait_f = 0, wait_t = 0;
            const long long t_begin = PLZ_PROF_ON(p.prof) ? clock64() : 0;
            for (int t = pair; t < p.n_tiles && ok; t += n_pairs, ++lt) {
                const uint32_t d_tmem = tmem_base + (uint32_t)(lt & 1) * 256u;
                const long long c_t = PLZ_PROF_ON(p.prof) ? clock64() : 0;
                ok = mbar_wait_lean(acc_empty(lt & 1), ((lt >> 1) & 1) ^ 1u, abort_flag, p.status, ST_TIMEOUT_ACCUM, 1);
                if (PLZ_PROF_ON(p.prof)) wait_t += clock64() - c_t;
                if (!ok) break;
                tc_fence_after_sync();
                for (int it = 0; it < nkb_total; ++it) {
                    const long long c0 = PLZ_PROF_ON(p.prof) ? clock64() : 0;
                    ok = mbar_wait_lean(full(s), ph, abort_flag, p.status, ST_TIMEOUT_FULL, 1);
                    if (PLZ_PROF_ON(p.prof)) wait_f += clock64() - c0;
                    if (!ok) break;
                    tc_fence_after_sync();
                    // k step ks: A and K-major B advance 32 bytes inside a 64-wide block and one block (16 KB) after four
                    // steps; MN-major B advances 16 rows of 128 bytes
                    if (it < nkb) {
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks) {
                            const uint32_t offk = (uint32_t)((ks >> 2) * (kBlkBytes >> 4) + (ks & 3) * 2);
                            const uint32_t offb = kBMn ? (uint32_t)(ks * (2048 >> 4)) : offk;
                            umma_bf16_words<2>(d_tmem, a_lo + offk, a_hi, b_lo + offb, b_hi, idesc, (ks > 0) ? 1u : (it > 0 ? 1u : 0u));
                        }
                    } else {
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {   // the LoRA block is 64 wide
                            const uint32_t offk = (uint32_t)(ks * 2);
                            const uint32_t offb = kBMn ? (uint32_t)(ks * (2048 >> 4)) : offk;
                            umma_bf16_words<2>(d_tmem, a_lo + offk, a_hi, b_lo + offb, b_hi, idesc, 1u);
                        }
                    }
                    umma_commit_pair(empty(s));
                    if (++s == kStages) { s = 0; ph ^= 1u; a_lo = a_lo0; b_lo = b_lo0; }
                    else { a_lo += kStageBytes >> 4; b_lo += kStageBytes >> 4; }
                }
                if (ok) umma_commit_pair(acc_full(lt & 1));
            }
            if (PLZ_PROF_ON(p.prof)) {
                unsigned long long* o = p.prof + 8ull * blockIdx.x;
                o[0] = wait_f; o[1] = 0; o[2] = wait_t; o[3] = clock64() - t_begin; o[4] = lt;
            }
        }
    } else if (warp < kFirstEpiWarp) {
        // ------------------------------------------------------------- decode warps
        // 512 threads produce this CTA's half of the B stage, 128 columns x 128 reduction elements: 32 weights (eight bytes of
        // packed indices, four 16-byte chunks of a 128-byte operand row) per thread and stage.
        //   forward  (rows of the operand = n, two 64-wide k blocks):  block b = t / 256, row n = (t % 256) / 2, half h = t % 2
        //   backward (rows of the operand = n of the stage, two 64-wide k column blocks): block b = t / 256, row = (t % 256) / 2, h
        // Eight consecutive lanes cover four rows x two halves of one block, whose swizzled chunk positions are all different.
        // The index / palette loads run three stages ahead of the stage being written, ACROSS tile boundaries: the sequence
        // of (tile, stage) positions of this pair is one stream, so a new tile does not start with an exposed load latency.
        const int t = threadIdx.x - 64;
        const int h = t & 1;
        const int rr = (t & 255) >> 1;
        const int b = t >> 8;
        const int blocks_per_kgroup = p.gs_k / 64;
        const int dj = n_pairs % p.tiles_j;                 // column-tile step from one tile of this pair to its next
        // Position in the stream of (tile, stage) pairs of this CTA pair, with the running addresses of this thread's
        // loads: per stage the index pointer moves by a constant (32 bytes along k in the forward product, 128 rows in the
        // backward one), so a load costs a compare and an add instead of the full address arithmetic.
        struct Pos {
            int tile, it, tj, kg, cnt;
            const uint8_t* ip;            // packed indices of this thread at stage `it`
            const __nv_bfloat16* pp;      // forward: palettes of this thread's row; backward: palette base + fixed k group
            bool ok;                      // the fixed coordinate (forward: n, backward: k) lies inside the matrix
        };
        const int koff = b * 64 + h * 32;
        // number of stages for which the running coordinate stays inside the matrix (forward: k, backward: n)
        const int it_lim = kBMn ? ((p.Wn - rr + kBK - 1) / kBK) : ((p.Wk - koff + kBK - 1) / kBK);
        const long long ip_step = kBMn ? (long long)kBK * p.packed_pitch : (long long)(kBK / 4);
        auto set_tile = [&](Pos& q) {
            const int jr = q.tj * 256 + 128 * (int)rank;
            if (kBMn) {
                const int k = jr + koff;
                q.ok = k < p.Wk;
                q.kg = q.ok ? (k / p.gs_k) : 0;
                q.cnt = 0;
                q.ip = p.packed + (long long)rr * p.packed_pitch + (k >> 2);
                q.pp = p.palette + (long long)q.kg * 4;
            } else {
                const int n = jr + rr;
                q.ok = n < p.Wn;
                q.kg = b / blocks_per_kgroup; q.cnt = b % blocks_per_kgroup;
                q.ip = p.packed + (long long)n * p.packed_pitch + (koff >> 2);
                const int ng = q.ok ? ((p.gs_n_shift >= 0) ? (n >> p.gs_n_shift) : (n / p.gs_n)) : 0;
                q.pp = p.palette + (long long)ng * p.n_kgroups * 4;
            }
        };
        auto pos_next = [&](Pos& q) {
            if (++q.it == nkb_total) {
                q.it = 0; q.tile += n_pairs; q.tj += dj; if (q.tj >= p.tiles_j) q.tj -= p.tiles_j;
                set_tile(q);
            } else {
                q.ip += ip_step;
                if (!kBMn) {
                    q.cnt += 2;
                    while (q.cnt >= blocks_per_kgroup) { q.cnt -= blocks_per_kgroup; ++q.kg; }
                }
            }
        };
        auto load_pos = [&](const Pos& q, uint2& idx, uint2& pal) {
            idx = make_uint2(0u, 0u); pal = make_uint2(0u, 0u);
            if (!q.ok || q.it >= it_lim || q.it >= nkb || q.tile >= p.n_tiles) return;
            idx = __ldg(reinterpret_cast<const uint2*>(q.ip));
            if (kBMn) {
                const int n = q.it * kBK + rr;
                const int ng = (p.gs_n_shift >= 0) ? (n >> p.gs_n_shift) : (n / p.gs_n);
                pal = __ldg(reinterpret_cast<const uint2*>(q.pp + (long long)ng * p.n_kgroups * 4));
            } else {
                pal = __ldg(reinterpret_cast<const uint2*>(q.pp + q.kg * 4));
            }
        };
        // The stream is walked three stages per trip (= the ring), so ring stage and queue slot of every step are compile-time
        // constants: no slot is ever copied, which would make the copy wait for a load that has just been issued.
        static_assert(kStages == 3, "the decode loop is unrolled by the depth of the ring");
        uint2 idx_q[3], pal_q[3];
        Pos pf; pf.tile = pair; pf.it = 0; pf.tj = pair % p.tiles_j; set_tile(pf);
        int c_tile = pair, c_it = 0;   // the position being written
#pragma unroll
        for (int u = 0; u < 3; ++u) { load_pos(pf, idx_q[u], pal_q[u]); pos_next(pf); }
        bool ok = true;
        for (int g0 = 0; ok && c_tile < p.n_tiles; g0 += 3) {
            const uint32_t ph = (uint32_t)((g0 / 3) & 1);
#pragma unroll
            for (int u = 0; u < 3; ++u) {
                if (c_tile >= p.n_tiles) break;
                const bool is_extra = c_it >= nkb;
                if (++c_it == nkb_total) { c_it = 0; c_tile += n_pairs; }
                const uint2 idx_cur = idx_q[u], pal_cur = pal_q[u];
                load_pos(pf, idx_q[u], pal_q[u]);
                pos_next(pf);
                ok = mbar_wait(empty(u), ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_EMPTY, 3);
                if (!ok) break;
                if (is_extra) {
                    // the LoRA block comes by TMA; arrive all the same, after the stage is free, to keep the phases in step
                    if (lane == 0) mbar_arrive_cluster(lead_full(u));
                    continue;
                }
                uint8_t* row = smem + u * kStageBytes + kABytes + b * kBlkBytes + rr * 128;
                const PalRegs pal = pal_split(pal_cur.x, pal_cur.y);
                const uint32_t w[2] = {idx_cur.x, idx_cur.y};
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    uint32_t o[8];
                    decode16(w[i], pal, o);
                    *reinterpret_cast<uint4*>(row + (((4 * h + 2 * i) ^ (rr & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<uint4*>(row + (((4 * h + 2 * i + 1) ^ (rr & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(lead_full(u));
            }
        }
    } else {
        // ------------------------------------------------------------- epilogue warps
        // warp e reads TMEM lanes 32 * (warp % 4) (its 32 output rows of this CTA's 128) and walks the 256 columns 64 at a
        // time: fp32 -> bf16 -> 128-byte-swizzled box in shared memory -> TMA store (clipped at M and J).
        const int e = warp - kFirstEpiWarp;
        const int lane_group = warp & 3;
        uint8_t* stage = smem + kEpiOff + e * kEpiStageBytes;
        const uint32_t stage_u32 = base + kEpiOff + e * kEpiStageBytes;
        bool ok = true;
        int lt = 0;
        for (int t = pair; t < p.n_tiles && ok; t += n_pairs, ++lt) {
            int m0, j0;
            tile_origin(t, m0, j0);
            const int buf = lt & 1;
            const int mrow = m0 + 128 * (int)rank + lane_group * 32;
            ok = mbar_wait(acc_full(buf), (lt >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_ACCUM, 4);
            if (!ok) break;
            tc_fence_after_sync();
#pragma unroll 1
            for (int b = 0; b < 4; ++b) {
                const int col = b * 64;
                if (lane == 0) tma_store_wait_read();
                __syncwarp();
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(lane_group * 32) << 16) + buf * 256u + col + c * 32, v);
                    if (b == 3 && c == 1) {
                        // last read of this accumulator: hand it back to the MMA thread of the leader
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(lead_acc_empty(buf));
                    }
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint4 o;
                        o.x = pack_bf16x2(__uint_as_float(v[g * 8 + 0]) * p.alpha, __uint_as_float(v[g * 8 + 1]) * p.alpha);
                        o.y = pack_bf16x2(__uint_as_float(v[g * 8 + 2]) * p.alpha, __uint_as_float(v[g * 8 + 3]) * p.alpha);
                        o.z = pack_bf16x2(__uint_as_float(v[g * 8 + 4]) * p.alpha, __uint_as_float(v[g * 8 + 5]) * p.alpha);
                        o.w = pack_bf16x2(__uint_as_float(v[g * 8 + 6]) * p.alpha, __uint_as_float(v[g * 8 + 7]) * p.alpha);
                        *reinterpret_cast<uint4*>(stage + swz128(lane, c * 4 + g)) = o;
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0 && j0 + col < p.J && mrow < p.M) {
                    tma_store_2d(&tmD, stage_u32, j0 + col, mrow);
                    tma_store_commit();
                }
            }
        }
        if (lane == 0) tma_store_wait_all();
    }
    // Neither CTA may leave while its partner can still touch its shared memory (operand reads of the pair MMA, remote
    // barrier arrivals) or its tensor memory.
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

template <int BMODE>
int launch_pair_t(const LutGemmArgs& a, cudaStream_t stream) {
    CUtensorMap tmA, tmA2, tmB2, tmD;
    int rc;
    if ((rc = make_tmap_bf16(&tmA, a.A, a.M, a.R, a.lda, 64, 128))) return rc;
    tmA2 = tmA; tmB2 = tmA;
    if (a.r2 > 0) {
        if ((rc = make_tmap_bf16(&tmA2, a.A2, a.M, a.r2, a.lda2, 64, 128))) return rc;
        if (BMODE == B_DECODE_MN) {
            if ((rc = make_tmap_bf16(&tmB2, a.B2, a.r2, a.J, a.ldb2, 64, 64))) return rc;
        } else {
            if ((rc = make_tmap_bf16(&tmB2, a.B2, a.J, a.r2, a.ldb2, 64, 128))) return rc;
        }
    }
    if ((rc = make_tmap_bf16(&tmD, a.out, a.M, a.J, a.ld_out, 64, 32))) return rc;
    PairParams p = {};
    p.M = a.M; p.J = a.J; p.R = a.R; p.n_extra = a.r2 > 0 ? 1 : 0;
    p.tiles_j = (a.J + 255) / 256;
    p.tiles_m = (a.M + 255) / 256;
    p.n_tiles = p.tiles_m * p.tiles_j;
    p.packed = (const uint8_t*)a.packed; p.packed_pitch = a.packed_pitch;
    p.palette = (const __nv_bfloat16*)a.palette;
    p.gs_n = a.gs_n > 0 ? a.gs_n : 1; p.gs_k = a.gs_k > 0 ? a.gs_k : kBK;
    p.n_kgroups = a.gs_k > 0 ? (a.Wk / a.gs_k) : 1;
    p.gs_n_shift = -1;
    for (int sh = 0; sh < 31; ++sh) if ((1 << sh) == p.gs_n) p.gs_n_shift = sh;
    p.Wn = a.Wn; p.Wk = a.Wk;
    p.alpha = a.alpha;
    p.status = device_status_ptr();
    p.prof = (unsigned long long*)a.prof;
    auto kern = lut_gemm_pair_kernel<BMODE>;
    static bool attr_set[64] = {};
    int dev = 0, sms = 0;
    PLZ_CUDA_CHECK(cudaGetDevice(&dev));
    if (!attr_set[dev & 63]) {
        PLZ_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        attr_set[dev & 63] = true;
    }
    PLZ_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (a.sm_limit > 0 && a.sm_limit < sms) sms = a.sm_limit;
    if (g_cta_limit > 0 && g_cta_limit < sms) sms = g_cta_limit;
    int pairs = sms / 2;
    if (pairs > p.n_tiles) pairs = p.n_tiles;
    if (pairs < 1) return PLZ_ERR_UNSUPPORTED;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = stream;
    PLZ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, tmA, tmA2, tmB2, tmD, p));
    ++g_launch_count;
    return PLZ_OK;
}

}  // namespace

// PLZ_ERR_UNSUPPORTED: not a shape for this kernel, the caller falls back to the single-CTA kernel.
int launch_lut_gemm_pair(const LutGemmArgs& a, cudaStream_t stream) {
    if (!g_pair_gemm) return PLZ_ERR_UNSUPPORTED;
    if (a.bmode != B_DECODE_K && a.bmode != B_DECODE_MN) return PLZ_ERR_UNSUPPORTED;
    if (a.fuse != 0 || a.M < 256 || a.J < 256) return PLZ_ERR_UNSUPPORTED;
    if (a.bmode == B_DECODE_MN && (a.J % 16)) return PLZ_ERR_UNSUPPORTED;
    if (a.bmode == B_DECODE_K && (a.Wk % 16)) return PLZ_ERR_UNSUPPORTED;
    return a.bmode == B_DECODE_K ? launch_pair_t<B_DECODE_K>(a, stream) : launch_pair_t<B_DECODE_MN>(a, stream);
}

}  // namespace plz
