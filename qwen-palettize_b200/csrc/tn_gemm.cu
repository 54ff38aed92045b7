// tn_gemm: D[I, J] = sum_m P[m, i] * Q[m, j]  -- a reduction over the token axis m of two row-major
// bf16 matrices (both operands MN-major for the tensor core), fp32 accumulation in TMEM, persistent
// CTAs with two TMEM accumulators so that the epilogue of one tile overlaps the main loop of the next.
//
// This is the weight-gradient product dW = x^T dY of the palettized Linear. dW never reaches HBM:
// the epilogue turns each fp32 tile into what the optimizer needs.
//
//   EPI_SOFT   dLogits[p] = dW * P[p] * (c[p] - W_soft),  dPalette[group][p] += sum dW * P[p]
//              with P recomputed from logits (+ the same noise the forward used)
//   EPI_HARD   dPalette[group][idx] += dW   (gradient of the hard gather)
//   EPI_STORE  plain fp32 store / atomic add (LoRA factor gradients dA, dB), optional split over m
//
// Layout B ("native"): D rows = k, columns = n; logits fp32 [N, K, 4]; one palette per (n, k / gs_k).
// Layout R (reference API): D rows = n, columns = k; logits fp16 [4, K, N]; one palette per n / gs_n.
// In both cases consecutive TMEM lanes (threads of a warp) touch consecutive addresses of the
// logits, so every global access of the epilogue is fully coalesced.
//
// Replaces, in the reference: grad_W = x^T dY (scripts/fused_lut_linear_cuda.py:952,
// scripts/triton_soft_backward.py:165-206), soft_bwd_elementwise_aos_kernel
// (scripts/fused_lut_kernel.cu:1877-1924), fused_soft_bwd_elementwise_kernel
// (scripts/triton_soft_backward.py:227-325) and fused_lut_linear_bwd_grad_palette_kernel
// (scripts/fused_lut_kernel.cu:902).
#include "plz_launch.h"
#include "soft_math.cuh"

namespace plz {


struct TnParams {
    int M, I, J;       // P is [M, I], Q is [M, J], D is [I, J]
    int n_whole, n_items;  // items [0, n_whole) are whole 128 x 256 tiles, the rest 128 x 128 halves (last round)
    int splits;        // EPI_STORE only: the m range is cut into `splits` chunks, results atomically added
    int m_chunk;       // rows of m per split (multiple of 64)
    // EPI_STORE
    float* out; long long out_si, out_sj; float alpha; int out_I, out_J;  // store bounds
    // EPI_SOFT / EPI_HARD
    const void* logits; void* dlogits;       // element strides below, dtype by template
    long long ls_row, ls_col, ls_p;          // strides of the logits for D row, D col, plane
    const float* noise; long long ns_row, ns_col, ns_p;
    int noise_mode; uint32_t seed; int hashN;  // hash noise index = (k * hashN + n) * 4 + p
    float inv_tau;
    const __nv_bfloat16* palette; float* dpalette;
    int gs_n, gs_k, n_kgroups;
    const uint8_t* packed; long long packed_pitch;  // EPI_HARD
    // Side jobs (the LoRA factor gradients): extra work items appended to the list, D[r, j] = sum_m S[m, r] * Qs[m, j]
    // with S a skinny [M, rank] matrix and Qs one of the two main operands; results are atomically added to `out`.
    struct Side {
        int tiles_j, splits, m_chunk, q_is_p, out_I, out_J, first_item;
        float* out; long long out_si, out_sj;
    } side[2];
    int n_side_items;
    // Tail of the persistent schedule. After the whole tiles come the half tiles (one per work unit, n_items - n_whole of
    // them) and then the side items, which are dealt only to the units that did not get a half tile: tail slots that fall on
    // a unit with a half tile stay empty, so that no unit carries a half tile AND a second side item while others idle.
    // tail_free = units without a half tile (0: the side items simply follow the halves); n_total = items including holes.
    int tail_free, n_total;
    // Fused reduce-scatter of dLogits over peer memory (rows = k layout only): weight row n belongs to rank
    // n / rows_per_rank; its gradient is stored into that rank's staging buffer, slot `rank`, instead of into `dlogits`.
    // scatter_add: the owner's buffer is one fp32 [rows_per_rank][K][4] accumulator (zeroed by its owner) and the partials
    // are added to it with vector reductions instead of being stored into per-source slots.
    float* peer_stage[8]; int world, rank, rows_per_rank, scatter_add; long long shard_elems;
    // Column tiles are walked from a rank-dependent start (rank * tiles_j / world), so that at any moment the ranks of a
    // node store into DIFFERENT owners: with a common order all of them write to the same one or two owners at once and
    // that GPU's NVLink ingress throttles everybody (measured at 8 ranks: the slowest rank's launch 1.4 ms against 0.8).
    int tj_rot;
    StatusWord* status;
    unsigned long long* prof;  // diagnostics build: [gridDim][8] cycle counters of the MMA thread
};

constexpr int kTnThreads = 320;  // warp 0: TMA, warp 1: MMA, warps 2..9: epilogue
constexpr int kTnStages = 4;
constexpr uint32_t kTnABytes = 128 * 64 * 2;  // 2 boxes of [64 m][64 i]
constexpr uint32_t kTnBBytes = 256 * 64 * 2;  // 4 boxes of [64 m][64 j]
constexpr uint32_t kTnStageBytes = kTnABytes + kTnBBytes;
constexpr uint32_t kTnRedBytes = 4 * 256 * 4 * 4;  // per-warp palette-gradient partials
constexpr uint32_t kTnSmemBytes = kTnStages * kTnStageBytes + kTnRedBytes + 1024 + 256;
// CTA-pair form (cta_group::2, one 256 x 256 tile per pair): each CTA stages its own 128 i columns and HALF of the j
// columns, 32 KB per 64 rows of m, so the ring holds six stages; every CTA reads 2/3 of the operand bytes of the one-CTA
// form for the same work, which matters because this product is bound by the L2 -> SM operand feed.
constexpr int kTnStagesPair = 6;
constexpr uint32_t kTnBBytesPair = 128 * 64 * 2;
constexpr uint32_t kTnStageBytesPair = kTnABytes + kTnBBytesPair;
constexpr uint32_t kTnSmemBytesPair = kTnStagesPair * kTnStageBytesPair + kTnRedBytes + 1024 + 256;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

template <int EPI, typename LogitT, bool ROWS_K, bool PAIR>
__global__ void __launch_bounds__(kTnThreads, 1)
tn_gemm_kernel(const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmQ,
               const __grid_constant__ CUtensorMap tmS0, const __grid_constant__ CUtensorMap tmS1, const TnParams p) {
    constexpr int kStages = PAIR ? kTnStagesPair : kTnStages;
    constexpr uint32_t kBBytes = PAIR ? kTnBBytesPair : kTnBBytes;
    constexpr uint32_t kStageBytes = kTnABytes + kBBytes;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    float* red = reinterpret_cast<float*>(smem + kStages * kStageBytes);
    const uint32_t bar_base = base + kStages * kStageBytes + kTnRedBytes;
    auto full = [&](int s) { return bar_base + 8u * s; };
    auto empty = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto acc_full = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
    auto acc_empty = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(
        smem + kStages * kStageBytes + kTnRedBytes + 8 * (2 * kStages + 4));
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // PAIR: the two CTAs of a cluster share every work item; full[] and acc_empty[] are used in the leader's copy only
    // (remote arrivals / TMA completions from the partner), empty[] and acc_full[] in each CTA's own copy (multicast commit)
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
    const uint32_t lead_bar_base = PAIR ? leader_addr(bar_base) : bar_base;
    auto lead_full = [&](int s) { return lead_bar_base + 8u * s; };
    auto lead_acc_empty = [&](int b) { return lead_bar_base + 8u * (2 * kStages + 2 + b); };
    const int unit = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int n_units = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const int tiles_i = PAIR ? (p.I + 255) / 256 : (p.I + 127) / 128;
    const int tiles_j = (p.J + 255) / 256;
    const int n_tiles = p.n_total;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), PAIR ? 16 : 8);
        }
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmP);
        tma_prefetch_desc(&tmQ);
        if (p.n_side_items) { tma_prefetch_desc(&tmS0); tma_prefetch_desc(&tmS1); }
    }
    if (warp == 1) {
        if (PAIR) { tmem_alloc_pair(smem_u32((const void*)tmem_slot), 512); tmem_relinquish_pair(); }
        else { tmem_alloc(smem_u32((const void*)tmem_slot), 512); tmem_relinquish(); }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (PAIR) cluster_sync_all();   // both CTAs' barriers exist before anyone arrives on the partner's
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    // tile -> (split, i tile, j tile); i fastest so that one wave of CTAs covers every i tile
    // item -> (split, i tile, j tile, first column inside the tile, columns); i fastest so that one wave of CTAs
    // covers every i tile. Items past n_whole are the two 128-column halves of a tile.
    auto tile_coords = [&](int item, int& sp, int& ti, int& tj, int& c_off, int& c_num, int& job) {
        c_off = 0; c_num = 256; job = -1;
        if (item >= p.n_items) {
            // side item number: tail slots on units that hold a half tile are holes (job -2: the unit is done)
            int sidx = item - p.n_items;
            if (p.tail_free > 0) {
                const int n_halves = p.n_items - p.n_whole;
                const int rt = item - p.n_whole, slot = rt % n_units, round = rt / n_units;
                if (slot < n_halves) { job = -2; sp = ti = tj = 0; return; }
                sidx = round * p.tail_free + slot - n_halves;
            }
            if (sidx >= p.n_side_items) { job = -2; sp = ti = tj = 0; return; }
            job = (p.side[1].splits > 0 && sidx >= p.side[1].first_item) ? 1 : 0;
            const int r = sidx - p.side[job].first_item;
            tj = r % p.side[job].tiles_j;
            sp = r / p.side[job].tiles_j;
            // PAIR: the operands change sides, D[big-matrix column, rank index]: the 256 rows of the pair are 256 columns of
            // x / dY (all of them useful) and the skinny matrix is the 128-column N side (16 or 32 real columns), so an MMA costs
            // half of what the 256-column shape with 240 padded rows would
            ti = PAIR ? 2 * tj + (int)rank : 0;
            if (PAIR) c_num = 128;
            return;
        }
        int t = item;
        if (item >= p.n_whole) {
            t = p.n_whole + ((item - p.n_whole) >> 1);
            c_off = ((item - p.n_whole) & 1) * 128;
            c_num = 128;
        }
        ti = t % tiles_i;
        const int r = t / tiles_i;
        tj = r % tiles_j + p.tj_rot;
        if (tj >= tiles_j) tj -= tiles_j;
        sp = r / tiles_j;
        if (PAIR) ti = 2 * ti + (int)rank;   // this CTA's 128 rows of the pair's 256
    };
    auto m_range = [&](int sp, int job, int& m_begin, int& nkb) {
        const int chunk = (job < 0) ? p.m_chunk : p.side[job].m_chunk;
        m_begin = sp * chunk;
        int m_end = m_begin + chunk;
        if (m_end > p.M) m_end = p.M;
        nkb = (m_end - m_begin + 63) / 64;
        if (nkb < 0) nkb = 0;
    };

    if (warp == 0) {
        if (lane == 0) {
            int last_fill[kStages];
            for (int s = 0; s < kStages; ++s) last_fill[s] = -1;
            bool ok = true;
            int git = 0;
            for (int t = unit; t < n_tiles && ok; t += n_units) {
                int sp, ti, tj, c_off, c_num, job, m_begin, nkb;
                tile_coords(t, sp, ti, tj, c_off, c_num, job);
                if (job == -2) break;      // a hole of the tail: nothing more for this unit
                m_range(sp, job, m_begin, nkb);
                const int c_mine = PAIR ? (c_num >> 1) : c_num;                  // j columns this CTA stages
                const bool swapped = PAIR && job >= 0;                           // side item of a pair: skinny matrix on the N side
                const int j_mine = swapped ? (int)rank * c_mine : tj * 256 + c_off + (PAIR ? (int)rank * c_mine : 0);
                for (int it = 0; it < nkb; ++it, ++git) {
                    const int s = git % kStages;
                    const uint32_t ph = (git / kStages) & 1;
                    ok = mbar_wait(empty(s), ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_EMPTY, 0);
                    if (!ok) break;
                    const uint32_t sA = base + s * kStageBytes;
                    const uint32_t sB = sA + kTnABytes;
                    // PAIR: the leader announces the bytes of both CTAs; each CTA's copies complete on the leader's barrier
                    if (!PAIR) mbar_arrive_expect_tx(full(s), kTnABytes + (uint32_t)c_num * 128u);
                    else if (rank == 0) mbar_arrive_expect_tx(full(s), 2u * (kTnABytes + (uint32_t)c_mine * 128u));
                    const int m = m_begin + it * 64;
                    const CUtensorMap* m_skinny = (job == 0) ? &tmS0 : &tmS1;
                    const CUtensorMap* m_big = (job >= 0 && p.side[job].q_is_p) ? &tmP : &tmQ;
                    const CUtensorMap* mp = (job < 0) ? &tmP : (swapped ? m_big : m_skinny);
                    const CUtensorMap* mq = (job < 0) ? &tmQ : (swapped ? m_skinny : m_big);
                    if (PAIR) {
#pragma unroll
                        for (int q = 0; q < 2; ++q) tma_load_2d_pair(sA + q * 8192u, mp, lead_full(s), ti * 128 + q * 64, m);
#pragma unroll
                        for (int q = 0; q < 2; ++q)
                            if (q * 64 < c_mine) tma_load_2d_pair(sB + q * 8192u, mq, lead_full(s), j_mine + q * 64, m);
                    } else {
#pragma unroll
                        for (int q = 0; q < 2; ++q) tma_load_2d(sA + q * 8192u, mp, full(s), ti * 128 + q * 64, m);
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            if (q * 64 < c_num) tma_load_2d(sB + q * 8192u, mq, full(s), j_mine + q * 64, m);
                    }
                    last_fill[s] = git;
                }
            }
            if (!ok && !PAIR) {
                for (int s = 0; s < kStages; ++s) {
                    if (last_fill[s] < 0) continue;
                    const uint32_t ph = (last_fill[s] / kStages) & 1;
                    const uint64_t t0 = globaltimer_ns();
                    while (!mbar_try_wait(full(s), ph)) {
                        if (globaltimer_ns() - t0 > 100000000ull) {
                            report(p.status, ST_TIMEOUT_DRAIN, 0);
                            break;
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // MMA issuer (PAIR: the leader's only). Kept lean on purpose: a lone thread retires a dependent instruction every
        // five or six cycles and an MMA lasts 128, so the descriptor words are precomputed (one integer add per operand
        // and MMA) and the usual, already-completed barrier costs a single try_wait.
        if (lane == 0 && rank == 0) {
            bool ok = true;
            int lt = 0, s = 0;
            uint32_t ph = 0;
            const uint64_t ad0 = make_sdesc(base, 8192u, 1024u);
            const uint64_t bd0 = make_sdesc(base + kTnABytes, 8192u, 1024u);
            const uint32_t a_hi = (uint32_t)(ad0 >> 32), b_hi = (uint32_t)(bd0 >> 32);
            const uint32_t a_lo0 = (uint32_t)ad0, b_lo0 = (uint32_t)bd0;
            uint32_t a_lo = a_lo0, b_lo = b_lo0;
            long long wait_f = 0, wait_t = 0, n_st = 0;
            const long long t_begin = PLZ_PROF_ON(p.prof) ? clock64() : 0;
            for (int t = unit; t < n_tiles && ok; t += n_units, ++lt) {
                int sp, ti, tj, c_off, c_num, job, m_begin, nkb;
                tile_coords(t, sp, ti, tj, c_off, c_num, job);
                if (job == -2) break;
                m_range(sp, job, m_begin, nkb);
                const int buf = lt & 1;
                const uint32_t idesc = make_idesc(PAIR ? 256 : 128, c_num, 1, 1);
                const uint32_t d_tmem = tmem_base + buf * 256u;
                const long long c_t = PLZ_PROF_ON(p.prof) ? clock64() : 0;
                ok = mbar_wait_lean(acc_empty(buf), ((lt >> 1) & 1) ^ 1u, abort_flag, p.status, ST_TIMEOUT_ACCUM, 1);
                if (PLZ_PROF_ON(p.prof)) wait_t += clock64() - c_t;
                if (!ok) break;
                tc_fence_after_sync();
                for (int it = 0; it < nkb; ++it) {
                    const long long c_f = PLZ_PROF_ON(p.prof) ? clock64() : 0;
                    ok = mbar_wait_lean(full(s), ph, abort_flag, p.status, ST_TIMEOUT_FULL, 1);
                    if (PLZ_PROF_ON(p.prof)) { wait_f += clock64() - c_f; ++n_st; }
                    if (!ok) break;
                    tc_fence_after_sync();
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks)   // 16 rows of m = 2048 bytes per step in both MN-major operands
                        umma_bf16_words<PAIR ? 2 : 1>(d_tmem, a_lo + ks * 128u, a_hi, b_lo + ks * 128u, b_hi, idesc,
                                                     (ks > 0) ? 1u : (it > 0 ? 1u : 0u));
                    if (PAIR) umma_commit_pair(empty(s)); else umma_commit(empty(s));
                    if (++s == kStages) { s = 0; ph ^= 1u; a_lo = a_lo0; b_lo = b_lo0; }
                    else { a_lo += kStageBytes >> 4; b_lo += kStageBytes >> 4; }
                }
                if (ok) { if (PAIR) umma_commit_pair(acc_full(buf)); else umma_commit(acc_full(buf)); }
            }
            if (PLZ_PROF_ON(p.prof)) {
                unsigned long long* o = p.prof + 8ull * blockIdx.x;
                o[0] = wait_f; o[1] = n_st; o[2] = wait_t; o[3] = clock64() - t_begin; o[4] = lt;
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps
        // Eight warps: warp w reads TMEM lanes 32*(w%4).., and the two warps of a lane group split the
        // 256 columns in halves. Columns are processed 8 at a time: all global loads of a batch are issued
        // before any arithmetic, so that each thread keeps 16 x 16 bytes in flight.
        const int lane_group = warp & 3;
        const int col_half = (warp - 2) >> 2;
        const int ew = warp - 2;  // 0..7
        bool ok = true;
        int lt = 0;
        for (int t = unit; t < n_tiles && ok; t += n_units, ++lt) {
            int sp, ti, tj, c_off, c_num, job, m_begin, nkb;
            tile_coords(t, sp, ti, tj, c_off, c_num, job);
            if (job == -2) break;
            m_range(sp, job, m_begin, nkb);
            const int buf = lt & 1;
            ok = mbar_wait(acc_full(buf), (lt >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_ACCUM, 2);
            if (!ok) break;
            tc_fence_after_sync();
            const int row = ti * 128 + lane_group * 32 + lane;  // D row of this thread
            const int wcols = c_num >> 1;  // columns per epilogue warp: 128, or 64 in a half tile
            const uint32_t trow = tmem_base + ((uint32_t)(lane_group * 32) << 16) + buf * 256u + col_half * wcols;
            const bool row_ok = row < p.I;
            const int colbase = (PAIR && job >= 0) ? col_half * wcols : tj * 256 + c_off + col_half * wcols;

            if (EPI == EPI_STORE || job >= 0) {
                float* o_ptr = (job < 0) ? p.out : p.side[job].out;
                const long long o_si = (job < 0) ? p.out_si : p.side[job].out_si, o_sj = (job < 0) ? p.out_sj : p.side[job].out_sj;
                const int o_I = (job < 0) ? p.out_I : p.side[job].out_I, o_J = (job < 0) ? p.out_J : p.side[job].out_J;
                const float o_alpha = (job < 0) ? p.alpha : 1.0f;
#pragma unroll 1
                for (int c0 = 0; c0 < wcols; c0 += 16) {
                    uint32_t v[16];
                    tmem_ld_32x16(trow + c0, v);
                    if (nkb > 0 && row < o_I) {
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            const int col = colbase + c0 + c;
                            if (col < o_J)
                                atomicAdd(o_ptr + (long long)row * o_si + (long long)col * o_sj, __uint_as_float(v[c]) * o_alpha);
                        }
                    }
                }
            } else if (ROWS_K) {
                // Interleaved logits [N, K, 4], one palette per (n, 256-wide k group): D rows are input columns k
                // (the 32 lanes of a warp read 32 consecutive float4 = 512 contiguous bytes), D columns are weight
                // rows n, each with its own palette. The palette gradient of a column is a sum over lanes: the 32
                // partials of a batch (8 columns x 4 entries) are reduced with a 31-shuffle transposing butterfly.
                const int k = row;
                const int kgi = (row_ok ? k : 0) / p.gs_k;
                const float* lbase = reinterpret_cast<const float*>(p.logits) + (long long)k * p.ls_row;
                float* dbase = p.dlogits ? reinterpret_cast<float*>(p.dlogits) + (long long)k * p.ls_row : nullptr;
                const float* nbase = p.noise ? p.noise + (long long)k * p.ns_row : nullptr;
#pragma unroll 1
                for (int c0 = 0; c0 < wcols; c0 += 8) {
                    uint32_t v[8];
                    tmem_ld_32x8(trow + c0, v);
                    const int nb = colbase + c0;  // first n of the batch
                    // fused reduce-scatter: the 8 rows of a batch have one owner (rows_per_rank % 8 == 0); its buffer, this
                    // rank's slot (or the accumulator) and this thread's k folded into one base pointer per batch
                    float* sbase = nullptr;
                    if (p.world > 1 && nb < p.J) {
                        const int owner = nb / p.rows_per_rank;
                        sbase = p.peer_stage[owner] + (p.scatter_add ? 0ll : (long long)p.rank * p.shard_elems) +
                                ((long long)(nb - owner * p.rows_per_rank) * p.I + k) * 4;
                    }
                    float4 lv[8], gv[8];
                    uint2 praw[8];
                    uint32_t hbyte[8];
                    // ---- phase 1: issue every load of the batch
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const int n = nb + c;
                        const bool valid = row_ok && n < p.J;
                        lv[c] = make_float4(0.f, 0.f, 0.f, 0.f);
                        gv[c] = make_float4(0.f, 0.f, 0.f, 0.f);
                        praw[c] = make_uint2(0u, 0u);
                        hbyte[c] = 0;
                        if (valid) {
                            if (EPI == EPI_SOFT) {
                                praw[c] = __ldg(reinterpret_cast<const uint2*>(p.palette + ((long long)n * p.n_kgroups + kgi) * 4));
                                lv[c] = __ldcs(reinterpret_cast<const float4*>(lbase + (long long)n * p.ls_col));
                                if (p.noise_mode == NOISE_TENSOR)
                                    gv[c] = __ldcs(reinterpret_cast<const float4*>(nbase + (long long)n * p.ns_col));
                            } else {
                                hbyte[c] = __ldg(p.packed + (long long)n * p.packed_pitch + (k >> 2));
                            }
                        }
                    }
                    // ---- phase 2: arithmetic and stores
                    float part[32];
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const int n = nb + c;
                        const bool valid = row_ok && n < p.J;
                        const float dw = valid ? __uint_as_float(v[c]) : 0.f;
                        if (EPI == EPI_SOFT) {
                            float cp[4], l[4], g[4];
                            cp[0] = __uint_as_float(praw[c].x << 16);
                            cp[1] = __uint_as_float(praw[c].x & 0xFFFF0000u);
                            cp[2] = __uint_as_float(praw[c].y << 16);
                            cp[3] = __uint_as_float(praw[c].y & 0xFFFF0000u);
                            l[0] = lv[c].x; l[1] = lv[c].y; l[2] = lv[c].z; l[3] = lv[c].w;
                            g[0] = gv[c].x; g[1] = gv[c].y; g[2] = gv[c].z; g[3] = gv[c].w;
                            if (p.noise_mode == NOISE_HASH) {
                                const uint32_t e = ((uint32_t)k * (uint32_t)p.hashN + (uint32_t)n) * 4u;
#pragma unroll
                                for (int q = 0; q < 4; ++q) g[q] = gumbel_hash(p.seed, e + q);
                            }
                            const Soft4 s4 = soft4(l, g, cp, p.inv_tau);
                            float dl[4];
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                part[c * 4 + q] = dw * s4.P[q];
                                dl[q] = part[c * 4 + q] * (cp[q] - s4.w_soft);
                            }
                            if (valid && p.world > 1) {
                                // plain (non-atomic) 16-byte store into the owner's staging slot of this rank: the 32 lanes
                                // of the warp cover 512 contiguous bytes there, peer or local alike
                                float* dst = sbase + (long long)c * p.I * 4;
                                if (p.scatter_add) {
                                    asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                                                 :: "l"(dst), "f"(dl[0]), "f"(dl[1]), "f"(dl[2]), "f"(dl[3]) : "memory");
                                } else {
                                    *reinterpret_cast<float4*>(dst) = make_float4(dl[0], dl[1], dl[2], dl[3]);
                                }
                            } else if (valid && dbase != nullptr)
                                __stcs(reinterpret_cast<float4*>(dbase + (long long)n * p.ls_col), make_float4(dl[0], dl[1], dl[2], dl[3]));
                        } else {
                            const int idx = (hbyte[c] >> (2 * (k & 3))) & 3;
#pragma unroll
                            for (int q = 0; q < 4; ++q) part[c * 4 + q] = (q == idx) ? dw : 0.f;
                        }
                    }
                    if (p.dpalette != nullptr) {
                        // transposing butterfly: afterwards lane L holds the sum over all 32 lanes of part[L]
#pragma unroll
                        for (int s = 16; s >= 1; s >>= 1) {
                            const bool up = (lane & s) != 0;
#pragma unroll
                            for (int j = 0; j < s; ++j) {
                                const float send = up ? part[j] : part[j + s];
                                const float keep = up ? part[j + s] : part[j];
                                part[j] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, s);
                            }
                        }
                        red[(lane_group * 256 + col_half * wcols + c0) * 4 + lane] = part[0];
                    }
                }
                if (p.dpalette != nullptr) {
                    epi_bar_sync();
                    // one thread per column: add the four lane groups' partials in a fixed order
                    const int et = threadIdx.x - 64;  // 0..255
                    const int n = tj * 256 + c_off + et;
                    const int k0 = ti * 128;
                    if (et < c_num && n < p.J && k0 < p.I) {
                        const long long pg = ((long long)n * p.n_kgroups + k0 / p.gs_k) * 4;
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float s = ((red[(0 * 256 + et) * 4 + q] + red[(1 * 256 + et) * 4 + q]) +
                                             red[(2 * 256 + et) * 4 + q]) + red[(3 * 256 + et) * 4 + q];
                            atomicAdd(p.dpalette + pg + q, s);
                        }
                    }
                    epi_bar_sync();
                }
            } else {
                // D rows are weight rows n, columns are input columns k. A thread owns one n and walks k, so the
                // palette (one per n-group and 256-wide k-group) is loaded once per tile and the palette-gradient
                // partial sums stay in registers for the whole tile.
                constexpr bool kVec = (sizeof(LogitT) == 4);
                const bool vec_l = kVec && p.ls_p == 1;
                const bool vec_n = p.ns_p == 1;
                const int n = row;
                const int k_tile0 = tj * 256 + c_off;
                const long long pg = ((long long)((row_ok ? n : 0) / p.gs_n) * p.n_kgroups + k_tile0 / p.gs_k) * 4;
                float cpal[4] = {0.f, 0.f, 0.f, 0.f};
                if (EPI == EPI_SOFT) {
                    const uint2 praw = __ldg(reinterpret_cast<const uint2*>(p.palette + pg));
                    cpal[0] = __uint_as_float(praw.x << 16);
                    cpal[1] = __uint_as_float(praw.x & 0xFFFF0000u);
                    cpal[2] = __uint_as_float(praw.y << 16);
                    cpal[3] = __uint_as_float(praw.y & 0xFFFF0000u);
                }
                const LogitT* lrow = reinterpret_cast<const LogitT*>(p.logits) + (long long)n * p.ls_row;
                LogitT* drow = p.dlogits ? reinterpret_cast<LogitT*>(p.dlogits) + (long long)n * p.ls_row : nullptr;
                const float* nrow = p.noise ? p.noise + (long long)n * p.ns_row : nullptr;
                const uint8_t* prow = p.packed ? p.packed + (long long)n * p.packed_pitch : nullptr;
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
                for (int c0 = 0; c0 < wcols; c0 += 8) {
                    uint32_t v[8];
                    tmem_ld_32x8(trow + c0, v);
                    const int kb = colbase + c0;  // first k of the batch
                    float l[8][4], g[8][4];
                    uint32_t hard_bits = 0;
                    // ---- phase 1: issue every load of the batch
                    if (EPI == EPI_SOFT) {
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            const bool valid = row_ok && (kb + c) < p.J;
#pragma unroll
                            for (int q = 0; q < 4; ++q) { l[c][q] = 0.f; g[c][q] = 0.f; }
                            if (valid) {
                                const long long lo = (long long)(kb + c) * p.ls_col;
                                if (vec_l) {
                                    const float4 lv = __ldcs(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(lrow) + lo));
                                    l[c][0] = lv.x; l[c][1] = lv.y; l[c][2] = lv.z; l[c][3] = lv.w;
                                } else {
#pragma unroll
                                    for (int q = 0; q < 4; ++q) l[c][q] = to_f32(lrow[lo + q * p.ls_p]);
                                }
                                if (p.noise_mode == NOISE_TENSOR) {
                                    const long long no = (long long)(kb + c) * p.ns_col;
                                    if (vec_n) {
                                        const float4 gv = __ldcs(reinterpret_cast<const float4*>(nrow + no));
                                        g[c][0] = gv.x; g[c][1] = gv.y; g[c][2] = gv.z; g[c][3] = gv.w;
                                    } else {
#pragma unroll
                                        for (int q = 0; q < 4; ++q) g[c][q] = __ldcs(nrow + no + q * p.ns_p);
                                    }
                                }
                            }
                        }
                    } else if (row_ok && kb < p.J) {
                        // 8 consecutive k = 16 bits of the packed row
                        hard_bits = __ldg(reinterpret_cast<const unsigned short*>(prow + (kb >> 2)));
                    }
                    // ---- phase 2: arithmetic and stores
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const bool valid = row_ok && (kb + c) < p.J;
                        const float dw = valid ? __uint_as_float(v[c]) : 0.f;
                        if (EPI == EPI_SOFT) {
                            if (p.noise_mode == NOISE_HASH) {
                                const uint32_t e = ((uint32_t)(kb + c) * (uint32_t)p.hashN + (uint32_t)n) * 4u;
#pragma unroll
                                for (int q = 0; q < 4; ++q) g[c][q] = gumbel_hash(p.seed, e + q);
                            }
                            const Soft4 s4 = soft4(l[c], g[c], cpal, p.inv_tau);
                            float dl[4];
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const float cq = dw * s4.P[q];
                                acc[q] += cq;
                                dl[q] = cq * (cpal[q] - s4.w_soft);
                            }
                            if (valid && drow != nullptr) {
                                const long long lo = (long long)(kb + c) * p.ls_col;
                                if (vec_l) {
                                    __stcs(reinterpret_cast<float4*>(reinterpret_cast<float*>(drow) + lo),
                                           make_float4(dl[0], dl[1], dl[2], dl[3]));
                                } else {
#pragma unroll
                                    for (int q = 0; q < 4; ++q) from_f32(drow[lo + q * p.ls_p], dl[q]);
                                }
                            }
                        } else {
                            const int idx = (hard_bits >> (2 * c)) & 3;
#pragma unroll
                            for (int q = 0; q < 4; ++q) acc[q] += (q == idx) ? dw : 0.f;
                        }
                    }
                }
                if (p.dpalette != nullptr) {
                    if (p.gs_n == 1) {
                        // this thread's row has its own palette: the two column halves add up in either order
                        if (row_ok) {
#pragma unroll
                            for (int q = 0; q < 4; ++q) atomicAdd(p.dpalette + pg + q, acc[q]);
                        }
                    } else {
                        // the whole 128-row tile lies in one palette group: shuffle-reduce, then one add per tile
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float s = warp_sum(acc[q]);
                            if (lane == 0) red[ew * 4 + q] = s;
                        }
                        epi_bar_sync();
                        const int et = threadIdx.x - 64;
                        if (et < 4 && ti * 128 < p.I) {
                            float s = 0.f;
#pragma unroll
                            for (int w8 = 0; w8 < 8; ++w8) s += red[w8 * 4 + et];
                            atomicAdd(p.dpalette + pg - 0 + et, s);
                        }
                        epi_bar_sync();
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) { if (PAIR) mbar_arrive_cluster(lead_acc_empty(buf)); else mbar_arrive(acc_empty(buf)); }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    // PAIR: neither CTA leaves while its partner may still read its shared memory (pair MMA operands), arrive on its
    // barriers or use its tensor memory
    if (PAIR) cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        if (PAIR) tmem_dealloc_pair(tmem_base, 512); else tmem_dealloc(tmem_base, 512);
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------

template <int EPI, typename LogitT, bool ROWS_K, bool PAIR>
static int launch_tn_t(const TnArgs& a, const TnParams& p, const CUtensorMap& tmP, const CUtensorMap& tmQ,
                       const CUtensorMap& tmS0, const CUtensorMap& tmS1, int grid, cudaStream_t stream) {
    auto kern = tn_gemm_kernel<EPI, LogitT, ROWS_K, PAIR>;
    constexpr uint32_t smem = PAIR ? kTnSmemBytesPair : kTnSmemBytes;
    static bool attr_set[64] = {};
    int dev = 0;
    PLZ_CUDA_CHECK(cudaGetDevice(&dev));
    if (!attr_set[dev & 63]) {
        PLZ_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attr_set[dev & 63] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kTnThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (PAIR) {
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
    }
    PLZ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, tmP, tmQ, tmS0, tmS1, p));
    ++g_launch_count;
    return PLZ_OK;
}

int launch_tn_gemm(const TnArgs& a, cudaStream_t stream) {
    if (a.M <= 0 || a.I <= 0 || a.J <= 0) { set_last_error("tn_gemm: empty problem"); return PLZ_ERR_BAD_SHAPE; }
    CUtensorMap tmP, tmQ;
    int rc;
    if ((rc = make_tmap_bf16(&tmP, a.P, a.M, a.I, a.ldp, 64, 64))) return rc;
    if ((rc = make_tmap_bf16(&tmQ, a.Q, a.M, a.J, a.ldq, 64, 64))) return rc;
    TnParams p = {};
    p.M = a.M; p.I = a.I; p.J = a.J;
    p.splits = 1; p.m_chunk = ((a.M + 63) / 64) * 64;
    if (a.epi == EPI_STORE) {
        if (!a.out) { set_last_error("tn_gemm: null output"); return PLZ_ERR_NULL; }
        int s = a.splits > 0 ? a.splits : 1;
        int blocks = (a.M + 63) / 64;
        if (s > blocks) s = blocks;
        p.m_chunk = ((blocks + s - 1) / s) * 64;
        p.splits = (a.M + p.m_chunk - 1) / p.m_chunk;
        p.out = a.out; p.out_si = a.out_si; p.out_sj = a.out_sj; p.alpha = a.alpha;
        p.out_I = a.out_I; p.out_J = a.out_J;
    } else {
        if (!a.palette) { set_last_error("tn_gemm: null palette"); return PLZ_ERR_NULL; }
        if (a.gs_n <= 0 || a.gs_k <= 0) { set_last_error("tn_gemm: bad group sizes"); return PLZ_ERR_BAD_SHAPE; }
        if (a.rows_are_k) {
            // rows of D are input columns k: every weight row n has its own palettes, a 128-row tile lies in one k-group
            if (a.gs_n != 1 || a.gs_k % 128) {
                set_last_error("tn_gemm: rows=k layout needs gs_n == 1 and gs_k %% 128 == 0 (got %d, %d)", a.gs_n, a.gs_k);
                return PLZ_ERR_UNSUPPORTED;
            }
            if (a.epi == EPI_SOFT && (a.logits_f16 || a.ls_p != 1 || (a.noise_mode == NOISE_TENSOR && a.ns_p != 1))) {
                set_last_error("tn_gemm: rows=k layout needs interleaved fp32 logits and noise");
                return PLZ_ERR_UNSUPPORTED;
            }
        } else if ((a.gs_n != 1 && a.gs_n % 128) || (a.gs_k % 256 && a.n_kgroups != 1)) {
            // rows of D are weight rows n: a 128-row tile lies in one n-group (or every row is its own group),
            // and a 256-column tile in one k-group
            set_last_error("tn_gemm: palette groups must be gs_n == 1 or gs_n %% 128 == 0, and gs_k %% 256 == 0 or gs_k == K (got %d, %d)", a.gs_n, a.gs_k);
            return PLZ_ERR_UNSUPPORTED;
        }
        p.logits = a.logits; p.dlogits = a.dlogits;
        p.ls_row = a.ls_row; p.ls_col = a.ls_col; p.ls_p = a.ls_p;
        p.noise = a.noise; p.ns_row = a.ns_row; p.ns_col = a.ns_col; p.ns_p = a.ns_p;
        p.noise_mode = a.noise_mode; p.seed = a.seed; p.hashN = a.hashN;
        p.inv_tau = 1.0f / a.tau;
        p.palette = (const __nv_bfloat16*)a.palette; p.dpalette = a.dpalette;
        p.gs_n = a.gs_n; p.gs_k = a.gs_k; p.n_kgroups = a.n_kgroups;
        p.packed = (const uint8_t*)a.packed; p.packed_pitch = a.packed_pitch;
        if (a.epi == EPI_SOFT) {
            if (!a.logits) { set_last_error("tn_gemm: null logits"); return PLZ_ERR_NULL; }
            if (a.noise_mode == NOISE_TENSOR && !a.noise) { set_last_error("tn_gemm: null noise"); return PLZ_ERR_NULL; }
            if (!(a.tau > 0.f)) { set_last_error("tn_gemm: tau must be positive"); return PLZ_ERR_BAD_SHAPE; }
            if (!a.logits_f16 && a.ls_p == 1) {
                if (((uintptr_t)a.logits & 15) || (a.dlogits && ((uintptr_t)a.dlogits & 15)) || (a.ls_row % 4) || (a.ls_col % 4)) {
                    set_last_error("tn_gemm: interleaved fp32 logits must be 16-byte aligned"); return PLZ_ERR_BAD_ALIGN;
                }
            }
            if (a.noise_mode == NOISE_TENSOR && a.ns_p == 1 && (((uintptr_t)a.noise & 15) || (a.ns_row % 4) || (a.ns_col % 4))) {
                set_last_error("tn_gemm: interleaved noise must be 16-byte aligned"); return PLZ_ERR_BAD_ALIGN;
            }
        } else if (!a.packed) { set_last_error("tn_gemm: null packed indices"); return PLZ_ERR_NULL; }
        if ((uintptr_t)a.palette & 7) { set_last_error("tn_gemm: palette must be 8-byte aligned"); return PLZ_ERR_BAD_ALIGN; }
    }
    p.world = 1; p.rank = 0; p.rows_per_rank = 1; p.shard_elems = 0; p.scatter_add = a.scatter_add;
    for (int r = 0; r < 8; ++r) p.peer_stage[r] = nullptr;
    if (a.world > 1) {
        if (a.epi != EPI_SOFT || !a.rows_are_k || a.world > 8 || a.J % (8 * a.world)) {
            set_last_error("tn_gemm: the fused reduce-scatter needs interleaved fp32 logits, world <= 8 and N %% (8 * world) == 0");
            return PLZ_ERR_UNSUPPORTED;
        }
        p.world = a.world; p.rank = a.rank; p.rows_per_rank = a.J / a.world;
        p.shard_elems = (long long)p.rows_per_rank * a.I * 4;
        p.tj_rot = (int)(((long long)a.rank * ((a.J + 255) / 256)) / a.world);
        for (int r = 0; r < a.world; ++r) {
            if (!a.peer_stage[r] || ((uintptr_t)a.peer_stage[r] & 15)) { set_last_error("tn_gemm: null or misaligned peer staging pointer"); return PLZ_ERR_NULL; }
            p.peer_stage[r] = a.peer_stage[r];
        }
    }
    p.status = device_status_ptr();
    p.prof = (unsigned long long*)a.prof;
    int sms = a.sm_count;
    if (sms <= 0) {
        int dev = 0;
        PLZ_CUDA_CHECK(cudaGetDevice(&dev));
        PLZ_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    }
    if (g_cta_limit > 0 && g_cta_limit < sms) sms = g_cta_limit;
    // CTA pairs (one 256 x 256 tile per two CTAs) for the fused weight-gradient launches; the plain store form and small
    // problems stay on one CTA per 128 x 256 tile
    const bool pair = g_pair_gemm && a.epi != EPI_STORE && a.I >= 256 && a.J >= 256 && sms >= 2;
    const int tiles = (pair ? (a.I + 255) / 256 : (a.I + 127) / 128) * ((a.J + 255) / 256) * p.splits;
    const int units = pair ? sms / 2 : sms;
    const int grid = tiles < units ? tiles : units;   // work units: CTAs, or pairs of CTAs
    p.n_whole = tiles; p.n_items = tiles;
    CUtensorMap tmS0 = tmP, tmS1 = tmP;
    p.n_side_items = 0;
    p.side[0].splits = p.side[1].splits = 0;
    for (int b = 0; b < 2; ++b) {
        if (a.epi == EPI_STORE || !a.side_S[b] || !a.side_out[b] || a.side_rank <= 0) continue;
        if ((rc = make_tmap_bf16(b == 0 ? &tmS0 : &tmS1, a.side_S[b], a.M, a.side_rank, a.side_ld[b], 64, 64))) return rc;
        TnParams::Side& sd = p.side[b];
        sd.q_is_p = a.side_q_is_p[b];
        const int width = sd.q_is_p ? a.I : a.J;
        sd.tiles_j = (width + 255) / 256;
        const int blocks = (a.M + 63) / 64;
        int sp = blocks >= 32 ? 2 : 1;  // two half-length items cost about as much as the half tiles of the last round
        sd.m_chunk = ((blocks + sp - 1) / sp) * 64;
        sd.splits = (a.M + sd.m_chunk - 1) / sd.m_chunk;
        sd.out = a.side_out[b]; sd.out_si = a.side_si[b]; sd.out_sj = a.side_sj[b];
        sd.out_I = a.side_rank; sd.out_J = width;
        if (pair) {   // the pair kernel computes the transposed product: D rows walk the big matrix's columns
            sd.out_si = a.side_sj[b]; sd.out_sj = a.side_si[b];
            sd.out_I = width; sd.out_J = a.side_rank;
        }
    }
    if (a.epi != EPI_STORE) {
        // the last, partially filled round of the persistent schedule is cut into half tiles
        const int rem = tiles % grid;
        if (tiles > grid && rem > 0 && 2 * rem <= grid) { p.n_whole = tiles - rem; p.n_items = p.n_whole + 2 * rem; }
    }
    {
        int next = 0;      // side items are numbered from 0
        for (int b = 0; b < 2; ++b) {
            p.side[b].first_item = next;
            next += p.side[b].splits * p.side[b].tiles_j * (p.side[b].splits > 0 ? 1 : 0);
        }
        p.n_side_items = next;
        if (p.side[0].splits == 0 && p.side[1].splits > 0) {
            // keep job 0 populated so that the item -> job mapping stays a simple threshold
            p.side[0] = p.side[1]; tmS0 = tmS1; p.side[1].splits = 0; p.side[0].first_item = 0;
        }
        const int n_halves = p.n_items - p.n_whole;
        p.tail_free = (n_halves > 0 && n_halves < grid && p.n_side_items > 0) ? grid - n_halves : 0;
        if (p.tail_free > 0) {
            const int full_rounds = p.n_side_items / p.tail_free, rest = p.n_side_items % p.tail_free;
            const int tail_len = full_rounds * grid + (rest > 0 ? n_halves + rest : 0);
            p.n_total = p.n_whole + (tail_len > n_halves ? tail_len : n_halves);
        } else {
            p.n_total = p.n_items + p.n_side_items;
        }
    }
    const int ctas = pair ? 2 * grid : grid;
    switch (a.epi) {
        case EPI_STORE: return launch_tn_t<EPI_STORE, float, false, false>(a, p, tmP, tmQ, tmS0, tmS1, ctas, stream);
        case EPI_HARD:
            if (pair) return a.rows_are_k ? launch_tn_t<EPI_HARD, float, true, true>(a, p, tmP, tmQ, tmS0, tmS1, ctas, stream)
                                          : launch_tn_t<EPI_HARD, float, false, true>(a, p, tmP, tmQ, tmS0, tmS1, ctas, stream);
            return a.rows_are_k ? launch_tn_t<EPI_HARD, float, true, false>(a, p, tmP, tmQ, tmS0, tmS1, ctas, stream)
                                : launch_tn_t<EPI_HARD, float, false, false>(a, p, tmP, tmQ, tmS0, tmS1, ctas, stream);
        case EPI_SOFT:
            if (pair) {
                if (a.rows_are_k) return launch_tn_t<EPI_SOFT, float, true, true>(a, p, tmP, tmQ, tmS0, tmS1, ctas, stream);
                return a.logits_f16 ? launch_tn_t<EPI_SOFT, __half, false, true>(a, p, tmP, tmQ, tmS0, tmS1, ctas, stream)
                                    : launch_tn_t<EPI_SOFT, float, false, true>(a, p, tmP, tmQ, tmS0, tmS1, ctas, stream);
            }
            if (a.rows_are_k) return launch_tn_t<EPI_SOFT, float, true, false>(a, p, tmP, tmQ, tmS0, tmS1, ctas, stream);
            return a.logits_f16 ? launch_tn_t<EPI_SOFT, __half, false, false>(a, p, tmP, tmQ, tmS0, tmS1, ctas, stream)
                                : launch_tn_t<EPI_SOFT, float, false, false>(a, p, tmP, tmQ, tmS0, tmS1, ctas, stream);
    }
    set_last_error("tn_gemm: unknown epilogue %d", a.epi);
    return PLZ_ERR_UNSUPPORTED;
}

}  // namespace plz
