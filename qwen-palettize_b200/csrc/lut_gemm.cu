// lut_gemm: D[M, J] = alpha * ( A[M, R] * B(R, J) (+ A2[M, R2] * B2(R2, J)) ), bf16 in, fp32 accumulate
// in TMEM, bf16 out, on the sm_100a tensor cores (tcgen05.mma, cta_group::1, 128 x 256 x 16).
//
// A always arrives by TMA (row-major, reduction index contiguous: the activations x or the
// upstream gradient dY). B is the palettized weight matrix W[N, K] and is *produced inside the
// kernel*: sixteen decode warps read the packed 2-bit indices and the 4-entry bf16 palettes from
// global memory and write bf16 tiles straight into the 128-byte-swizzled shared-memory layout the
// tensor core reads, so no decoded weight ever exists in HBM.
//
//   B_DECODE_K   forward     y  = x  * W^T   reduction over K, B tile rows = n (K-major operand)
//   B_DECODE_MN  backward    dX = dY * W     reduction over N, B tile rows = n (MN-major operand)
//   B_TMA_K / B_TMA_MN       same two products with a dense bf16 W (soft weights, LoRA factors)
//
// The optional second product (A2, B2) is one extra 64-wide reduction block appended to the main
// loop: the LoRA branch y += (s x A^T) B^T, or dX += dt A, accumulated into the same TMEM tile.
//
// Persistent: one CTA per SM walks the 256 x 256 output tiles (column tile fastest, so the CTAs that run
// together share the same rows of A in L2). Roles: warp 0 TMA producer, warp 1 MMA issuer, warps 2..17
// decode, warps 18..25 epilogue. While the epilogue warps drain a finished accumulator (TMEM -> bf16 ->
// swizzled shared memory -> TMA store, full 128-byte lines), the producer and decode warps already fill
// the pipeline for the next tile; the MMA resumes as soon as the last tcgen05.ld of the tile has retired.
//
// Replaces, in the reference: fused_lut_linear_fwd_tc_kernel (scripts/fused_lut_kernel.cu:309),
// fused_lut_linear_bwd_grad_x_tc_kernel (:551), the cuBLAS calls of the soft path
// (scripts/fused_lut_linear_cuda.py:912, :944) and the eager LoRA matmuls (scripts/qwen_model.py:300-304).
#include "plz_launch.h"

namespace plz {

int g_cta_limit = 0;  // > 0: persistent kernels use at most this many CTAs (plz_set_cta_limit)

struct LutGemmParams {
    int M, J, R;         // D is [M, J]; R = reduction length of the main product (multiple of 64)
    int n_extra;         // 64-wide reduction blocks taken from (A2, B2): 0 or 1
    int tiles_m, tiles_j;
    int n_whole;         // tiles [0, n_whole) are whole (MT row blocks); the rest of the list are single 128-row blocks
    int n_items;         // length of the tile list
    int mma_n;           // MMA N extent: 256, or the output width rounded up to 16 when it is narrower
    const uint8_t* packed;  // W indices, [Wn, packed_pitch] bytes, 4 per byte along K, LSB first
    long long packed_pitch;
    const __nv_bfloat16* palette;  // [(n / gs_n) * n_kgroups + k / gs_k][4]
    int gs_n, gs_k, n_kgroups;
    int gs_n_shift;      // log2(gs_n) when gs_n is a power of two, else -1
    int Wn, Wk;          // weight matrix extents (N, K)
    float alpha;
    // fused MLP front end (FUSE != 0): optional RMSNorm factors and, for FUSE == 1, a second weight matrix
    const uint8_t* packed2; const __nv_bfloat16* palette2;  // "up" projection, same shape and grouping as the first
    __nv_bfloat16* gate_out; __nv_bfloat16* up_out; long long ld_gu;  // FUSE == 1: optional copies of the two pre-activations
    const __nv_bfloat16* col_scale;  // [K]: norm weight g[k], multiplied into the decoded weights (may be null)
    const float* row_scale;          // [M]: 1 / rms(x[m, :]), applied to the accumulator rows (may be null)
    const __nv_bfloat16* bias;       // FUSE == 2: [J], added in fp32 before the bf16 store (may be null)
    StatusWord* status;
    unsigned long long* prof;  // optional [gridDim][8] cycle counters of the MMA thread (diagnostics)
};

constexpr int kDecodeWarps = 16;
constexpr int kEpiWarps = 8;
constexpr int kDecodeThreads = kDecodeWarps * 32;
constexpr int kFirstEpiWarp = 2 + kDecodeWarps;
constexpr int kThreads = (2 + kDecodeWarps + kEpiWarps) * 32;  // 832
constexpr int kBK = 64;             // reduction elements per stage (128 bytes of bf16)
constexpr int kBN = 256;            // D columns per tile
constexpr uint32_t kBBytes = kBN * kBK * 2;
constexpr uint32_t kEpiStageBytes = 32 * 64 * 2;  // one 32-row x 64-column bf16 box per epilogue warp

// NARROW: dense-B products whose output is at most 64 columns wide (the LoRA projections). Their B stage shrinks to
// one 64 x 64 box, which leaves room for eight stages: these products are bound by streaming A, i.e. by bytes in flight.
template <int MT, bool NARROW>
struct Cfg {
    static constexpr int STAGES = NARROW ? 8 : ((MT == 2) ? 3 : 4);
    static constexpr uint32_t A_BYTES = MT * 128 * kBK * 2;
    static constexpr uint32_t B_BYTES = NARROW ? 64 * kBK * 2 : kBBytes;
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr uint32_t TMEM_COLS = MT * 256;
    static constexpr uint32_t EPI_OFF = STAGES * STAGE_BYTES;
    static constexpr uint32_t BAR_OFF = EPI_OFF + kEpiWarps * kEpiStageBytes;
    static constexpr uint32_t SMEM_BYTES = BAR_OFF + 1024 /*align*/ + 256 /*barriers*/;
};

template <int MT, int BMODE, bool NARROW, int FUSE>
__global__ void __launch_bounds__(kThreads, 1)
lut_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
                const __grid_constant__ CUtensorMap tmD, const LutGemmParams p) {
    using C = Cfg<MT, NARROW>;
    constexpr bool kDecode = (BMODE == B_DECODE_K || BMODE == B_DECODE_MN);
    constexpr bool kBMn = (BMODE == B_DECODE_MN || BMODE == B_TMA_MN);
    constexpr int kIssuers = NARROW ? 4 : 1;  // MMA-issuing warps (see the MMA role below)

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    const uint32_t bar_base = base + C::BAR_OFF;
    auto full_a = [&](int s) { return bar_base + 8u * s; };
    auto full_b = [&](int s) { return bar_base + 8u * (C::STAGES + s); };
    auto empty = [&](int s) { return bar_base + 8u * (2 * C::STAGES + s); };
    const uint32_t accum_full = bar_base + 8u * (3 * C::STAGES);
    const uint32_t tmem_empty = bar_base + 8u * (3 * C::STAGES + 1);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + C::BAR_OFF + 8 * (3 * C::STAGES + 2));
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int nkb = p.R / kBK;
    const int nkb_total = nkb + p.n_extra;
    const int n_tiles = p.n_items;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(full_a(s), 1);
            mbar_init(full_b(s), kDecodeWarps);
            mbar_init(empty(s), 1);
        }
        mbar_init(accum_full, kIssuers);
        mbar_init(tmem_empty, kEpiWarps);
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmD);
        if (!kDecode) tma_prefetch_desc(&tmB);
        if (p.n_extra) {
            tma_prefetch_desc(&tmA2);
            tma_prefetch_desc(&tmB2);
        }
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void*)tmem_slot), C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    // work item t -> (first row, first column, number of 128-row blocks); column tile fastest. The items of the last,
    // partially filled round are cut into single 128-row blocks so that the round costs half as much.
    auto tile_origin = [&](int t, int& m0, int& j0, int& nmt) {
        int tile = t, half = 0;
        nmt = MT;
        if (MT == 2 && t >= p.n_whole) {
            tile = p.n_whole + ((t - p.n_whole) >> 1);
            half = (t - p.n_whole) & 1;
            nmt = 1;
        }
        j0 = (tile % p.tiles_j) * kBN;
        m0 = (tile / p.tiles_j) * (128 * MT) + half * 128;
    };

    if (warp == 0) {
        // ------------------------------------------------------------- TMA producer
        if (lane == 0) {
            int last_fill[C::STAGES];
            for (int s = 0; s < C::STAGES; ++s) last_fill[s] = -1;
            bool ok = true;
            int git = 0;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
                int m0, j0, nmt;
                tile_origin(t, m0, j0, nmt);
                for (int it = 0; it < nkb_total; ++it, ++git) {
                    const int s = git % C::STAGES;
                    const uint32_t ph = (git / C::STAGES) & 1;
                    ok = mbar_wait(empty(s), ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_EMPTY, 0);
                    if (!ok) break;
                    const uint32_t sA = base + s * C::STAGE_BYTES;
                    const uint32_t sB = sA + C::A_BYTES;
                    const bool extra = it >= nkb;
                    const uint32_t bytes = nmt * 16384u + ((extra || !kDecode) ? C::B_BYTES : 0u);
                    mbar_arrive_expect_tx(full_a(s), bytes);
                    const CUtensorMap* ma = extra ? &tmA2 : &tmA;
                    const CUtensorMap* mb = extra ? &tmB2 : &tmB;
                    const int r0 = (extra ? (it - nkb) : it) * kBK;
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
                        if (mt < nmt) tma_load_2d(sA + mt * 16384u, ma, full_a(s), r0, m0 + mt * 128);
                    if (extra || !kDecode) {
                        if (kBMn) {
#pragma unroll
                            for (int q = 0; q < (NARROW ? 1 : 4); ++q) tma_load_2d(sB + q * 8192u, mb, full_a(s), j0 + q * 64, r0);
                        } else {
                            tma_load_2d(sB, mb, full_a(s), r0, j0);
                        }
                    }
                    last_fill[s] = git;
                }
            }
            if (!ok) {
                // give copies already in flight a bounded chance to land before the CTA exits
                for (int s = 0; s < C::STAGES; ++s) {
                    if (last_fill[s] < 0) continue;
                    const uint32_t ph = (last_fill[s] / C::STAGES) & 1;
                    const uint64_t t0 = globaltimer_ns();
                    while (!mbar_try_wait(full_a(s), ph)) {
                        if (globaltimer_ns() - t0 > 100000000ull) {
                            report(p.status, ST_TIMEOUT_DRAIN, 0);
                            break;
                        }
                    }
                }
            }
        }
    } else if (warp == 1 || (kIssuers > 1 && warp < 1 + kIssuers)) {
        // ------------------------------------------------------------- MMA issuer(s)
        // A narrow tcgen05.mma (N <= 64) retires in a few tens of cycles but costs its issuing thread several times
        // that, so for the rank-16/32 products four warps issue in parallel: issuer q takes the blocks q, q + 4, ...
        // and accumulates into its own 64 TMEM columns; the epilogue adds the four partial tiles.
        const int q = warp - 1;
        if (lane == 0) {
            const uint32_t idesc_main = make_idesc(128, p.mma_n, 0, kBMn ? 1 : 0);
            const uint64_t ad0 = make_sdesc(base, 16u, 1024u);
            const uint64_t bd0 = kBMn ? make_sdesc(base + C::A_BYTES, 8192u, 1024u) : make_sdesc(base + C::A_BYTES, 16u, 1024u);
            const uint32_t a_hi = (uint32_t)(ad0 >> 32), b_hi = (uint32_t)(bd0 >> 32);
            const uint32_t a_lo0 = (uint32_t)ad0, b_lo0 = (uint32_t)bd0;
            bool ok = true;
            long long wait_a = 0, wait_b = 0, wait_t = 0;
            const long long t_begin = PLZ_PROF_ON(p.prof) ? clock64() : 0;
            int git = 0, lt = 0;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++lt) {
                int m0, j0, nmt;
                tile_origin(t, m0, j0, nmt);
                if (lt > 0) {
                    // the epilogue warps must have read the previous tile out of TMEM
                    const long long c0 = PLZ_PROF_ON(p.prof) ? clock64() : 0;
                    ok = mbar_wait(tmem_empty, (lt - 1) & 1, abort_flag, p.status, ST_TIMEOUT_ACCUM, 1);
                    if (PLZ_PROF_ON(p.prof)) wait_t += clock64() - c0;
                    if (!ok) break;
                    tc_fence_after_sync();
                }
                for (int it = 0; it < nkb_total; ++it, ++git) {
                    if (kIssuers > 1 && (it % kIssuers) != q) continue;
                    const int s = git % C::STAGES;
                    const uint32_t ph = (git / C::STAGES) & 1;
                    const bool extra = it >= nkb;
                    const long long c0 = PLZ_PROF_ON(p.prof) ? clock64() : 0;
                    ok = mbar_wait(full_a(s), ph, abort_flag, p.status, ST_TIMEOUT_FULL, 1);
                    const long long c1 = PLZ_PROF_ON(p.prof) ? clock64() : 0;
                    if (ok && kDecode && !extra)
                        ok = mbar_wait(full_b(s), ph, abort_flag, p.status, ST_TIMEOUT_FULL, 2);
                    if (PLZ_PROF_ON(p.prof)) { wait_a += c1 - c0; wait_b += clock64() - c1; }
                    if (!ok) break;
                    tc_fence_after_sync();
                    // precomputed descriptor words: only the low word moves (stage base, then a constant per k step)
                    const uint32_t a_lo = a_lo0 + (uint32_t)s * (C::STAGE_BYTES >> 4);
                    const uint32_t b_lo = b_lo0 + (uint32_t)s * (C::STAGE_BYTES >> 4);
                    const uint32_t acc0 = (it >= kIssuers) ? 1u : 0u;
#pragma unroll
                    for (int ks = 0; ks < kBK / 16; ++ks) {
                        const uint32_t offb = kBMn ? (uint32_t)(ks * 128) : (uint32_t)(ks * 2);
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            if (mt >= nmt) break;
                            umma_bf16_words<1>(tmem_base + mt * 256u + (kIssuers > 1 ? q * 64u : 0u), a_lo + (uint32_t)(mt * 1024 + ks * 2), a_hi,
                                               b_lo + offb, b_hi, idesc_main, (ks > 0) ? 1u : acc0);
                        }
                    }
                    umma_commit(empty(s));
                }
                if (ok) umma_commit(accum_full);
            }
            if (PLZ_PROF_ON(p.prof) && q == 0) {
                unsigned long long* q = p.prof + 8ull * blockIdx.x;
                q[0] = wait_a; q[1] = wait_b; q[2] = wait_t; q[3] = clock64() - t_begin; q[4] = lt;
            }
        }
    } else if (warp < kFirstEpiWarp) {
        // ------------------------------------------------------------- decode warps (idle in the dense-B modes)
        if (kDecode) {
            // Each of the 512 decode threads produces 32 weights (four 16-byte chunks of one 128-byte operand row)
            // per stage from 8 bytes of packed indices.
            // forward:  row = tile row n - j0 = t / 2, chunks 4*(t%2)..; k runs with the stage.
            // backward: 64-wide k block a = t / 128, row = n - it*64 = (t % 128) / 2, chunks 4*(t%2)..; n runs with the stage.
            const int t = threadIdx.x - 64;
            // In both mappings eight consecutive lanes cover four rows x two halves of ONE 64-wide block, so that
            // their 16-byte stores land on eight different swizzled chunk positions (a 128-bit store is served a
            // quarter warp at a time; with one row per quarter warp it would be a 4-way bank conflict).
            const int h = t & 1;
            const int rr = (BMODE == B_DECODE_K) ? (t >> 1) : ((t & 127) >> 1);
            const int a = t >> 7;
            const int blocks_per_kgroup = p.gs_k / kBK;
            bool ok = true;
            int git = 0;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                int m0, j0, nmt;
                tile_origin(tile, m0, j0, nmt);
                const int k_fixed = j0 + a * 64 + h * 32;  // backward only
                // FUSE == 1: the 256 tile rows are 128 rows of the gate matrix followed by the same 128 rows of the up matrix
                const int n_fused = (j0 >> 1) + (rr & 127);
                const uint8_t* packed_src = (FUSE == 1 && rr >= 128) ? p.packed2 : p.packed;
                const __nv_bfloat16* palette_src = (FUSE == 1 && rr >= 128) ? p.palette2 : p.palette;
                auto src_n = [&](int it) { return (BMODE == B_DECODE_K) ? (FUSE == 1 ? n_fused : (j0 + rr)) : (it * kBK + rr); };
                auto src_k = [&](int it) { return (BMODE == B_DECODE_K) ? (it * kBK + h * 32) : k_fixed; };
                auto in_range = [&](int it) { return it < nkb && src_n(it) < p.Wn && src_k(it) < p.Wk; };
                auto load_idx = [&](int it) -> uint2 {
                    if (!in_range(it)) return make_uint2(0, 0);
                    return __ldg(reinterpret_cast<const uint2*>(packed_src + (long long)src_n(it) * p.packed_pitch +
                                                                (src_k(it) >> 2)));
                };
                // palette group of the stage: one of (n / gs_n, k / gs_k) is fixed per thread, the other advances
                const int ng_fixed = (BMODE == B_DECODE_K) ? ((FUSE == 1 ? n_fused : (j0 + rr)) / p.gs_n) : 0;
                const int kg_fixed = (BMODE == B_DECODE_K) ? 0 : (k_fixed / p.gs_k);
                // kg = k group of stage `it` (forward only), carried incrementally to keep divisions out of the loop
                auto load_pal = [&](int it, int kg) -> uint2 {
                    if (!in_range(it)) return make_uint2(0, 0);
                    long long g;
                    if (BMODE == B_DECODE_K) g = (long long)ng_fixed * p.n_kgroups + kg;
                    else g = (long long)((p.gs_n_shift >= 0) ? ((it * kBK + rr) >> p.gs_n_shift) : ((it * kBK + rr) / p.gs_n)) * p.n_kgroups + kg_fixed;
                    return __ldg(reinterpret_cast<const uint2*>(palette_src + g * 4));
                };
                int pf_kg = 0, pf_cnt = 0;  // k group and position inside it of the next stage to prefetch
                auto advance_kg = [&]() { if (++pf_cnt == blocks_per_kgroup) { pf_cnt = 0; ++pf_kg; } };
                // software prefetch kPF stages ahead: the index / palette loads come from L2 or HBM and one stage
                // of MMA work (about a thousand cycles) does not cover their latency
                constexpr int kPF = 4;
                uint2 idx_q[kPF], pal_q[kPF];
#pragma unroll
                for (int j = 0; j < kPF; ++j) { idx_q[j] = load_idx(j); pal_q[j] = load_pal(j, pf_kg); advance_kg(); }
                for (int it = 0; it < nkb_total; ++it, ++git) {
                    const int s = git % C::STAGES;
                    const uint32_t ph = (git / C::STAGES) & 1;
                    if (it >= nkb) {
                        // the extra (LoRA) block is filled by TMA; arrive all the same (after the stage is free, like
                        // any other use of it) so that this barrier's phase keeps step with the ring position
                        ok = mbar_wait(empty(s), ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_EMPTY, 3);
                        if (!ok) break;
                        if (lane == 0) mbar_arrive(full_b(s));
                        continue;
                    }
                    const uint2 idx_cur = idx_q[0], pal_cur = pal_q[0];
#pragma unroll
                    for (int j = 0; j + 1 < kPF; ++j) { idx_q[j] = idx_q[j + 1]; pal_q[j] = pal_q[j + 1]; }
                    idx_q[kPF - 1] = load_idx(it + kPF);
                    pal_q[kPF - 1] = load_pal(it + kPF, pf_kg);
                    advance_kg();
                    ok = mbar_wait(empty(s), ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_EMPTY, 3);
                    if (!ok) break;
                    uint8_t* sB = smem + s * C::STAGE_BYTES + C::A_BYTES;
                    uint8_t* row = (BMODE == B_DECODE_K) ? (sB + rr * 128) : (sB + a * 8192 + rr * 128);
                    const PalRegs pal = pal_split(pal_cur.x, pal_cur.y);
                    const uint32_t w[2] = {idx_cur.x, idx_cur.y};
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        uint32_t o[8];
                        decode16(w[i], pal, o);
                        if (FUSE != 0 && p.col_scale != nullptr) {
                            // RMSNorm weight folded into the operand: W[n, k] * g[k] (one bf16 rounding)
                            const uint4* gp = reinterpret_cast<const uint4*>(p.col_scale + it * kBK + h * 32 + i * 16);
                            const uint4 g0 = __ldg(gp), g1 = __ldg(gp + 1);
                            const uint32_t gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const __nv_bfloat162 prod = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&o[j]),
                                                                    *reinterpret_cast<const __nv_bfloat162*>(&gg[j]));
                                o[j] = *reinterpret_cast<const uint32_t*>(&prod);
                            }
                        }
                        // word i covers 16 elements = 16-byte chunks 4h + 2i and 4h + 2i + 1 of the 128-byte row
                        *reinterpret_cast<uint4*>(row + (((4 * h + 2 * i) ^ (rr & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                        *reinterpret_cast<uint4*>(row + (((4 * h + 2 * i + 1) ^ (rr & 7)) << 4)) =
                            make_uint4(o[4], o[5], o[6], o[7]);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(full_b(s));
                }
            }
        }
    } else {
        // ------------------------------------------------------------- epilogue warps
        // warp e reads TMEM lanes 32*(warp%4).. (its 32 output rows) and one half of the 256 columns, 64 columns
        // at a time: fp32 -> bf16 -> 128-byte-swizzled box in shared memory -> TMA store (clipped at M and J).
        const int e = warp - kFirstEpiWarp;
        const int lane_group = warp & 3;
        const int col_half = e >> 2;
        uint8_t* stage = smem + C::EPI_OFF + e * kEpiStageBytes;
        const uint32_t stage_u32 = base + C::EPI_OFF + e * kEpiStageBytes;
        bool ok = true;
        int lt = 0;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++lt) {
            int m0, j0, nmt;
            tile_origin(t, m0, j0, nmt);
            ok = mbar_wait(accum_full, lt & 1, abort_flag, p.status, ST_TIMEOUT_ACCUM, 4);
            if (!ok) break;
            tc_fence_after_sync();
            if (FUSE == 1) {
                // SwiGLU: accumulator columns [0,128) hold the gate product, [128,256) the up product of the same 128
                // output columns; this warp writes out[:, n0 + 64*col_half .. +64) = silu(s*gate) * (s*up).
                const int n0 = j0 >> 1;
#pragma unroll 1
                for (int mt = 0; mt < nmt; ++mt) {
                    const int m = m0 + mt * 128 + lane_group * 32 + lane;
                    const float rs = (p.row_scale != nullptr && m < p.M) ? __ldg(p.row_scale + m) : 1.0f;
                    if (lane == 0) tma_store_wait_read();
                    __syncwarp();
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t vg[16], vu[16];
                        const uint32_t ta = tmem_base + ((uint32_t)(lane_group * 32) << 16) + mt * 256u + col_half * 64 + c * 16;
                        tmem_ld_32x16(ta, vg);
                        tmem_ld_32x16(ta + 128u, vu);
                        if (mt == nmt - 1 && c == 3) {
                            tc_fence_before_sync();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(tmem_empty);
                        }
                        uint32_t o[8];
                        if (p.gate_out != nullptr && m < p.M) {
                            // keep rs * gate and rs * up (bf16) for the backward: 32 contiguous bytes of this thread's row each
                            const int n = n0 + col_half * 64 + c * 16;
                            if (n < p.Wn) {
                                uint32_t kg[8], ku[8];
#pragma unroll
                                for (int i = 0; i < 8; ++i) {
                                    kg[i] = pack_bf16x2(__uint_as_float(vg[2 * i]) * rs, __uint_as_float(vg[2 * i + 1]) * rs);
                                    ku[i] = pack_bf16x2(__uint_as_float(vu[2 * i]) * rs, __uint_as_float(vu[2 * i + 1]) * rs);
                                }
                                uint4* dg = reinterpret_cast<uint4*>(p.gate_out + (long long)m * p.ld_gu + n);
                                uint4* du = reinterpret_cast<uint4*>(p.up_out + (long long)m * p.ld_gu + n);
                                dg[0] = make_uint4(kg[0], kg[1], kg[2], kg[3]); dg[1] = make_uint4(kg[4], kg[5], kg[6], kg[7]);
                                du[0] = make_uint4(ku[0], ku[1], ku[2], ku[3]); du[1] = make_uint4(ku[4], ku[5], ku[6], ku[7]);
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            float a0 = __uint_as_float(vg[2 * i]) * rs, a1 = __uint_as_float(vg[2 * i + 1]) * rs;
                            a0 = __fdividef(a0, 1.0f + __expf(-a0));
                            a1 = __fdividef(a1, 1.0f + __expf(-a1));
                            o[i] = pack_bf16x2(a0 * (__uint_as_float(vu[2 * i]) * rs), a1 * (__uint_as_float(vu[2 * i + 1]) * rs));
                        }
                        *reinterpret_cast<uint4*>(stage + swz128(lane, c * 2)) = make_uint4(o[0], o[1], o[2], o[3]);
                        *reinterpret_cast<uint4*>(stage + swz128(lane, c * 2 + 1)) = make_uint4(o[4], o[5], o[6], o[7]);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && n0 + col_half * 64 < p.J && m0 + mt * 128 + lane_group * 32 < p.M) {
                        tma_store_2d(&tmD, stage_u32, n0 + col_half * 64, m0 + mt * 128 + lane_group * 32);
                        tma_store_commit();
                    }
                }
                continue;
            }
#pragma unroll 1
            for (int mt = 0; mt < nmt; ++mt) {
                float rs = 1.0f;
                if (FUSE == 2 && p.row_scale != nullptr) {
                    const int m = m0 + mt * 128 + lane_group * 32 + lane;
                    if (m < p.M) rs = __ldg(p.row_scale + m);
                }
                const float scale = p.alpha * rs;
#pragma unroll 1
                for (int b = 0; b < 2; ++b) {
                    const int col = col_half * 128 + b * 64;
                    // the previous box must have been read out of the staging buffer
                    if (lane == 0) tma_store_wait_read();
                    __syncwarp();
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        uint32_t v[32];
                        tmem_ld_32x32(tmem_base + ((uint32_t)(lane_group * 32) << 16) + mt * 256u + col + c * 32, v);
                        if (NARROW && col == 0) {
                            // the four issuers' partial tiles sit 64 columns apart
                            const int used = nkb_total < kIssuers ? nkb_total : kIssuers;
                            for (int qq = 1; qq < used; ++qq) {
#pragma unroll
                                for (int hh = 0; hh < 2; ++hh) {
                                    uint32_t u[16];
                                    tmem_ld_32x16(tmem_base + ((uint32_t)(lane_group * 32) << 16) + qq * 64u + c * 32 + hh * 16, u);
#pragma unroll
                                    for (int i = 0; i < 16; ++i)
                                        v[hh * 16 + i] = __float_as_uint(__uint_as_float(v[hh * 16 + i]) + __uint_as_float(u[i]));
                                }
                            }
                        }
                        if (mt == nmt - 1 && b == 1 && c == 1) {
                            // last read of this tile's accumulators: hand TMEM back to the MMA warp
                            tc_fence_before_sync();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(tmem_empty);
                        }
                        if (FUSE == 2 && p.bias != nullptr) {
                            // bias in fp32 before the rounding (scripts/fused_lut_kernel.cu:512-514); columns past J are
                            // clipped by the TMA store, so only the loads need the bound
                            const int jc = j0 + col + c * 32;
#pragma unroll
                            for (int g = 0; g < 4; ++g) {
                                uint4 bb = make_uint4(0u, 0u, 0u, 0u);
                                if (jc + g * 8 < p.J) bb = __ldg(reinterpret_cast<const uint4*>(p.bias + jc + g * 8));
                                const uint32_t bw[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    v[g * 8 + 2 * i] = __float_as_uint(__uint_as_float(v[g * 8 + 2 * i]) * scale + __uint_as_float(bw[i] << 16));
                                    v[g * 8 + 2 * i + 1] = __float_as_uint(__uint_as_float(v[g * 8 + 2 * i + 1]) * scale + __uint_as_float(bw[i] & 0xFFFF0000u));
                                }
                            }
#pragma unroll
                            for (int g = 0; g < 4; ++g) {
                                uint4 o;
                                o.x = pack_bf16x2(__uint_as_float(v[g * 8 + 0]), __uint_as_float(v[g * 8 + 1]));
                                o.y = pack_bf16x2(__uint_as_float(v[g * 8 + 2]), __uint_as_float(v[g * 8 + 3]));
                                o.z = pack_bf16x2(__uint_as_float(v[g * 8 + 4]), __uint_as_float(v[g * 8 + 5]));
                                o.w = pack_bf16x2(__uint_as_float(v[g * 8 + 6]), __uint_as_float(v[g * 8 + 7]));
                                *reinterpret_cast<uint4*>(stage + swz128(lane, c * 4 + g)) = o;
                            }
                            continue;
                        }
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            uint4 o;
                            o.x = pack_bf16x2(__uint_as_float(v[g * 8 + 0]) * scale, __uint_as_float(v[g * 8 + 1]) * scale);
                            o.y = pack_bf16x2(__uint_as_float(v[g * 8 + 2]) * scale, __uint_as_float(v[g * 8 + 3]) * scale);
                            o.z = pack_bf16x2(__uint_as_float(v[g * 8 + 4]) * scale, __uint_as_float(v[g * 8 + 5]) * scale);
                            o.w = pack_bf16x2(__uint_as_float(v[g * 8 + 6]) * scale, __uint_as_float(v[g * 8 + 7]) * scale);
                            *reinterpret_cast<uint4*>(stage + swz128(lane, c * 4 + g)) = o;
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && j0 + col < p.J && m0 + mt * 128 + lane_group * 32 < p.M) {
                        tma_store_2d(&tmD, stage_u32, j0 + col, m0 + mt * 128 + lane_group * 32);
                        tma_store_commit();
                    }
                }
            }
        }
        if (lane == 0) tma_store_wait_all();
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------

template <int MT, int BMODE, bool NARROW, int FUSE = 0>
static int launch_t(const LutGemmArgs& a, cudaStream_t stream) {
    using C = Cfg<MT, NARROW>;
    CUtensorMap tmA, tmB, tmA2, tmB2, tmD;
    int rc;
    if ((rc = make_tmap_bf16(&tmA, a.A, a.M, a.R, a.lda, 64, 128))) return rc;
    tmB = tmA; tmA2 = tmA; tmB2 = tmA;
    constexpr bool kMn = (BMODE == B_DECODE_MN || BMODE == B_TMA_MN);
    if (BMODE == B_TMA_K) {
        if ((rc = make_tmap_bf16(&tmB, a.Bdense, a.J, a.R, a.ldb, 64, NARROW ? 64 : 256))) return rc;
    } else if (BMODE == B_TMA_MN) {
        if ((rc = make_tmap_bf16(&tmB, a.Bdense, a.R, a.J, a.ldb, 64, 64))) return rc;
    }
    if (a.r2 > 0) {
        if ((rc = make_tmap_bf16(&tmA2, a.A2, a.M, a.r2, a.lda2, 64, 128))) return rc;
        if (kMn) {
            if ((rc = make_tmap_bf16(&tmB2, a.B2, a.r2, a.J, a.ldb2, 64, 64))) return rc;
        } else {
            if ((rc = make_tmap_bf16(&tmB2, a.B2, a.J, a.r2, a.ldb2, 64, 256))) return rc;
        }
    }
    const int out_cols = (FUSE == 1) ? a.J / 2 : a.J;  // the SwiGLU form writes one column per gate/up pair
    if ((rc = make_tmap_bf16(&tmD, a.out, a.M, out_cols, a.ld_out, 64, 32))) return rc;
    LutGemmParams p;
    p.M = a.M; p.J = out_cols; p.R = a.R; p.n_extra = a.r2 > 0 ? 1 : 0;
    p.tiles_j = (a.J + kBN - 1) / kBN;
    p.tiles_m = (a.M + 128 * MT - 1) / (128 * MT);
    p.packed = (const uint8_t*)a.packed; p.packed_pitch = a.packed_pitch;
    p.palette = (const __nv_bfloat16*)a.palette;
    p.gs_n = a.gs_n > 0 ? a.gs_n : 1; p.gs_k = a.gs_k > 0 ? a.gs_k : kBK;
    p.n_kgroups = a.gs_k > 0 ? (a.Wk / a.gs_k) : 1;
    p.gs_n_shift = -1;
    for (int sh = 0; sh < 31; ++sh) if ((1 << sh) == p.gs_n) p.gs_n_shift = sh;
    p.Wn = a.Wn; p.Wk = a.Wk;
    p.alpha = a.alpha;
    p.packed2 = (const uint8_t*)a.packed2; p.palette2 = (const __nv_bfloat16*)a.palette2;
    p.gate_out = (__nv_bfloat16*)a.gate_out; p.up_out = (__nv_bfloat16*)a.up_out; p.ld_gu = a.ld_gu;
    p.col_scale = (const __nv_bfloat16*)a.col_scale; p.row_scale = a.row_scale;
    p.bias = (const __nv_bfloat16*)a.bias;
    p.status = device_status_ptr();
    p.prof = (unsigned long long*)a.prof;
    auto kern = lut_gemm_kernel<MT, BMODE, NARROW, FUSE>;
    static bool attr_set[64] = {};
    int dev = 0, sms = 0;
    PLZ_CUDA_CHECK(cudaGetDevice(&dev));
    if (!attr_set[dev & 63]) {
        PLZ_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
        attr_set[dev & 63] = true;
    }
    PLZ_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (a.sm_limit > 0 && a.sm_limit < sms) sms = a.sm_limit;
    if (g_cta_limit > 0 && g_cta_limit < sms) sms = g_cta_limit;
    const int tiles = p.tiles_m * p.tiles_j;
    const int grid = tiles < sms ? tiles : sms;
    p.n_whole = tiles; p.n_items = tiles;
    p.mma_n = (a.J >= kBN) ? kBN : ((a.J + 15) / 16) * 16;
    if (MT == 2) {
        const int rem = tiles % grid;
        if (tiles > grid && rem > 0 && 2 * rem <= grid) { p.n_whole = tiles - rem; p.n_items = p.n_whole + 2 * rem; }
    }
    kern<<<grid, kThreads, C::SMEM_BYTES, stream>>>(tmA, tmB, tmA2, tmB2, tmD, p);
    PLZ_LAUNCH_CHECK();
    return PLZ_OK;
}

int launch_lut_gemm(const LutGemmArgs& a, cudaStream_t stream) {
    if (a.M <= 0 || a.J <= 0 || a.R <= 0) { set_last_error("lut_gemm: empty problem"); return PLZ_ERR_BAD_SHAPE; }
    if (a.R % kBK) { set_last_error("lut_gemm: reduction length %d is not a multiple of 64", a.R); return PLZ_ERR_BAD_SHAPE; }
    if (a.J % 8) { set_last_error("lut_gemm: output width %d is not a multiple of 8", a.J); return PLZ_ERR_BAD_SHAPE; }
    if (a.r2 < 0 || a.r2 > 64 || (a.r2 % 8)) { set_last_error("lut_gemm: extra rank %d must be a multiple of 8 in [0, 64]", a.r2); return PLZ_ERR_BAD_SHAPE; }
    if (((uintptr_t)a.out & 15) || ((a.ld_out * 2) & 15)) { set_last_error("lut_gemm: output must be 16-byte aligned"); return PLZ_ERR_BAD_ALIGN; }
    const bool decode = (a.bmode == B_DECODE_K || a.bmode == B_DECODE_MN);
    if (decode) {
        if (!a.packed || !a.palette) { set_last_error("lut_gemm: null packed weights"); return PLZ_ERR_NULL; }
        if (((uintptr_t)a.packed & 15) || (a.packed_pitch & 15)) { set_last_error("lut_gemm: packed index rows must be 16-byte aligned"); return PLZ_ERR_BAD_ALIGN; }
        if ((uintptr_t)a.palette & 7) { set_last_error("lut_gemm: palette must be 8-byte aligned"); return PLZ_ERR_BAD_ALIGN; }
        if (a.gs_k % 64 || a.Wk % a.gs_k || a.Wk % 64) { set_last_error("lut_gemm: K group size %d must be a multiple of 64 dividing K=%d", a.gs_k, a.Wk); return PLZ_ERR_BAD_SHAPE; }
    }
    if (decode && a.fuse == 0) {
        // the large products run on CTA pairs (lut_gemm_pair.cu); everything else, and shapes it declines, stays here
        const int rc = launch_lut_gemm_pair(a, stream);
        if (rc != PLZ_ERR_UNSUPPORTED) return rc;
    }
    // narrow outputs (the rank-16/32 LoRA products) are bound by streaming A: 128-row tiles give twice the CTAs
    const bool big = a.M > 128 && a.J > 64;
    const bool narrow = !decode && a.J <= 64 && a.r2 == 0;
    switch (a.bmode) {
        case B_DECODE_K:
            if (a.fuse == 1) return big ? launch_t<2, B_DECODE_K, false, 1>(a, stream) : launch_t<1, B_DECODE_K, false, 1>(a, stream);
            if (a.fuse == 2) return big ? launch_t<2, B_DECODE_K, false, 2>(a, stream) : launch_t<1, B_DECODE_K, false, 2>(a, stream);
            return big ? launch_t<2, B_DECODE_K, false>(a, stream) : launch_t<1, B_DECODE_K, false>(a, stream);
        case B_DECODE_MN: return big ? launch_t<2, B_DECODE_MN, false>(a, stream) : launch_t<1, B_DECODE_MN, false>(a, stream);
        case B_TMA_K:
            if (narrow) return launch_t<1, B_TMA_K, true>(a, stream);
            return big ? launch_t<2, B_TMA_K, false>(a, stream) : launch_t<1, B_TMA_K, false>(a, stream);
        case B_TMA_MN:
            if (narrow) return launch_t<1, B_TMA_MN, true>(a, stream);
            return big ? launch_t<2, B_TMA_MN, false>(a, stream) : launch_t<1, B_TMA_MN, false>(a, stream);
    }
    set_last_error("lut_gemm: unknown B mode %d", a.bmode);
    return PLZ_ERR_UNSUPPORTED;
}

}  // namespace plz
