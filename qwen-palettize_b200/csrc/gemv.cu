// Small-M hard forward (token decode): y[M, N] = x[M, K] W^T for M <= 64, bound by the HBM read of the
// packed 2-bit weights (N*K/4 bytes of indices + the palettes), each read exactly once.
//
// One CTA per SM owns a contiguous range of weight rows (any length up to 128, so that N rows split
// evenly over the SMs whatever N is). At entry every thread issues cp.async copies for the CTA's
// whole block of packed indices -- tens of KB in flight per SM, which is what it takes to cover
// HBM latency at full bandwidth -- in one commit group per 256 input columns. As each group lands,
// the decode warps expand it (byte permutes against the 4-entry palettes) into the swizzled A tile of
// a tcgen05 MMA whose B operand is the TMA-loaded activation tile: D[n, m] += W[n, k] x[m, k]
// ("swap-AB": the 128 TMEM lanes are weight rows, the <= 64 columns are tokens). The tensor core
// does the multiply-accumulate for every token at once, so the cost per weight does not grow with M.
//
// Replaces the reference's hard forward at decode batch sizes (scripts/qwen_model.py:164-192 dispatching to
// fused_lut_linear_fwd_tc_kernel, scripts/fused_lut_kernel.cu:309, which reads 1 byte per weight).
#include "plz_launch.h"

namespace plz {

struct GemvParams {
    int M, N, K;
    int mpad;       // 16, 32 or 64: MMA N extent
    const uint8_t* packed; long long packed_pitch;
    const __nv_bfloat16* palette; int gs_n, gs_k, n_kgroups;
    __nv_bfloat16* out; long long ld_out;
    uint32_t idx_bytes;  // shared-memory bytes reserved for the packed block (rows_max * K/4, 16-aligned)
    uint32_t pal_bytes;  // shared-memory bytes reserved for palettes (rows_max * n_kgroups_per_row * 8)
    StatusWord* status;
    unsigned long long* prof;  // optional [gridDim][8] cycle counters of the MMA thread (diagnostics)
};

constexpr int kGvMmaWarps = 4;   // MMA issuers: k-blocks round-robin, two accumulators each
constexpr int kGvDecodeWarps = 16;  // two per ring stage
constexpr int kGvFirstExtraMma = 2 + kGvDecodeWarps;
constexpr int kGvThreads = (2 + kGvDecodeWarps + kGvMmaWarps - 1) * 32;  // warp 0 TMA, warp 1 MMA, 16 decode warps, 3 more MMA issuers
constexpr int kGvStages = 8;                     // decoded-weight ring: one stage per decode warp
constexpr uint32_t kGvXRingBytes = 32 * 1024;   // activation ring (2..8 KB per stage)
constexpr uint32_t kGvABytes = 128 * 64 * 2;
constexpr uint32_t kGvStageBytes = kGvABytes;
constexpr int kGvMaxGroups = 64;  // commit groups (256 input columns each): K <= 16384

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// wait until at most `n` of this thread's most recent commit groups are pending (n runtime, <= 63)
__device__ __forceinline__ void cp_async_wait_pending(int n) {
    switch (n) {
#define PLZ_CASE(i) case i: asm volatile("cp.async.wait_group " #i ";" ::: "memory"); break;
        PLZ_CASE(0) PLZ_CASE(1) PLZ_CASE(2) PLZ_CASE(3) PLZ_CASE(4) PLZ_CASE(5) PLZ_CASE(6) PLZ_CASE(7)
        PLZ_CASE(8) PLZ_CASE(9) PLZ_CASE(10) PLZ_CASE(11) PLZ_CASE(12) PLZ_CASE(13) PLZ_CASE(14) PLZ_CASE(15)
        PLZ_CASE(16) PLZ_CASE(17) PLZ_CASE(18) PLZ_CASE(19) PLZ_CASE(20) PLZ_CASE(21) PLZ_CASE(22) PLZ_CASE(23)
        PLZ_CASE(24) PLZ_CASE(25) PLZ_CASE(26) PLZ_CASE(27) PLZ_CASE(28) PLZ_CASE(29) PLZ_CASE(30) PLZ_CASE(31)
        PLZ_CASE(32) PLZ_CASE(33) PLZ_CASE(34) PLZ_CASE(35) PLZ_CASE(36) PLZ_CASE(37) PLZ_CASE(38) PLZ_CASE(39)
        PLZ_CASE(40) PLZ_CASE(41) PLZ_CASE(42) PLZ_CASE(43) PLZ_CASE(44) PLZ_CASE(45) PLZ_CASE(46) PLZ_CASE(47)
        PLZ_CASE(48) PLZ_CASE(49) PLZ_CASE(50) PLZ_CASE(51) PLZ_CASE(52) PLZ_CASE(53) PLZ_CASE(54) PLZ_CASE(55)
        PLZ_CASE(56) PLZ_CASE(57) PLZ_CASE(58) PLZ_CASE(59) PLZ_CASE(60) PLZ_CASE(61) PLZ_CASE(62) PLZ_CASE(63)
#undef PLZ_CASE
        default: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    }
}

__global__ void __launch_bounds__(kGvThreads, 1)
lut_gemv_kernel(const __grid_constant__ CUtensorMap tmX, const GemvParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    // layout: decoded-weight ring | activation ring | packed block | palettes | barriers
    const uint32_t x_off = kGvStages * kGvStageBytes;
    const uint32_t idx_off = x_off + kGvXRingBytes;
    const uint32_t pal_off = idx_off + p.idx_bytes;
    const uint32_t bar_off = pal_off + p.pal_bytes;
    const uint32_t bar_base = base + bar_off;
    const uint32_t x_stage_bytes = (uint32_t)p.mpad * 128u;
    const int x_stages = (int)(kGvXRingBytes / x_stage_bytes);  // 16, 8 or 4
    auto full_w = [&](int s) { return bar_base + 8u * s; };                       // weights of stage s decoded
    auto empty_w = [&](int s) { return bar_base + 8u * (kGvStages + s); };        // MMAs reading stage s retired
    auto full_x = [&](int s) { return bar_base + 8u * (2 * kGvStages + s); };     // activation tile landed
    auto empty_x = [&](int s) { return bar_base + 8u * (2 * kGvStages + 16 + s); };
    const uint32_t accum_full = bar_base + 8u * (2 * kGvStages + 32);
    const uint32_t grp_ready = bar_base + 8u * (2 * kGvStages + 33);  // all decode threads' copies of a group landed
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + bar_off + 8 * (2 * kGvStages + 34));
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const long long t_entry = PLZ_PROF_ON(p.prof) ? clock64() : 0;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n_begin = (int)(((long long)blockIdx.x * p.N) / gridDim.x);
    const int n_end = (int)(((long long)(blockIdx.x + 1) * p.N) / gridDim.x);
    const int rows = n_end - n_begin;  // <= 128 by construction of the grid
    const int nkb = p.K / 64;
    const int kb_per_grp = 4;          // 256 input columns per commit group
    const int n_grp = (nkb + kb_per_grp - 1) / kb_per_grp;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kGvStages; ++s) {
            mbar_init(full_w(s), kGvDecodeWarps / kGvStages);
            mbar_init(empty_w(s), 1);
        }
        for (int s = 0; s < 16; ++s) {
            mbar_init(full_x(s), 1);
            mbar_init(empty_x(s), 1);
        }
        mbar_init(accum_full, kGvMmaWarps);
        mbar_init(grp_ready, kGvDecodeWarps);
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmX);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void*)tmem_slot), 8u * p.mpad);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (rows > 0) {
        if (warp == 0) {
            // ---------------------------------------------------------- TMA producer: activation tiles
            if (lane == 0) {
                bool ok = true;
                int issued = 0;
                for (int it = 0; it < nkb && ok; ++it) {
                    const int s = it % x_stages;
                    const uint32_t ph = (it / x_stages) & 1;
                    ok = mbar_wait(empty_x(s), ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_EMPTY, 0);
                    if (!ok) break;
                    mbar_arrive_expect_tx(full_x(s), x_stage_bytes);
                    tma_load_2d(base + x_off + s * x_stage_bytes, &tmX, full_x(s), it * 64, 0);
                    issued = it + 1;
                }
                if (!ok) {
                    // give copies already in flight a bounded chance to land before the CTA exits
                    for (int it = (issued > x_stages ? issued - x_stages : 0); it < issued; ++it) {
                        const uint64_t t0 = globaltimer_ns();
                        while (!mbar_try_wait(full_x(it % x_stages), (it / x_stages) & 1)) {
                            if (globaltimer_ns() - t0 > 100000000ull) {
                                report(p.status, ST_TIMEOUT_DRAIN, 0);
                                break;
                            }
                        }
                    }
                }
            }
        } else if (warp == 1 || warp >= kGvFirstExtraMma) {
            // ---------------------------------------------------------- MMA issuers
            // A tcgen05.mma this narrow occupies the tensor pipe for a few tens of cycles but costs its issuing thread
            // far longer, so four warps issue in parallel: issuer q takes the k-blocks q, q + 4, ... and owns the
            // accumulators 2q and 2q + 1 (alternating with the 64-column half of the block).
            const int q = (warp == 1) ? 0 : (warp - kGvFirstExtraMma + 1);
            if (lane == 0) {
                const uint32_t idesc = make_idesc(128, p.mpad, 0, 0);
                bool ok = true;
                long long wait_x = 0, wait_w = 0;
                const long long t_begin = PLZ_PROF_ON(p.prof) ? clock64() : 0;
                for (int it = q; it < nkb && ok; it += kGvMmaWarps) {
                    const int s = it % kGvStages, xs = it % x_stages;
                    const long long c0 = PLZ_PROF_ON(p.prof) ? clock64() : 0;
                    ok = mbar_wait(full_x(xs), (it / x_stages) & 1, abort_flag, p.status, ST_TIMEOUT_FULL, 1);
                    const long long c1 = PLZ_PROF_ON(p.prof) ? clock64() : 0;
                    if (ok) ok = mbar_wait(full_w(s), (it / kGvStages) & 1, abort_flag, p.status, ST_TIMEOUT_FULL, 2);
                    if (PLZ_PROF_ON(p.prof)) { wait_x += c1 - c0; wait_w += clock64() - c1; }
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t sW = base + s * kGvStageBytes;         // decoded weights: MMA operand A
                    const uint32_t sX = base + x_off + xs * x_stage_bytes;  // activations: MMA operand B
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        // A narrow MMA (N = 16..64) retires in a few cycles, but accumulating into the tile the previous
                        // MMA is still writing costs the full TMEM round trip. Eight independent accumulators (four per
                        // block, alternating with the block parity) keep eight chains in flight; the epilogue adds them.
                        const uint32_t acc = (uint32_t)((q * 2 + (ks & 1)) * p.mpad);
                        umma_bf16(tmem_base + acc, make_sdesc(sW + ks * 32u, 16u, 1024u), make_sdesc(sX + ks * 32u, 16u, 1024u),
                                  idesc, (it >= kGvMmaWarps || ks > 1) ? 1u : 0u);
                    }
                    umma_commit(empty_w(s));
                    umma_commit(empty_x(xs));
                }
                if (ok) umma_commit(accum_full);
                if (PLZ_PROF_ON(p.prof) && q == 0) {
                    unsigned long long* q = p.prof + 8ull * blockIdx.x;
                    q[0] = wait_x; q[1] = wait_w; q[2] = clock64() - t_begin; q[3] = t_begin - t_entry;
                }
            }
        } else {
            // ---------------------------------------------------------- decode warps
            const int t = threadIdx.x - 64;
            const int dw = (warp - 2) % kGvStages;  // ring stage of this warp
            const int dh = (warp - 2) / kGvStages;  // which half of the stage's units
            const uint32_t s_idx = base + idx_off;  // [kb][row][16 bytes]
            const uint32_t s_pal = base + pal_off;  // [kgroup][row][8 bytes]
            const int kg_per_row = (p.K + p.gs_k - 1) / p.gs_k;
            // 1) put the whole packed block (and the palettes) in flight
            for (int u = t; u < rows * kg_per_row; u += kGvDecodeWarps * 32) {
                const int r = u % rows, kg = u / rows;
                const long long g = (long long)((n_begin + r) / p.gs_n) * p.n_kgroups + kg;
                cp_async8(s_pal + (uint32_t)(kg * rows + r) * 8u, p.palette + g * 4);
            }
            for (int grp = 0; grp < n_grp; ++grp) {
                const int kb0 = grp * kb_per_grp;
                const int nb = (nkb - kb0 < kb_per_grp) ? (nkb - kb0) : kb_per_grp;
                for (int u = t; u < rows * nb; u += kGvDecodeWarps * 32) {
                    const int r = u / nb, j = u % nb;  // consecutive threads: consecutive 16 bytes of one row
                    cp_async16(s_idx + (uint32_t)((kb0 + j) * rows + r) * 16u,
                               p.packed + (long long)(n_begin + r) * p.packed_pitch + (kb0 + j) * 16);
                }
                cp_async_commit();
            }
            // 2) warp w decodes the 64-column blocks w, w + 8, ... into ring stage w, so eight blocks are in work at once
            bool ok = true;
            const int units = rows * 4;  // (row, 16-column word) per 64-column block
            int grp_done = -1;           // commit groups known to have landed
            for (int it = dw; it < nkb && ok; it += kGvStages) {
                const int grp = it / kb_per_grp;
                while (grp_done < grp && ok) {
                    // every decode warp passes here for every group, in order
                    ++grp_done;
                    cp_async_wait_pending(n_grp - 1 - grp_done);
                    __syncwarp();  // every lane's copies of the group have landed: one arrival per warp
                    if (lane == 0) mbar_arrive(grp_ready);
                    ok = mbar_wait(grp_ready, grp_done & 1, abort_flag, p.status, ST_TIMEOUT_FULL, 5);
                }
                if (!ok) break;
                const int s = dw;
                const uint32_t ph = (it / kGvStages) & 1;
                ok = mbar_wait(empty_w(s), ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_EMPTY, 3);
                if (!ok) break;
                uint8_t* sW = smem + s * kGvStageBytes;
                const int kg = (it * 64) / p.gs_k;
                for (int u = dh * 32 + lane; u < units; u += 64) {
                    const int r = u >> 2, w = u & 3;
                    const uint32_t word = *reinterpret_cast<const uint32_t*>(smem + idx_off + (uint32_t)(it * rows + r) * 16u + w * 4u);
                    const uint2 praw = *reinterpret_cast<const uint2*>(smem + pal_off + (uint32_t)(kg * rows + r) * 8u);
                    const PalRegs pal = pal_split(praw.x, praw.y);
                    uint32_t o[8];
                    decode16(word, pal, o);
                    uint8_t* row = sW + r * 128;
                    *reinterpret_cast<uint4*>(row + (((2 * w) ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<uint4*>(row + (((2 * w + 1) ^ (r & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(full_w(s));
            }
            // groups this warp did not need still have to be passed so that the other warps' barrier completes
            while (grp_done < n_grp - 1 && ok) {
                ++grp_done;
                cp_async_wait_pending(n_grp - 1 - grp_done);
                __syncwarp();
                if (lane == 0) mbar_arrive(grp_ready);
                ok = mbar_wait(grp_ready, grp_done & 1, abort_flag, p.status, ST_TIMEOUT_FULL, 5);
            }
            if (!ok) cp_async_wait_pending(0);
            // 3) epilogue: warps 2..5 cover the 128 TMEM lanes (weight rows); columns are tokens
            if (warp < 6) {
                if (ok) ok = mbar_wait(accum_full, 0, abort_flag, p.status, ST_TIMEOUT_ACCUM, 4);
                if (ok) {
                    tc_fence_after_sync();
                    const int lane_group = warp & 3;
                    const int r = lane_group * 32 + lane;
                    const int n_acc = 2 * (nkb < kGvMmaWarps ? nkb : kGvMmaWarps);  // accumulators that have been written
                    for (int c0 = 0; c0 < p.mpad; c0 += 16) {
                        float sum[16];
#pragma unroll
                        for (int c = 0; c < 16; ++c) sum[c] = 0.f;
                        for (int a = 0; a < n_acc; ++a) {
                            uint32_t v[16];
                            tmem_ld_32x16(tmem_base + ((uint32_t)(lane_group * 32) << 16) + a * p.mpad + c0, v);
#pragma unroll
                            for (int c = 0; c < 16; ++c) sum[c] += __uint_as_float(v[c]);
                        }
                        if (r < rows) {
#pragma unroll
                            for (int c = 0; c < 16; ++c) {
                                const int m = c0 + c;
                                if (m < p.M) p.out[(long long)m * p.ld_out + n_begin + r] = __float2bfloat16_rn(sum[c]);
                            }
                        }
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 8u * p.mpad);
    }
    if (PLZ_PROF_ON(p.prof) && threadIdx.x == 0) p.prof[8ull * blockIdx.x + 4] = clock64() - t_entry;
}

// ---------------------------------------------------------------------------------------------
// M <= 4 (single-token decode): no tensor cores, no barriers. One warp per weight row at a time; the warp reads
// 128 bytes of packed indices (512 weights) per step with one coalesced load, shuffles them so that lane L owns
// bytes L, L+32, L+64, L+96 (its activations are then 16 contiguous bytes per lane: conflict-free float4 reads of
// the fp32 activations staged in shared memory), decodes with the same byte permutes and accumulates in fp32.
// ---------------------------------------------------------------------------------------------
template <int MM>
__global__ void __launch_bounds__(512)
lut_gemv_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int M, int N, int K,
                     const uint8_t* __restrict__ packed, long long pitch, const __nv_bfloat16* __restrict__ palette,
                     int gs_n, int gs_k, int gs_k_shift, int n_kgroups, __nv_bfloat16* __restrict__ out, long long ld_out) {
    extern __shared__ float xs[];  // [MM][K]
    for (int i = threadIdx.x; i < MM * K; i += blockDim.x) {
        const int m = i / K, k = i - m * K;
        xs[i] = (m < M) ? __bfloat162float(x[(long long)m * ldx + k]) : 0.f;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int warps_per_block = blockDim.x >> 5;
    const int gw = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int total_warps = gridDim.x * warps_per_block;
    const int segs = (K + 511) / 512;  // 128-byte segments per row
    for (int n = gw; n < N; n += total_warps) {
        const uint8_t* prow = packed + (long long)n * pitch;
        const __nv_bfloat16* pal_row = palette + (long long)(n / gs_n) * n_kgroups * 4;
        float acc[MM];
#pragma unroll
        for (int m = 0; m < MM; ++m) acc[m] = 0.f;
        uint32_t word = (lane * 16 < K) ? __ldg(reinterpret_cast<const uint32_t*>(prow) + lane) : 0u;
        for (int sg = 0; sg < segs; ++sg) {
            const int k_seg = sg * 512;
            uint32_t next = 0u;
            if (sg + 1 < segs && (k_seg + 512 + lane * 16) < K)
                next = __ldg(reinterpret_cast<const uint32_t*>(prow + (sg + 1) * 128) + lane);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // byte lane + 32 j of the segment lives in word (lane / 4 + 8 j), byte lane % 4
                const uint32_t wj = __shfl_sync(0xFFFFFFFFu, word, (lane >> 2) + 8 * j);
                const uint32_t b = (wj >> (8 * (lane & 3))) & 0xFFu;
                const int k = k_seg + 4 * (lane + 32 * j);
                if (k < K) {
                    const int kg = (gs_k_shift >= 0) ? (k >> gs_k_shift) : (k / gs_k);
                    const uint2 praw = __ldg(reinterpret_cast<const uint2*>(pal_row + kg * 4));
                    // index of weight k + e into byte e, then the selector bytes 0x22 * i + 0x10 (palette bytes 2i, 2i + 1)
                    const uint32_t v = (b & 0x3u) | ((b & 0xCu) << 6) | ((b & 0x30u) << 12) | ((b & 0xC0u) << 18);
                    const uint32_t s = v * 0x22u + 0x10101010u;
                    const uint32_t w01 = prmt_raw(praw.x, praw.y, s), w23 = prmt_raw(praw.x, praw.y, s >> 16);
                    const float w0 = __uint_as_float(w01 << 16), w1 = __uint_as_float(w01 & 0xFFFF0000u);
                    const float w2 = __uint_as_float(w23 << 16), w3 = __uint_as_float(w23 & 0xFFFF0000u);
#pragma unroll
                    for (int m = 0; m < MM; ++m) {
                        const float4 xv = *reinterpret_cast<const float4*>(xs + m * K + k);
                        acc[m] = fmaf(w0, xv.x, acc[m]);
                        acc[m] = fmaf(w1, xv.y, acc[m]);
                        acc[m] = fmaf(w2, xv.z, acc[m]);
                        acc[m] = fmaf(w3, xv.w, acc[m]);
                    }
                }
            }
            word = next;
        }
#pragma unroll
        for (int m = 0; m < MM; ++m) {
            float v = acc[m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
            if (lane == 0 && m < M) out[(long long)m * ld_out + n] = __float2bfloat16_rn(v);
        }
    }
}

template <int MM>
static int launch_rows(const GemvArgs& a, cudaStream_t stream) {
    const size_t smem = (size_t)MM * a.K * sizeof(float);
    auto kern = lut_gemv_rows_kernel<MM>;
    static int attr_smem[64] = {};
    int dev = 0;
    PLZ_CUDA_CHECK(cudaGetDevice(&dev));
    if (smem > 48 * 1024 && attr_smem[dev & 63] < (int)smem) {
        PLZ_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_smem[dev & 63] = (int)smem;
    }
    const int sms = a.sm_count > 0 ? a.sm_count : 1;
    int blocks_per_sm = (int)((200u * 1024u) / (smem + 1024));
    if (blocks_per_sm > 4) blocks_per_sm = 4;
    if (blocks_per_sm < 1) blocks_per_sm = 1;
    int grid = sms * blocks_per_sm;
    const int max_grid = (a.N + 15) / 16;
    if (grid > max_grid) grid = max_grid;
    int shift = -1;
    for (int sh = 0; sh < 31; ++sh) if ((1 << sh) == a.gs_k) shift = sh;
    kern<<<grid, 512, smem, stream>>>((const __nv_bfloat16*)a.x, a.ldx, a.M, a.N, a.K, (const uint8_t*)a.packed,
                                      a.packed_pitch, (const __nv_bfloat16*)a.palette, a.gs_n, a.gs_k, shift, a.K / a.gs_k,
                                      (__nv_bfloat16*)a.out, a.ld_out);
    PLZ_LAUNCH_CHECK();
    return PLZ_OK;
}

int g_debug_smallm_variant = 0;

int launch_lut_gemv(const GemvArgs& a, cudaStream_t stream) {
    if (a.M <= 0 || a.M > 64) { set_last_error("small-M forward handles 1 <= M <= 64 (M=%d)", a.M); return PLZ_ERR_BAD_SHAPE; }
    // up to 16 rows: weights go from registers straight into mma.sync fragments, all loads in flight at once
    if (a.M <= 16 && g_debug_smallm_variant != 1) {
        const int rc = launch_lut_smallm_mma(a, stream);
        if (rc != PLZ_ERR_UNSUPPORTED) return rc;
    }
    // one to four rows, activations fit in shared memory as fp32: the barrier-free CUDA-core kernel is faster
    if (a.M <= 4 && (size_t)a.K * 4 * (a.M <= 1 ? 1 : (a.M <= 2 ? 2 : 4)) <= 160 * 1024 && a.K % 16 == 0 && (a.packed_pitch % 4) == 0) {
        if (a.M <= 1) return launch_rows<1>(a, stream);
        if (a.M <= 2) return launch_rows<2>(a, stream);
        return launch_rows<4>(a, stream);
    }
    if (a.K % 64 || a.K / 256 + 1 > kGvMaxGroups) { set_last_error("small-M forward needs K %% 64 == 0 and K <= 16128 (K=%d)", a.K); return PLZ_ERR_BAD_SHAPE; }
    CUtensorMap tmX;
    const int mpad = a.M <= 16 ? 16 : (a.M <= 32 ? 32 : 64);
    int rc;
    if ((rc = make_tmap_bf16(&tmX, a.x, a.M, a.K, a.ldx, 64, mpad))) return rc;
    // grid: one CTA per SM unless a CTA's packed block would not fit in shared memory or exceed 128 rows
    const int row_bytes = a.K / 4;
    const int kg_per_row = (a.K + a.gs_k - 1) / a.gs_k;
    const uint32_t budget = 227 * 1024 - (kGvStages * kGvStageBytes + kGvXRingBytes + 1024 + 768 + 64);
    int max_rows = (int)(budget / (uint32_t)(row_bytes + kg_per_row * 8));
    if (max_rows > 128) max_rows = 128;
    if (max_rows < 1) { set_last_error("small-M forward: K=%d too large for shared memory", a.K); return PLZ_ERR_TOO_LARGE; }
    int sms = a.sm_count > 0 ? a.sm_count : 1;
    int grid = sms;
    if ((a.N + grid - 1) / grid > max_rows) grid = (a.N + max_rows - 1) / max_rows;
    if (grid > a.N) grid = a.N;
    const int rows_max = (a.N + grid - 1) / grid;
    GemvParams p = {};
    p.M = a.M; p.N = a.N; p.K = a.K; p.mpad = mpad;
    p.packed = (const uint8_t*)a.packed; p.packed_pitch = a.packed_pitch;
    p.palette = (const __nv_bfloat16*)a.palette; p.gs_n = a.gs_n; p.gs_k = a.gs_k; p.n_kgroups = a.K / a.gs_k;
    p.out = (__nv_bfloat16*)a.out; p.ld_out = a.ld_out;
    p.idx_bytes = (uint32_t)(rows_max * row_bytes + 15) & ~15u;
    p.pal_bytes = (uint32_t)(rows_max * kg_per_row * 8 + 15) & ~15u;
    p.status = device_status_ptr();
    p.prof = (unsigned long long*)a.prof;
    const uint32_t smem = kGvStages * kGvStageBytes + kGvXRingBytes + p.idx_bytes + p.pal_bytes + 768 + 1024;
    static int attr_smem[64] = {};
    int dev = 0;
    PLZ_CUDA_CHECK(cudaGetDevice(&dev));
    if (attr_smem[dev & 63] < (int)smem) {
        PLZ_CUDA_CHECK(cudaFuncSetAttribute(lut_gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        attr_smem[dev & 63] = 227 * 1024;
    }
    lut_gemv_kernel<<<grid, kGvThreads, smem, stream>>>(tmX, p);
    PLZ_LAUNCH_CHECK();
    return PLZ_OK;
}

}  // namespace plz
