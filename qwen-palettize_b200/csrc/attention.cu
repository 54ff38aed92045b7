// Causal grouped-query attention, forward and backward, for the decoder layers around the palettized Linears
// (head_dim 128, tokens-major activations: q [B*S, Hq*128], k / v [B*S, Hkv*128], exactly what the q/k/v projections
// write and what o_proj reads, so nothing is transposed).
//
// The reference has no attention code of its own: it trains through the HuggingFace decoder layer
// (scripts/train_qwen.py:1259-1266) with SDPA selected at scripts/qwen_model.py:454. Semantics follow
// transformers' Qwen3Attention: softmax(q k^T / sqrt(d) + causal mask) v, fp32 softmax, bf16 operands.
//
// All products run on the 5th-generation tensor cores (tcgen05.mma, 128 x 128 x 16, accumulators in TMEM), operands
// staged by TMA in 128-byte-swizzled tiles. One CTA handles one (batch, head) and one or two 128-token tiles:
//   forward        two neighbouring query tiles per CTA: S = Q K^T -> online softmax by 128 threads per tile (one row each,
//                  TMEM -> registers) -> P (bf16) to shared memory -> O += P V, O rescaled in TMEM when a row maximum grows;
//                  the softmax of one tile runs under the MMAs of the other; also writes the row log-sum-exp.
//   backward dQ    per q tile: S, dP = dO V^T -> dS = P (dP - D) / sqrt(d) -> dQ += dS K
//   backward dKdV  per kv tile and kv head, over the q heads of the group and the q tiles at or after it:
//                  S, dP -> P, dS to shared memory -> dV += P^T dO, dK += dS^T Q  (P^T / dS^T are the same bytes read
//                  through an MN-major operand descriptor)
// D[row] = sum_d dO O is a small pre-pass. Every barrier wait is bounded (status word, as in the GEMM kernels).
#include "plz_launch.h"

namespace plz {
namespace {

constexpr int kT = 128;                         // tokens per tile
constexpr int kD = 128;                         // head dimension
constexpr uint32_t kBlk = kT * 64 * 2;          // one 64-column block of a 128-row bf16 tile: 16 KB
constexpr uint32_t kTile = 2 * kBlk;            // a 128 x 128 bf16 tile: 32 KB
constexpr float kLog2e = 1.4426950408889634f;

struct AttnParams {
    int B, S, Hq, Hkv;
    float scale;          // 1 / sqrt(head_dim)
    float* lse;           // [B, Hq, S] natural-log sum-exp of the scaled scores
    const float* dsum;    // [B, Hq, S] sum_d dO * O (backward)
    StatusWord* status;
};

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n\t"
        "tcgen05.wait::st.sync.aligned;"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
          "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
          "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void bar_sync_128() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// eight MMAs of one 128 x 128 x 128 product. A / B tiles are 128-row bf16 tiles of two 64-column blocks.
//   K-major operand (rows = M or N index, reduction along the 128-byte row):  step ks -> block ks / 4, 32 bytes * (ks % 4)
//   MN-major operand (rows = reduction index, M or N along the row): step ks -> 16 rows = 2048 bytes, blocks 16 KB apart
__device__ __forceinline__ void mma_128(uint32_t d_tmem, uint32_t sA, bool a_mn, uint32_t sB, bool b_mn, bool accumulate) {
    const uint32_t idesc = make_idesc(128, 128, a_mn ? 1 : 0, b_mn ? 1 : 0);
    const uint64_t ad0 = a_mn ? make_sdesc(sA, kBlk, 1024u) : make_sdesc(sA, 16u, 1024u);
    const uint64_t bd0 = b_mn ? make_sdesc(sB, kBlk, 1024u) : make_sdesc(sB, 16u, 1024u);
    const uint32_t a_hi = (uint32_t)(ad0 >> 32), b_hi = (uint32_t)(bd0 >> 32), a_lo = (uint32_t)ad0, b_lo = (uint32_t)bd0;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        const uint32_t off_k = (uint32_t)((ks >> 2) * (kBlk >> 4) + (ks & 3) * 2);
        const uint32_t off_mn = (uint32_t)(ks * 128);
        umma_bf16_words<1>(d_tmem, a_lo + (a_mn ? off_mn : off_k), a_hi, b_lo + (b_mn ? off_mn : off_k), b_hi, idesc,
                           (ks > 0 || accumulate) ? 1u : 0u);
    }
}

// 16-byte chunk c (8 bf16) of row r of a two-block K-major tile, 128-byte swizzle
__device__ __forceinline__ uint8_t* tile_chunk(uint8_t* tile, int r, int c16) {
    return tile + (c16 >> 3) * kBlk + r * 128 + (((c16 & 7) ^ (r & 7)) << 4);
}
__device__ __forceinline__ void load_tile(uint32_t dst, const CUtensorMap* map, uint32_t bar, int col0, int row0) {
    tma_load_2d(dst, map, bar, col0, row0);
    tma_load_2d(dst + kBlk, map, bar, col0 + 64, row0);
}

// ---------------------------------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------------------------------
// One CTA takes TWO neighbouring 128-query tiles (A = tile 2i, B = tile 2i + 1) of one head and walks the key / value tiles
// they share once. Warps 0-3 are the softmax group of A, warps 4-7 of B (thread = query row = TMEM lane), warp 8 issues the
// TMA copies and the MMAs. S_A, S_B, O_A, O_B fill the 512 TMEM columns; Q_A, Q_B, two K stages, one V stage and one P tile
// per group (7 x 32 KB) fill the shared memory. While one group runs its softmax on S(j), the tensor core runs the other group's O += P V(j - 1... j)
// and S(j + 1): the exponentials (MUFU, 16 per clock) and the MMAs cost about the same per tile, so each hides the other.
constexpr int kFwdThreads = 288;   // warps 0..3 / 4..7: softmax of tile A / B, warp 8: TMA + MMA
constexpr uint32_t kFwdSmem = 7 * kTile + 1024 + 256;   // Q x 2, K x 2, V, P x 2

struct FwdGroup {          // what one softmax group works on
    uint32_t tS, tO;       // TMEM columns of its score and output accumulators
    uint32_t s_full, p_full, o_full;
    uint8_t* pP; uint32_t sP;
    int qt;                // its query tile; it attends key tiles 0 .. qt
};

__device__ __forceinline__ void fwd_softmax_group(const FwdGroup& G, const AttnParams& p, const CUtensorMap* tmO, int h, int b, int row0,
                                                  int warp_in_group, int lane, int bar_id, volatile uint32_t* abort_flag) {
    const int r = warp_in_group * 32 + lane;                       // query row of the tile = TMEM lane
    const uint32_t lane_off = (uint32_t)(warp_in_group * 32) << 16;
    const float c = p.scale * kLog2e;
    const int n_kv = G.qt + 1;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
        ok = mbar_wait(G.s_full, j & 1, abort_flag, p.status, ST_TIMEOUT_ACCUM, 20);
        if (!ok) break;
        tc_fence_after_sync();
        const bool diag = (j == G.qt);
        // pass 1: row maximum of this tile
        float m_tile = -INFINITY;
#pragma unroll 1
        for (int cb = 0; cb < 4; ++cb) {
            uint32_t v[32];
            tmem_ld_32x32(G.tS + lane_off + cb * 32, v);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float sc = __uint_as_float(v[i]);
                if (!diag || cb * 32 + i <= r) m_tile = fmaxf(m_tile, sc);
            }
        }
        const float m_new = fmaxf(m_run, m_tile);
        const float alpha = (m_run == -INFINITY) ? 0.f : exp2f((m_run - m_new) * c);
        // the previous P V product must have landed before O is rescaled and before P is overwritten
        if (j > 0) {
            ok = mbar_wait(G.o_full, (j - 1) & 1, abort_flag, p.status, ST_TIMEOUT_ACCUM, 21);
            if (!ok) break;
            tc_fence_after_sync();
            if (__any_sync(0xFFFFFFFFu, m_new > m_run)) {
#pragma unroll 1
                for (int cb = 0; cb < 4; ++cb) {
                    uint32_t v[32];
                    tmem_ld_32x32(G.tO + lane_off + cb * 32, v);
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                    tmem_st_32x32(G.tO + lane_off + cb * 32, v);
                }
            }
        }
        // pass 2: P = exp2(s c - m c), row sum, bf16 row into the swizzled P tile
        const float mc = m_new * c;
        float l_tile = 0.f;
#pragma unroll 1
        for (int cb = 0; cb < 4; ++cb) {
            uint32_t v[32];
            tmem_ld_32x32(G.tS + lane_off + cb * 32, v);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                uint32_t o[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int c0 = cb * 32 + g * 8 + 2 * i;
                    float p0 = exp2f(fmaf(__uint_as_float(v[g * 8 + 2 * i]), c, -mc));
                    float p1 = exp2f(fmaf(__uint_as_float(v[g * 8 + 2 * i + 1]), c, -mc));
                    if (diag) { if (c0 > r) p0 = 0.f; if (c0 + 1 > r) p1 = 0.f; }
                    l_tile += p0 + p1;
                    o[i] = pack_bf16x2(p0, p1);
                }
                *reinterpret_cast<uint4*>(tile_chunk(G.pP, r, cb * 4 + g)) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
        l_run = l_run * alpha + l_tile;
        m_run = m_new;
        tc_fence_before_sync();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(G.p_full);
    }
    // epilogue: O / l -> bf16 -> the P tile as staging -> TMA store; log-sum-exp for the backward
    if (ok) ok = mbar_wait(G.o_full, (n_kv - 1) & 1, abort_flag, p.status, ST_TIMEOUT_ACCUM, 22);
    if (ok) {
        tc_fence_after_sync();
        const float inv_l = 1.0f / l_run;
#pragma unroll 1
        for (int cb = 0; cb < 4; ++cb) {
            uint32_t v[32];
            tmem_ld_32x32(G.tO + lane_off + cb * 32, v);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                uint32_t o[4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    o[i] = pack_bf16x2(__uint_as_float(v[g * 8 + 2 * i]) * inv_l, __uint_as_float(v[g * 8 + 2 * i + 1]) * inv_l);
                *reinterpret_cast<uint4*>(tile_chunk(G.pP, r, cb * 4 + g)) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
        if (p.lse) p.lse[((long long)b * p.Hq + h) * p.S + G.qt * kT + r] = m_run * p.scale + logf(l_run);
        fence_proxy_async_smem();
        asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
        if (r == 0) {
            tma_store_2d(tmO, G.sP, h * kD, row0 + G.qt * kT);
            tma_store_2d(tmO, G.sP + kBlk, h * kD + 64, row0 + G.qt * kT);
            tma_store_commit();
            tma_store_wait_all();
        }
    }
}

__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                const __grid_constant__ CUtensorMap tmO, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    const uint32_t sQ0 = base, sK0 = base + 2 * kTile, sV = base + 4 * kTile, sP0 = base + 5 * kTile;
    const uint32_t bar = base + 7 * kTile;
    const uint32_t q_full = bar, k_full0 = bar + 8, k_empty0 = bar + 24, v_full = bar + 40, v_empty = bar + 48;
    auto s_full = [&](int g) { return bar + 56u + 8u * g; };
    auto p_full = [&](int g) { return bar + 72u + 8u * g; };
    auto o_full = [&](int g) { return bar + 88u + 8u * g; };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + 7 * kTile + 112);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_qt = p.S / kT;
    const int n_pairs = (n_qt + 1) / 2;
    const int pi = n_pairs - 1 - (int)blockIdx.x;   // heavy pairs first
    const int qtA = 2 * pi, qtB = 2 * pi + 1;
    const bool hasB = qtB < n_qt;
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (p.Hq / p.Hkv);
    const int n_kvA = qtA + 1;
    const int n_kv = hasB ? qtB + 1 : n_kvA;
    const int row0 = b * p.S;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1); mbar_init(v_full, 1); mbar_init(v_empty, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(k_full0 + 8 * i, 1); mbar_init(k_empty0 + 8 * i, 1);
            mbar_init(s_full(i), 1); mbar_init(p_full(i), 4); mbar_init(o_full(i), 1);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 8) { tmem_alloc(smem_u32((const void*)tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    auto tS = [&](int g) { return tmem + 128u * g; };
    auto tO = [&](int g) { return tmem + 256u + 128u * g; };

    if (warp == 8) {
        if (lane == 0) {
            tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
            mbar_arrive_expect_tx(q_full, hasB ? 2 * kTile : kTile);
            load_tile(sQ0, &tmQ, q_full, h * kD, row0 + qtA * kT);
            if (hasB) load_tile(sQ0 + kTile, &tmQ, q_full, h * kD, row0 + qtB * kT);
            bool ok = true;
            for (int j = 0; j < 2 && j < n_kv; ++j) {
                mbar_arrive_expect_tx(k_full0 + 8 * j, kTile);
                load_tile(sK0 + j * kTile, &tmK, k_full0 + 8 * j, hk * kD, row0 + j * kT);
            }
            mbar_arrive_expect_tx(v_full, kTile);
            load_tile(sV, &tmV, v_full, hk * kD, row0);
            ok = mbar_wait(q_full, 0, abort_flag, p.status, ST_TIMEOUT_FULL, 10);
            if (ok) ok = mbar_wait(k_full0, 0, abort_flag, p.status, ST_TIMEOUT_FULL, 11);
            if (ok) {
                tc_fence_after_sync();
                mma_128(tS(0), sQ0, false, sK0, false, false);                    // S_A(0) = Q_A K_0^T
                umma_commit(s_full(0));
                if (hasB) { mma_128(tS(1), sQ0 + kTile, false, sK0, false, false); umma_commit(s_full(1)); }
            }
            for (int j = 0; j < n_kv && ok; ++j) {
                const int s = j & 1, s1 = (j + 1) & 1;
                ok = mbar_wait(v_full, j & 1, abort_flag, p.status, ST_TIMEOUT_FULL, 15);
                if (!ok) break;
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    const int n_g = g == 0 ? n_kvA : n_kv;
                    if ((g == 1 && !hasB) || j >= n_g) continue;
                    // P_g(j) is ready (and S_g(j) has been read): O_g += P_g V_j, then S_g(j + 1) while the other group's softmax runs
                    ok = mbar_wait(p_full(g), j & 1, abort_flag, p.status, ST_TIMEOUT_FULL, 12);
                    if (!ok) break;
                    tc_fence_after_sync();
                    mma_128(tO(g), sP0 + g * kTile, false, sV, true, j > 0);      // V: rows = kv = reduction index
                    umma_commit(o_full(g));
                    if (j + 1 < n_g) {
                        ok = mbar_wait(k_full0 + 8 * s1, ((j + 1) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_FULL, 13);
                        if (!ok) break;
                        tc_fence_after_sync();
                        mma_128(tS(g), sQ0 + g * kTile, false, sK0 + s1 * kTile, false, false);
                        umma_commit(s_full(g));
                    }
                }
                if (!ok) break;
                // every product that reads V_j and K_j has been issued: the two buffers are free once those have completed
                umma_commit(v_empty);
                umma_commit(k_empty0 + 8 * s);
                if (j + 1 < n_kv) {
                    ok = mbar_wait(v_empty, j & 1, abort_flag, p.status, ST_TIMEOUT_EMPTY, 16);
                    if (!ok) break;
                    mbar_arrive_expect_tx(v_full, kTile);
                    load_tile(sV, &tmV, v_full, hk * kD, row0 + (j + 1) * kT);
                }
                if (j + 2 < n_kv) {
                    ok = mbar_wait(k_empty0 + 8 * s, (j >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_EMPTY, 14);
                    if (!ok) break;
                    mbar_arrive_expect_tx(k_full0 + 8 * s, kTile);
                    load_tile(sK0 + s * kTile, &tmK, k_full0 + 8 * s, hk * kD, row0 + (j + 2) * kT);
                }
            }
        }
    } else {
        const int g = warp >> 2;
        if (g == 0 || hasB) {
            FwdGroup G;
            G.tS = tS(g); G.tO = tO(g); G.s_full = s_full(g); G.p_full = p_full(g); G.o_full = o_full(g);
            G.pP = smem + 5 * kTile + g * kTile; G.sP = sP0 + g * kTile; G.qt = g == 0 ? qtA : qtB;
            fwd_softmax_group(G, p, &tmO, h, b, row0, warp & 3, lane, 1 + g, abort_flag);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 8) { tc_fence_after_sync(); tmem_dealloc(tmem, 512); }
}

// ---------------------------------------------------------------------------------------------------------------------
// backward pre-pass: dsum[b, h, s] = sum_d dO * O   (one warp per (token, head) row)
// ---------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
attn_dsum_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o, long long ld, int B, int S, int Hq,
                 float* __restrict__ dsum) {
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);   // over B * S * Hq
    if (row >= (long long)B * S * Hq) return;
    const int h = (int)(row % Hq);
    const long long tok = row / Hq;
    const uint2 a = *reinterpret_cast<const uint2*>(o + tok * ld + h * kD + lane * 4);
    const uint2 g = *reinterpret_cast<const uint2*>(d_o + tok * ld + h * kD + lane * 4);
    float s = __uint_as_float(a.x << 16) * __uint_as_float(g.x << 16) + __uint_as_float(a.x & 0xFFFF0000u) * __uint_as_float(g.x & 0xFFFF0000u) +
              __uint_as_float(a.y << 16) * __uint_as_float(g.y << 16) + __uint_as_float(a.y & 0xFFFF0000u) * __uint_as_float(g.y & 0xFFFF0000u);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, off);
    if (lane == 0) {
        const int b = (int)(tok / S), sidx = (int)(tok % S);
        dsum[((long long)b * Hq + h) * S + sidx] = s;
    }
}

// The element-wise middle of both backward kernels: thread r (row = query r of the q tile) turns the score row in tS and
// the dP row in tdP into P (optional) and dS = P (dP - D) scale, written as bf16 rows of swizzled K-major tiles.
__device__ __forceinline__ void bwd_rows(uint32_t tS, uint32_t tdP, uint32_t lane_off, int r, bool diag, float c, float lse_l2, float dsum_r,
                                         float scale, uint8_t* pP, uint8_t* pdS) {
#pragma unroll 1
    for (int cb = 0; cb < 4; ++cb) {
        uint32_t vs[32], vd[32];
        tmem_ld_32x32(tS + lane_off + cb * 32, vs);
        tmem_ld_32x32(tdP + lane_off + cb * 32, vd);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            uint32_t op[4], od[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int c0 = cb * 32 + g * 8 + 2 * i;
                float p0 = exp2f(__uint_as_float(vs[g * 8 + 2 * i]) * c - lse_l2);
                float p1 = exp2f(__uint_as_float(vs[g * 8 + 2 * i + 1]) * c - lse_l2);
                if (diag) { if (c0 > r) p0 = 0.f; if (c0 + 1 > r) p1 = 0.f; }
                const float d0 = p0 * (__uint_as_float(vd[g * 8 + 2 * i]) - dsum_r) * scale;
                const float d1 = p1 * (__uint_as_float(vd[g * 8 + 2 * i + 1]) - dsum_r) * scale;
                op[i] = pack_bf16x2(p0, p1);
                od[i] = pack_bf16x2(d0, d1);
            }
            if (pP) *reinterpret_cast<uint4*>(tile_chunk(pP, r, cb * 4 + g)) = make_uint4(op[0], op[1], op[2], op[3]);
            *reinterpret_cast<uint4*>(tile_chunk(pdS, r, cb * 4 + g)) = make_uint4(od[0], od[1], od[2], od[3]);
        }
    }
}

// write a finished 128 x 128 fp32 accumulator (TMEM) as bf16 through a staging tile and two TMA boxes
__device__ __forceinline__ void store_acc_tile(uint32_t tacc, uint32_t lane_off, int r, uint8_t* stage, uint32_t stage_u32,
                                               const CUtensorMap* map, int col0, int row0) {
#pragma unroll 1
    for (int cb = 0; cb < 4; ++cb) {
        uint32_t v[32];
        tmem_ld_32x32(tacc + lane_off + cb * 32, v);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) o[i] = pack_bf16x2(__uint_as_float(v[g * 8 + 2 * i]), __uint_as_float(v[g * 8 + 2 * i + 1]));
            *reinterpret_cast<uint4*>(tile_chunk(stage, r, cb * 4 + g)) = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
    fence_proxy_async_smem();
    bar_sync_128();
    if (threadIdx.x == 0) {
        tma_store_2d(map, stage_u32, col0, row0);
        tma_store_2d(map, stage_u32 + kBlk, col0 + 64, row0);
        tma_store_commit();
        tma_store_wait_all();
    }
    bar_sync_128();
}

// ---------------------------------------------------------------------------------------------------------------------
// backward, dQ: one CTA per (q tile, q head, batch)
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kBwdThreads = 160;
constexpr uint32_t kDqSmem = 7 * kTile + 1024 + 256;   // Q, dO, K x 2, V x 2, dS

__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   const __grid_constant__ CUtensorMap tmdO, const __grid_constant__ CUtensorMap tmdQ, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    const uint32_t sQ = base, sdO = base + kTile, sK0 = base + 2 * kTile, sV0 = base + 4 * kTile, sdS = base + 6 * kTile;
    uint8_t* pdS = smem + 6 * kTile;
    const uint32_t bar = base + 7 * kTile;
    const uint32_t q_full = bar, kv_full0 = bar + 8, kv_empty0 = bar + 24, sd_full = bar + 40, ds_full = bar + 48, dq_full = bar + 56;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + 7 * kTile + 64);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_qt = p.S / kT;
    const int qt = n_qt - 1 - (int)blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (p.Hq / p.Hkv);
    const int n_kv = qt + 1;
    const int row0 = b * p.S;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) { mbar_init(kv_full0 + 8 * i, 1); mbar_init(kv_empty0 + 8 * i, 1); }
        mbar_init(sd_full, 1); mbar_init(ds_full, 4); mbar_init(dq_full, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 4) { tmem_alloc(smem_u32((const void*)tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tS = tmem, tdP = tmem + 128, tdQ = tmem + 256;

    if (warp == 4) {
        if (lane == 0) {
            mbar_arrive_expect_tx(q_full, 2 * kTile);
            load_tile(sQ, &tmQ, q_full, h * kD, row0 + qt * kT);
            load_tile(sdO, &tmdO, q_full, h * kD, row0 + qt * kT);
            for (int j = 0; j < 2 && j < n_kv; ++j) {
                mbar_arrive_expect_tx(kv_full0 + 8 * j, 2 * kTile);
                load_tile(sK0 + j * kTile, &tmK, kv_full0 + 8 * j, hk * kD, row0 + j * kT);
                load_tile(sV0 + j * kTile, &tmV, kv_full0 + 8 * j, hk * kD, row0 + j * kT);
            }
            bool ok = mbar_wait(q_full, 0, abort_flag, p.status, ST_TIMEOUT_FULL, 30);
            for (int j = 0; j < n_kv && ok; ++j) {
                const int s = j & 1;
                ok = mbar_wait(kv_full0 + 8 * s, (j >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_FULL, 31);
                if (!ok) break;
                if (j > 0) {
                    // the threads have read S / dP of the previous tile (they arrived on ds_full) before these are overwritten
                    ok = mbar_wait(ds_full, (j - 1) & 1, abort_flag, p.status, ST_TIMEOUT_FULL, 32);
                    if (!ok) break;
                }
                tc_fence_after_sync();
                if (j > 0) {
                    mma_128(tdQ, sdS, false, sK0 + ((j - 1) & 1) * kTile, true, j > 1);   // dQ += dS_{j-1} K_{j-1}
                    umma_commit(kv_empty0 + 8 * ((j - 1) & 1));
                }
                mma_128(tS, sQ, false, sK0 + s * kTile, false, false);        // S  = Q K_j^T
                mma_128(tdP, sdO, false, sV0 + s * kTile, false, false);      // dP = dO V_j^T
                umma_commit(sd_full);
                if (j >= 1 && j + 1 < n_kv) {
                    // stage (j - 1) & 1 == (j + 1) & 1 is free once dQ += dS_{j-1} K_{j-1} has completed
                    const int s1 = (j + 1) & 1;
                    ok = mbar_wait(kv_empty0 + 8 * s1, ((j - 1) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_EMPTY, 33);
                    if (!ok) break;
                    mbar_arrive_expect_tx(kv_full0 + 8 * s1, 2 * kTile);
                    load_tile(sK0 + s1 * kTile, &tmK, kv_full0 + 8 * s1, hk * kD, row0 + (j + 1) * kT);
                    load_tile(sV0 + s1 * kTile, &tmV, kv_full0 + 8 * s1, hk * kD, row0 + (j + 1) * kT);
                }
            }
            if (ok) ok = mbar_wait(ds_full, (n_kv - 1) & 1, abort_flag, p.status, ST_TIMEOUT_FULL, 34);
            if (ok) {
                tc_fence_after_sync();
                mma_128(tdQ, sdS, false, sK0 + ((n_kv - 1) & 1) * kTile, true, n_kv > 1);
                umma_commit(dq_full);
            }
        }
    } else {
        const int r = threadIdx.x;
        const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
        const float c = p.scale * kLog2e;
        const long long stat = ((long long)b * p.Hq + h) * p.S + qt * kT + r;
        const float lse_l2 = p.lse[stat] * kLog2e, dsum_r = p.dsum[stat];
        bool ok = true;
        for (int j = 0; j < n_kv && ok; ++j) {
            ok = mbar_wait(sd_full, j & 1, abort_flag, p.status, ST_TIMEOUT_ACCUM, 40);
            if (!ok) break;
            tc_fence_after_sync();
            // dS_{j-1} must have been consumed (dQ product issued AND completed) before the dS tile is rewritten: the
            // S / dP products of this tile were issued after it in the same thread, so sd_full implies it
            bwd_rows(tS, tdP, lane_off, r, j == qt, c, lse_l2, dsum_r, p.scale, nullptr, pdS);
            tc_fence_before_sync();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(ds_full);
        }
        if (ok) ok = mbar_wait(dq_full, 0, abort_flag, p.status, ST_TIMEOUT_ACCUM, 41);
        if (ok) {
            tc_fence_after_sync();
            store_acc_tile(tdQ, lane_off, r, pdS, sdS, &tmdQ, h * kD, row0 + qt * kT);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 4) { tc_fence_after_sync(); tmem_dealloc(tmem, 512); }
}

// ---------------------------------------------------------------------------------------------------------------------
// backward, dK and dV: one CTA per (kv tile, kv head, batch); inner loop over the q heads of the group and the q tiles
// ---------------------------------------------------------------------------------------------------------------------
constexpr uint32_t kDkvSmem = 6 * kTile + 1024 + 256;   // K, V, Q, dO, P, dS

__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                    const __grid_constant__ CUtensorMap tmdO, const __grid_constant__ CUtensorMap tmdK, const __grid_constant__ CUtensorMap tmdV,
                    const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    const uint32_t sK = base, sV = base + kTile, sQ = base + 2 * kTile, sdO = base + 3 * kTile, sP = base + 4 * kTile, sdS = base + 5 * kTile;
    uint8_t* pP = smem + 4 * kTile;
    uint8_t* pdS = smem + 5 * kTile;
    const uint32_t bar = base + 6 * kTile;
    const uint32_t kv_full = bar, q_full = bar + 8, q_empty = bar + 16, sd_full = bar + 24, ds_full = bar + 32, acc_full = bar + 40;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + 6 * kTile + 64);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_qt = p.S / kT;
    const int jt = blockIdx.x;                    // kv tile (the first ones have the most q tiles)
    const int hk = blockIdx.y, b = blockIdx.z;
    const int group = p.Hq / p.Hkv;
    const int n_i = n_qt - jt;                    // q tiles at or after the kv tile
    const int n_it = group * n_i;                 // inner iterations: (q head of the group) x (q tile)
    const int row0 = b * p.S;

    if (threadIdx.x == 0) {
        mbar_init(kv_full, 1); mbar_init(q_full, 1); mbar_init(q_empty, 1);
        mbar_init(sd_full, 1); mbar_init(ds_full, 4); mbar_init(acc_full, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 4) { tmem_alloc(smem_u32((const void*)tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tS = tmem, tdP = tmem + 128, tdV = tmem + 256, tdK = tmem + 384;

    if (warp == 4) {
        if (lane == 0) {
            mbar_arrive_expect_tx(kv_full, 2 * kTile);
            load_tile(sK, &tmK, kv_full, hk * kD, row0 + jt * kT);
            load_tile(sV, &tmV, kv_full, hk * kD, row0 + jt * kT);
            bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, ST_TIMEOUT_FULL, 50);
            for (int it = 0; it < n_it && ok; ++it) {
                const int h = hk * group + it / n_i, qi = jt + it % n_i;
                // Q / dO of the previous iteration are free once its dV / dK products have completed
                if (it > 0) {
                    ok = mbar_wait(q_empty, (it - 1) & 1, abort_flag, p.status, ST_TIMEOUT_EMPTY, 51);
                    if (!ok) break;
                }
                mbar_arrive_expect_tx(q_full, 2 * kTile);
                load_tile(sQ, &tmQ, q_full, h * kD, row0 + qi * kT);
                load_tile(sdO, &tmdO, q_full, h * kD, row0 + qi * kT);
                ok = mbar_wait(q_full, it & 1, abort_flag, p.status, ST_TIMEOUT_FULL, 52);
                if (!ok) break;
                tc_fence_after_sync();
                mma_128(tS, sQ, false, sK, false, false);          // S  = Q K^T      (rows = queries)
                mma_128(tdP, sdO, false, sV, false, false);        // dP = dO V^T
                umma_commit(sd_full);
                ok = mbar_wait(ds_full, it & 1, abort_flag, p.status, ST_TIMEOUT_FULL, 53);
                if (!ok) break;
                tc_fence_after_sync();
                mma_128(tdV, sP, true, sdO, true, it > 0);         // dV += P^T dO    (P^T: the P tile read MN-major)
                mma_128(tdK, sdS, true, sQ, true, it > 0);         // dK += dS^T Q
                umma_commit(q_empty);
                if (it == n_it - 1) umma_commit(acc_full);
            }
        }
    } else {
        const int r = threadIdx.x;
        const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
        const float c = p.scale * kLog2e;
        bool ok = true;
        for (int it = 0; it < n_it && ok; ++it) {
            const int h = hk * group + it / n_i, qi = jt + it % n_i;
            const long long stat = ((long long)b * p.Hq + h) * p.S + qi * kT + r;
            const float lse_l2 = p.lse[stat] * kLog2e, dsum_r = p.dsum[stat];
            ok = mbar_wait(sd_full, it & 1, abort_flag, p.status, ST_TIMEOUT_ACCUM, 60);
            if (!ok) break;
            tc_fence_after_sync();
            // the P / dS tiles of the previous iteration have been consumed: S / dP of this one were issued after the
            // previous dV / dK products by the same thread and have completed
            bwd_rows(tS, tdP, lane_off, r, qi == jt, c, lse_l2, dsum_r, p.scale, pP, pdS);
            tc_fence_before_sync();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(ds_full);
        }
        if (ok) ok = mbar_wait(acc_full, 0, abort_flag, p.status, ST_TIMEOUT_ACCUM, 61);
        if (ok) {
            tc_fence_after_sync();
            store_acc_tile(tdV, lane_off, r, pP, sP, &tmdV, hk * kD, row0 + jt * kT);
            store_acc_tile(tdK, lane_off, r, pdS, sdS, &tmdK, hk * kD, row0 + jt * kT);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 4) { tc_fence_after_sync(); tmem_dealloc(tmem, 512); }
}

int check_attn(const AttnArgs& a) {
    if (a.B <= 0 || a.S <= 0 || a.Hq <= 0 || a.Hkv <= 0 || a.Hq % a.Hkv) { set_last_error("attention: bad shape B=%d S=%d Hq=%d Hkv=%d", a.B, a.S, a.Hq, a.Hkv); return PLZ_ERR_BAD_SHAPE; }
    if (a.S % kT) { set_last_error("attention: the sequence length %d must be a multiple of 128", a.S); return PLZ_ERR_BAD_SHAPE; }
    if (a.head_dim != kD) { set_last_error("attention: head_dim %d (only 128 is built)", a.head_dim); return PLZ_ERR_UNSUPPORTED; }
    return PLZ_OK;
}

template <typename K>
int set_smem(K kern, uint32_t bytes) {
    PLZ_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    return PLZ_OK;
}

}  // namespace

int launch_attn_fwd(const AttnArgs& a, cudaStream_t stream) {
    int rc = check_attn(a);
    if (rc) return rc;
    if (!a.q || !a.k || !a.v || !a.o) { set_last_error("attention: null pointer"); return PLZ_ERR_NULL; }
    const uint64_t rows = (uint64_t)a.B * a.S;
    CUtensorMap tmQ, tmK, tmV, tmO;
    if ((rc = make_tmap_bf16(&tmQ, a.q, rows, (uint64_t)a.Hq * kD, a.ldq, 64, kT))) return rc;
    if ((rc = make_tmap_bf16(&tmK, a.k, rows, (uint64_t)a.Hkv * kD, a.ldk, 64, kT))) return rc;
    if ((rc = make_tmap_bf16(&tmV, a.v, rows, (uint64_t)a.Hkv * kD, a.ldv, 64, kT))) return rc;
    if ((rc = make_tmap_bf16(&tmO, a.o, rows, (uint64_t)a.Hq * kD, a.ldo, 64, kT))) return rc;
    AttnParams p = {};
    p.B = a.B; p.S = a.S; p.Hq = a.Hq; p.Hkv = a.Hkv; p.scale = a.scale; p.lse = a.lse; p.status = device_status_ptr();
    static bool once = false;
    if (!once) { if ((rc = set_smem(attn_fwd_kernel, kFwdSmem))) return rc; once = true; }
    attn_fwd_kernel<<<dim3((a.S / kT + 1) / 2, a.Hq, a.B), kFwdThreads, kFwdSmem, stream>>>(tmQ, tmK, tmV, tmO, p);
    PLZ_LAUNCH_CHECK();
    return PLZ_OK;
}

int launch_attn_bwd(const AttnArgs& a, cudaStream_t stream) {
    int rc = check_attn(a);
    if (rc) return rc;
    if (!a.q || !a.k || !a.v || !a.o || !a.d_o || !a.dq || !a.dk || !a.dv || !a.lse || !a.dsum) { set_last_error("attention backward: null pointer"); return PLZ_ERR_NULL; }
    const uint64_t rows = (uint64_t)a.B * a.S;
    CUtensorMap tmQ, tmK, tmV, tmdO, tmdQ, tmdK, tmdV;
    if ((rc = make_tmap_bf16(&tmQ, a.q, rows, (uint64_t)a.Hq * kD, a.ldq, 64, kT))) return rc;
    if ((rc = make_tmap_bf16(&tmK, a.k, rows, (uint64_t)a.Hkv * kD, a.ldk, 64, kT))) return rc;
    if ((rc = make_tmap_bf16(&tmV, a.v, rows, (uint64_t)a.Hkv * kD, a.ldv, 64, kT))) return rc;
    if ((rc = make_tmap_bf16(&tmdO, a.d_o, rows, (uint64_t)a.Hq * kD, a.ldo, 64, kT))) return rc;
    if ((rc = make_tmap_bf16(&tmdQ, a.dq, rows, (uint64_t)a.Hq * kD, a.ldq, 64, kT))) return rc;
    if ((rc = make_tmap_bf16(&tmdK, a.dk, rows, (uint64_t)a.Hkv * kD, a.ldk, 64, kT))) return rc;
    if ((rc = make_tmap_bf16(&tmdV, a.dv, rows, (uint64_t)a.Hkv * kD, a.ldv, 64, kT))) return rc;
    AttnParams p = {};
    p.B = a.B; p.S = a.S; p.Hq = a.Hq; p.Hkv = a.Hkv; p.scale = a.scale; p.lse = a.lse; p.dsum = a.dsum; p.status = device_status_ptr();
    static bool once = false;
    if (!once) {
        if ((rc = set_smem(attn_bwd_dq_kernel, kDqSmem))) return rc;
        if ((rc = set_smem(attn_bwd_dkv_kernel, kDkvSmem))) return rc;
        once = true;
    }
    const long long n_rows = (long long)a.B * a.S * a.Hq;
    attn_dsum_kernel<<<(unsigned)((n_rows + 7) / 8), 256, 0, stream>>>((const __nv_bfloat16*)a.o, (const __nv_bfloat16*)a.d_o, a.ldo, a.B, a.S,
                                                                       a.Hq, a.dsum);
    PLZ_LAUNCH_CHECK();
    attn_bwd_dq_kernel<<<dim3(a.S / kT, a.Hq, a.B), kBwdThreads, kDqSmem, stream>>>(tmQ, tmK, tmV, tmdO, tmdQ, p);
    PLZ_LAUNCH_CHECK();
    attn_bwd_dkv_kernel<<<dim3(a.S / kT, a.Hkv, a.B), kBwdThreads, kDkvSmem, stream>>>(tmQ, tmK, tmV, tmdO, tmdK, tmdV, p);
    PLZ_LAUNCH_CHECK();
    return PLZ_OK;
}

}  // namespace plz
