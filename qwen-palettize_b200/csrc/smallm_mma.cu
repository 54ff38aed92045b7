// Small-M hard forward for decode batches of up to 16 rows: y[M, N] = x[M, K] W^T with W 2-bit palettized.
//
// A 9728 x 2560 Linear is 7 MB of packed indices: one microsecond at HBM speed, so the kernel is built to have every
// byte of its weights in flight right after it starts and to do nothing that costs a fixed latency on top (no TMEM
// allocation, no tensor map, no producer / consumer hand-over between warps):
//
//   * one CTA per SM owns a contiguous range of weight rows; warp 0 starts one bulk copy (cp.async.bulk, mbarrier
//     complete_tx) per 16-row strip into shared memory before anything else happens, each strip with its own
//     mbarrier so that its items start as soon as its 16 rows have landed.  Loading the rows into registers with
//     ordinary 16-byte loads instead was measured to take 4400 cycles just to ISSUE (the SM's outstanding-load
//     capacity, not HBM, was the limit), and one bulk copy per row 50 cycles of issue each;
//   * while the rows are in flight all warps stage x in shared memory, in the permuted order below;
//   * a work item is 16 rows x 256 input columns (one palette group per row); the items are dealt round-robin to the
//     warps (32 of them up to eight rows, 16 beyond).  Weights go from shared memory straight into mma.sync.m16n8k16 A fragments (the 128-row tcgen05 tile
//     would be 7/8 padding here): the reduction dimension may be permuted freely as long as x is permuted alike, so
//     lane (g, t) simply takes the 16 bytes at columns 64 t.. of rows g and g + 8 of the group; k-step 4 w + e uses bit
//     pair e of each of the four bytes of word w (the weights 16 w + e, + 4, + 8, + 12 of the lane's 64 columns).  One mask
//     and one multiply-add turn those four indices into four selector bytes (0x22 i + 0x10 = palette bytes 2i, 2i + 1),
//     and a byte permute of the row's palette per selector half gives two bf16 weights: 19 ALU instructions and 4
//     multiply-adds per 16 weights;
//   * x sits in shared memory in the matching order, 8 bytes per (k-step, lane quad), so that a B fragment is one
//     conflict-free 8-byte load;
//   * partial sums of an item are added to the CTA's fp32 output tile in shared memory (red.shared; the order in which
//     the K groups of a row meet there is not fixed, so the last bit of y may differ between runs), and the tile is
//     written out as bf16 once at the end.
#include <cuda_bf16.h>
#include <stdint.h>

#include "plz_host.h"
#include "plz_launch.h"
#include "plz_sm100.cuh"

namespace plz {

namespace {

// Up to eight rows (MT = 1) the kernel runs 1024 threads of 64 registers (measured 5 % faster than 512: more warps to cover the
// dependent decode -> mma chains); with sixteen rows the second accumulator set needs the registers of 512 threads.
template <int MT> struct SmallmCfg {
    static constexpr int kThreads = MT == 1 ? 1024 : 512;
    static constexpr int kWarps = kThreads / 32;
    static constexpr int kBatch = MT == 1 ? 2 : 4;    // items whose palette loads a warp keeps in flight together
};
constexpr int kHeader = 1024;        // mbarriers (one per strip, up to 126) and the abort flags

constexpr int kMaxMats = 4;

// Up to four weight matrices with the same K and palette grouping, all multiplied by the same x (gate and up, or q, k and
// v): their rows form one virtual row space [0, row_start[n_mats]) that is cut evenly over the CTAs.
struct SmallmParams {
    const __nv_bfloat16* x; long long ldx;
    const uint8_t* packed[kMaxMats]; long long pitch[kMaxMats];
    const __nv_bfloat16* palette[kMaxMats];
    __nv_bfloat16* out[kMaxMats]; long long ld_out[kMaxMats];
    int row_start[kMaxMats + 1];
    int n_mats;
    int M, N, K, gs_n, gs_k, n_kgroups;  // N: rows of the virtual row space; n_kgroups: palette groups per row group
    int gs_n_shift, gs_k_shift;          // log2 of gs_n / gs_k when they are powers of two, else -1 (division)
    int rows_per_cta, rows_alloc;        // rows_alloc: packed rows reserved in shared memory (rows_per_cta up to 16)
    StatusWord* status;
    uint32_t x_pitch;                    // bytes per token row of the staged x (K * 2 + 32)
    unsigned long long* prof;            // optional [gridDim][8] cycle counters of warp 0 (diagnostics)
};

__device__ __forceinline__ int mat_of(const SmallmParams& p, int v) {
    int mi = 0;
#pragma unroll
    for (int i = 1; i < kMaxMats; ++i) mi += (i < p.n_mats && v >= p.row_start[i]) ? 1 : 0;
    return mi;
}

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

template <int MT>  // MT m8 tiles: M <= 8 * MT
__global__ void __launch_bounds__(SmallmCfg<MT>::kThreads, 1)
lut_smallm_mma_kernel(const SmallmParams p) {
    constexpr int kThreads = SmallmCfg<MT>::kThreads, kWarps = SmallmCfg<MT>::kWarps, kBatch = SmallmCfg<MT>::kBatch;
    extern __shared__ __align__(128) uint8_t smem[];
    // [0, kHeader): one mbarrier per 16-row strip + abort flags | packed rows | x rows | fp32 output tile
    const uint32_t bar0 = smem_u32(smem);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + kHeader - 16);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int r0 = blockIdx.x * p.rows_per_cta;
    const int r1 = min(p.N, r0 + p.rows_per_cta);
    const int rows = r1 - r0;
    const int strips = (rows + 15) >> 4;
    const int kgs = p.K >> 8;               // 256-column groups along K
    const int n_items = strips * kgs;
    const int rows_pad = strips * 16;
    const uint32_t row_bytes = (uint32_t)p.K >> 2;
    uint8_t* wsm = smem + kHeader;          // rows back to back (row_bytes each), as in global memory
    uint8_t* xs = wsm + (size_t)p.rows_alloc * row_bytes;
    float* acc_s = reinterpret_cast<float*>(xs + (size_t)p.M * p.x_pitch);

    const long long t_entry = PLZ_PROF_ON(p.prof) ? clock64() : 0;
    // ---- the CTA's packed rows: one bulk copy per 16-row strip (rows of a matrix are contiguous when its pitch is the
    // row size; otherwise, and where a strip crosses into the next matrix, one copy per contiguous piece), each strip
    // with its own mbarrier so that its items can start as soon as its 16 rows have landed
    if (warp == 0) {
        for (int s = lane; s < strips; s += 32) mbar_init(bar0 + 8u * s, 1);
        if (lane == 0) { abort_flag[0] = 0u; abort_flag[1] = 0u; }
        mbar_fence_init();
        __syncwarp();
        if (PLZ_PROF_ON(p.prof) && threadIdx.x == 0) p.prof[8ull * blockIdx.x + 5] = clock64() - t_entry;
        for (int s = lane; s < strips; s += 32) {
            const int a = s * 16, b = min(rows, a + 16);
            mbar_arrive_expect_tx(bar0 + 8u * s, (uint32_t)(b - a) * row_bytes);
            int r = a;
            while (r < b) {
                const int mi = mat_of(p, r0 + r), lr = r0 + r - p.row_start[mi];
                const long long pitch = p.pitch[mi];
                int n = 1;  // rows of this piece
                if (pitch == (long long)row_bytes) n = min(b - r, p.row_start[mi + 1] - (r0 + r));
                bulk_load(smem_u32(wsm) + (uint32_t)r * row_bytes, p.packed[mi] + (long long)lr * pitch, (uint32_t)n * row_bytes,
                          bar0 + 8u * s);
                r += n;
            }
        }
    }
    if (PLZ_PROF_ON(p.prof) && threadIdx.x == 0) p.prof[8ull * blockIdx.x + 6] = clock64() - t_entry;
    // Programmatic dependent launch (no-ops unless the launch carries the attribute): the next kernel of the stream may
    // start its own weight copies now; this one must not read x, nor write y, before the previous kernel has finished.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (PLZ_PROF_ON(p.prof) && threadIdx.x == 0) p.prof[8ull * blockIdx.x + 7] = clock64() - t_entry;
    uint2 pa[kBatch], pb[kBatch];
    // (strip, k group) of an item without a division: a warp's items are 16 apart
    auto advance = [&](int& s, int& kg) {
        kg += kWarps;
        while (kg >= kgs) { kg -= kgs; ++s; }
    };
    auto palette_of = [&](int v, int kg) -> uint2 {
        const int mi = mat_of(p, v), lr = v - p.row_start[mi];
        const int ng = p.gs_n_shift >= 0 ? (lr >> p.gs_n_shift) : (lr / p.gs_n);
        const int pg = p.gs_k_shift >= 0 ? ((kg << 8) >> p.gs_k_shift) : ((kg << 8) / p.gs_k);
        return __ldg(reinterpret_cast<const uint2*>(p.palette[mi] + ((long long)ng * p.n_kgroups + pg) * 4));
    };
    auto load_palettes = [&](int first_item, int s, int kg) {
#pragma unroll
        for (int q = 0; q < kBatch; ++q) {
            const int item = first_item + q * kWarps;
            pa[q] = make_uint2(0u, 0u); pb[q] = pa[q];
            if (item < n_items) {
                const int ra = r0 + s * 16 + g, rb = ra + 8;
                if (ra < r1) pa[q] = palette_of(ra, kg);
                if (rb < r1) pb[q] = palette_of(rb, kg);
            }
            advance(s, kg);
        }
    };
    int s_cur = 0, kg_cur = warp;  // (strip, k group) of the warp's next item
    while (kg_cur >= kgs) { kg_cur -= kgs; ++s_cur; }
    const long long t_a = PLZ_PROF_ON(p.prof) ? clock64() : 0;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    {
        // x in the permuted order of the fragments. A 16-byte chunk = 8 consecutive k of one token = bytes 2 hh, 2 hh + 1 of word
        // wi of lane quad tq, all four bit pairs e: its elements (byte c, pair e) go to k-step 4 wi + e, slot c of the quad's
        // 8-byte unit. Up to eight loads (one per row) per thread in flight together. Only the M real rows are staged: a
        // column n >= M of an mma only ever reaches the same column of D, which is never written out, so the lanes of those
        // columns simply read row 0
        const int chunks_per_row = p.K >> 3;
        for (int c = threadIdx.x; c < chunks_per_row; c += kThreads) {
            const int k = c << 3;
            const int kg = k >> 8, r = k & 255, tq = r >> 6, wi = (r & 63) >> 4, hh = (r >> 3) & 1;
            uint8_t* dst = xs + (size_t)(((kg * 16 + wi * 4) * 4 + tq) * 8 + hh * 4);
            const __nv_bfloat16* src = p.x + k;
#pragma unroll
            for (int m0 = 0; m0 < 8 * MT; m0 += 8) {
                uint4 v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (m0 + u < p.M) v[u] = __ldg(reinterpret_cast<const uint4*>(src + (long long)(m0 + u) * p.ldx));
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    if (m0 + u < p.M) {
                        uint8_t* d = dst + (size_t)(m0 + u) * p.x_pitch;
                        // v.x = (byte 2hh: pairs 0, 1), v.y = (byte 2hh: pairs 2, 3), v.z / v.w the same of byte 2hh + 1
                        *reinterpret_cast<uint32_t*>(d) = prmt_raw(v[u].x, v[u].z, 0x5410u);        // pair 0 of both bytes
                        *reinterpret_cast<uint32_t*>(d + 32) = prmt_raw(v[u].x, v[u].z, 0x7632u);   // pair 1 (next k-step, same quad)
                        *reinterpret_cast<uint32_t*>(d + 64) = prmt_raw(v[u].y, v[u].w, 0x5410u);
                        *reinterpret_cast<uint32_t*>(d + 96) = prmt_raw(v[u].y, v[u].w, 0x7632u);
                    }
                }
            }
        }
    }
    load_palettes(warp, s_cur, kg_cur);
    for (int i = threadIdx.x; i < rows_pad * 8 * MT; i += kThreads) acc_s[i] = 0.f;
    const long long t_pro = PLZ_PROF_ON(p.prof) ? clock64() : 0;
    __syncthreads();
    const long long t_sync = PLZ_PROF_ON(p.prof) ? clock64() : 0;
    bool ok = true;
    int strip_ready = -1;  // strips up to this one have been waited for by this warp

    uint32_t xs_base[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
        xs_base[mt] = smem_u32(xs) + (uint32_t)((mt * 8 + g) < p.M ? (mt * 8 + g) : 0) * p.x_pitch + (uint32_t)t * 8u;
    const uint32_t w_base = smem_u32(wsm) + (uint32_t)g * row_bytes + (uint32_t)t * 16u;
    for (int first = warp; ok && first < n_items; first += kBatch * kWarps) {
        if (first != warp) load_palettes(first, s_cur, kg_cur);
#pragma unroll
        for (int q = 0; q < kBatch; ++q) {
            const int item = first + q * kWarps;
            if (item >= n_items) break;
            const int s = s_cur, kg = kg_cur;
            advance(s_cur, kg_cur);
            if (s > strip_ready) {
                // bounded wait for the strip's rows: on a timeout the status word is set and the CTA writes nothing
                for (int w = strip_ready + 1; ok && w <= s; ++w) ok = mbar_wait(bar0 + 8u * w, 0, abort_flag, p.status, ST_TIMEOUT_FULL, 1);
                strip_ready = s;
                if (!ok) break;
            }
            // two accumulators per m-tile (even / odd k-steps) so that consecutive mma do not wait on each other
            float d[MT][4], e_acc[MT][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                d[mt][0] = d[mt][1] = d[mt][2] = d[mt][3] = 0.f;
                e_acc[mt][0] = e_acc[mt][1] = e_acc[mt][2] = e_acc[mt][3] = 0.f;
            }
            uint32_t wra[4], wrb[4];
            const uint32_t wadr = w_base + (uint32_t)(s * 16) * row_bytes + (uint32_t)kg * 64u;
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(wra[0]), "=r"(wra[1]), "=r"(wra[2]), "=r"(wra[3]) : "r"(wadr));
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(wrb[0]), "=r"(wrb[1]), "=r"(wrb[2]), "=r"(wrb[3]) : "r"(wadr + 8u * row_bytes));
            const uint32_t xoff = (uint32_t)kg * (16u * 4u * 8u);
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = wi * 4 + e;
                    const uint32_t sa = ((wra[wi] >> (2 * e)) & 0x03030303u) * 0x22u + 0x10101010u;
                    const uint32_t sb = ((wrb[wi] >> (2 * e)) & 0x03030303u) * 0x22u + 0x10101010u;
                    uint32_t a[4];
                    a[0] = prmt_raw(pa[q].x, pa[q].y, sa);
                    a[1] = prmt_raw(pb[q].x, pb[q].y, sb);
                    a[2] = prmt_raw(pa[q].x, pa[q].y, sa >> 16);
                    a[3] = prmt_raw(pb[q].x, pb[q].y, sb >> 16);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        uint32_t b0, b1;
                        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(xs_base[mt] + xoff + (uint32_t)j * 32u));
                        if (j & 1) mma_bf16_16816(e_acc[mt], a, b0, b1);
                        else mma_bf16_16816(d[mt], a, b0, b1);
                    }
                }
            }
            float* o = acc_s + (size_t)(s * 16 + g) * (8 * MT) + 2 * t;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                atomicAdd(o + mt * 8, d[mt][0] + e_acc[mt][0]);
                atomicAdd(o + mt * 8 + 1, d[mt][1] + e_acc[mt][1]);
                atomicAdd(o + 8 * (8 * MT) + mt * 8, d[mt][2] + e_acc[mt][2]);
                atomicAdd(o + 8 * (8 * MT) + mt * 8 + 1, d[mt][3] + e_acc[mt][3]);
            }
        }
    }
    const long long t_comp = PLZ_PROF_ON(p.prof) ? clock64() : 0;
    // a CTA must not exit with copies in flight into its shared memory: every warp has waited for every strip it used;
    // warp 0 waits for all of them (again bounded), and a timeout anywhere disables the output below
    if (warp == 0) {
        for (int w = 0; w < strips; ++w)
            if (!mbar_wait(bar0 + 8u * w, 0, abort_flag + 1, p.status, ST_TIMEOUT_DRAIN, 1)) break;
    }
    __syncthreads();
    ok = (abort_flag[0] == 0u) && (abort_flag[1] == 0u);
    // ---- write the tile: consecutive threads walk the weight rows of one token (contiguous in y)
    for (int i = threadIdx.x; ok && i < p.M * rows; i += kThreads) {
        const int m = i / rows, r = i - m * rows;
        const int mi = mat_of(p, r0 + r), lr = r0 + r - p.row_start[mi];
        p.out[mi][(long long)m * p.ld_out[mi] + lr] = __float2bfloat16_rn(acc_s[(size_t)r * (8 * MT) + m]);
    }
    if (PLZ_PROF_ON(p.prof) && threadIdx.x == 0) {
        unsigned long long* o = p.prof + 8ull * blockIdx.x;
        o[0] = t_a - t_entry; o[1] = t_pro - t_entry; o[2] = t_sync - t_entry; o[3] = t_comp - t_entry;
        o[4] = clock64() - t_entry;
    }
}

}  // namespace

int g_smallm_overlap = 0;  // plz_set_smallm_overlap

// Returns PLZ_OK, or PLZ_ERR_UNSUPPORTED (without setting the error text) when the shape is outside this kernel's
// domain and the caller should use another small-M kernel. `mats` matrices (1..4) share x, K and the palette grouping.
int launch_lut_smallm_mma_multi(const GemvArgs* mats, int count, cudaStream_t stream) {
    if (count < 1 || count > kMaxMats) return PLZ_ERR_UNSUPPORTED;
    const GemvArgs& a = mats[0];
    if (a.M < 1 || a.M > 16 || a.K % 256 || a.gs_k % 256 || ((uintptr_t)a.x & 15) || (a.ldx & 7)) return PLZ_ERR_UNSUPPORTED;
    SmallmParams p = {};
    int total = 0;
    for (int i = 0; i < count; ++i) {
        const GemvArgs& b = mats[i];
        if (b.K != a.K || b.gs_n != a.gs_n || b.gs_k != a.gs_k || b.M != a.M || b.x != a.x || b.ldx != a.ldx) return PLZ_ERR_UNSUPPORTED;
        if ((b.packed_pitch & 15) || ((uintptr_t)b.packed & 15) || ((uintptr_t)b.palette & 7)) return PLZ_ERR_UNSUPPORTED;
        p.packed[i] = (const uint8_t*)b.packed; p.pitch[i] = b.packed_pitch;
        p.palette[i] = (const __nv_bfloat16*)b.palette;
        p.out[i] = (__nv_bfloat16*)b.out; p.ld_out[i] = b.ld_out;
        p.row_start[i] = total;
        total += b.N;
    }
    for (int i = count; i <= kMaxMats; ++i) p.row_start[i] = total;
    p.n_mats = count;
    const int mt = a.M <= 8 ? 1 : 2;
    const int sms = a.sm_count > 0 ? a.sm_count : 1;
    int grid = sms;
    if (grid > (total + 15) / 16) grid = (total + 15) / 16;
    int rows_per_cta = (total + grid - 1) / grid;
    grid = (total + rows_per_cta - 1) / rows_per_cta;
    const int rows_pad = ((rows_per_cta + 15) / 16) * 16;
    p.x = (const __nv_bfloat16*)a.x; p.ldx = a.ldx;
    p.M = a.M; p.N = total; p.K = a.K; p.gs_n = a.gs_n; p.gs_k = a.gs_k; p.n_kgroups = a.K / a.gs_k;
    p.rows_per_cta = rows_per_cta;
    p.gs_n_shift = p.gs_k_shift = -1;
    for (int sh = 0; sh < 31; ++sh) {
        if ((1 << sh) == a.gs_n) p.gs_n_shift = sh;
        if ((1 << sh) == a.gs_k) p.gs_k_shift = sh;
    }
    p.x_pitch = (uint32_t)a.K * 2u + 32u;
    p.prof = (unsigned long long*)a.prof;
    p.status = device_status_ptr();
    // Shared memory: header | packed rows | x (M rows) | fp32 tile. The last strip may be ragged: its missing rows are read
    // (and ignored) all the same, so whatever follows the packed rows must cover 15 more rows: true with rows_pad rows
    // reserved; when that does not fit, reserve the exact rows and make the tail at least that long.
    const size_t rb = (size_t)a.K / 4;
    const size_t tail = (size_t)a.M * p.x_pitch + (size_t)rows_pad * 8 * mt * sizeof(float);
    size_t smem = kHeader + (size_t)rows_pad * rb + tail;
    p.rows_alloc = rows_pad;
    if (smem > 227u * 1024u) {
        p.rows_alloc = rows_per_cta;
        smem = kHeader + (size_t)rows_per_cta * rb + (tail > 16 * rb ? tail : 16 * rb);
    }
    if (rows_pad / 16 > (kHeader - 16) / 8) return PLZ_ERR_UNSUPPORTED;
    if (smem > 227u * 1024u) {
        // nine to sixteen rows of a wide x: two passes of up to eight rows each fit where one pass of sixteen does not
        if (a.M <= 8) return PLZ_ERR_UNSUPPORTED;
        GemvArgs half[kMaxMats];
        for (int pass = 0; pass < 2; ++pass) {
            const int m0 = pass * 8, mcount = pass == 0 ? 8 : a.M - 8;
            for (int i = 0; i < count; ++i) {
                half[i] = mats[i];
                half[i].M = mcount;
                half[i].x = (const __nv_bfloat16*)mats[i].x + (long long)m0 * mats[i].ldx;
                half[i].out = (__nv_bfloat16*)mats[i].out + (long long)m0 * mats[i].ld_out;
            }
            const int rc = launch_lut_smallm_mma_multi(half, count, stream);
            if (rc != PLZ_OK) return rc;
        }
        return PLZ_OK;
    }
    static int attr_smem[2][64] = {};
    int dev = 0;
    PLZ_CUDA_CHECK(cudaGetDevice(&dev));
    if (attr_smem[mt - 1][dev & 63] < (int)smem) {
        if (mt == 1) PLZ_CUDA_CHECK(cudaFuncSetAttribute(lut_smallm_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        else PLZ_CUDA_CHECK(cudaFuncSetAttribute(lut_smallm_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        attr_smem[mt - 1][dev & 63] = 227 * 1024;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(mt == 1 ? SmallmCfg<1>::kThreads : SmallmCfg<2>::kThreads); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = g_smallm_overlap ? 1 : 0;
    if (mt == 1) PLZ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, lut_smallm_mma_kernel<1>, p));
    else PLZ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, lut_smallm_mma_kernel<2>, p));
    ++g_launch_count;
    return PLZ_OK;
}

int launch_lut_smallm_mma(const GemvArgs& a, cudaStream_t stream) { return launch_lut_smallm_mma_multi(&a, 1, stream); }

}  // namespace plz
