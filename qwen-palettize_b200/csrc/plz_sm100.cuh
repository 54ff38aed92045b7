// Device-side primitives for the sm_100a kernels of this library: mbarrier with
// bounded waits, TMA (cp.async.bulk.tensor, never multicast), tcgen05 MMA / TMEM,
// shared-memory matrix descriptors and the 2-bit palette decode.
//
// Every wait in here is bounded: after PLZ_WAIT_LIMIT_NS without progress the
// waiter records an error code in the global status word and returns false, so
// that the caller can leave its loop, release TMEM and exit with the context intact.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#ifndef PLZ_WAIT_LIMIT_NS
#define PLZ_WAIT_LIMIT_NS 2000000000ull  // 2 s
#endif

// Cycle counters inside the kernels exist only in a diagnostics build (-DPLZ_DIAGNOSTICS); otherwise the
// condition is a compile-time false and the counter code disappears.
#ifdef PLZ_DIAGNOSTICS
#define PLZ_PROF_ON(ptr) ((ptr) != nullptr)
#else
#define PLZ_PROF_ON(ptr) false
#endif

namespace plz {

// ---------------------------------------------------------------------------
// status word (one per loaded library, static device memory)
// ---------------------------------------------------------------------------
enum : uint32_t {
    ST_OK = 0,
    ST_TIMEOUT_FULL = 1,    // consumer gave up waiting for a filled stage
    ST_TIMEOUT_EMPTY = 2,   // producer gave up waiting for a free stage
    ST_TIMEOUT_ACCUM = 3,   // epilogue gave up waiting for the accumulator
    ST_TIMEOUT_DRAIN = 4,   // teardown gave up waiting for copies in flight
};

struct StatusWord {
    unsigned int code;   // first error code seen (0 = ok)
    unsigned int where;  // blockIdx.x | role << 24
    unsigned int count;  // number of errors
    unsigned int pad;
};

// Programmatic dependent launch: let the next kernel of the stream start (it will wait for this one to finish before it
// reads what this one writes), and wait for the previous kernel to have finished. Both are no-ops in a launch without the
// programmatic-stream-serialization attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void report(StatusWord* st, uint32_t code, uint32_t role) {
    if (st == nullptr) return;
    atomicAdd(&st->count, 1u);
    if (atomicCAS(&st->code, 0u, code) == 0u) st->where = (blockIdx.x & 0xFFFFFFu) | (role << 24);
}

// ---------------------------------------------------------------------------
// small helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\telect.sync _|p, 0xFFFFFFFF;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait. `abort_flag` is a CTA-shared word: once any role has given up,
// the others stop waiting as soon as they poll it.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          StatusWord* st, uint32_t code, uint32_t role) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
    uint32_t polls = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++polls & 63u) == 0u) {
            if (*abort_flag != 0u) return false;
            if (globaltimer_ns() - t0 > PLZ_WAIT_LIMIT_NS) {
                *abort_flag = 1u;
                report(st, code, role);
                return false;
            }
        }
    }
}

// The same bounded wait for the one thread that issues the MMAs: every instruction on its path delays the tensor
// pipe (a lone thread retires a dependent instruction every five or six cycles, and a 128 x 256 x 16 MMA lasts 128), so
// the usual case -- the barrier has already completed -- is a single try_wait and the polling loop is kept out of line.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, StatusWord* st,
                                            uint32_t code, uint32_t role) {
    return mbar_wait(bar, parity, abort_flag, st, code, role);
}
__device__ __forceinline__ bool mbar_wait_lean(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, StatusWord* st,
                                               uint32_t code, uint32_t role) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, st, code, role);
}

// ---------------------------------------------------------------------------
// proxies and fences
// ---------------------------------------------------------------------------
// generic-proxy writes to shared memory -> visible to the async proxy (UMMA / TMA)
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------
// TMA: 2-D tiled load into this CTA's shared memory, completion on an mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar,
                                            int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
        "%4}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
// TMA store of one box from this CTA's shared memory; elements outside the tensor are clipped.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src_smem, int32_t x, int32_t y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src_smem), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all of this thread's bulk stores have finished READING shared memory (the source may be overwritten)
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all of this thread's bulk stores are complete (writes visible)
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---------------------------------------------------------------------------
// TMEM + tcgen05
// ---------------------------------------------------------------------------
// Executed by one full warp. ncols: power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t result_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_smem),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc], bf16 inputs, fp32 accumulate. One thread issues.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The same instruction with each 64-bit shared-memory descriptor given as its two 32-bit words. Only the low word
// (start address >> 4, leading byte offset) changes inside a main loop, by a constant per 16-element step, so the issuing
// thread spends one integer add per operand and MMA instead of rebuilding descriptors.
template <int CTA_GROUP>
__device__ __forceinline__ void umma_bf16_words(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                                uint32_t idesc, uint32_t accumulate) {
    if (CTA_GROUP == 2) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t}"
            ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
            ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}
// mbarrier arrives once every tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// ---------------------------------------------------------------------------
// CTA pairs (clusters of two, tcgen05 cta_group::2)
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the LEADER's (cluster rank 0) copy of a shared-memory location of this CTA
__device__ __forceinline__ uint32_t leader_addr(uint32_t own_addr) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(r) : "r"(own_addr));
    return r;
}
// arrive on a barrier given by its shared::cluster address (the leader's copy, from either CTA of the pair)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
// 2-D TMA load into THIS CTA's shared memory whose bytes complete on a barrier that may live in the partner CTA
// (no multicast: every CTA issues its own copies)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar_cluster_addr, int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}
// executed by the same warp of BOTH CTAs of the pair
__device__ __forceinline__ void tmem_alloc_pair(uint32_t result_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// the barrier at this offset in BOTH CTAs arrives once every tcgen05 operation issued so far by this thread has completed
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3)
                 : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives lane (base_lane + i).
// The load and its wait sit in one asm statement so that no use of the results can be scheduled
// between them.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
          "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
          "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
          "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
          "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(taddr)
        : "memory");
}

// ---------------------------------------------------------------------------
// descriptors
// ---------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1 (Blackwell).
//   bits [0,14)  start address >> 4        bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4   bits [46,48) version = 1
//   bits [61,64) layout type: 2 = SWIZZLE_128B
// K-major tile (rows = M or N index, 64 bf16 = 128 B of K per row): 8 rows form a
// 1024-byte swizzle atom; SBO = 1024 (next 8 rows); LBO unused.
// MN-major tile (rows = K index, 64 bf16 of M/N per row): atom = 64 MN x 8 K = 1024 B;
// SBO = 1024 (next 8 K rows); LBO = bytes between 64-wide MN column blocks.
__device__ __forceinline__ uint64_t make_sdesc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor for kind::f16, bf16 x bf16 -> fp32.
//   bits [4,6) D format (1 = f32), [7,10) A format (1 = bf16), [10,13) B format (1 = bf16),
//   bit 15 A major (1 = MN), bit 16 B major (1 = MN), bits [17,23) N >> 3, bits [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc(int M, int N, int a_mn_major, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// byte offset of 16-byte chunk `c` (0..7) in row `r` of a 128-byte-swizzled tile whose
// rows are 128 bytes and whose base is 1024-byte aligned (same pattern TMA SWIZZLE_128B writes)
__device__ __forceinline__ uint32_t swz128(uint32_t r, uint32_t c) {
    return r * 128u + ((c ^ (r & 7u)) << 4);
}

// ---------------------------------------------------------------------------
// 2-bit palette decode (bit-exact: pure byte permutes of the palette entries)
// ---------------------------------------------------------------------------
// Palette of one group as loaded from memory: p01 = {c0, c1}, p23 = {c2, c3} (bf16 pairs), i.e. entry i is bytes 2i, 2i + 1
// of the 8-byte pair {p01, p23}.
struct PalRegs {
    uint32_t lo;  // p01
    uint32_t hi;  // p23
};
__device__ __forceinline__ PalRegs pal_split(uint32_t p01, uint32_t p23) {
    PalRegs r;
    r.lo = p01;
    r.hi = p23;
    return r;
}
// prmt.b32 without the selector mask that the __byte_perm intrinsic adds: every selector nibble here is 0..7 by construction
__device__ __forceinline__ uint32_t prmt_raw(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
// 16 packed indices (element j in bits 2j..2j+1) -> 16 bf16 (out[j/2] holds elements j, j+1).
// An element with index i is the two palette bytes 2i, 2i + 1: selector byte 0x22 * i + 0x10. One mask + multiply-add makes the
// selector bytes of four elements at once (elements e, 4 + e, 8 + e, 12 + e for the bit pair e of every byte); two byte
// permutes interleave them into the order of the elements, and one permute of the palette per element pair does the
// look-up: 23 ALU instructions and 4 multiply-adds per 16 weights.
__device__ __forceinline__ void decode16(uint32_t w, const PalRegs& pal, uint32_t* out) {
    const uint32_t sa = (w & 0x03030303u) * 0x22u + 0x10101010u;          // elements 0, 4, 8, 12
    const uint32_t sb = ((w >> 2) & 0x03030303u) * 0x22u + 0x10101010u;   // 1, 5, 9, 13
    const uint32_t sc = ((w >> 4) & 0x03030303u) * 0x22u + 0x10101010u;   // 2, 6, 10, 14
    const uint32_t sd = ((w >> 6) & 0x03030303u) * 0x22u + 0x10101010u;   // 3, 7, 11, 15
    const uint32_t ab0 = prmt_raw(sa, sb, 0x5140u), ab1 = prmt_raw(sa, sb, 0x7362u);   // (0,1 | 4,5), (8,9 | 12,13)
    const uint32_t cd0 = prmt_raw(sc, sd, 0x5140u), cd1 = prmt_raw(sc, sd, 0x7362u);   // (2,3 | 6,7), (10,11 | 14,15)
    out[0] = prmt_raw(pal.lo, pal.hi, ab0);
    out[1] = prmt_raw(pal.lo, pal.hi, cd0);
    out[2] = prmt_raw(pal.lo, pal.hi, ab0 >> 16);
    out[3] = prmt_raw(pal.lo, pal.hi, cd0 >> 16);
    out[4] = prmt_raw(pal.lo, pal.hi, ab1);
    out[5] = prmt_raw(pal.lo, pal.hi, cd1);
    out[6] = prmt_raw(pal.lo, pal.hi, ab1 >> 16);
    out[7] = prmt_raw(pal.lo, pal.hi, cd1 >> 16);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

}  // namespace plz
