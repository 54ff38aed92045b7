// Bandwidth-bound companions of the GEMM kernels: index packing, hard-index selection and soft-weight
// construction from the index logits, and a dequantizer used by the bit-exactness tests.
//
// Packed format (identical to the reference's .idx2 bit order, scripts/palettize_core.py:31-42):
// element k of a row lives in byte k / 4, bits 2 * (k % 4) .. 2 * (k % 4) + 1. Rows are weight
// rows n (K contiguous), i.e. packed[n, k / 4].
#include "plz_launch.h"
#include "soft_math.cuh"

namespace plz {

// ---------------------------------------------------------------------------------------------
// pack: unpacked int8 indices -> packed [N, K/4]
//   src element (n, k) at src[n * s_n + k * s_k]; layout R (K, N) row-major: s_n = 1, s_k = N.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
pack_indices_kernel(const int8_t* __restrict__ src, long long s_n, long long s_k, int N, int K,
                    uint8_t* __restrict__ dst, long long pitch) {
    __shared__ uint8_t tile[32][33];
    const int n0 = blockIdx.x * 32, kb0 = blockIdx.y * 32;  // kb = byte index along K
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    if (s_n == 1) {
        // n fastest in memory: threads of a warp walk n, then transpose through shared memory
        for (int b = ty; b < 32; b += 8) {
            const int n = n0 + tx, kb = kb0 + b;
            uint8_t v = 0;
            if (n < N && kb * 4 < K) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int k = kb * 4 + j;
                    if (k < K) v |= (uint8_t)((src[(long long)n * s_n + (long long)k * s_k] & 3) << (2 * j));
                }
            }
            tile[tx][b] = v;
        }
        __syncthreads();
        for (int r = ty; r < 32; r += 8) {
            const int n = n0 + r, kb = kb0 + tx;
            if (n < N && kb * 4 < K) dst[(long long)n * pitch + kb] = tile[r][tx];
        }
    } else {
        for (int r = ty; r < 32; r += 8) {
            const int n = n0 + r, kb = kb0 + tx;
            if (n < N && kb * 4 < K) {
                uint8_t v = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int k = kb * 4 + j;
                    if (k < K) v |= (uint8_t)((src[(long long)n * s_n + (long long)k * s_k] & 3) << (2 * j));
                }
                dst[(long long)n * pitch + kb] = v;
            }
        }
    }
}

int launch_pack_indices(const void* src, long long s_n, long long s_k, int N, int K, void* dst, long long pitch,
                        cudaStream_t stream) {
    if (N <= 0 || K <= 0) return PLZ_OK;
    dim3 grid((N + 31) / 32, ((K + 3) / 4 + 31) / 32);
    pack_indices_kernel<<<grid, 256, 0, stream>>>((const int8_t*)src, s_n, s_k, N, K, (uint8_t*)dst, pitch);
    PLZ_LAUNCH_CHECK();
    return PLZ_OK;
}

// unpack: packed [N, K/4] -> int8 at dst[n * s_n + k * s_k]
__global__ void __launch_bounds__(256)
unpack_indices_kernel(const uint8_t* __restrict__ src, long long pitch, int N, int K, int8_t* __restrict__ dst,
                      long long s_n, long long s_k) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)N * K;
    if (i >= total) return;
    // walk the fastest destination axis with consecutive threads
    int n, k;
    if (s_n == 1) { n = (int)(i % N); k = (int)(i / N); }
    else { k = (int)(i % K); n = (int)(i / K); }
    const uint8_t b = src[(long long)n * pitch + (k >> 2)];
    dst[(long long)n * s_n + (long long)k * s_k] = (int8_t)((b >> (2 * (k & 3))) & 3);
}

int launch_unpack_indices(const void* src, long long pitch, int N, int K, void* dst, long long s_n, long long s_k,
                          cudaStream_t stream) {
    const long long total = (long long)N * K;
    if (total <= 0) return PLZ_OK;
    unpack_indices_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>((const uint8_t*)src, pitch, N, K,
                                                                               (int8_t*)dst, s_n, s_k);
    PLZ_LAUNCH_CHECK();
    return PLZ_OK;
}

// ---------------------------------------------------------------------------------------------
// dequantize: W[n, k] = palette[(n / gs_n) * n_kgroups + k / gs_k][idx[n, k]] as bf16, written at
// dst[n * d_n + k * d_k]. Uses the same byte-permute decode as the GEMM producer warps.
// One thread per 16 consecutive k.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
dequant_kernel(const uint8_t* __restrict__ packed, long long pitch, const __nv_bfloat16* __restrict__ palette,
               int gs_n, int gs_k, int n_kgroups, int N, int K, __nv_bfloat16* __restrict__ dst, long long d_n,
               long long d_k) {
    const int words = K / 16;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)N * words) return;
    const int n = (int)(i / words), wq = (int)(i % words);
    const int k0 = wq * 16;
    const uint32_t w = *reinterpret_cast<const uint32_t*>(packed + (long long)n * pitch + wq * 4);
    const long long g = (long long)(n / gs_n) * n_kgroups + k0 / gs_k;
    const uint2 praw = *reinterpret_cast<const uint2*>(palette + g * 4);
    const PalRegs pal = pal_split(praw.x, praw.y);
    uint32_t o[8];
    decode16(w, pal, o);
    if (d_k == 1) {
        uint4* d = reinterpret_cast<uint4*>(dst + (long long)n * d_n + k0);
        d[0] = make_uint4(o[0], o[1], o[2], o[3]);
        d[1] = make_uint4(o[4], o[5], o[6], o[7]);
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint16_t h = (uint16_t)(o[j >> 1] >> (16 * (j & 1)));
            reinterpret_cast<uint16_t*>(dst)[(long long)n * d_n + (long long)(k0 + j) * d_k] = h;
        }
    }
}

int launch_dequant(const void* packed, long long pitch, const void* palette, int gs_n, int gs_k, int N, int K,
                   void* dst, long long d_n, long long d_k, cudaStream_t stream) {
    if (N <= 0 || K <= 0) return PLZ_OK;
    if (K % 16 || gs_k % 16 || K % gs_k) { set_last_error("dequant: K and gs_k must be multiples of 16, gs_k | K"); return PLZ_ERR_BAD_SHAPE; }
    if ((pitch & 3) || ((uintptr_t)packed & 3) || ((uintptr_t)palette & 7)) { set_last_error("dequant: misaligned input"); return PLZ_ERR_BAD_ALIGN; }
    if (d_k == 1 && ((d_n & 7) || ((uintptr_t)dst & 15))) { set_last_error("dequant: misaligned output"); return PLZ_ERR_BAD_ALIGN; }
    const long long total = (long long)N * (K / 16);
    dequant_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
        (const uint8_t*)packed, pitch, (const __nv_bfloat16*)palette, gs_n, gs_k, K / gs_k, N, K,
        (__nv_bfloat16*)dst, d_n, d_k);
    PLZ_LAUNCH_CHECK();
    return PLZ_OK;
}

// ---------------------------------------------------------------------------------------------
// soft_select: from the index logits build, in one pass over them,
//   * the packed hard indices argmax_p logits[p] (plain logits, first maximum wins), and / or
//   * the soft weights W_soft[n, k] = sum_p softmax((logits + g) / tau)[p] * palette[p] as bf16 [N, K].
// Logit element (n, k, p) at logits[n * ls_n + k * ls_k + p * ls_p]; same for the noise tensor.
// Two thread mappings: k fastest (interleaved fp32 [N, K, 4]) and n fastest (planar [4, K, N]);
// the planar one transposes the packed bytes through shared memory so both sides stay coalesced.
// ---------------------------------------------------------------------------------------------

template <typename LogitT>
__device__ __forceinline__ void select_one(const SelectParams& p, int n, int k, int& hard, uint16_t& wsoft_bits) {
    const LogitT* lg = reinterpret_cast<const LogitT*>(p.logits);
    const long long lo = (long long)n * p.ls_n + (long long)k * p.ls_k;
    float l[4];
    if (sizeof(LogitT) == 4 && p.ls_p == 1) {
        const float4 v = __ldcs(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.logits) + lo));
        l[0] = v.x; l[1] = v.y; l[2] = v.z; l[3] = v.w;
    } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) l[q] = to_f32(lg[lo + q * p.ls_p]);
    }
    hard = argmax4_first(l[0], l[1], l[2], l[3]);
    if (p.w_soft != nullptr) {
        float g[4] = {0.f, 0.f, 0.f, 0.f};
        if (p.noise_mode == NOISE_TENSOR) {
            const long long no = (long long)n * p.ns_n + (long long)k * p.ns_k;
            if (p.ns_p == 1) {
                const float4 v = __ldcs(reinterpret_cast<const float4*>(p.noise + no));
                g[0] = v.x; g[1] = v.y; g[2] = v.z; g[3] = v.w;
            } else {
#pragma unroll
                for (int q = 0; q < 4; ++q) g[q] = __ldcs(p.noise + no + q * p.ns_p);
            }
        } else if (p.noise_mode == NOISE_HASH) {
            const uint32_t e = ((uint32_t)k * (uint32_t)p.N + (uint32_t)n) * 4u;
#pragma unroll
            for (int q = 0; q < 4; ++q) g[q] = gumbel_hash(p.seed, e + q);
        }
        const long long pg = ((long long)(n / p.gs_n) * p.n_kgroups + k / p.gs_k) * 4;
        const uint2 praw = __ldg(reinterpret_cast<const uint2*>(p.palette + pg));
        float c[4];
        c[0] = __uint_as_float(praw.x << 16);
        c[1] = __uint_as_float(praw.x & 0xFFFF0000u);
        c[2] = __uint_as_float(praw.y << 16);
        c[3] = __uint_as_float(praw.y & 0xFFFF0000u);
        const Soft4 s = soft4(l, g, c, p.inv_tau);
        const __nv_bfloat16 b = __float2bfloat16_rn(s.w_soft);
        wsoft_bits = *reinterpret_cast<const uint16_t*>(&b);
    }
}

// k fastest: one thread per 4 consecutive k (one packed byte)
template <typename LogitT>
__global__ void __launch_bounds__(256) soft_select_kfast_kernel(const SelectParams p) {
    const int kbytes = (p.K + 3) / 4;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)p.N * kbytes) return;
    const int n = (int)(i / kbytes), kb = (int)(i % kbytes);
    uint8_t byte = 0;
    uint16_t ws[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int k = kb * 4 + j;
        if (k < p.K) {
            int hard;
            select_one<LogitT>(p, n, k, hard, ws[j]);
            byte |= (uint8_t)(hard << (2 * j));
        }
    }
    if (p.packed) p.packed[(long long)n * p.pitch + kb] = byte;
    if (p.w_soft) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = kb * 4 + j;
            if (k < p.K) reinterpret_cast<uint16_t*>(p.w_soft)[(long long)n * p.ws_n + (long long)k * p.ws_k] = ws[j];
        }
    }
}

// n fastest: block = 32 n x 32 bytes of k (128 k); warps walk n
template <typename LogitT>
__global__ void __launch_bounds__(256) soft_select_nfast_kernel(const SelectParams p) {
    __shared__ uint8_t tile[32][33];
    const int n0 = blockIdx.x * 32, kb0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int b = ty; b < 32; b += 8) {
        const int n = n0 + tx, kb = kb0 + b;
        uint8_t byte = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = kb * 4 + j;
            if (n < p.N && k < p.K) {
                int hard;
                uint16_t ws = 0;
                select_one<LogitT>(p, n, k, hard, ws);
                byte |= (uint8_t)(hard << (2 * j));
                if (p.w_soft) reinterpret_cast<uint16_t*>(p.w_soft)[(long long)n * p.ws_n + (long long)k * p.ws_k] = ws;
            }
        }
        tile[tx][b] = byte;
    }
    if (p.packed) {
        __syncthreads();
        for (int r = ty; r < 32; r += 8) {
            const int n = n0 + r, kb = kb0 + tx;
            if (n < p.N && kb * 4 < p.K) p.packed[(long long)n * p.pitch + kb] = tile[r][tx];
        }
    }
}

int launch_soft_select(const SelectParams& p, int logits_f16, cudaStream_t stream) {
    if (p.N <= 0 || p.K <= 0) return PLZ_OK;
    if (!p.logits) { set_last_error("soft_select: null logits"); return PLZ_ERR_NULL; }
    if (p.w_soft && !p.palette) { set_last_error("soft_select: null palette"); return PLZ_ERR_NULL; }
    if (p.w_soft && p.noise_mode == NOISE_TENSOR && !p.noise) { set_last_error("soft_select: null noise"); return PLZ_ERR_NULL; }
    if (!logits_f16 && p.ls_p == 1 && (((uintptr_t)p.logits & 15) || (p.ls_n % 4) || (p.ls_k % 4))) {
        set_last_error("soft_select: interleaved fp32 logits must be 16-byte aligned"); return PLZ_ERR_BAD_ALIGN;
    }
    if (p.w_soft && p.noise_mode == NOISE_TENSOR && p.ns_p == 1 && (((uintptr_t)p.noise & 15) || (p.ns_n % 4) || (p.ns_k % 4))) {
        set_last_error("soft_select: interleaved noise must be 16-byte aligned"); return PLZ_ERR_BAD_ALIGN;
    }
    const bool nfast = (p.ls_n == 1);
    if (nfast) {
        dim3 grid((p.N + 31) / 32, ((p.K + 3) / 4 + 31) / 32);
        if (logits_f16) soft_select_nfast_kernel<__half><<<grid, 256, 0, stream>>>(p);
        else soft_select_nfast_kernel<float><<<grid, 256, 0, stream>>>(p);
    } else {
        const long long total = (long long)p.N * ((p.K + 3) / 4);
        const unsigned grid = (unsigned)((total + 255) / 256);
        if (logits_f16) soft_select_kfast_kernel<__half><<<grid, 256, 0, stream>>>(p);
        else soft_select_kfast_kernel<float><<<grid, 256, 0, stream>>>(p);
    }
    PLZ_LAUNCH_CHECK();
    return PLZ_OK;
}

}  // namespace plz
