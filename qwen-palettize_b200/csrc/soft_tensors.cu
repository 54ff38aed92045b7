// The soft path with its intermediates AS TENSORS: P = softmax((logits + g) / tau), W_soft and W_hard written to
// memory, and the element-wise backward that reads P and a materialised dW. The training path of this library never
// needs them (it recomputes P inside the weight-gradient epilogue and keeps dW in TMEM); they exist for callers of the
// reference's lower-level extension functions, which exchange exactly these tensors:
//   compute_P_W kernels            scripts/fused_lut_kernel.cu:1946-2004 (P AoS + W_soft + W_hard), :2097-2158 (batched)
//   soft_bwd_elementwise_aos       scripts/fused_lut_kernel.cu:1877-1924
// All tensors are addressed through element strides, so the reference's planar (4, K, N) / AoS (K, N, 4) layouts and
// this library's interleaved [N, K, 4] are the same code. Both kernels are single passes bound by HBM.
#include "plz_launch.h"
#include "soft_math.cuh"

namespace plz {

constexpr int kPwMaxItems = 12;  // descriptors per launch (they travel as kernel parameters)

struct PwTable {
    PwItem it[kPwMaxItems];
    long long first_block[kPwMaxItems + 1];
    int count;
    float inv_tau;
    int hard_from_noisy;
};

__device__ __forceinline__ void load4(const void* base, int f16, long long off, long long sp, float (&v)[4]) {
    if (f16) {
        const __half* p = reinterpret_cast<const __half*>(base) + off;
        if (sp == 1 && ((reinterpret_cast<uintptr_t>(p) & 7) == 0)) {
            const uint2 r = *reinterpret_cast<const uint2*>(p);
            const __half2 a = *reinterpret_cast<const __half2*>(&r.x), b = *reinterpret_cast<const __half2*>(&r.y);
            v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) v[q] = __half2float(p[q * sp]);
        }
    } else {
        const float* p = reinterpret_cast<const float*>(base) + off;
        if (sp == 1 && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
            const float4 r = *reinterpret_cast<const float4*>(p);
            v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) v[q] = p[q * sp];
        }
    }
}
__device__ __forceinline__ void store4(void* base, int f16, long long off, long long sp, const float (&v)[4]) {
    if (f16) {
        __half* p = reinterpret_cast<__half*>(base) + off;
        if (sp == 1 && ((reinterpret_cast<uintptr_t>(p) & 7) == 0)) {
            const __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
            uint2 r;
            r.x = *reinterpret_cast<const uint32_t*>(&a); r.y = *reinterpret_cast<const uint32_t*>(&b);
            *reinterpret_cast<uint2*>(p) = r;
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) p[q * sp] = __float2half_rn(v[q]);
        }
    } else {
        float* p = reinterpret_cast<float*>(base) + off;
        if (sp == 1 && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
            *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) p[q * sp] = v[q];
        }
    }
}
__device__ __forceinline__ void palette4(const __nv_bfloat16* palette, long long g, float (&c)[4]) {
    const uint2 praw = __ldg(reinterpret_cast<const uint2*>(palette + g * 4));
    c[0] = __uint_as_float(praw.x << 16);
    c[1] = __uint_as_float(praw.x & 0xFFFF0000u);
    c[2] = __uint_as_float(praw.y << 16);
    c[3] = __uint_as_float(praw.y & 0xFFFF0000u);
}

// One thread per weight. Consecutive threads walk the axis along which the logits are contiguous.
__global__ void __launch_bounds__(256) soft_weights_kernel(const __grid_constant__ PwTable t) {
    int li = 0;
#pragma unroll 1
    while (li + 1 < t.count && (long long)blockIdx.x >= t.first_block[li + 1]) ++li;
    const PwItem& d = t.it[li];
    const long long i = ((long long)blockIdx.x - t.first_block[li]) * 256 + threadIdx.x;
    if (i >= (long long)d.N * d.K) return;
    int n, k;
    if (d.n_fast) { n = (int)(i % d.N); k = (int)(i / d.N); }
    else { k = (int)(i % d.K); n = (int)(i / d.K); }
    float l[4], g[4] = {0.f, 0.f, 0.f, 0.f}, c[4];
    load4(d.logits, d.logits_f16, (long long)n * d.ls_n + (long long)k * d.ls_k, d.ls_p, l);
    if (d.noise_mode == NOISE_TENSOR) {
        load4(d.noise, 0, (long long)n * d.ns_n + (long long)k * d.ns_k, d.ns_p, g);
    } else if (d.noise_mode == NOISE_HASH) {
        const uint32_t e = ((uint32_t)k * (uint32_t)d.N + (uint32_t)n) * 4u;
#pragma unroll
        for (int q = 0; q < 4; ++q) g[q] = gumbel_hash(d.seed, e + q);
    }
    palette4(d.palette, (long long)(n / d.gs_n) * d.n_kgroups + k / d.gs_k, c);
    const Soft4 s = soft4(l, g, c, t.inv_tau);
    if (d.P) store4(d.P, 1, (long long)n * d.p_n + (long long)k * d.p_k, d.p_p, s.P);
    if (d.w_soft) d.w_soft[(long long)n * d.ws_n + (long long)k * d.ws_k] = __float2bfloat16_rn(s.w_soft);
    if (d.w_hard) {
        const int h = t.hard_from_noisy ? argmax4_first(s.P[0], s.P[1], s.P[2], s.P[3]) : argmax4_first(l[0], l[1], l[2], l[3]);
        d.w_hard[(long long)n * d.wh_n + (long long)k * d.wh_k] = __float2bfloat16_rn(c[h]);
    }
}

int launch_soft_weights(const PwItem* items, int count, float tau, int hard_from_noisy, cudaStream_t stream) {
    if (!(tau > 0.f)) { set_last_error("soft_weights: tau must be positive"); return PLZ_ERR_BAD_SHAPE; }
    for (int first = 0; first < count; first += kPwMaxItems) {
        PwTable t = {};
        t.count = (count - first < kPwMaxItems) ? (count - first) : kPwMaxItems;
        t.inv_tau = 1.0f / tau;
        t.hard_from_noisy = hard_from_noisy;
        long long blocks = 0;
        for (int i = 0; i < t.count; ++i) {
            const PwItem& d = items[first + i];
            if (d.N <= 0 || d.K <= 0 || d.gs_n <= 0 || d.gs_k <= 0 || d.N % d.gs_n || d.K % d.gs_k) {
                set_last_error("soft_weights: bad shape or grouping in matrix %d", first + i); return PLZ_ERR_BAD_SHAPE;
            }
            if (!d.logits || !d.palette) { set_last_error("soft_weights: null logits or palette in matrix %d", first + i); return PLZ_ERR_NULL; }
            if (d.noise_mode == NOISE_TENSOR && !d.noise) { set_last_error("soft_weights: null noise tensor"); return PLZ_ERR_NULL; }
            if ((uintptr_t)d.palette & 7) { set_last_error("soft_weights: palette must be 8-byte aligned"); return PLZ_ERR_BAD_ALIGN; }
            t.it[i] = d;
            t.first_block[i] = blocks;
            blocks += ((long long)d.N * d.K + 255) / 256;
        }
        t.first_block[t.count] = blocks;
        if (blocks == 0) continue;
        if (blocks > 0x7FFFFFFFll) { set_last_error("soft_weights: too many elements for one launch"); return PLZ_ERR_TOO_LARGE; }
        soft_weights_kernel<<<(unsigned)blocks, 256, 0, stream>>>(t);
        PLZ_LAUNCH_CHECK();
    }
    return PLZ_OK;
}

// dLogits[p] = dW * P[p] * (c[p] - sum_q P[q] c[q]);  dPalette[group][p] += dW * P[p]
// The palette-gradient partials of a warp are summed with shuffles when all its lanes fall into one group (always the
// case for the reference layout, where 256 consecutive n share a palette), then one atomic per entry and warp.
struct BwdElemParams {
    const void* dW; int dw_dtype; long long dw_n, dw_k;  // 0 fp32, 2 bf16
    const __half* P; long long p_n, p_k, p_p;
    const __nv_bfloat16* palette; int gs_n, gs_k, n_kgroups;
    int N, K, n_fast;
    void* dlogits; int dl_f16; long long dl_n, dl_k, dl_p;
    float* dpalette;
};

__global__ void __launch_bounds__(256) soft_bwd_elementwise_kernel(const BwdElemParams d) {
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    const bool in = i < (long long)d.N * d.K;
    int n = 0, k = 0;
    if (in) {
        if (d.n_fast) { n = (int)(i % d.N); k = (int)(i / d.N); }
        else { k = (int)(i % d.K); n = (int)(i / d.K); }
    }
    float part[4] = {0.f, 0.f, 0.f, 0.f};
    const long long grp = (long long)(n / d.gs_n) * d.n_kgroups + k / d.gs_k;
    if (in) {
        const long long wo = (long long)n * d.dw_n + (long long)k * d.dw_k;
        const float gw = d.dw_dtype == 0 ? reinterpret_cast<const float*>(d.dW)[wo]
                                         : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(d.dW)[wo]);
        float p[4], c[4], dl[4];
        load4(d.P, 1, (long long)n * d.p_n + (long long)k * d.p_k, d.p_p, p);
        palette4(d.palette, grp, c);
        const float w_soft = p[0] * c[0] + p[1] * c[1] + p[2] * c[2] + p[3] * c[3];
#pragma unroll
        for (int q = 0; q < 4; ++q) { part[q] = gw * p[q]; dl[q] = part[q] * (c[q] - w_soft); }
        if (d.dlogits) store4(d.dlogits, d.dl_f16, (long long)n * d.dl_n + (long long)k * d.dl_k, d.dl_p, dl);
    }
    if (d.dpalette == nullptr) return;
    const long long g0 = __shfl_sync(0xFFFFFFFFu, grp, 0);
    const bool uniform = __all_sync(0xFFFFFFFFu, !in || grp == g0);
    if (uniform) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float v = part[q];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
            if ((threadIdx.x & 31) == 0) atomicAdd(d.dpalette + g0 * 4 + q, v);
        }
    } else if (in) {
#pragma unroll
        for (int q = 0; q < 4; ++q) atomicAdd(d.dpalette + grp * 4 + q, part[q]);
    }
}

int launch_soft_bwd_elementwise(const BwdElemArgs& a, cudaStream_t stream) {
    if (a.N <= 0 || a.K <= 0) return PLZ_OK;
    if (!a.dW || !a.P || !a.palette) { set_last_error("soft_bwd_elementwise: null input"); return PLZ_ERR_NULL; }
    if (a.dw_dtype != 0 && a.dw_dtype != 2) { set_last_error("soft_bwd_elementwise: dW must be fp32 (0) or bf16 (2)"); return PLZ_ERR_UNSUPPORTED; }
    if (a.gs_n <= 0 || a.gs_k <= 0 || a.N % a.gs_n || a.K % a.gs_k) { set_last_error("soft_bwd_elementwise: bad grouping"); return PLZ_ERR_BAD_SHAPE; }
    if ((uintptr_t)a.palette & 7) { set_last_error("soft_bwd_elementwise: palette must be 8-byte aligned"); return PLZ_ERR_BAD_ALIGN; }
    BwdElemParams d;
    d.dW = a.dW; d.dw_dtype = a.dw_dtype; d.dw_n = a.dw_n; d.dw_k = a.dw_k;
    d.P = (const __half*)a.P; d.p_n = a.p_n; d.p_k = a.p_k; d.p_p = a.p_p;
    d.palette = (const __nv_bfloat16*)a.palette; d.gs_n = a.gs_n; d.gs_k = a.gs_k; d.n_kgroups = a.K / a.gs_k;
    d.N = a.N; d.K = a.K;
    d.n_fast = (a.p_n <= a.p_k) ? 1 : 0;  // walk the axis along which P is denser
    d.dlogits = a.dlogits; d.dl_f16 = a.dl_f16; d.dl_n = a.dl_n; d.dl_k = a.dl_k; d.dl_p = a.dl_p;
    d.dpalette = a.dpalette;
    const long long blocks = ((long long)a.N * a.K + 255) / 256;
    if (blocks > 0x7FFFFFFFll) { set_last_error("soft_bwd_elementwise: too many elements"); return PLZ_ERR_TOO_LARGE; }
    soft_bwd_elementwise_kernel<<<(unsigned)blocks, 256, 0, stream>>>(d);
    PLZ_LAUNCH_CHECK();
    return PLZ_OK;
}

// out[n] += sum_m dY[m, n] (the bias gradient, scripts/fused_lut_kernel.cu:1129: grad_bias = grad_y.sum(0)).
// One block per 64 columns x a slice of rows; 8 row-lanes x 32 column-pairs per block, fp32 partials, one atomic per
// column and block.
__global__ void __launch_bounds__(256) col_sum_kernel(const __nv_bfloat16* __restrict__ dY, long long ld, int M, int N,
                                                      int rows_per_block, float* __restrict__ out) {
    __shared__ float red[8][64];
    const int c0 = blockIdx.x * 64 + (threadIdx.x & 31) * 2;
    const int r_lane = threadIdx.x >> 5;
    const int m0 = blockIdx.y * rows_per_block;
    int m1 = m0 + rows_per_block;
    if (m1 > M) m1 = M;
    float s0 = 0.f, s1 = 0.f;
    if (c0 < N) {
        for (int m = m0 + r_lane; m < m1; m += 8) {
            const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(dY + (long long)m * ld + c0);
            s0 += __low2float(v); s1 += __high2float(v);
        }
    }
    red[r_lane][(threadIdx.x & 31) * 2] = s0;
    red[r_lane][(threadIdx.x & 31) * 2 + 1] = s1;
    __syncthreads();
    if (threadIdx.x < 64) {
        float s = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) s += red[r][threadIdx.x];
        const int c = blockIdx.x * 64 + threadIdx.x;
        if (c < N) atomicAdd(out + c, s);
    }
}

int launch_col_sum(const void* dY, long long ld, int M, int N, float* out, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return PLZ_OK;
    const int col_blocks = (N + 63) / 64;
    int dev = 0, sms = 0;
    PLZ_CUDA_CHECK(cudaGetDevice(&dev));
    PLZ_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    int row_blocks = (sms * 8 + col_blocks - 1) / col_blocks;  // about eight blocks per SM
    if (row_blocks < 1) row_blocks = 1;
    int rows_per_block = (M + row_blocks - 1) / row_blocks;
    if (rows_per_block < 64) rows_per_block = 64;
    row_blocks = (M + rows_per_block - 1) / rows_per_block;
    col_sum_kernel<<<dim3(col_blocks, row_blocks), 256, 0, stream>>>((const __nv_bfloat16*)dY, ld, M, N, rows_per_block, out);
    PLZ_LAUNCH_CHECK();
    return PLZ_OK;
}

}  // namespace plz
