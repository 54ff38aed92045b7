// The two bandwidth-bound steps on either side of the Linear in the distillation loop:
//
//   adamw_clamp   fp32-master AdamW on a flat parameter (index logits, palettes, LoRA factors) with the gradient
//                 clip coefficient, bias correction, decoupled weight decay and the post-step clamp to +-5 tau
//                 folded into ONE pass over (grad, master, m, v) that also writes the model-dtype copy.
//                 Reference: FP32MasterAdamW = torch.optim.AdamW on fp32 masters + copy back
//                 (scripts/train_qwen.py:154-215, betas/eps :600), clip_grad_norm_ (:1303-1319),
//                 par.data.clamp_(-5 tau, 5 tau) (:1343-1348) -- eight separate passes there.
//   distill_loss  per-token 1 - cos plus MSE normalised by mean(t^2), fp32 math, forward and gradient
//                 (compute_loss, scripts/train_qwen.py:229-249).
#include "plz_launch.h"
#include "soft_math.cuh"

namespace plz {

// number of SMs of the current device (grid sizing of the grid-stride kernels below)
static int sm_count_of_current_device() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 1;
    dev &= 63;
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
        cached[dev] = n;
    }
    return cached[dev];
}

__device__ __forceinline__ float ld_as_f32(const float* p, long long i) { return p[i]; }
__device__ __forceinline__ float ld_as_f32(const __half* p, long long i) { return __half2float(p[i]); }
__device__ __forceinline__ float ld_as_f32(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void st_from_f32(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void st_from_f32(__half* p, long long i, float v) { p[i] = __float2half_rn(v); }
__device__ __forceinline__ void st_from_f32(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

template <typename GradT, typename ParamT>
__global__ void __launch_bounds__(256) adamw_clamp_kernel(const AdamParams p) {
    const GradT* g = reinterpret_cast<const GradT*>(p.grad);
    ParamT* out = reinterpret_cast<ParamT*>(p.param);
    const float step_size = p.lr / p.bias_c1;
    const bool do_clamp = p.clamp_lo <= p.clamp_hi;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < p.n; i += (long long)gridDim.x * blockDim.x) {
        const float gr = ld_as_f32(g, i) * p.grad_scale;
        float w = p.master[i];
        w *= 1.0f - p.lr * p.weight_decay;                       // decoupled weight decay (torch.optim.AdamW order)
        const float m = p.beta1 * p.m[i] + (1.0f - p.beta1) * gr;
        const float v = p.beta2 * p.v[i] + (1.0f - p.beta2) * gr * gr;
        const float denom = sqrtf(v) / p.sqrt_bias_c2 + p.eps;
        w -= step_size * (m / denom);
        float wc = w;
        if (do_clamp) wc = fminf(fmaxf(w, p.clamp_lo), p.clamp_hi);
        p.m[i] = m;
        p.v[i] = v;
        p.master[i] = p.clamp_master ? wc : w;
        if (out != nullptr) st_from_f32(out, i, wc);
    }
}

int launch_adamw(const AdamParams& p, int grad_dtype, int param_dtype, cudaStream_t stream) {
    if (p.n <= 0) return PLZ_OK;
    long long blocks = (p.n + 255) / 256;
    if (blocks > sm_count_of_current_device() * 16) blocks = sm_count_of_current_device() * 16;
#define PLZ_ADAM(GT, PT) adamw_clamp_kernel<GT, PT><<<(unsigned)blocks, 256, 0, stream>>>(p)
    if (grad_dtype == 0) {
        if (param_dtype == 0) PLZ_ADAM(float, float); else if (param_dtype == 1) PLZ_ADAM(float, __half); else PLZ_ADAM(float, __nv_bfloat16);
    } else if (grad_dtype == 1) {
        if (param_dtype == 0) PLZ_ADAM(__half, float); else if (param_dtype == 1) PLZ_ADAM(__half, __half); else PLZ_ADAM(__half, __nv_bfloat16);
    } else {
        if (param_dtype == 0) PLZ_ADAM(__nv_bfloat16, float); else if (param_dtype == 1) PLZ_ADAM(__nv_bfloat16, __half); else PLZ_ADAM(__nv_bfloat16, __nv_bfloat16);
    }
#undef PLZ_ADAM
    PLZ_LAUNCH_CHECK();
    return PLZ_OK;
}

// ---------------------------------------------------------------------------------------------
// distillation loss. ws layout (fp32): [0] sum(1 - cos), [1] sum((s-t)^2), [2] sum(t^2), [3] unused,
// then per token: dot, |s|^2, |t|^2, |s - t|^2 (4 floats). The three totals are summed by ONE block in a fixed order
// (no atomics), so the loss and everything scaled by it are bit-identical from run to run.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

// one warp per token row
__global__ void __launch_bounds__(256)
distill_stats_kernel(const __nv_bfloat16* __restrict__ s, long long lds, const __nv_bfloat16* __restrict__ t, long long ldt,
                     int M, int H, float eps, float* __restrict__ ws) {
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    for (int row = blockIdx.x * 8 + wib; row < M; row += gridDim.x * 8) {
        const __nv_bfloat16* sr = s + (long long)row * lds;
        const __nv_bfloat16* tr = t + (long long)row * ldt;
        float dot = 0.f, s2 = 0.f, t2 = 0.f, d2 = 0.f;
        for (int c = lane * 2; c < H; c += 64) {
            const float2 sv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(sr + c));
            const float2 tv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(tr + c));
            dot += sv.x * tv.x + sv.y * tv.y;
            s2 += sv.x * sv.x + sv.y * sv.y;
            t2 += tv.x * tv.x + tv.y * tv.y;
            const float dx = sv.x - tv.x, dy = sv.y - tv.y;
            d2 += dx * dx + dy * dy;
        }
        dot = warp_sum_f(dot); s2 = warp_sum_f(s2); t2 = warp_sum_f(t2); d2 = warp_sum_f(d2);
        if (lane == 0) *reinterpret_cast<float4*>(ws + 4 + 4ll * row) = make_float4(dot, s2, t2, d2);
    }
}

// one block: thread i sums rows i, i + 1024, ...; then a fixed tree over the 1024 partials
__global__ void __launch_bounds__(1024)
distill_reduce_kernel(int M, float eps, float* __restrict__ ws) {
    __shared__ float part[3][1024];
    float a_cos = 0.f, a_d2 = 0.f, a_t2 = 0.f;
    for (int row = threadIdx.x; row < M; row += 1024) {
        const float4 st = *reinterpret_cast<const float4*>(ws + 4 + 4ll * row);
        const float cosv = st.x / (fmaxf(sqrtf(st.y), eps) * fmaxf(sqrtf(st.z), eps));
        a_cos += 1.0f - cosv; a_d2 += st.w; a_t2 += st.z;
    }
    part[0][threadIdx.x] = a_cos; part[1][threadIdx.x] = a_d2; part[2][threadIdx.x] = a_t2;
    __syncthreads();
    for (int w = 512; w > 0; w >>= 1) {
        if (threadIdx.x < w) {
#pragma unroll
            for (int q = 0; q < 3; ++q) part[q][threadIdx.x] += part[q][threadIdx.x + w];
        }
        __syncthreads();
    }
    if (threadIdx.x < 3) ws[threadIdx.x] = part[threadIdx.x][0];
}

template <typename GradT>
__global__ void __launch_bounds__(256)
distill_grad_kernel(const __nv_bfloat16* __restrict__ s, long long lds, const __nv_bfloat16* __restrict__ t, long long ldt,
                    int M, int H, float eps, float w_cos, float w_mse, float upstream, const float* __restrict__ ws,
                    float* __restrict__ out4, GradT* __restrict__ ds, long long ldds) {
    const float inv_m = 1.0f / (float)M, inv_mh = 1.0f / ((float)M * (float)H);
    const float t_var = fmaxf(ws[2] * inv_mh, 1e-6f);
    if (blockIdx.x == 0 && threadIdx.x == 0 && out4 != nullptr) {
        const float l_cos = ws[0] * inv_m, l_mse = ws[1] * inv_mh / t_var;
        out4[0] = w_cos * l_cos + w_mse * l_mse; out4[1] = l_cos; out4[2] = l_mse; out4[3] = t_var;
    }
    if (ds == nullptr) return;
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const float c_mse = upstream * w_mse * 2.0f * inv_mh / t_var;
    for (int row = blockIdx.x * 8 + wib; row < M; row += gridDim.x * 8) {
        const float4 st = *reinterpret_cast<const float4*>(ws + 4 + 4ll * row);
        const float dot = st.x, s2 = st.y, t2 = st.z;
        const float ns = sqrtf(s2), nt = sqrtf(t2);
        const float cs = fmaxf(ns, eps), ct = fmaxf(nt, eps);
        // cos = dot / (cs * ct); d cos / d s = t / (cs ct) - [ns >= eps] * cos * s / ns^2 (the clamp has no slope below eps)
        const float a = 1.0f / (cs * ct);
        const float b = (ns >= eps) ? (dot * a) / s2 : 0.f;
        const float c_cos = -upstream * w_cos * inv_m;
        const __nv_bfloat16* sr = s + (long long)row * lds;
        const __nv_bfloat16* tr = t + (long long)row * ldt;
        for (int c = lane * 2; c < H; c += 64) {
            const float2 sv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(sr + c));
            const float2 tv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(tr + c));
            const float g0 = c_cos * (tv.x * a - sv.x * b) + c_mse * (sv.x - tv.x);
            const float g1 = c_cos * (tv.y * a - sv.y * b) + c_mse * (sv.y - tv.y);
            st_from_f32(ds, (long long)row * ldds + c, g0);
            st_from_f32(ds, (long long)row * ldds + c + 1, g1);
        }
    }
}

int launch_distill_loss(const void* s, long long lds, const void* t, long long ldt, int M, int H, float eps, float w_cos,
                        float w_mse, float upstream, float* ws, float* out4, void* ds, long long ldds, int ds_dtype,
                        cudaStream_t stream) {
    if (M <= 0 || H <= 0) return PLZ_OK;
    int blocks = (M + 7) / 8;
    if (blocks > sm_count_of_current_device() * 8) blocks = sm_count_of_current_device() * 8;
    distill_stats_kernel<<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)s, lds, (const __nv_bfloat16*)t, ldt, M, H, eps, ws);
    PLZ_LAUNCH_CHECK();
    distill_reduce_kernel<<<1, 1024, 0, stream>>>(M, eps, ws);
    PLZ_LAUNCH_CHECK();
    if (ds_dtype == 0)
        distill_grad_kernel<float><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)s, lds, (const __nv_bfloat16*)t, ldt, M, H, eps,
                                                                w_cos, w_mse, upstream, ws, out4, (float*)ds, ldds);
    else
        distill_grad_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)s, lds, (const __nv_bfloat16*)t, ldt, M, H,
                                                                        eps, w_cos, w_mse, upstream, ws, out4, (__nv_bfloat16*)ds, ldds);
    PLZ_LAUNCH_CHECK();
    return PLZ_OK;
}

// ---------------------------------------------------------------------------------------------
// rstd[m] = 1 / sqrt(mean_k x[m, k]^2 + eps): the per-row factor of RMSNorm. The normalisation itself is folded into
// the GEMM that consumes x (row factor in its epilogue, norm weight in its decoded operand).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
rms_rstd_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int M, int K, float eps, float* __restrict__ rstd) {
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    for (int row = blockIdx.x * 8 + wib; row < M; row += gridDim.x * 8) {
        const __nv_bfloat16* xr = x + (long long)row * ldx;
        float s2 = 0.f;
        for (int c = lane * 2; c < K; c += 64) {
            const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + c));
            s2 += v.x * v.x + v.y * v.y;
        }
        s2 = warp_sum_f(s2);
        if (lane == 0) rstd[row] = rsqrtf(s2 / (float)K + eps);
    }
}

int launch_rms_rstd(const void* x, long long ldx, int M, int K, float eps, float* rstd, cudaStream_t stream) {
    if (M <= 0) return PLZ_OK;
    int blocks = (M + 7) / 8;
    if (blocks > sm_count_of_current_device() * 8) blocks = sm_count_of_current_device() * 8;
    rms_rstd_kernel<<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, M, K, eps, rstd);
    PLZ_LAUNCH_CHECK();
    return PLZ_OK;
}

// Backward of act = silu(gate) * up, elementwise, fp32 arithmetic on bf16 operands:
//   dGate = dAct * up * sigma(gate) * (1 + gate * (1 - sigma(gate))),   dUp = dAct * silu(gate).
// Eight elements (16 bytes) per thread and step; rows may be pitched.
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gate, long long ldg, const __nv_bfloat16* __restrict__ up, long long ldu,
                  const __nv_bfloat16* __restrict__ dact, long long ldd, int M, int N, __nv_bfloat16* __restrict__ dgate,
                  long long lddg, __nv_bfloat16* __restrict__ dup, long long lddu) {
    const int vec_per_row = N >> 3;
    const long long total = (long long)M * vec_per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int m = (int)(i / vec_per_row), c = (int)(i - (long long)m * vec_per_row) << 3;
        const uint4 gv = __ldcs(reinterpret_cast<const uint4*>(gate + (long long)m * ldg + c));
        const uint4 uv = __ldcs(reinterpret_cast<const uint4*>(up + (long long)m * ldu + c));
        const uint4 dv = __ldcs(reinterpret_cast<const uint4*>(dact + (long long)m * ldd + c));
        const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w}, dw[4] = {dv.x, dv.y, dv.z, dv.w};
        uint32_t og[4], ou[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float r[2][2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float g = __uint_as_float(h ? (gw[q] & 0xFFFF0000u) : (gw[q] << 16));
                const float u = __uint_as_float(h ? (uw[q] & 0xFFFF0000u) : (uw[q] << 16));
                const float d = __uint_as_float(h ? (dw[q] & 0xFFFF0000u) : (dw[q] << 16));
                const float sg = 1.0f / (1.0f + __expf(-g));
                r[0][h] = d * u * sg * (1.0f + g * (1.0f - sg));
                r[1][h] = d * g * sg;
            }
            const __nv_bfloat162 a = __floats2bfloat162_rn(r[0][0], r[0][1]), b = __floats2bfloat162_rn(r[1][0], r[1][1]);
            og[q] = *reinterpret_cast<const uint32_t*>(&a);
            ou[q] = *reinterpret_cast<const uint32_t*>(&b);
        }
        __stcs(reinterpret_cast<uint4*>(dgate + (long long)m * lddg + c), make_uint4(og[0], og[1], og[2], og[3]));
        __stcs(reinterpret_cast<uint4*>(dup + (long long)m * lddu + c), make_uint4(ou[0], ou[1], ou[2], ou[3]));
    }
}

int launch_swiglu_bwd(const void* gate, long long ldg, const void* up, long long ldu, const void* dact, long long ldd, int M, int N,
                      void* dgate, long long lddg, void* dup, long long lddu, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return PLZ_OK;
    long long blocks = ((long long)M * (N >> 3) + 255) / 256;
    if (blocks > sm_count_of_current_device() * 16) blocks = sm_count_of_current_device() * 16;
    swiglu_bwd_kernel<<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)gate, ldg, (const __nv_bfloat16*)up, ldu,
                                                        (const __nv_bfloat16*)dact, ldd, M, N, (__nv_bfloat16*)dgate, lddg,
                                                        (__nv_bfloat16*)dup, lddu);
    PLZ_LAUNCH_CHECK();
    return PLZ_OK;
}

// Backward of h = x * rstd[m] * g[k] (RMSNorm) given dh:
//   dx[m, k] = rstd * g[k] * dh[m, k] - x[m, k] * rstd^3 / K * sum_k (x * g * dh)[m, k]
//   dg[k]   += sum_m dh[m, k] * x[m, k] * rstd[m]                       (fp32, accumulated with atomics)
// A block of 256 threads walks rows; thread t owns the column pairs 2t + 512 i, keeps its dg partial sums in registers over
// all its rows and adds them to memory once at the end.
constexpr int kNormPairsMax = 20;  // K <= 512 * 20
template <int kNormPairs>  // column pairs per thread: K <= 512 * kNormPairs
__global__ void __launch_bounds__(256)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ dh, long long lddh,
                   const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ g, int M, int K,
                   __nv_bfloat16* __restrict__ dx, long long lddx, float* __restrict__ dg) {
    __shared__ float red[8];
    const int t = threadIdx.x, lane = t & 31, wib = t >> 5;
    float gk[kNormPairs][2], acc[kNormPairs][2];
#pragma unroll
    for (int i = 0; i < kNormPairs; ++i) {
        const int c = 2 * t + 512 * i;
        acc[i][0] = acc[i][1] = 0.f;
        gk[i][0] = gk[i][1] = 0.f;
        if (c < K) {
            const float2 v = g ? __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(g + c)) : make_float2(1.f, 1.f);
            gk[i][0] = v.x; gk[i][1] = v.y;
        }
    }
    for (int row = blockIdx.x; row < M; row += gridDim.x) {
        const float rs = rstd[row];
        float xv[kNormPairs][2], dv[kNormPairs][2];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < kNormPairs; ++i) {
            const int c = 2 * t + 512 * i;
            xv[i][0] = xv[i][1] = dv[i][0] = dv[i][1] = 0.f;
            if (c < K) {
                const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + (long long)row * ldx + c));
                const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dh + (long long)row * lddh + c));
                xv[i][0] = a.x; xv[i][1] = a.y; dv[i][0] = b.x; dv[i][1] = b.y;
                s += a.x * gk[i][0] * b.x + a.y * gk[i][1] * b.y;
                acc[i][0] += b.x * a.x * rs; acc[i][1] += b.y * a.y * rs;
            }
        }
        s = warp_sum_f(s);
        __syncthreads();  // red is free again (previous row's readers are done)
        if (lane == 0) red[wib] = s;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) tot += red[w];
        const float coef = tot * rs * rs * rs / (float)K;
#pragma unroll
        for (int i = 0; i < kNormPairs; ++i) {
            const int c = 2 * t + 512 * i;
            if (c < K) {
                const __nv_bfloat162 o = __floats2bfloat162_rn(rs * gk[i][0] * dv[i][0] - xv[i][0] * coef,
                                                               rs * gk[i][1] * dv[i][1] - xv[i][1] * coef);
                *reinterpret_cast<__nv_bfloat162*>(dx + (long long)row * lddx + c) = o;
            }
        }
    }
    if (dg) {
#pragma unroll
        for (int i = 0; i < kNormPairs; ++i) {
            const int c = 2 * t + 512 * i;
            if (c < K) { atomicAdd(dg + c, acc[i][0]); atomicAdd(dg + c + 1, acc[i][1]); }
        }
    }
}

int launch_rmsnorm_bwd(const void* x, long long ldx, const void* dh, long long lddh, const float* rstd, const void* g, int M, int K,
                       void* dx, long long lddx, float* dg, cudaStream_t stream) {
    if (M <= 0) return PLZ_OK;
    if (K > 512 * kNormPairsMax) { set_last_error("rmsnorm_bwd: K=%d exceeds %d", K, 512 * kNormPairsMax); return PLZ_ERR_TOO_LARGE; }
    int blocks = M < sm_count_of_current_device() * 8 ? M : sm_count_of_current_device() * 8;
    const __nv_bfloat16 *xp = (const __nv_bfloat16*)x, *dp = (const __nv_bfloat16*)dh, *gp = (const __nv_bfloat16*)g;
    if (K <= 512 * 5) rmsnorm_bwd_kernel<5><<<blocks, 256, 0, stream>>>(xp, ldx, dp, lddh, rstd, gp, M, K, (__nv_bfloat16*)dx, lddx, dg);
    else if (K <= 512 * 10) rmsnorm_bwd_kernel<10><<<blocks, 256, 0, stream>>>(xp, ldx, dp, lddh, rstd, gp, M, K, (__nv_bfloat16*)dx, lddx, dg);
    else rmsnorm_bwd_kernel<20><<<blocks, 256, 0, stream>>>(xp, ldx, dp, lddh, rstd, gp, M, K, (__nv_bfloat16*)dx, lddx, dg);
    PLZ_LAUNCH_CHECK();
    return PLZ_OK;
}

// out[i] = scale * (slot 0 + slot 1 + ... + slot world-1)[i], slots `shard_elems` floats apart: the second half of the
// reduce-scatter whose first half is the weight-gradient epilogue storing every rank's partial into the owner's slots.
// Fixed summation order, so every run and every rank count gives the same bits for the same partials.
__global__ void __launch_bounds__(256)
reduce_slots_kernel(const float4* __restrict__ stage, int world, long long shard_vec, float4* __restrict__ out, float scale) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < shard_vec; i += stride) {
        float4 acc = __ldcs(stage + i);
        for (int r = 1; r < world; ++r) {
            const float4 v = __ldcs(stage + (long long)r * shard_vec + i);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
        out[i] = acc;
    }
}

int launch_reduce_slots(const float* stage, int world, long long shard_elems, float* out, float scale, cudaStream_t stream) {
    if (shard_elems <= 0) return PLZ_OK;
    const long long vec = shard_elems / 4;
    long long blocks = (vec + 255) / 256;
    if (blocks > sm_count_of_current_device() * 16) blocks = sm_count_of_current_device() * 16;
    reduce_slots_kernel<<<(int)blocks, 256, 0, stream>>>((const float4*)stage, world, vec, (float4*)out, scale);
    PLZ_LAUNCH_CHECK();
    return PLZ_OK;
}

}  // namespace plz
