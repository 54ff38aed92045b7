// Element-wise companions of the Linears and the attention inside a decoder layer: RMSNorm forward, per-head q/k RMSNorm
// fused with the rotary embedding (forward and backward), SwiGLU forward and the residual add. All are single passes bound
// by HBM; 16-byte accesses, one warp per row where a row statistic is needed.
//
// The reference has no code for these: it calls the HuggingFace decoder layer (scripts/train_qwen.py:1259-1266). Semantics
// follow transformers' Qwen3RMSNorm (fp32 statistics, x * rstd rounded to bf16, then times the bf16 weight), Qwen3Attention
// (q_norm / k_norm over the head dimension, then apply_rotary_pos_emb with rotate_half) and Qwen3MLP (silu(gate) * up).
#include "plz_launch.h"

namespace plz {
namespace {

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// h[m, k] = bf16( bf16(s[m, k] * rstd[m]) * g[k] ),  rstd[m] = rsqrt(mean_k s^2 + eps), where s = x, or with ADD
// s = bf16(x + addend) (fp32 sum rounded once), which is also written out: the residual add and the norm that follows it in
// one pass. A row belongs to one warp (many rows: training, prefill) or, with BLOCK, to a whole 256-thread block (a handful
// of rows: token decode, where one warp per row would leave the row's 5 KB to 32 lanes).
template <bool BLOCK, bool ADD>
__global__ void __launch_bounds__(256)
rms_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ addend, long long lda,
           __nv_bfloat16* __restrict__ sum_out, long long lds, const __nv_bfloat16* __restrict__ g, int M, int K, float eps,
           __nv_bfloat16* __restrict__ h, long long ldh, float* __restrict__ rstd) {
    __shared__ float part[8];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int t = BLOCK ? (int)threadIdx.x : lane, team = BLOCK ? 256 : 32;
    pdl_launch_dependents();
    pdl_wait();
    for (int row = BLOCK ? (int)blockIdx.x : (int)blockIdx.x * 8 + wib; row < M; row += BLOCK ? (int)gridDim.x : (int)gridDim.x * 8) {
        const __nv_bfloat16* xr = x + (long long)row * ldx;
        const __nv_bfloat16* sr = ADD ? sum_out + (long long)row * lds : xr;
        float s2 = 0.f;
        for (int c = t * 8; c < K; c += team * 8) {
            uint4 v = *reinterpret_cast<const uint4*>(xr + c);
            uint32_t w[4] = {v.x, v.y, v.z, v.w};
            if (ADD) {
                const uint4 av = *reinterpret_cast<const uint4*>(addend + (long long)row * lda + c);
                const uint32_t aw[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) w[i] = pack_bf16x2(bf_lo(w[i]) + bf_lo(aw[i]), bf_hi(w[i]) + bf_hi(aw[i]));
                *reinterpret_cast<uint4*>(sum_out + (long long)row * lds + c) = make_uint4(w[0], w[1], w[2], w[3]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) s2 += bf_lo(w[i]) * bf_lo(w[i]) + bf_hi(w[i]) * bf_hi(w[i]);
        }
        s2 = wsum(s2);
        if (BLOCK) {
            __syncthreads();           // the previous row's readers of part[] are done
            if (lane == 0) part[wib] = s2;
            __syncthreads();
            s2 = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) s2 += part[i];
        }
        const float rs = rsqrtf(s2 / (float)K + eps);
        if (t == 0 && rstd) rstd[row] = rs;
        __nv_bfloat16* hr = h + (long long)row * ldh;
        for (int c = t * 8; c < K; c += team * 8) {
            const uint4 v = *reinterpret_cast<const uint4*>(sr + c);   // with ADD: this thread's own stores of the loop above
            const uint4 gv = g ? __ldg(reinterpret_cast<const uint4*>(g + c)) : make_uint4(0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w}, gw[4] = {gv.x, gv.y, gv.z, gv.w};
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                o[i] = pack_bf16x2(round_bf16(bf_lo(w[i]) * rs) * bf_lo(gw[i]), round_bf16(bf_hi(w[i]) * rs) * bf_hi(gw[i]));
            *reinterpret_cast<uint4*>(hr + c) = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

// q/k norm + rotary embedding, head_dim 128. One warp per (token, head): lane l holds elements 2l, 2l+1 (first half) and
// 64 + 2l, 65 + 2l (second half), i.e. the two rotation pairs (i, i + 64).
//   xn = bf16(x * rstd) ; y = bf16(w * xn) ; out[i] = y[i] cos_i - y[i+64] sin_i ; out[i+64] = y[i+64] cos_i + y[i] sin_i
// cos / sin: fp32 [S, 64] tables, position = token index inside its sequence.
struct QkSide { const __nv_bfloat16* x; long long ldx; const __nv_bfloat16* w; __nv_bfloat16* out; long long ldo; int H; };

// One launch may carry two tensors (the q and the k projection of the same tokens): heads [0, a.H) are a's, the rest b's.
__global__ void __launch_bounds__(256)
qknorm_rope_fwd_kernel(const QkSide a, const QkSide b, const float* __restrict__ cs, const float* __restrict__ sn, long long rows, int S, float eps) {
    const int lane = threadIdx.x & 31;
    const long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);   // over tokens * heads
    pdl_launch_dependents();
    pdl_wait();
    if (r >= rows) return;
    const int H = a.H + b.H;
    const long long tok = r / H;
    int h = (int)(r % H);
    const int pos = (int)(tok % S);
    const bool second = h >= a.H;
    const QkSide& q = second ? b : a;
    if (second) h -= a.H;
    const __nv_bfloat16* xr = q.x + tok * q.ldx + h * 128;
    const uint32_t xa = *reinterpret_cast<const uint32_t*>(xr + 2 * lane), xb = *reinterpret_cast<const uint32_t*>(xr + 64 + 2 * lane);
    const float x0 = bf_lo(xa), x1 = bf_hi(xa), x2 = bf_lo(xb), x3 = bf_hi(xb);
    const float rs = rsqrtf(wsum(x0 * x0 + x1 * x1 + x2 * x2 + x3 * x3) * (1.0f / 128.0f) + eps);
    const uint32_t wa = q.w ? *reinterpret_cast<const uint32_t*>(q.w + 2 * lane) : 0x3F803F80u;
    const uint32_t wb = q.w ? *reinterpret_cast<const uint32_t*>(q.w + 64 + 2 * lane) : 0x3F803F80u;
    const float y0 = round_bf16(round_bf16(x0 * rs) * bf_lo(wa)), y1 = round_bf16(round_bf16(x1 * rs) * bf_hi(wa));
    const float y2 = round_bf16(round_bf16(x2 * rs) * bf_lo(wb)), y3 = round_bf16(round_bf16(x3 * rs) * bf_hi(wb));
    const float2 c = *reinterpret_cast<const float2*>(cs + (long long)pos * 64 + 2 * lane);
    const float2 s = *reinterpret_cast<const float2*>(sn + (long long)pos * 64 + 2 * lane);
    __nv_bfloat16* orow = q.out + tok * q.ldo + h * 128;
    *reinterpret_cast<uint32_t*>(orow + 2 * lane) = pack_bf16x2(y0 * c.x - y2 * s.x, y1 * c.y - y3 * s.y);
    *reinterpret_cast<uint32_t*>(orow + 64 + 2 * lane) = pack_bf16x2(y2 * c.x + y0 * s.x, y3 * c.y + y1 * s.y);
}

// backward of the above: dy (gradient of the rotated output) -> dx (gradient of the raw projection output), dw[128] +=
__global__ void __launch_bounds__(256)
qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ w, const float* __restrict__ cs,
                       const float* __restrict__ sn, const __nv_bfloat16* __restrict__ dy, long long lddy, long long rows, int H, int S,
                       float eps, __nv_bfloat16* __restrict__ dx, long long lddx, float* __restrict__ dw) {
    __shared__ float acc[8][128];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    float g0 = 0.f, g1 = 0.f, g2 = 0.f, g3 = 0.f;   // this lane's four weight-gradient partials
    for (long long r = (long long)blockIdx.x * 8 + wib; r < rows; r += (long long)gridDim.x * 8) {
        const long long tok = r / H;
        const int h = (int)(r % H), pos = (int)(tok % S);
        const __nv_bfloat16* xr = x + tok * ldx + h * 128;
        const __nv_bfloat16* gr = dy + tok * lddy + h * 128;
        const uint32_t a = *reinterpret_cast<const uint32_t*>(xr + 2 * lane), b = *reinterpret_cast<const uint32_t*>(xr + 64 + 2 * lane);
        const uint32_t da = *reinterpret_cast<const uint32_t*>(gr + 2 * lane), db = *reinterpret_cast<const uint32_t*>(gr + 64 + 2 * lane);
        const float x0 = bf_lo(a), x1 = bf_hi(a), x2 = bf_lo(b), x3 = bf_hi(b);
        const float rs = rsqrtf(wsum(x0 * x0 + x1 * x1 + x2 * x2 + x3 * x3) * (1.0f / 128.0f) + eps);
        const float2 c = *reinterpret_cast<const float2*>(cs + (long long)pos * 64 + 2 * lane);
        const float2 s = *reinterpret_cast<const float2*>(sn + (long long)pos * 64 + 2 * lane);
        // inverse rotation: gradient with respect to y = w * xn
        const float e0 = bf_lo(da), e1 = bf_hi(da), e2 = bf_lo(db), e3 = bf_hi(db);
        const float t0 = e0 * c.x + e2 * s.x, t1 = e1 * c.y + e3 * s.y, t2 = e2 * c.x - e0 * s.x, t3 = e3 * c.y - e1 * s.y;
        const uint32_t wa = w ? *reinterpret_cast<const uint32_t*>(w + 2 * lane) : 0x3F803F80u;
        const uint32_t wb = w ? *reinterpret_cast<const uint32_t*>(w + 64 + 2 * lane) : 0x3F803F80u;
        const float n0 = x0 * rs, n1 = x1 * rs, n2 = x2 * rs, n3 = x3 * rs;          // x hat
        g0 += t0 * n0; g1 += t1 * n1; g2 += t2 * n2; g3 += t3 * n3;
        const float u0 = t0 * bf_lo(wa), u1 = t1 * bf_hi(wa), u2 = t2 * bf_lo(wb), u3 = t3 * bf_hi(wb);   // d / d xhat
        const float mean = wsum(u0 * n0 + u1 * n1 + u2 * n2 + u3 * n3) * (1.0f / 128.0f);
        __nv_bfloat16* drow = dx + tok * lddx + h * 128;
        *reinterpret_cast<uint32_t*>(drow + 2 * lane) = pack_bf16x2(rs * (u0 - n0 * mean), rs * (u1 - n1 * mean));
        *reinterpret_cast<uint32_t*>(drow + 64 + 2 * lane) = pack_bf16x2(rs * (u2 - n2 * mean), rs * (u3 - n3 * mean));
    }
    if (dw == nullptr) return;
    acc[wib][2 * lane] = g0; acc[wib][2 * lane + 1] = g1; acc[wib][64 + 2 * lane] = g2; acc[wib][65 + 2 * lane] = g3;
    __syncthreads();
    if (threadIdx.x < 128) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) s += acc[i][threadIdx.x];
        atomicAdd(dw + threadIdx.x, s);
    }
}

// act = silu(gate) * up, bf16, eight elements per thread and step
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gate, long long ldg, const __nv_bfloat16* __restrict__ up, long long ldu, int M, int N,
                  __nv_bfloat16* __restrict__ act, long long lda) {
    const int vec = N >> 3;
    const long long total = (long long)M * vec;
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int m = (int)(i / vec), c = (int)(i - (long long)m * vec) << 3;
        const uint4 gv = __ldcs(reinterpret_cast<const uint4*>(gate + (long long)m * ldg + c));
        const uint4 uv = __ldcs(reinterpret_cast<const uint4*>(up + (long long)m * ldu + c));
        const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float a0 = bf_lo(gw[q]), a1 = bf_hi(gw[q]);
            // silu rounded to bf16 before the product, as the eager act_fn(gate) * up does
            const float s0 = round_bf16(__fdividef(a0, 1.0f + __expf(-a0))), s1 = round_bf16(__fdividef(a1, 1.0f + __expf(-a1)));
            o[q] = pack_bf16x2(s0 * bf_lo(uw[q]), s1 * bf_hi(uw[q]));
        }
        *reinterpret_cast<uint4*>(act + (long long)m * lda + c) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// out = a + b (+ c), bf16 rows, fp32 sum rounded once
__global__ void __launch_bounds__(256)
add_kernel(const __nv_bfloat16* __restrict__ a, long long lda, const __nv_bfloat16* __restrict__ b, long long ldb,
           const __nv_bfloat16* __restrict__ c3, long long ldc, int M, int N, __nv_bfloat16* __restrict__ out, long long ldo) {
    const int vec = N >> 3;
    const long long total = (long long)M * vec;
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int m = (int)(i / vec), c = (int)(i - (long long)m * vec) << 3;
        const uint4 av = *reinterpret_cast<const uint4*>(a + (long long)m * lda + c);
        const uint4 bv = *reinterpret_cast<const uint4*>(b + (long long)m * ldb + c);
        uint4 cv = make_uint4(0u, 0u, 0u, 0u);
        if (c3) cv = *reinterpret_cast<const uint4*>(c3 + (long long)m * ldc + c);
        const uint32_t aw[4] = {av.x, av.y, av.z, av.w}, bw[4] = {bv.x, bv.y, bv.z, bv.w}, cw[4] = {cv.x, cv.y, cv.z, cv.w};
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
            o[q] = pack_bf16x2(bf_lo(aw[q]) + bf_lo(bw[q]) + bf_lo(cw[q]), bf_hi(aw[q]) + bf_hi(bw[q]) + bf_hi(cw[q]));
        *reinterpret_cast<uint4*>(out + (long long)m * ldo + c) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

int grid_for(long long work_items, int per_block) {
    int dev = 0, sms = 1;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    long long blocks = (work_items + per_block - 1) / per_block;
    const long long cap = (long long)sms * 16;
    return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace

static int sm_count_here() {
    int dev = 0, sms = 1;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms;
}

int launch_rmsnorm_fwd(const void* x, long long ldx, const void* g, int M, int K, float eps, void* h, long long ldh, float* rstd,
                       cudaStream_t stream) {
    return launch_add_rmsnorm(x, ldx, nullptr, 0, nullptr, 0, g, M, K, eps, h, ldh, rstd, stream);
}
// addend == nullptr: plain RMSNorm of x; else sum_out = x + addend and h = rmsnorm(sum_out) * g
int launch_add_rmsnorm(const void* x, long long ldx, const void* addend, long long lda, void* sum_out, long long lds, const void* g, int M,
                       int K, float eps, void* h, long long ldh, float* rstd, cudaStream_t stream) {
    if (M <= 0) return PLZ_OK;
    const __nv_bfloat16 *xp = (const __nv_bfloat16*)x, *ap = (const __nv_bfloat16*)addend, *gp = (const __nv_bfloat16*)g;
    __nv_bfloat16 *sp = (__nv_bfloat16*)sum_out, *hp = (__nv_bfloat16*)h;
    const bool block = M <= 4 * sm_count_here();   // few rows: a block per row
    const dim3 grid(block ? M : grid_for(M, 8));
    if (addend) {
        if (block) PLZ_LAUNCH_CHAIN(rms_kernel<true, true>, grid, dim3(256), 0, stream, xp, ldx, ap, lda, sp, lds, gp, M, K, eps, hp, ldh, rstd);
        else PLZ_LAUNCH_CHAIN(rms_kernel<false, true>, grid, dim3(256), 0, stream, xp, ldx, ap, lda, sp, lds, gp, M, K, eps, hp, ldh, rstd);
    } else {
        if (block) PLZ_LAUNCH_CHAIN(rms_kernel<true, false>, grid, dim3(256), 0, stream, xp, ldx, ap, lda, sp, lds, gp, M, K, eps, hp, ldh, rstd);
        else PLZ_LAUNCH_CHAIN(rms_kernel<false, false>, grid, dim3(256), 0, stream, xp, ldx, ap, lda, sp, lds, gp, M, K, eps, hp, ldh, rstd);
    }
    return PLZ_OK;
}
int launch_qknorm_rope(int backward, const void* x, long long ldx, const void* w, const float* cs, const float* sn, const void* dy,
                       long long lddy, long long tokens, int H, int S, float eps, void* out, long long ldo, float* dw, cudaStream_t stream) {
    if (!backward) return launch_qknorm_rope2(x, ldx, w, H, out, ldo, nullptr, 0, nullptr, 0, nullptr, 0, cs, sn, tokens, S, eps, stream);
    const long long rows = tokens * H;
    if (rows <= 0) return PLZ_OK;
    qknorm_rope_bwd_kernel<<<grid_for(rows, 8 * 16), 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, cs, sn,
                                                                       (const __nv_bfloat16*)dy, lddy, rows, H, S, eps, (__nv_bfloat16*)out, ldo, dw);
    PLZ_LAUNCH_CHECK();
    return PLZ_OK;
}
// forward for one tensor (H2 == 0) or two (q and k of the same tokens) in one launch
int launch_qknorm_rope2(const void* x1, long long ldx1, const void* w1, int H1, void* out1, long long ldo1, const void* x2, long long ldx2,
                        const void* w2, int H2, void* out2, long long ldo2, const float* cs, const float* sn, long long tokens, int S, float eps,
                        cudaStream_t stream) {
    const long long rows = tokens * (H1 + H2);
    if (rows <= 0) return PLZ_OK;
    const long long blocks = (rows + 7) / 8;
    if (blocks > 0x7FFFFFFFll) { set_last_error("qknorm_rope: too many rows"); return PLZ_ERR_TOO_LARGE; }
    const QkSide a = {(const __nv_bfloat16*)x1, ldx1, (const __nv_bfloat16*)w1, (__nv_bfloat16*)out1, ldo1, H1};
    const QkSide b = {(const __nv_bfloat16*)x2, ldx2, (const __nv_bfloat16*)w2, (__nv_bfloat16*)out2, ldo2, H2};
    PLZ_LAUNCH_CHAIN(qknorm_rope_fwd_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, a, b, cs, sn, rows, S, eps);
    return PLZ_OK;
}
int launch_swiglu_fwd(const void* gate, long long ldg, const void* up, long long ldu, int M, int N, void* act, long long lda, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return PLZ_OK;
    PLZ_LAUNCH_CHAIN(swiglu_fwd_kernel, dim3(grid_for((long long)M * (N >> 3), 256)), dim3(256), 0, stream, (const __nv_bfloat16*)gate, ldg,
                     (const __nv_bfloat16*)up, ldu, M, N, (__nv_bfloat16*)act, lda);
    return PLZ_OK;
}
int launch_add(const void* a, long long lda, const void* b, long long ldb, const void* c, long long ldc, int M, int N, void* out, long long ldo,
               cudaStream_t stream) {
    if (M <= 0 || N <= 0) return PLZ_OK;
    PLZ_LAUNCH_CHAIN(add_kernel, dim3(grid_for((long long)M * (N >> 3), 256)), dim3(256), 0, stream, (const __nv_bfloat16*)a, lda,
                     (const __nv_bfloat16*)b, ldb, (const __nv_bfloat16*)c, ldc, M, N, (__nv_bfloat16*)out, ldo);
    return PLZ_OK;
}

}  // namespace plz
