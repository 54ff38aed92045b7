// Attention of one new token per sequence against a key / value cache (token decode), and the embedding-row gather that
// opens a forward pass. Both are single passes bound by HBM: a decode step reads every cached key and value once
// (B * T * Hkv * 128 * 2 * 2 bytes per layer), no tensor core involved.
//
//   attn_decode_partial_kernel  grid (splits, Hkv, B), 4 warps. The sequence is cut into `splits` contiguous chunks so that
//     the launch has a few CTAs per SM whatever B is. Inside a CTA a warp takes 8 tokens per step: 16 lanes per token, each
//     lane the 16 bytes (8 dims) of the key and of the value row that belong to it, so one load instruction of a warp covers
//     two whole 256-byte rows, and four such loads for K and four for V are in flight per lane before anything is used. The
//     up-to-4 query heads of the group share every key / value byte. The 16 partial scores of a step (4 heads x 4 token
//     slots) are summed over the 16 lanes by recursive halving (15 shuffles, after which lane i owns score i), so exp2 is
//     evaluated once per score; online softmax (running max and sum per head) across steps; the warps' partial results meet in
//     shared memory. With one split the CTA writes the bf16 output itself, else an unnormalised fp32 partial (o, max, sum).
//   attn_decode_combine_kernel  merges the splits.
//
// The reference has no attention code (it calls the HuggingFace layer, scripts/qwen_model.py:454 selects SDPA); semantics are
// those of transformers' Qwen3Attention at q_len = 1 with a DynamicCache: softmax over all T cached positions, no mask.
#include "plz_launch.h"

namespace plz {
namespace {

constexpr float kLog2eDec = 1.4426950408889634f;
constexpr float kNegBig = -1.0e30f;
constexpr int kDecWarps = 4;
constexpr int kStepTokens = 8;                     // tokens of one warp step
constexpr int kCtaStep = kDecWarps * kStepTokens;  // tokens a CTA advances per step of its warps

struct DecParams {
    const __nv_bfloat16* q; long long ldq;
    const __nv_bfloat16* k; const __nv_bfloat16* v; long long batch_stride, tok_stride;
    __nv_bfloat16* out; long long ldo;
    float* ws_o; float* ws_ml;       // [B, Hq, splits, 128] and [B, Hq, splits, 2]
    int T, Hq, Hkv, G, chunk, splits, g0;   // G: q heads of a group handled by this launch (<= 4), first of them g0
    int group;                               // Hq / Hkv
    float scale_log2e;
};

__device__ __forceinline__ float ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ void unpack8(const uint4& r, float (&f)[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
}

__global__ void __launch_bounds__(kDecWarps * 32)
attn_decode_partial_kernel(const DecParams p) {
    __shared__ float sm_o[kDecWarps][4][128];
    __shared__ float sm_ml[kDecWarps][4][2];
    const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tl = lane >> 4, dl = lane & 15;
    const int t0 = split * p.chunk, t1 = min(p.T, t0 + p.chunk);
    const int head0 = hk * p.group + p.g0;          // first q head of this launch's part of the group
    pdl_launch_dependents();
    pdl_wait();

    float q[4][8];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        if (g < p.G) {
            const uint4 r = __ldg(reinterpret_cast<const uint4*>(p.q + (long long)b * p.ldq + (long long)(head0 + g) * 128 + dl * 8));
            unpack8(r, q[g]);
#pragma unroll
            for (int d = 0; d < 8; ++d) q[g][d] *= p.scale_log2e;
        } else {
#pragma unroll
            for (int d = 0; d < 8; ++d) q[g][d] = 0.f;
        }
    }
    float o[4][8];
#pragma unroll
    for (int g = 0; g < 4; ++g)
#pragma unroll
        for (int d = 0; d < 8; ++d) o[g][d] = 0.f;
    float m_own = kNegBig, l_own = 0.f;             // of head dl >> 2, this lane's share of the sum
    const __nv_bfloat16* kb = p.k + (long long)b * p.batch_stride + (long long)hk * 128 + dl * 8;
    const __nv_bfloat16* vb = p.v + (long long)b * p.batch_stride + (long long)hk * 128 + dl * 8;

    for (int base = t0 + warp * kStepTokens; base < t1; base += kCtaStep) {
        uint4 kr[4], vr[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int t = base + 2 * u + tl;
            kr[u] = make_uint4(0u, 0u, 0u, 0u); vr[u] = kr[u];
            if (t < t1) {
                kr[u] = __ldcs(reinterpret_cast<const uint4*>(kb + (long long)t * p.tok_stride));
                vr[u] = __ldcs(reinterpret_cast<const uint4*>(vb + (long long)t * p.tok_stride));
            }
        }
        float val[16];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            float kf[8];
            unpack8(kr[u], kf);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                float s = 0.f;
#pragma unroll
                for (int d = 0; d < 8; ++d) s = fmaf(q[g][d], kf[d], s);
                val[g * 4 + u] = s;
            }
        }
        // sum over the 16 lanes of a token by recursive halving: afterwards lane dl holds the total of val[dl]
#pragma unroll
        for (int half = 8; half >= 1; half >>= 1) {
            const bool up = (dl & half) != 0;
#pragma unroll
            for (int i = 0; i < half; ++i) {
                const float send = up ? val[i] : val[i + half];
                const float keep = up ? val[i + half] : val[i];
                val[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, half);
            }
        }
        const int u_own = dl & 3;
        const bool ok = (base + 2 * u_own + tl) < t1;
        const float s = ok ? val[0] : kNegBig;
        float mx = fmaxf(s, __shfl_xor_sync(0xFFFFFFFFu, s, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 16));
        const float m_new = fmaxf(m_own, mx);
        const float corr = ex2(m_own - m_new);
        const float pr = ok ? ex2(s - m_new) : 0.f;
        l_own = l_own * corr + pr;
        m_own = m_new;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const float cg = __shfl_sync(0xFFFFFFFFu, corr, g * 4);
#pragma unroll
            for (int d = 0; d < 8; ++d) o[g][d] *= cg;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            float vf[8];
            unpack8(vr[u], vf);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const float pgu = __shfl_sync(0xFFFFFFFFu, pr, (tl << 4) + g * 4 + u);
#pragma unroll
                for (int d = 0; d < 8; ++d) o[g][d] = fmaf(pgu, vf[d], o[g][d]);
            }
        }
    }
    // the two token slots of a warp, then the sum of a head over its lanes
#pragma unroll
    for (int g = 0; g < 4; ++g)
#pragma unroll
        for (int d = 0; d < 8; ++d) o[g][d] += __shfl_xor_sync(0xFFFFFFFFu, o[g][d], 16);
    l_own += __shfl_xor_sync(0xFFFFFFFFu, l_own, 1);
    l_own += __shfl_xor_sync(0xFFFFFFFFu, l_own, 2);
    l_own += __shfl_xor_sync(0xFFFFFFFFu, l_own, 16);
    if (tl == 0) {
#pragma unroll
        for (int g = 0; g < 4; ++g)
#pragma unroll
            for (int d = 0; d < 8; ++d) sm_o[warp][g][dl * 8 + d] = o[g][d];
        if ((dl & 3) == 0) { sm_ml[warp][dl >> 2][0] = m_own; sm_ml[warp][dl >> 2][1] = l_own; }
    }
    __syncthreads();
    // merge the warps: thread d of 128 takes dimension d of every head
    const int d = threadIdx.x;
    for (int g = 0; g < p.G; ++g) {
        float M = kNegBig;
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) M = fmaxf(M, sm_ml[w][g][0]);
        float acc = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) {
            const float c = ex2(sm_ml[w][g][0] - M);
            acc = fmaf(c, sm_o[w][g][d], acc);
            l = fmaf(c, sm_ml[w][g][1], l);
        }
        const int head = head0 + g;
        if (p.splits == 1) {
            p.out[(long long)b * p.ldo + (long long)head * 128 + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
        } else {
            const long long slot = ((long long)b * p.Hq + head) * p.splits + split;
            p.ws_o[slot * 128 + d] = acc;
            if (d == 0) { p.ws_ml[slot * 2] = M; p.ws_ml[slot * 2 + 1] = l; }
        }
    }
}

// Merge of the splits: one block per (head, sequence), thread d = dimension d. The weights exp2(m_s - M) of the splits are
// computed once (thread s for split s, at most kMaxSplits of them) and shared; the sum over splits then has independent loads.
constexpr int kMaxSplits = 128;
__global__ void __launch_bounds__(128)
attn_decode_combine_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml, int splits, int Hq, __nv_bfloat16* __restrict__ out,
                           long long ldo) {
    __shared__ float wgt[kMaxSplits];
    __shared__ float red[8];
    const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x, lane = d & 31, wib = d >> 5;
    const long long slot0 = ((long long)b * Hq + head) * splits;
    pdl_launch_dependents();
    pdl_wait();
    const float m = d < splits ? ws_ml[(slot0 + d) * 2] : kNegBig;
    const float l = d < splits ? ws_ml[(slot0 + d) * 2 + 1] : 0.f;
    float M = m;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xFFFFFFFFu, M, o));
    if (lane == 0) red[wib] = M;
    __syncthreads();
    M = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    const float c = ex2(m - M);
    wgt[d] = c;
    float ls = c * l;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ls += __shfl_xor_sync(0xFFFFFFFFu, ls, o);
    if (lane == 0) red[4 + wib] = ls;
    __syncthreads();
    const float L = red[4] + red[5] + red[6] + red[7];
    float acc = 0.f;
    const float* src = ws_o + slot0 * 128 + d;
#pragma unroll 8
    for (int s = 0; s < splits; ++s) acc = fmaf(wgt[s], __ldcs(src + (long long)s * 128), acc);
    out[(long long)b * ldo + (long long)head * 128 + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
}

// out[i, :] = table[ids[i], :] (bf16 rows of `width`, width % 8 == 0); an id outside [0, vocab) gives a zero row and sets *bad
__global__ void __launch_bounds__(256)
embed_gather_kernel(const __nv_bfloat16* __restrict__ table, long long ldt, const long long* __restrict__ ids, long long n, int width,
                    long long vocab, __nv_bfloat16* __restrict__ out, long long ldo, int* __restrict__ bad) {
    const int vec = width >> 3;
    const long long total = n * vec;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / vec;
        const int c = (int)(i - r * vec) << 3;
        const long long id = ids[r];
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (id >= 0 && id < vocab) v = __ldg(reinterpret_cast<const uint4*>(table + id * ldt + c));
        else if (bad && c == 0) *bad = 1;
        *reinterpret_cast<uint4*>(out + r * ldo + c) = v;
    }
}

int sm_count_now() {
    int dev = 0, sms = 1;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms;
}

// tokens per split (a multiple of the CTA step) and the number of splits for a launch of B * Hkv groups over T tokens
void decode_split(int B, int Hkv, int T, int* chunk, int* splits) {
    const int want_ctas = 2 * sm_count_now();
    int s = (want_ctas + B * Hkv - 1) / (B * Hkv);
    const int max_s = (T + kCtaStep - 1) / kCtaStep;
    if (s > max_s) s = max_s;
    if (s > kMaxSplits) s = kMaxSplits;
    if (s < 1) s = 1;
    int c = (T + s - 1) / s;
    c = ((c + kCtaStep - 1) / kCtaStep) * kCtaStep;
    *chunk = c;
    *splits = (T + c - 1) / c;
}

}  // namespace

long long attn_decode_ws_bytes(int B, int T, int Hq, int Hkv) {
    int chunk = 0, splits = 1;
    decode_split(B, Hkv, T, &chunk, &splits);
    return splits == 1 ? 0 : (long long)B * Hq * splits * 130 * (long long)sizeof(float);
}

int launch_attn_decode(const AttnDecodeArgs& a, cudaStream_t stream) {
    if (a.B <= 0) return PLZ_OK;
    DecParams p = {};
    decode_split(a.B, a.Hkv, a.T, &p.chunk, &p.splits);
    const long long need = p.splits == 1 ? 0 : (long long)a.B * a.Hq * p.splits * 130 * (long long)sizeof(float);
    if (need > a.ws_bytes) { set_last_error("attn_decode: workspace of %lld bytes needed, %lld given", need, a.ws_bytes); return PLZ_ERR_TOO_LARGE; }
    p.q = (const __nv_bfloat16*)a.q; p.ldq = a.ldq;
    p.k = (const __nv_bfloat16*)a.k; p.v = (const __nv_bfloat16*)a.v; p.batch_stride = a.batch_stride; p.tok_stride = a.tok_stride;
    p.out = (__nv_bfloat16*)a.out; p.ldo = a.ldo;
    p.ws_o = (float*)a.ws;
    p.ws_ml = p.ws_o ? p.ws_o + (long long)a.B * a.Hq * p.splits * 128 : nullptr;
    p.T = a.T; p.Hq = a.Hq; p.Hkv = a.Hkv; p.group = a.Hq / a.Hkv;
    p.scale_log2e = a.scale * kLog2eDec;
    for (int g0 = 0; g0 < p.group; g0 += 4) {   // groups of more than four q heads: four at a time
        p.g0 = g0; p.G = p.group - g0 < 4 ? p.group - g0 : 4;
        PLZ_LAUNCH_CHAIN(attn_decode_partial_kernel, dim3(p.splits, a.Hkv, a.B), dim3(kDecWarps * 32), 0, stream, p);
    }
    if (p.splits > 1) {
        PLZ_LAUNCH_CHAIN(attn_decode_combine_kernel, dim3(a.Hq, a.B), dim3(128), 0, stream, (const float*)p.ws_o, (const float*)p.ws_ml, p.splits,
                         a.Hq, p.out, p.ldo);
    }
    return PLZ_OK;
}

int launch_embed_gather(const void* table, long long ldt, const long long* ids, long long n, int width, long long vocab, void* out,
                        long long ldo, int* bad, cudaStream_t stream) {
    if (n <= 0) return PLZ_OK;
    long long blocks = (n * (width >> 3) + 255) / 256;
    const long long cap = (long long)sm_count_now() * 16;
    if (blocks > cap) blocks = cap;
    embed_gather_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const __nv_bfloat16*)table, ldt, ids, n, width, vocab, (__nv_bfloat16*)out, ldo, bad);
    PLZ_LAUNCH_CHECK();
    return PLZ_OK;
}

}  // namespace plz
