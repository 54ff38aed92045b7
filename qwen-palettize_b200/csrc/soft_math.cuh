// Per-weight arithmetic of the Gumbel-Softmax relaxation, shared by the weight-construction
// kernels and by the gradient epilogue so that forward and backward see identical numbers.
//
// Semantics follow the reference's PyTorch/Triton path:
//   P = softmax((logits + g) / tau) in fp32, max-subtracted   (scripts/triton_soft_forward.py:119-141)
//   W_soft = sum_p P[p] * palette[p]                          (scripts/bench_triton_kernels.py:77-78)
//   hard index = argmax over the *plain* logits, ties -> lowest index (scripts/triton_soft_forward.py:160-168)
//   dLogits[p] = dW * P[p] * (palette[p] - W_soft), no 1/tau   (scripts/bench_triton_kernels.py:108-111)
//   dPalette[p] += dW * P[p]                                   (scripts/bench_triton_kernels.py:114-118)
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace plz {

enum NoiseMode { NOISE_NONE = 0, NOISE_TENSOR = 1, NOISE_HASH = 2 };

// Counter-based Gumbel(0,1) sample: the 32-bit hash-LCG of the reference sampler
// (scripts/fused_lut_kernel.cu:1245-1256), integer part bit-exact; the float part uses
// the device's logf, so values agree with the reference to a few ulp.
__device__ __forceinline__ float gumbel_hash(uint32_t seed, uint32_t idx) {
    uint32_t x = seed ^ (idx * 0x9E3779B9u);
    x ^= x >> 13;
    x = x * 1103515245u + 12345u;
    x ^= x >> 17;
    x = x * 1103515245u + 12345u;
    float u = (float)(x & 0xFFFFFFu) * (1.0f / 16777216.0f);
    u = fmaxf(u, 1e-7f);
    return -__logf(-__logf(u));
}

__device__ __forceinline__ int argmax4_first(float a, float b, float c, float d) {
    int i = 0;
    float m = a;
    if (b > m) { m = b; i = 1; }
    if (c > m) { m = c; i = 2; }
    if (d > m) { m = d; i = 3; }
    return i;
}

struct Soft4 {
    float P[4];
    float w_soft;
};

// l: logits already converted to fp32; g: noise; c: palette entries in fp32
__device__ __forceinline__ Soft4 soft4(const float (&l)[4], const float (&g)[4], const float (&c)[4],
                                       float inv_tau) {
    float z[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) z[p] = (l[p] + g[p]) * inv_tau;
    const float mx = fmaxf(fmaxf(z[0], z[1]), fmaxf(z[2], z[3]));
    float e[4];
    float sum = 0.f;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        e[p] = __expf(z[p] - mx);
        sum += e[p];
    }
    const float inv = __fdividef(1.0f, sum);
    Soft4 r;
    r.w_soft = 0.f;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        r.P[p] = e[p] * inv;
        r.w_soft += r.P[p] * c[p];
    }
    return r;
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ void from_f32(float& d, float v) { d = v; }
__device__ __forceinline__ void from_f32(__half& d, float v) { d = __float2half_rn(v); }

}  // namespace plz
