// Argument structures and prototypes of the kernel launchers (one per .cu file).
#pragma once
#include "plz_host.h"

namespace plz {

// ---- lut_gemm.cu ------------------------------------------------------------------------------
enum BMode { B_DECODE_K = 0, B_DECODE_MN = 1, B_TMA_K = 2, B_TMA_MN = 3 };
struct LutGemmArgs {
    int bmode;
    int M, J, R;
    const void* A; long long lda;           // [M, R] bf16
    // dense B (TMA modes): B_TMA_K: [J, R] row-major; B_TMA_MN: [R, J] row-major
    const void* Bdense; long long ldb;
    // packed B (decode modes)
    const void* packed; long long packed_pitch; const void* palette;
    int gs_n, gs_k, Wn, Wk;
    // optional extra block: A2 [M, r2] (pitch lda2); B2: K-major modes [J, r2], MN-major modes [r2, J]
    int r2; const void* A2; long long lda2; const void* B2; long long ldb2;
    void* out; long long ld_out; float alpha;
    // fused MLP front end (forward decode mode only): fuse 1 = gate/up pair + SwiGLU (J = 2 N), 2 = one matrix;
    // col_scale bf16 [K] and row_scale fp32 [M] are the RMSNorm factors (either may be null)
    int fuse; const void* packed2; const void* palette2; const void* col_scale; const float* row_scale;
    void* gate_out; void* up_out; long long ld_gu;  // fuse == 1: optional bf16 copies of the two pre-activations
    const void* bias;  // fuse == 2: optional bf16 [J], added in fp32 before the bf16 store
    int sm_limit;  // > 0: use at most this many CTAs (tests of the multi-tile schedule)
    void* prof;  // optional device buffer of cycle counters, 8 x uint64 per CTA (diagnostics)
};
int launch_lut_gemm(const LutGemmArgs& a, cudaStream_t stream);
// lut_gemm_pair.cu: the decode modes on CTA pairs (cta_group::2); PLZ_ERR_UNSUPPORTED = not a shape for it
int launch_lut_gemm_pair(const LutGemmArgs& a, cudaStream_t stream);
extern int g_pair_gemm;  // 0: keep every product on the single-CTA kernel
extern int g_cta_limit;

// ---- tn_gemm.cu -------------------------------------------------------------------------------
enum Epi { EPI_STORE = 0, EPI_SOFT = 1, EPI_HARD = 2 };
struct TnArgs {
    int epi;
    int M, I, J;
    const void* P; long long ldp;  // [M, I] bf16
    const void* Q; long long ldq;  // [M, J] bf16
    // EPI_STORE (results are atomically added to `out`)
    float* out; long long out_si, out_sj; float alpha; int out_I, out_J; int splits;
    // EPI_SOFT / EPI_HARD
    int rows_are_k;  // 1: D rows = input columns k (interleaved logits); 0: D rows = weight rows n
    int logits_f16;
    const void* logits; void* dlogits; long long ls_row, ls_col, ls_p;
    const float* noise; long long ns_row, ns_col, ns_p; int noise_mode; uint32_t seed; int hashN;
    float tau;
    const void* palette; float* dpalette; int gs_n, gs_k, n_kgroups;
    const void* packed; long long packed_pitch;
    int sm_count;
    // optional side jobs appended to a dW launch: out[r, j] += sum_m S[m, r] * (q_is_p ? P : Q)[m, j]
    const void* side_S[2]; long long side_ld[2]; int side_rank; int side_q_is_p[2];
    float* side_out[2]; long long side_si[2], side_sj[2];
    // fused reduce-scatter of dLogits over peer memory (world > 1): staging base of every rank, as mapped in THIS process
    int world, rank, scatter_add; float* peer_stage[8];
    void* prof;  // optional device buffer of cycle counters (diagnostics build)
};
int launch_tn_gemm(const TnArgs& a, cudaStream_t stream);

// ---- gemv.cu ----------------------------------------------------------------------------------
struct GemvArgs {
    int M, N, K;
    const void* x; long long ldx;
    const void* packed; long long packed_pitch; const void* palette;
    int gs_n, gs_k;
    void* out; long long ld_out;
    int sm_count;
    void* prof;  // optional device buffer of cycle counters (diagnostics)
};
int launch_lut_gemv(const GemvArgs& a, cudaStream_t stream);
// smallm_mma.cu: M <= 16 on mma.sync fragments; PLZ_ERR_UNSUPPORTED = shape outside its domain, use launch_lut_gemv's kernels
int launch_lut_smallm_mma(const GemvArgs& a, cudaStream_t stream);
int launch_lut_smallm_mma_multi(const GemvArgs* mats, int count, cudaStream_t stream);  // 1..4 matrices sharing x
extern int g_smallm_overlap;        // 1: launch the mma.sync small-M kernel with programmatic stream serialization
extern int g_debug_smallm_variant;  // 0 = automatic choice, 1 = never use the mma.sync kernel (comparisons)

// ---- elementwise.cu ---------------------------------------------------------------------------
struct SelectParams {
    const void* logits; long long ls_n, ls_k, ls_p;
    const float* noise; long long ns_n, ns_k, ns_p;
    int noise_mode; uint32_t seed; float inv_tau;
    const __nv_bfloat16* palette; int gs_n, gs_k, n_kgroups;
    int N, K;
    uint8_t* packed; long long pitch;             // may be null
    __nv_bfloat16* w_soft; long long ws_n, ws_k;  // may be null; element (n, k) at n * ws_n + k * ws_k
};
int launch_soft_select(const SelectParams& p, int logits_f16, cudaStream_t stream);
int launch_pack_indices(const void* src, long long s_n, long long s_k, int N, int K, void* dst, long long pitch,
                        cudaStream_t stream);
int launch_unpack_indices(const void* src, long long pitch, int N, int K, void* dst, long long s_n, long long s_k,
                          cudaStream_t stream);
int launch_dequant(const void* packed, long long pitch, const void* palette, int gs_n, int gs_k, int N, int K,
                   void* dst, long long d_n, long long d_k, cudaStream_t stream);

// ---- soft_tensors.cu ---------------------------------------------------------------------------
// One matrix of a (batched) soft-weight pass; every tensor through element strides, any output may be null.
struct PwItem {
    const void* logits; long long ls_n, ls_k, ls_p; int logits_f16;
    const float* noise; long long ns_n, ns_k, ns_p; int noise_mode; uint32_t seed;
    const __nv_bfloat16* palette; int gs_n, gs_k, n_kgroups;
    int N, K, n_fast;  // n_fast: consecutive threads walk n (planar (4, K, N) logits), else k
    void* P; long long p_n, p_k, p_p;                 // fp16
    __nv_bfloat16* w_soft; long long ws_n, ws_k;
    __nv_bfloat16* w_hard; long long wh_n, wh_k;
};
int launch_soft_weights(const PwItem* items, int count, float tau, int hard_from_noisy, cudaStream_t stream);
struct BwdElemArgs {
    const void* dW; int dw_dtype; long long dw_n, dw_k;
    const void* P; long long p_n, p_k, p_p;
    const void* palette; int gs_n, gs_k;
    int N, K;
    void* dlogits; int dl_f16; long long dl_n, dl_k, dl_p;
    float* dpalette;
};
int launch_soft_bwd_elementwise(const BwdElemArgs& a, cudaStream_t stream);
int launch_col_sum(const void* dY, long long ld, int M, int N, float* out, cudaStream_t stream);

// ---- attention.cu -------------------------------------------------------------------------------
struct AttnArgs {
    int B, S, Hq, Hkv, head_dim;
    float scale;
    const void* q; long long ldq;     // bf16 [B * S, Hq * head_dim]
    const void* k; long long ldk;     // bf16 [B * S, Hkv * head_dim]
    const void* v; long long ldv;
    void* o; long long ldo;           // forward output / backward input, layout of q
    float* lse;                       // fp32 [B, Hq, S]
    // backward
    const void* d_o; void* dq; void* dk; void* dv; float* dsum;   // gradients in the layouts (and pitches) of o, q, k, v
};
int launch_attn_fwd(const AttnArgs& a, cudaStream_t stream);
int launch_attn_bwd(const AttnArgs& a, cudaStream_t stream);

// ---- attention_decode.cu ------------------------------------------------------------------------
struct AttnDecodeArgs {
    int B, T, Hq, Hkv;
    float scale;
    const void* q; long long ldq;                 // bf16 [B, Hq * 128]: the new token of every sequence
    const void* k; const void* v;                 // bf16 caches [B, T_max, Hkv * 128]
    long long batch_stride, tok_stride;           // elements between sequences / between positions
    void* out; long long ldo;                     // bf16 [B, Hq * 128]
    void* ws; long long ws_bytes;
};
long long attn_decode_ws_bytes(int B, int T, int Hq, int Hkv);
int launch_attn_decode(const AttnDecodeArgs& a, cudaStream_t stream);
int launch_embed_gather(const void* table, long long ldt, const long long* ids, long long n, int width, long long vocab, void* out,
                        long long ldo, int* bad, cudaStream_t stream);

// ---- layer_ops.cu -------------------------------------------------------------------------------
int launch_rmsnorm_fwd(const void* x, long long ldx, const void* g, int M, int K, float eps, void* h, long long ldh, float* rstd,
                       cudaStream_t stream);
int launch_add_rmsnorm(const void* x, long long ldx, const void* addend, long long lda, void* sum_out, long long lds, const void* g, int M,
                       int K, float eps, void* h, long long ldh, float* rstd, cudaStream_t stream);
int launch_qknorm_rope2(const void* x1, long long ldx1, const void* w1, int H1, void* out1, long long ldo1, const void* x2, long long ldx2,
                        const void* w2, int H2, void* out2, long long ldo2, const float* cs, const float* sn, long long tokens, int S, float eps,
                        cudaStream_t stream);
int launch_qknorm_rope(int backward, const void* x, long long ldx, const void* w, const float* cs, const float* sn, const void* dy,
                       long long lddy, long long tokens, int H, int S, float eps, void* out, long long ldo, float* dw, cudaStream_t stream);
int launch_swiglu_fwd(const void* gate, long long ldg, const void* up, long long ldu, int M, int N, void* act, long long lda, cudaStream_t stream);
int launch_add(const void* a, long long lda, const void* b, long long ldb, const void* c, long long ldc, int M, int N, void* out, long long ldo,
               cudaStream_t stream);

// ---- train_ops.cu ------------------------------------------------------------------------------
struct AdamParams {
    float* master; float* m; float* v;
    const void* grad; void* param;
    long long n;
    float grad_scale, lr, beta1, beta2, eps, weight_decay;
    float bias_c1, sqrt_bias_c2;  // 1 - beta1^t, sqrt(1 - beta2^t)
    float clamp_lo, clamp_hi; int clamp_master;
};

int launch_adamw(const AdamParams& p, int grad_dtype, int param_dtype, cudaStream_t stream);
int launch_reduce_slots(const float* stage, int world, long long shard_elems, float* out, float scale, cudaStream_t stream);
int launch_swiglu_bwd(const void* gate, long long ldg, const void* up, long long ldu, const void* dact, long long ldd, int M, int N,
                      void* dgate, long long lddg, void* dup, long long lddu, cudaStream_t stream);
int launch_rmsnorm_bwd(const void* x, long long ldx, const void* dh, long long lddh, const float* rstd, const void* g, int M, int K,
                       void* dx, long long lddx, float* dg, cudaStream_t stream);
int launch_rms_rstd(const void* x, long long ldx, int M, int K, float eps, float* rstd, cudaStream_t stream);
int launch_distill_loss(const void* s, long long lds, const void* t, long long ldt, int M, int H, float eps, float w_cos,
                        float w_mse, float upstream, float* ws, float* out4, void* ds, long long ldds, int ds_dtype,
                        cudaStream_t stream);

}  // namespace plz
