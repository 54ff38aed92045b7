/* plz.h -- C ABI of libplz.so: the PalettizedLinear hot path (2-bit palette look-up-table Linear)
 * on NVIDIA B200 (sm_100a).
 *
 * Conventions
 *   - Every pointer is a CUDA device pointer on the current device unless stated otherwise.
 *   - Every entry point enqueues work on `stream` (a cudaStream_t passed as void*; NULL = legacy
 *     default stream) and returns without synchronizing. Nothing here allocates device memory:
 *     outputs and workspaces come from the caller.
 *   - Return value: 0 on success, a PLZ_ERR_* code otherwise; plz_last_error() gives the text.
 *     Nothing throws. Launch errors are checked (cudaGetLastError) on every call.
 *   - Device-side waits are bounded. A kernel that gives up records a code in a per-device status
 *     word; plz_device_status() synchronizes the device and reads (and clears) it.
 *   - bf16 matrices are row-major with an explicit row pitch in ELEMENTS; bases and pitches must be
 *     multiples of 16 bytes (TMA requirement).
 *
 * Weight format (plz_weight_t)
 *   W[n, k] = palette[(n / gs_n) * (K / gs_k) + k / gs_k][ idx[n, k] ],  idx in {0,1,2,3}
 *   packed: N rows of `packed_pitch` bytes; element k of a row is bits 2*(k%4)..2*(k%4)+1 of byte k/4
 *           (the bit order of the reference's .idx2 files, scripts/palettize_core.py:31-42).
 *   palette: bf16, 4 entries per group, groups ordered (n-group major, k-group minor).
 *   The reference's runtime layout -- one palette per 256 output columns, shared by every input row
 *   (scripts/qwen_model.py:98-102) -- is gs_n = 256, gs_k = K. One palette per output row and 256
 *   input columns is gs_n = 1, gs_k = 256.
 */
#ifndef PLZ_H_
#define PLZ_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PLZ_OK 0
#define PLZ_ERR_BAD_SHAPE 1
#define PLZ_ERR_BAD_ALIGN 2
#define PLZ_ERR_UNSUPPORTED 3
#define PLZ_ERR_CUDA 4
#define PLZ_ERR_WORKSPACE 5
#define PLZ_ERR_DEVICE_WAIT 6
#define PLZ_ERR_NULL 7
#define PLZ_ERR_TOO_LARGE 8

typedef struct plz_weight {
    int32_t N, K;          /* out features, in features */
    int32_t gs_n, gs_k;    /* palette group extents along n and k; gs_k % 64 == 0, K % gs_k == 0 */
    const void* packed;    /* uint8 [N][packed_pitch], 16-byte aligned rows */
    int64_t packed_pitch;  /* bytes, >= K/4, multiple of 16 */
    const void* palette;   /* bf16 [(N/gs_n) * (K/gs_k)][4], 8-byte aligned */
} plz_weight_t;

/* LoRA branch y += (scale * x A^T) B^T.  A: [rank, K] bf16, B: [N, rank] bf16 (both row-major).
 * rank must be a multiple of 8, at most 64. The reference stores lora_A as (K, rank)
 * (scripts/qwen_model.py:262-277); its transpose is what goes here. */
typedef struct plz_lora {
    int32_t rank;
    float scale;
    const void* A; int64_t lda;
    const void* B; int64_t ldb;
} plz_lora_t;

/* Index logits: element (n, k, p) at ptr[n * s_n + k * s_k + p * s_p] (strides in elements).
 * dtype 0 = fp32, 1 = fp16. Interleaved fp32 [N, K, 4]: (4K, 4, 1). The reference's planar
 * fp16 (4, K, N) (scripts/qwen_model.py:135-143): (1, N, K*N). */
typedef struct plz_logits {
    void* ptr;
    int32_t dtype;
    int64_t s_n, s_k, s_p;
} plz_logits_t;

/* Gumbel noise. mode 0: none (g = 0). mode 1: explicit fp32 tensor with its own strides.
 * mode 2: counter-based, g = gumbel(seed, (k * N + n) * 4 + p) -- the reference's sampler
 * (scripts/fused_lut_kernel.cu:1245-1256, noise index :1296-1299). */
typedef struct plz_noise {
    int32_t mode;
    uint32_t seed;
    const float* ptr;
    int64_t s_n, s_k, s_p;
} plz_noise_t;

int32_t plz_version(void);
/* Number of kernels this library has launched in this process so far (all entry points, all devices, all threads; not
 * synchronized across threads: read it from the thread that makes the calls). For callers that report how many device
 * kernels a region of their program ran. */
uint64_t plz_launch_count(void);
const char* plz_last_error(void);
/* Synchronizes the current device, copies the 4-word status {code, where, count, 0} to the HOST
 * array `out4` (may be NULL) and clears it. Returns PLZ_ERR_DEVICE_WAIT if a kernel gave up. */
int32_t plz_device_status(uint32_t* out4);

/* The GEMM kernels are persistent: one CTA per SM, holding most of its shared memory for the whole launch, so nothing
 * else can run beside them. plz_set_cta_limit(n) makes later launches use at most n CTAs (0 = all SMs again), which
 * leaves the other SMs to a communication library: set it around the dX product while the gradient all-reduce of the
 * same Linear is in flight. Process-wide. (No counterpart in the reference, which is single-GPU.) */
int32_t plz_set_cta_limit(int32_t n);
/* The large forward / dX products run on pairs of CTAs that share one 256 x 256 tile (tcgen05 cta_group::2). on = 0 keeps
 * them on the one-CTA-per-tile kernel that serves all other shapes (for comparisons and tests); default 1. Process-wide.
 * (No counterpart in the reference.) */
int32_t plz_set_pair_gemm(int32_t on);

/* ---- formats ---------------------------------------------------------------------------------
 * Pack unpacked int8/uint8 indices, element (n, k) at src[n * s_n + k * s_k], into `dst`.
 * Replaces pack_indices_2bit (scripts/palettize_core.py:31-42) as a device kernel; the reference
 * keeps int8 (K, N) on the GPU (scripts/qwen_model.py:80). */
int32_t plz_pack_indices(const void* src, int64_t s_n, int64_t s_k, int32_t N, int32_t K, void* dst,
                         int64_t pitch, void* stream);
/* Inverse of plz_pack_indices (unpack_indices_2bit, scripts/palettize_core.py:45-56). */
int32_t plz_unpack_indices(const void* src, int64_t pitch, int32_t N, int32_t K, void* dst, int64_t s_n,
                           int64_t s_k, void* stream);
/* Materialize W as bf16, element (n, k) at dst[n * d_n + k * d_k]. The gather of the reference's
 * fallback forward (scripts/qwen_model.py:183-186) / compute_hard_W_kernel
 * (scripts/triton_hard_forward.py:48). Used by tests to check the decode bit for bit. */
int32_t plz_dequantize(const plz_weight_t* w, void* dst, int64_t d_n, int64_t d_k, void* stream);

/* ---- forward ---------------------------------------------------------------------------------
 * y[M, N] = x[M, K] W^T (+ LoRA). Hard forward of PalettizedLinear: fused_lut_linear_fwd
 * (scripts/fused_lut_linear_cuda.py:74-117), fallback scripts/qwen_model.py:183-192, plus
 * QwenLoRA.forward (scripts/qwen_model.py:291-304) when `lora` is not NULL.
 * With LoRA, `t` is a caller-provided bf16 [M, rank] workspace (pitch = rank) that receives
 * scale * x A^T; keep it for plz_lora_bwd. */
int32_t plz_hard_fwd(const plz_weight_t* w, const void* x, int64_t ldx, int32_t M, const plz_lora_t* lora,
                     void* t, void* y, int64_t ldy, void* stream);

/* plz_hard_fwd with LoRA for callers that must not allocate. (No counterpart in the reference: its wrappers
 * allocate every intermediate through torch.)  Some hosts hand an operator its inputs and outputs and nothing
 * else: the host owns the whole device-memory pool, so a cudaMalloc inside the operator can fail or stall the
 * device, and there is no workspace argument to pass `t` through. For them the [M, rank] intermediate
 * scale * x A^T lives in a fixed 512 KiB array inside the library (every GPU that loads libplz.so holds it until
 * the process exits). Limits: M * rank <= 262144 elements (4096 rows at rank 64, 16384 rows at rank 16); larger
 * calls return PLZ_ERR_TOO_LARGE and change nothing. The first call on each device looks up the array's device
 * address (cudaGetSymbolAddress); make that first call outside any stream capture. The call itself performs no
 * cudaMalloc / cudaFree and uses no allocating library routine. All calls on a device share the one array and it
 * keeps the previous call's contents: rows [0, M) are rewritten before they are read, nothing needs to start at
 * zero, but two calls whose kernels overlap on the GPU (different streams) race on it -- serialize them. */
int32_t plz_hard_fwd_lora_static(const plz_weight_t* w, const void* x, int64_t ldx, int32_t M, const plz_lora_t* lora,
                                 void* y, int64_t ldy, void* stream);

/* Same product for 1 <= M <= 64 rows (token decode), written for the HBM roofline of the packed
 * weights: every SM streams its own range of weight rows exactly once. No LoRA branch. The
 * reference has no separate small-batch kernel: its hard forward (scripts/qwen_model.py:164-192,
 * scripts/fused_lut_kernel.cu:309) serves every batch size and reads one byte per weight. */
int32_t plz_hard_fwd_smallm(const plz_weight_t* w, const void* x, int64_t ldx, int32_t M, void* y, int64_t ldy,
                            void* stream);
/* The same for 1 to 4 weight matrices that multiply the SAME x (gate_proj and up_proj of the MLP; q, k and v projections of the
 * attention: separate Linears of the same input in the reference's model, listed with their shapes in
 * scripts/bench_triton_kernels.py:9 and :141-142, each wrapped on its own by scripts/qwen_model.py:769-794):
 * one launch streams all of them, ys[i] = x W_i^T (bf16 [M, N_i], pitch ldys[i]). M <= 16; all matrices share K and
 * the palette grouping. A decode step is bound by launch latency, not bandwidth, at 7 MB per Linear. */
int32_t plz_hard_fwd_smallm_multi(const plz_weight_t* const* ws, int32_t count, const void* x, int64_t ldx, int32_t M,
                                  void* const* ys, const int64_t* ldys, void* stream);
/* on = 1: small-M launches (M <= 16) carry the programmatic-stream-serialization attribute, so a launch may start while the
 * previous kernel of the stream is still running: it issues the loads of its weights and builds its tables at once, and
 * waits for the previous kernel to finish (griddepcontrol.wait) only before it reads x or writes y. This hides the
 * launch latency between the Linears of a decode step. Only valid when the kernel that precedes a small-M call in its
 * stream does not write that call's packed indices or palettes (true in inference; not right after plz_soft_select or
 * plz_pack_indices). Process-wide, default 0. */
int32_t plz_set_smallm_overlap(int32_t on);

/* One pass over the index logits: packed hard indices (argmax over the plain logits, first maximum
 * wins: scripts/triton_soft_forward.py:160-168) into w->packed (written!), and/or the soft weights
 * W_soft = softmax((logits + g) / tau) . palette as bf16 at w_soft[n * ws_n + k * ws_k]
 * (compute_P_W kernels, scripts/fused_lut_kernel.cu:1946-2004; scripts/triton_soft_forward.py:83-181).
 * Either output may be skipped (want_packed = 0 / w_soft = NULL). */
int32_t plz_soft_select(const plz_weight_t* w, const plz_logits_t* logits, const plz_noise_t* noise, float tau,
                        int32_t want_packed, void* w_soft, int64_t ws_n, int64_t ws_k, void* stream);

/* y = x Wd^T (+ LoRA) with a dense bf16 Wd [N, K] (pitch ldw): the soft forward without the
 * straight-through estimator, y = x W_soft (scripts/fused_lut_linear_cuda.py:239-275). */
int32_t plz_dense_fwd(const void* Wd, int64_t ldw, int32_t N, int32_t K, const void* x, int64_t ldx, int32_t M,
                      const plz_lora_t* lora, void* t, void* y, int64_t ldy, void* stream);

/* ---- backward --------------------------------------------------------------------------------
 * dX[M, K] = dY[M, N] W (+ LoRA: dt = scale * dY B into the bf16 [M, rank] workspace `dt`, then
 * dX += dt A). fused_lut_linear_bwd_grad_x_tc_kernel (scripts/fused_lut_kernel.cu:551) and
 * grad_x = grad_y @ W.T (scripts/fused_lut_linear_cuda.py:944). */
int32_t plz_bwd_dx(const plz_weight_t* w, const void* dY, int64_t lddy, int32_t M, const plz_lora_t* lora,
                   void* dt, void* dX, int64_t lddx, void* stream);
/* The two halves of plz_bwd_dx for callers that want dt early (it is also an input of the LoRA factor gradients, so
 * computing it first lets plz_bwd_dw_soft_lora run before the dX product and the gradient exchange overlap with dX):
 * plz_lora_dt: dt[M, rank] = scale * dY B;  plz_bwd_dx_with_dt: dX = dY W + dt A with dt as given. */
int32_t plz_lora_dt(const plz_lora_t* lora, const void* dY, int64_t lddy, int32_t M, int32_t N, void* dt, void* stream);
int32_t plz_bwd_dx_with_dt(const plz_weight_t* w, const void* dY, int64_t lddy, int32_t M, const plz_lora_t* lora, const void* dt,
                           void* dX, int64_t lddx, void* stream);
int32_t plz_dense_bwd_dx(const void* Wd, int64_t ldw, int32_t N, int32_t K, const void* dY, int64_t lddy,
                         int32_t M, const plz_lora_t* lora, void* dt, void* dX, int64_t lddx, void* stream);

/* Weight-gradient product dW = x^T dY, never written to memory, fused with the soft backward:
 *   dLogits[n,k,p] = dW[n,k] * P[p] * (palette[p] - W_soft)   (same dtype/strides as `logits`)
 *   dPalette[group][p] += sum dW * P[p]                        (fp32, ACCUMULATED: zero it first)
 * P is recomputed from logits and noise. Either output pointer may be NULL.
 * grad_W + soft_bwd_elementwise (scripts/fused_lut_linear_cuda.py:952-961,
 * scripts/fused_lut_kernel.cu:1877-1924; scripts/triton_soft_backward.py:165-325). */
int32_t plz_bwd_dw_soft(const plz_weight_t* w, const void* x, int64_t ldx, const void* dY, int64_t lddy,
                        int32_t M, const plz_logits_t* logits, const plz_noise_t* noise, float tau,
                        void* dlogits, float* dpalette, void* stream);
/* plz_bwd_dw_soft plus the LoRA factor gradients in the same launch: dA[rank, K] += dt^T x and dB[N, rank] += dY^T t
 * (fp32, accumulated) are computed by extra work items that fill the last, partially occupied round of the persistent
 * weight-gradient kernel, so x and dY are not streamed a second time. t / dt as left by plz_hard_fwd / plz_bwd_dx.
 * Autograd of scripts/qwen_model.py:300-304 fused with scripts/fused_lut_linear_cuda.py:952-961. */
int32_t plz_bwd_dw_soft_lora(const plz_weight_t* w, const void* x, int64_t ldx, const void* dY, int64_t lddy, int32_t M,
                             const plz_logits_t* logits, const plz_noise_t* noise, float tau, void* dlogits, float* dpalette,
                             const void* t, const void* dt, int32_t rank, float* dA, float* dB, void* stream);
/* Hard-mode palette gradient dPalette[group][idx[n,k]] += dW[n,k] (fp32, accumulated):
 * fused_lut_linear_bwd_grad_palette_kernel (scripts/fused_lut_kernel.cu:902-1127). */
int32_t plz_bwd_dw_hard(const plz_weight_t* w, const void* x, int64_t ldx, const void* dY, int64_t lddy,
                        int32_t M, float* dpalette, void* stream);
/* Data-parallel form of plz_bwd_dw_soft_lora: the weight-gradient product fused with the reduce-scatter of dLogits
 * over peer memory. Rank `my_rank` of `world` (2..8, N % (8 * world) == 0) owns weight rows [my_rank * N/world, ...).
 * stage[r] is rank r's staging buffer AS MAPPED IN THIS PROCESS (a peer mapping for r != my_rank; CUDA IPC or any other
 * peer-accessible allocation), fp32 [world][N/world][K][4]. The epilogue stores this rank's partial dLogits of row n
 * into stage[n / (N/world)], slot my_rank, with plain coalesced 16-byte stores: the partials cross NVLink while the
 * tensor cores work on the next tile, nothing is read back, and no dLogits buffer of the full size exists.
 * After every rank's launch has completed (the caller orders this, e.g. with a small collective on the stream),
 * plz_reduce_slots sums the `world` slots of a rank's own buffer in a fixed order into its shard,
 * out[shard_elems] = scale * sum_r stage_own[r][...]  (shard_elems = N/world * K * 4).
 * accumulate = 1 instead ADDS the partials (16-byte vector reductions, performed by the owner's L2) into ONE fp32
 * [N/world][K][4] accumulator per rank, stage[r], which its owner zeroes beforehand: no slots (1/world of the memory),
 * no reduction pass, but the order of the `world` additions per element, and so the last bit, varies from run to run.
 * Needs the native layout (gs_n = 1, interleaved fp32 logits). dPalette, dA, dB as in plz_bwd_dw_soft_lora
 * (rank = 0: no LoRA). No reference counterpart: the reference is single-process and leaves the whole gradient in
 * index_logits.grad (scripts/fused_lut_linear_cuda.py:952-961); this is that step for data-parallel ranks. */
int32_t plz_bwd_dw_soft_scatter(const plz_weight_t* w, const void* x, int64_t ldx, const void* dY, int64_t lddy, int32_t M,
                                const plz_logits_t* logits, const plz_noise_t* noise, float tau, float* const* stage,
                                int32_t world, int32_t my_rank, int32_t accumulate, float* dpalette, const void* t, const void* dt,
                                int32_t rank, float* dA, float* dB, void* stream);
/* Staging memory that the other ranks of the node can map (CUDA IPC): plz_peer_alloc allocates `bytes` of zeroed device
 * memory on the current device and fills the 64-byte handle to send to the peers (any host channel); plz_peer_open maps
 * a peer's handle into this process (peer access is enabled on first use); plz_peer_close / plz_peer_free undo them.
 * plz_peer_copy is one asynchronous copy-engine transfer between two such buffers (either side may be a peer mapping):
 * the all-gather of the reduced shards is `world - 1` of them per rank and takes no SM from the dX product beside it.
 * Only plz_peer_alloc / plz_peer_open allocate or map memory. */
int32_t plz_peer_alloc(int64_t bytes, void** ptr, uint8_t* handle64);
int32_t plz_peer_copy(void* dst, const void* src, int64_t bytes, void* stream);
int32_t plz_peer_zero(void* ptr, int64_t bytes, void* stream); /* asynchronous memset to 0 (accumulator of accumulate = 1) */
int32_t plz_peer_open(const uint8_t* handle64, void** ptr);
int32_t plz_peer_close(void* ptr);
int32_t plz_peer_free(void* ptr);
int32_t plz_reduce_slots(const float* stage, int32_t world, int64_t shard_elems, float* out, float scale, void* stream);
/* LoRA factor gradients, fp32, ACCUMULATED (zero them first):
 *   dA[rank, K] += dt^T x,   dB[N, rank] += dY^T t     (t, dt as left by plz_hard_fwd / plz_bwd_dx).
 * Autograd of scripts/qwen_model.py:300-304. */
int32_t plz_lora_bwd(const void* x, int64_t ldx, const void* dY, int64_t lddy, const void* t, const void* dt,
                     int32_t M, int32_t N, int32_t K, int32_t rank, float* dA, float* dB, void* stream);

/* ---- the ops around the Linears of a decoder layer, folded into the hard forward -------------------------
 * The reference has no code for these: it calls the HuggingFace decoder layer (scripts/train_qwen.py:1259-1266), whose
 * RMSNorm, SwiGLU and Linears are separate eager ops; the fusions were only planned there
 * (agent-ctx/agent-layer-fusion/TASKS.md). Semantics follow transformers' Qwen3RMSNorm / Qwen3MLP:
 *   rmsnorm(x)[m, k] = x[m, k] * rstd[m] * g[k],  rstd[m] = 1 / sqrt(mean_k x[m, k]^2 + eps);   mlp = down(silu(gate(h)) * up(h)).
 * plz_rms_rstd writes rstd (fp32 [M]).
 * plz_hard_fwd_norm: y = rmsnorm(x) W^T without materialising rmsnorm(x): g[k] is multiplied into the decoded weight tile
 *   (one bf16 rounding of W*g), rstd[m] scales the accumulator row in the epilogue. Either factor may be NULL.
 * plz_mlp_gate_up_fwd: act[M, N] = silu(h Wg^T) * (h Wu^T) with h = rmsnorm(x) (factors optional as above): one launch, the
 *   gate and up tiles share the x tiles and sit side by side in TMEM, the epilogue applies SwiGLU; the two [M, N]
 *   intermediates never reach HBM. Wg, Wu: same shape / grouping / pitch, N % 128 == 0. */
int32_t plz_rms_rstd(const void* x, int64_t ldx, int32_t M, int32_t K, float eps, float* rstd, void* stream);
int32_t plz_hard_fwd_norm(const plz_weight_t* w, const void* x, int64_t ldx, int32_t M, const float* row_scale,
                          const void* col_scale, void* y, int64_t ldy, void* stream);
int32_t plz_mlp_gate_up_fwd(const plz_weight_t* w_gate, const plz_weight_t* w_up, const void* x, int64_t ldx, int32_t M,
                            const float* row_scale, const void* col_scale, void* act, int64_t ldact, void* stream);
/* plz_mlp_gate_up_fwd that also writes the two pre-activations gate = h Wg^T and up = h Wu^T (bf16 [M, N], common pitch
 * ldgu) from the same accumulators, for a backward that does not recompute them (plz_swiglu_bwd). */
int32_t plz_mlp_gate_up_fwd_keep(const plz_weight_t* w_gate, const plz_weight_t* w_up, const void* x, int64_t ldx, int32_t M,
                                 const float* row_scale, const void* col_scale, void* act, int64_t ldact, void* gate, void* up,
                                 int64_t ldgu, void* stream);

/* Backward of the two element-wise ops above (the Linears between them use plz_bwd_dx / plz_bwd_dw_*):
 * plz_swiglu_bwd: from the pre-activations gate = h Wg^T, up = h Wu^T (bf16 [M, N], recomputed with plz_hard_fwd_norm
 *   or kept from an unfused forward) and dAct: dGate = dAct * up * silu'(gate), dUp = dAct * silu(gate)  (bf16 [M, N]).
 * plz_rmsnorm_bwd: from dH, the gradient with respect to h = rmsnorm(x): dX (bf16 [M, K]) and dG[K] += sum_m dH * x * rstd
 *   (fp32, ACCUMULATED: zero it first; NULL to skip). g may be NULL (no norm weight).
 * Semantics: autograd of transformers' Qwen3MLP / Qwen3RMSNorm, which the reference trains through
 * (scripts/train_qwen.py:1259-1266); no reference kernel exists for them. */
int32_t plz_swiglu_bwd(const void* gate, int64_t ldg, const void* up, int64_t ldu, const void* dact, int64_t ldd, int32_t M,
                       int32_t N, void* dgate, int64_t lddg, void* dup, int64_t lddu, void* stream);
int32_t plz_rmsnorm_bwd(const void* x, int64_t ldx, const void* dh, int64_t lddh, const float* rstd, const void* g, int32_t M,
                        int32_t K, void* dx, int64_t lddx, float* dg, void* stream);

/* ---- the steps around the Linear in the distillation loop ------------------------------------
 * One fused pass of fp32-master AdamW over a flat parameter of n elements:
 *   g = grad * grad_scale (grad_scale carries the gradient-clipping coefficient and 1/world_size);
 *   master *= 1 - lr*weight_decay; m, v updated; master -= lr/(1-beta1^step) * m / (sqrt(v)/sqrt(1-beta2^step) + eps);
 *   param (may be NULL) = master clamped to [clamp_lo, clamp_hi] (no clamp if clamp_lo > clamp_hi), cast to param_dtype;
 *   clamp_master != 0 also stores the clamped value in the master.
 * dtype codes: 0 fp32, 1 fp16, 2 bf16. Replaces FP32MasterAdamW.step (scripts/train_qwen.py:154-215, torch.optim.AdamW
 * with betas/eps of :600), clip_grad_norm_'s in-place scaling (:1303-1319) and the index-logit clamp to +-5 tau
 * (:1343-1348), which cost eight passes over the state there. */
int32_t plz_adamw_step(float* master, float* m, float* v, const void* grad, int32_t grad_dtype, float grad_scale, int64_t n,
                       float lr, float beta1, float beta2, float eps, float weight_decay, int32_t step, float clamp_lo,
                       float clamp_hi, int32_t clamp_master, void* param, int32_t param_dtype, void* stream);

/* Distillation loss of compute_loss (scripts/train_qwen.py:229-249), type "1-cos+norm_mse", fp32 math on bf16
 * student / teacher states s, t [M, H]:  loss = w_cos * mean_tokens(1 - cos(s, t)) + w_mse * mean((s-t)^2) / max(mean(t^2), 1e-6),
 * cosine with each norm clamped at 1e-4. out4 (device, may be NULL) receives {loss, l_cos, l_mse, mean(t^2)}.
 * ds (may be NULL) receives upstream * dLoss/ds in ds_dtype (0 fp32, 2 bf16). ws: caller workspace of 4 + 4*M floats, 16-byte aligned; the three sums are reduced in a fixed order, so the loss is
 * bit-identical from run to run. */
int32_t plz_distill_loss(const void* s, int64_t lds, const void* t, int64_t ldt, int32_t M, int32_t H, float w_cos, float w_mse,
                         float upstream, float* ws, float* out4, void* ds, int64_t ldds, int32_t ds_dtype, void* stream);

/* ---- bias -------------------------------------------------------------------------------------
 * plz_hard_fwd_bias: y = x W^T + bias with the bias (bf16 [N], 16-byte aligned, may be NULL) added in fp32 before the
 * bf16 store, as fused_lut_linear_fwd_tc_kernel does (scripts/fused_lut_kernel.cu:512-514; wrapper
 * scripts/fused_lut_linear_cuda.py:74-117). No LoRA branch (the reference's LoRA wraps a bias-carrying Linear from outside).
 * plz_col_sum: out[n] += sum_m dY[m, n] (fp32, ACCUMULATED): the bias gradient grad_y.sum(0),
 * fused_lut_linear_bwd_grad_bias (scripts/fused_lut_kernel.cu:1129). */
int32_t plz_hard_fwd_bias(const plz_weight_t* w, const void* x, int64_t ldx, int32_t M, const void* bias, void* y, int64_t ldy,
                          void* stream);
int32_t plz_col_sum(const void* dY, int64_t lddy, int32_t M, int32_t N, float* out, void* stream);

/* ---- the soft path with its intermediates as tensors -----------------------------------------
 * For callers of the reference's lower-level extension functions (scripts/fused_lut_linear_cuda.py:721-732), which pass
 * P, W_soft / W_hard and a materialised dW between calls. The training path above needs none of them.
 * Outputs of one matrix, each through element strides (element (n, k[, p])), each may be NULL:
 *   P fp16 = softmax((logits + g) / tau);  w_soft bf16 = sum_p P[p] palette[p];  w_hard bf16 = palette[hard index]. */
typedef struct plz_soft_out {
    void* P; int64_t p_n, p_k, p_p;
    void* w_soft; int64_t ws_n, ws_k;
    void* w_hard; int64_t wh_n, wh_k;
} plz_soft_out_t;
/* One launch (per 12 matrices) over `count` matrices: the compute_P_W kernels (scripts/fused_lut_kernel.cu:1946-2004) and
 * their batched form fused_compute_P_W_batched (:2097-2158; the caller passes noise[i]->seed = step_seed ^ (i * 0x9E3779B9u)
 * to reproduce its per-layer seeds). ws[i]->packed is not used. noise may be NULL (no noise), as may any noise[i].
 * hard_from_noisy = 1: hard index = argmax of P, i.e. of the NOISED logits, as compute_P_W_hard_aos_kernel does
 * (:1996-2003); 0: argmax of the plain logits (scripts/triton_soft_forward.py:160-168), the rule of plz_soft_select. */
int32_t plz_soft_weights(int32_t count, const plz_weight_t* const* ws, const plz_logits_t* const* logits,
                         const plz_noise_t* const* noise, float tau, int32_t hard_from_noisy, const plz_soft_out_t* const* outs,
                         void* stream);
/* Element-wise soft backward from a materialised dW (dtype 0 fp32 / 2 bf16, element (n, k) at dW[n * dw_n + k * dw_k]) and
 * P (fp16, strides as above): dLogits[p] = dW P[p] (palette[p] - W_soft) into `dlogits` (dtype / strides of a logits
 * descriptor; NULL to skip) and dPalette[group][p] += dW P[p] (fp32, ACCUMULATED; NULL to skip).
 * soft_bwd_elementwise_aos_kernel (scripts/fused_lut_kernel.cu:1877-1924), fused_lut_linear_soft_bwd (wrappers in
 * scripts/fused_lut_linear_cuda.py:275-340). */
int32_t plz_soft_bwd_elementwise(const plz_weight_t* w, const void* dW, int32_t dw_dtype, int64_t dw_n, int64_t dw_k, const void* P,
                                 int64_t p_n, int64_t p_k, int64_t p_p, const plz_logits_t* dlogits, float* dpalette, void* stream);
/* dW[n * dw_n + k * dw_k] += sum_m dY[m, n] x[m, k] (fp32, ACCUMULATED: zero it first): grad_W = x^T grad_y as a tensor
 * (scripts/fused_lut_linear_cuda.py:952). N and K multiples of 8. */
int32_t plz_weight_grad(const void* x, int64_t ldx, const void* dY, int64_t lddy, int32_t M, int32_t N, int32_t K, float* dW,
                        int64_t dw_n, int64_t dw_k, void* stream);

/* ---- attention of the decoder layers -----------------------------------------------------------
 * Causal grouped-query attention on tokens-major activations: q bf16 [B * S, Hq * 128] (row pitch ldq), k / v bf16
 * [B * S, Hkv * 128], o in the layout of q: exactly what the q/k/v projections write and o_proj reads. S % 128 == 0,
 * head_dim = 128, Hq % Hkv == 0. o = softmax(q k^T * scale + causal mask) v per (batch, head), fp32 softmax.
 * lse (fp32 [B, Hq, S], may be NULL in the forward) receives the natural-log sum-exp of the scaled scores; the backward
 * needs it, together with o, and a workspace dsum_ws of B * Hq * S floats. Gradients dq / dk / dv have the layouts and
 * pitches of q / k / v and are WRITTEN (dk, dv already summed over the q heads of a group).
 * The reference has no attention code: it calls the HuggingFace decoder layer (scripts/train_qwen.py:1259-1266; SDPA
 * selected at scripts/qwen_model.py:454); semantics are those of transformers' Qwen3Attention after q/k norm and RoPE. */
int32_t plz_attn_fwd(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, int32_t B, int32_t S,
                     int32_t Hq, int32_t Hkv, int32_t head_dim, float scale, void* o, int64_t ldo, float* lse, void* stream);
int32_t plz_attn_bwd(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, const void* o, const void* d_o,
                     int64_t ldo, const float* lse, int32_t B, int32_t S, int32_t Hq, int32_t Hkv, int32_t head_dim, float scale,
                     float* dsum_ws, void* dq, void* dk, void* dv, void* stream);

/* Attention of ONE new token per sequence against a key / value cache (token decode; transformers' Qwen3Attention at
 * q_len = 1 with a DynamicCache): out[b, h] = softmax(q[b, h] . K[b, 0..T, h / group] * scale) V[b, 0..T, h / group].
 * q / out: bf16 [B, Hq * 128]; caches bf16 [B, T_max, Hkv * 128] given by the element strides between sequences and between
 * positions; T counts the positions to attend to (the new token's key and value already stored). head_dim = 128.
 * ws: plz_attn_decode_ws_bytes(B, T, Hq, Hkv) bytes of scratch (the sequence is split over several CTAs when B * Hkv alone
 * would not fill the GPU; 0 bytes when it is not split), 16-byte aligned. */
int64_t plz_attn_decode_ws_bytes(int32_t B, int32_t T, int32_t Hq, int32_t Hkv);
int32_t plz_attn_decode(const void* q, int64_t ldq, const void* k_cache, const void* v_cache, int64_t batch_stride, int64_t tok_stride,
                        int32_t B, int32_t T, int32_t Hq, int32_t Hkv, int32_t head_dim, float scale, void* out, int64_t ldo, void* ws,
                        int64_t ws_bytes, void* stream);
/* out[i, :] = table[ids[i], :], bf16 rows of `width` elements (embed_tokens of the HuggingFace model the reference wraps,
 * scripts/qwen_model.py:897-951). An id outside [0, vocab) gives a zero row and stores 1 to *bad (device int32, may be NULL). */
int32_t plz_embed_gather(const void* table, int64_t ldt, const int64_t* ids, int64_t n, int32_t width, int64_t vocab, void* out, int64_t ldo,
                         int32_t* bad, void* stream);

/* ---- element-wise ops of a decoder layer -------------------------------------------------------
 * The reference has no code for these (it calls the HuggingFace decoder layer, scripts/train_qwen.py:1259-1266);
 * semantics follow transformers' Qwen3RMSNorm / Qwen3Attention (q_norm, k_norm, apply_rotary_pos_emb) / Qwen3MLP.
 * plz_rmsnorm_fwd: h = bf16(bf16(x * rstd) * g), rstd = 1 / sqrt(mean x^2 + eps) also written to rstd (fp32 [M], may be NULL);
 *   the materialised form of the norm that plz_hard_fwd_norm folds into a GEMM, for Linears that carry a LoRA branch.
 * plz_qknorm_rope_fwd: per (token, head) vector of 128: RMSNorm with weight w (bf16 [128], may be NULL), then the rotary
 *   embedding out[i] = y[i] cos_i - y[i+64] sin_i, out[i+64] = y[i+64] cos_i + y[i] sin_i with cos / sin fp32 [S, 64] tables
 *   indexed by the token's position inside its sequence (token index % S). x / out: bf16 [tokens, H * 128].
 * plz_qknorm_rope_bwd: dy -> dx, and dw[128] += (fp32, ACCUMULATED; NULL to skip).
 * plz_swiglu_fwd: act = bf16(silu(gate)) * up.  plz_add: out = a + b (+ c if not NULL), fp32 sum rounded once (residuals,
 *   sums of input gradients).
 * plz_bwd_dw_hard_lora: plz_bwd_dw_hard plus the LoRA factor gradients in the same launch (as plz_bwd_dw_soft_lora). */
int32_t plz_rmsnorm_fwd(const void* x, int64_t ldx, const void* g, int32_t M, int32_t K, float eps, void* h, int64_t ldh, float* rstd,
                        void* stream);
/* sum_out = bf16(x + addend) and h = rmsnorm(sum_out) * g in one pass: a residual add and the norm that follows it. */
int32_t plz_add_rmsnorm_fwd(const void* x, int64_t ldx, const void* addend, int64_t lda, void* sum_out, int64_t lds, const void* g, int32_t M,
                            int32_t K, float eps, void* h, int64_t ldh, float* rstd, void* stream);
/* plz_qknorm_rope_fwd for the q and the k projection of the same tokens in one launch. */
int32_t plz_qknorm_rope_fwd2(const void* xq, int64_t ldxq, const void* wq, int32_t Hq, void* outq, int64_t ldoq, const void* xk, int64_t ldxk,
                             const void* wk, int32_t Hk, void* outk, int64_t ldok, const float* cos_tab, const float* sin_tab, int64_t tokens,
                             int32_t S, int32_t head_dim, float eps, void* stream);
int32_t plz_qknorm_rope_fwd(const void* x, int64_t ldx, const void* w, const float* cos_tab, const float* sin_tab, int64_t tokens,
                            int32_t H, int32_t S, int32_t head_dim, float eps, void* out, int64_t ldo, void* stream);
int32_t plz_qknorm_rope_bwd(const void* x, int64_t ldx, const void* w, const float* cos_tab, const float* sin_tab, const void* dy,
                            int64_t lddy, int64_t tokens, int32_t H, int32_t S, int32_t head_dim, float eps, void* dx, int64_t lddx,
                            float* dw, void* stream);
int32_t plz_swiglu_fwd(const void* gate, int64_t ldg, const void* up, int64_t ldu, int32_t M, int32_t N, void* act, int64_t lda, void* stream);
int32_t plz_add(const void* a, int64_t lda, const void* b, int64_t ldb, const void* c, int64_t ldc, int32_t M, int32_t N, void* out,
                int64_t ldo, void* stream);
int32_t plz_bwd_dw_hard_lora(const plz_weight_t* w, const void* x, int64_t ldx, const void* dY, int64_t lddy, int32_t M, float* dpalette,
                             const void* t, const void* dt, int32_t rank, float* dA, float* dB, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PLZ_H_ */
