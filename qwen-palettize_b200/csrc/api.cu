// extern "C" entry points of libplz.so (declared and documented in include/plz.h) and the small amount
// of host state behind them: last-error text, the per-device status word, the tensor-map encoder.
#include <stdarg.h>
#include <string.h>

#include "../../include/plz.h"
#include "plz_launch.h"
#include "soft_math.cuh"

namespace plz {

// ---- host state ------------------------------------------------------------------------------
static thread_local char g_err[512] = "";

void set_last_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

unsigned long long g_launch_count = 0;

__device__ StatusWord g_status_word;

StatusWord* device_status_ptr() {
    static StatusWord* ptrs[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    dev &= 63;
    if (!ptrs[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
        ptrs[dev] = (StatusWord*)p;
    }
    return ptrs[dev];
}

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

int make_tmap_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                   uint32_t box_cols, uint32_t box_rows) {
    EncodeTiledFn enc = get_encode_fn();
    // The driver call needs the device's primary context current on the calling thread; a thread that has
    // only been handed a device by cudaSetDevice (e.g. an autograd worker) may not have it bound yet.
    static thread_local int bound_dev = -1;
    int dev = -1;
    if (cudaGetDevice(&dev) == cudaSuccess && dev != bound_dev) {
        cudaSetDevice(dev);  // binds the primary context to this thread (allocates nothing)
        bound_dev = dev;
    }
    if (!enc) { set_last_error("cuTensorMapEncodeTiled is not available from the driver"); return PLZ_ERR_CUDA; }
    if (!base) { set_last_error("null matrix pointer"); return PLZ_ERR_NULL; }
    if (((uintptr_t)base & 15) || ((ld * 2) & 15)) {
        set_last_error("bf16 matrix base (%p) and row pitch (%llu elements) must be multiples of 16 bytes", base,
                       (unsigned long long)ld);
        return PLZ_ERR_BAD_ALIGN;
    }
    if (ld < cols) { set_last_error("row pitch %llu < columns %llu", (unsigned long long)ld, (unsigned long long)cols); return PLZ_ERR_BAD_SHAPE; }
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("cuTensorMapEncodeTiled failed with CUresult %d (rows %llu cols %llu ld %llu box %ux%u)", (int)r,
                       (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld, box_cols, box_rows);
        return PLZ_ERR_CUDA;
    }
    return PLZ_OK;
}

static int check_weight(const plz_weight_t* w, bool need_packed) {
    if (!w) { set_last_error("null weight descriptor"); return PLZ_ERR_NULL; }
    if (w->N <= 0 || w->K <= 0) { set_last_error("weight is empty (N=%d, K=%d)", w->N, w->K); return PLZ_ERR_BAD_SHAPE; }
    if (w->K % 64) { set_last_error("K=%d must be a multiple of 64", w->K); return PLZ_ERR_BAD_SHAPE; }
    if (w->N % 8) { set_last_error("N=%d must be a multiple of 8", w->N); return PLZ_ERR_BAD_SHAPE; }
    if (w->gs_n <= 0 || w->gs_k <= 0 || w->gs_k % 64 || w->K % w->gs_k || w->N % w->gs_n) {
        set_last_error("palette groups (gs_n=%d, gs_k=%d) must tile (N=%d, K=%d); gs_k %% 64 == 0", w->gs_n, w->gs_k, w->N, w->K);
        return PLZ_ERR_BAD_SHAPE;
    }
    if (need_packed) {
        if (!w->packed) { set_last_error("null packed indices"); return PLZ_ERR_NULL; }
        if (w->packed_pitch < w->K / 4 || (w->packed_pitch & 15) || ((uintptr_t)w->packed & 15)) {
            set_last_error("packed rows must be 16-byte aligned with pitch >= K/4 (pitch=%lld)", (long long)w->packed_pitch);
            return PLZ_ERR_BAD_ALIGN;
        }
    }
    if (!w->palette) { set_last_error("null palette"); return PLZ_ERR_NULL; }
    if ((uintptr_t)w->palette & 7) { set_last_error("palette must be 8-byte aligned"); return PLZ_ERR_BAD_ALIGN; }
    return PLZ_OK;
}

static int check_lora(const plz_lora_t* l, const void* ws) {
    if (!l) return PLZ_OK;
    if (l->rank <= 0 || l->rank > 64 || l->rank % 8) { set_last_error("LoRA rank %d must be a multiple of 8 in [8, 64]", l->rank); return PLZ_ERR_BAD_SHAPE; }
    if (!l->A || !l->B) { set_last_error("null LoRA factor"); return PLZ_ERR_NULL; }
    if (!ws) { set_last_error("LoRA needs the [M, rank] bf16 workspace"); return PLZ_ERR_WORKSPACE; }
    if ((uintptr_t)ws & 15) { set_last_error("LoRA workspace must be 16-byte aligned"); return PLZ_ERR_BAD_ALIGN; }
    return PLZ_OK;
}

// t = scale * x A^T  (bf16 [M, rank])
static int lora_down(const plz_lora_t* l, const void* x, long long ldx, int M, int K, void* t, cudaStream_t s) {
    LutGemmArgs g = {};
    g.bmode = B_TMA_K; g.M = M; g.J = l->rank; g.R = K;
    g.A = x; g.lda = ldx; g.Bdense = l->A; g.ldb = l->lda;
    g.out = t; g.ld_out = l->rank; g.alpha = l->scale;
    return launch_lut_gemm(g, s);
}
// dt = scale * dY B  (bf16 [M, rank]); reduction over N, B is [N, rank] -> MN-major operand
static int lora_up_bwd(const plz_lora_t* l, const void* dY, long long lddy, int M, int N, void* dt, cudaStream_t s) {
    if (N % 64) { set_last_error("LoRA backward needs N %% 64 == 0 (N=%d)", N); return PLZ_ERR_BAD_SHAPE; }
    LutGemmArgs g = {};
    g.bmode = B_TMA_MN; g.M = M; g.J = l->rank; g.R = N;
    g.A = dY; g.lda = lddy; g.Bdense = l->B; g.ldb = l->ldb;
    g.out = dt; g.ld_out = l->rank; g.alpha = l->scale;
    return launch_lut_gemm(g, s);
}

}  // namespace plz

using namespace plz;

#ifdef PLZ_DIAGNOSTICS
static void* g_prof_buffer = nullptr;
#else
static void* const g_prof_buffer = nullptr;
#endif

extern "C" {

#ifdef PLZ_DIAGNOSTICS
// Diagnostics build only (-DPLZ_DIAGNOSTICS): point the kernels at a device buffer of 8 x uint64 per CTA that receives
// cycle counts of their issuing threads; keep the small-M forward off the mma.sync kernel. Not part of the ABI.
void plz_debug_set_profile_buffer(void* dev_ptr) { g_prof_buffer = dev_ptr; }
void plz_debug_set_smallm_variant(int v) { g_debug_smallm_variant = v; }
#endif
int32_t plz_set_cta_limit(int32_t n) { g_cta_limit = n > 0 ? n : 0; return PLZ_OK; }

int32_t plz_set_pair_gemm(int32_t on) { g_pair_gemm = on ? 1 : 0; return PLZ_OK; }

int32_t plz_set_smallm_overlap(int32_t on) { g_smallm_overlap = on ? 1 : 0; return PLZ_OK; }

int32_t plz_version(void) { return 110; }
uint64_t plz_launch_count(void) { return g_launch_count; }
const char* plz_last_error(void) { return g_err; }

int32_t plz_device_status(uint32_t* out4) {
    StatusWord* d = device_status_ptr();
    if (!d) { set_last_error("no CUDA device / status word unavailable"); return PLZ_ERR_CUDA; }
    PLZ_CUDA_CHECK(cudaDeviceSynchronize());
    StatusWord h;
    PLZ_CUDA_CHECK(cudaMemcpy(&h, d, sizeof(h), cudaMemcpyDeviceToHost));
    if (out4) { out4[0] = h.code; out4[1] = h.where; out4[2] = h.count; out4[3] = 0; }
    if (h.code != 0) {
        PLZ_CUDA_CHECK(cudaMemset(d, 0, sizeof(h)));
        set_last_error("a kernel gave up waiting: code %u, block %u, role %u, %u reports", h.code, h.where & 0xFFFFFFu,
                       h.where >> 24, h.count);
        return PLZ_ERR_DEVICE_WAIT;
    }
    return PLZ_OK;
}

int32_t plz_pack_indices(const void* src, int64_t s_n, int64_t s_k, int32_t N, int32_t K, void* dst, int64_t pitch,
                         void* stream) {
    if (N < 0 || K < 0) { set_last_error("negative extent"); return PLZ_ERR_BAD_SHAPE; }
    if (N == 0 || K == 0) return PLZ_OK;
    if (!src || !dst) { set_last_error("null pointer"); return PLZ_ERR_NULL; }
    if (pitch < (K + 3) / 4) { set_last_error("pitch %lld < K/4", (long long)pitch); return PLZ_ERR_BAD_SHAPE; }
    return launch_pack_indices(src, s_n, s_k, N, K, dst, pitch, (cudaStream_t)stream);
}

int32_t plz_unpack_indices(const void* src, int64_t pitch, int32_t N, int32_t K, void* dst, int64_t s_n, int64_t s_k,
                           void* stream) {
    if (N < 0 || K < 0) { set_last_error("negative extent"); return PLZ_ERR_BAD_SHAPE; }
    if (N == 0 || K == 0) return PLZ_OK;
    if (!src || !dst) { set_last_error("null pointer"); return PLZ_ERR_NULL; }
    return launch_unpack_indices(src, pitch, N, K, dst, s_n, s_k, (cudaStream_t)stream);
}

int32_t plz_dequantize(const plz_weight_t* w, void* dst, int64_t d_n, int64_t d_k, void* stream) {
    int rc = check_weight(w, true);
    if (rc) return rc;
    if (!dst) { set_last_error("null output"); return PLZ_ERR_NULL; }
    return launch_dequant(w->packed, w->packed_pitch, w->palette, w->gs_n, w->gs_k, w->N, w->K, dst, d_n, d_k,
                          (cudaStream_t)stream);
}

int32_t plz_hard_fwd(const plz_weight_t* w, const void* x, int64_t ldx, int32_t M, const plz_lora_t* lora, void* t,
                     void* y, int64_t ldy, void* stream) {
    int rc = check_weight(w, true);
    if (rc) return rc;
    if (M < 0) { set_last_error("negative M"); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0) return PLZ_OK;
    if (!x || !y) { set_last_error("null activation pointer"); return PLZ_ERR_NULL; }
    if ((rc = check_lora(lora, t))) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (lora && (rc = lora_down(lora, x, ldx, M, w->K, t, s))) return rc;
    LutGemmArgs g = {};
    g.bmode = B_DECODE_K; g.M = M; g.J = w->N; g.R = w->K;
    g.A = x; g.lda = ldx;
    g.packed = w->packed; g.packed_pitch = w->packed_pitch; g.palette = w->palette;
    g.gs_n = w->gs_n; g.gs_k = w->gs_k; g.Wn = w->N; g.Wk = w->K;
    if (lora) { g.r2 = lora->rank; g.A2 = t; g.lda2 = lora->rank; g.B2 = lora->B; g.ldb2 = lora->ldb; }
    g.out = y; g.ld_out = ldy; g.alpha = 1.0f; g.prof = g_prof_buffer;
    return launch_lut_gemm(g, s);
}

// ---- allocation-free LoRA forward ---------------------------------------------------------------
// Scratch for plz_hard_fwd_lora_static: the [M, rank] bf16 intermediate scale * x A^T. It lives in the
// library image, so every GPU that loads libplz.so carries these 512 KiB until the process exits.
#define PLZ_STATIC_LORA_ELEMS (4096 * 64)
static __device__ __align__(256) __nv_bfloat16 g_lora_scratch[PLZ_STATIC_LORA_ELEMS];

// In host code `g_lora_scratch` is only a handle for the runtime, never an address a kernel may use: the
// device address is looked up once per device (with that device current) and cached.
static int lora_scratch_ptr(void** out) {
    static void* ptrs[64] = {};
    int dev = 0;
    PLZ_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) { set_last_error("device index %d out of range", dev); return PLZ_ERR_UNSUPPORTED; }
    if (!ptrs[dev]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_lora_scratch);
        if (e != cudaSuccess || !p) {
            set_last_error("cudaGetSymbolAddress(g_lora_scratch) failed: %s", cudaGetErrorString(e));
            return PLZ_ERR_CUDA;
        }
        ptrs[dev] = p;
    }
    *out = ptrs[dev];
    return PLZ_OK;
}

int32_t plz_hard_fwd_lora_static(const plz_weight_t* w, const void* x, int64_t ldx, int32_t M, const plz_lora_t* lora,
                                 void* y, int64_t ldy, void* stream) {
    if (!lora) { set_last_error("plz_hard_fwd_lora_static needs a LoRA descriptor; without LoRA call plz_hard_fwd"); return PLZ_ERR_NULL; }
    if (M < 0) { set_last_error("negative M"); return PLZ_ERR_BAD_SHAPE; }
    if (lora->rank > 0 && (long long)M * lora->rank > PLZ_STATIC_LORA_ELEMS) {
        set_last_error("plz_hard_fwd_lora_static: M * rank = %lld exceeds the built-in scratch of %d elements "
                       "(e.g. 4096 rows at rank 64, 16384 rows at rank 16); use plz_hard_fwd with your own workspace",
                       (long long)M * lora->rank, PLZ_STATIC_LORA_ELEMS);
        return PLZ_ERR_TOO_LARGE;
    }
    void* t = nullptr;
    int rc = lora_scratch_ptr(&t);
    if (rc) return rc;
    return plz_hard_fwd(w, x, ldx, M, lora, t, y, ldy, stream);
}

int32_t plz_hard_fwd_smallm(const plz_weight_t* w, const void* x, int64_t ldx, int32_t M, void* y, int64_t ldy,
                            void* stream) {
    int rc = check_weight(w, true);
    if (rc) return rc;
    if (M < 0 || M > 64) { set_last_error("plz_hard_fwd_smallm handles 0 <= M <= 64 (M=%d); use plz_hard_fwd", M); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0) return PLZ_OK;
    if (!x || !y) { set_last_error("null activation pointer"); return PLZ_ERR_NULL; }
    GemvArgs g = {};
    g.M = M; g.N = w->N; g.K = w->K; g.x = x; g.ldx = ldx;
    g.packed = w->packed; g.packed_pitch = w->packed_pitch; g.palette = w->palette;
    g.gs_n = w->gs_n; g.gs_k = w->gs_k; g.out = y; g.ld_out = ldy;
    int dev = 0, sms = 0;
    PLZ_CUDA_CHECK(cudaGetDevice(&dev));
    PLZ_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    g.sm_count = sms; g.prof = g_prof_buffer;
    return launch_lut_gemv(g, (cudaStream_t)stream);
}

int32_t plz_hard_fwd_smallm_multi(const plz_weight_t* const* ws, int32_t count, const void* x, int64_t ldx, int32_t M,
                                  void* const* ys, const int64_t* ldys, void* stream) {
    if (count < 1 || count > 4 || !ws || !ys || !ldys) { set_last_error("smallm_multi: 1 to 4 weight matrices"); return PLZ_ERR_BAD_SHAPE; }
    if (M < 0 || M > 16) { set_last_error("plz_hard_fwd_smallm_multi handles 0 <= M <= 16 (M=%d)", M); return PLZ_ERR_BAD_SHAPE; }
    GemvArgs g[4] = {};
    int dev = 0, sms = 0;
    PLZ_CUDA_CHECK(cudaGetDevice(&dev));
    PLZ_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    for (int i = 0; i < count; ++i) {
        int rc = check_weight(ws[i], true);
        if (rc) return rc;
        if (!ys[i]) { set_last_error("null output pointer"); return PLZ_ERR_NULL; }
        if (ws[i]->K != ws[0]->K || ws[i]->gs_n != ws[0]->gs_n || ws[i]->gs_k != ws[0]->gs_k) {
            set_last_error("smallm_multi: all matrices must share K and the palette grouping"); return PLZ_ERR_BAD_SHAPE;
        }
        g[i].M = M; g[i].N = ws[i]->N; g[i].K = ws[i]->K; g[i].x = x; g[i].ldx = ldx;
        g[i].packed = ws[i]->packed; g[i].packed_pitch = ws[i]->packed_pitch; g[i].palette = ws[i]->palette;
        g[i].gs_n = ws[i]->gs_n; g[i].gs_k = ws[i]->gs_k; g[i].out = ys[i]; g[i].ld_out = ldys[i];
        g[i].sm_count = sms;
    }
    if (M == 0) return PLZ_OK;
    if (!x) { set_last_error("null activation pointer"); return PLZ_ERR_NULL; }
    int rc = launch_lut_smallm_mma_multi(g, count, (cudaStream_t)stream);
    if (rc == PLZ_ERR_UNSUPPORTED)
        set_last_error("smallm_multi: needs K %% 256 == 0, palette groups of a multiple of 256 columns, 16-byte aligned x rows "
                       "and M * K small enough for shared memory; call plz_hard_fwd_smallm per matrix instead");
    return rc;
}

int32_t plz_dense_fwd(const void* Wd, int64_t ldw, int32_t N, int32_t K, const void* x, int64_t ldx, int32_t M,
                      const plz_lora_t* lora, void* t, void* y, int64_t ldy, void* stream) {
    if (N <= 0 || K <= 0 || M < 0 || K % 64 || N % 8) { set_last_error("dense_fwd: bad shape M=%d N=%d K=%d", M, N, K); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0) return PLZ_OK;
    if (!Wd || !x || !y) { set_last_error("null pointer"); return PLZ_ERR_NULL; }
    int rc;
    if ((rc = check_lora(lora, t))) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (lora && (rc = lora_down(lora, x, ldx, M, K, t, s))) return rc;
    LutGemmArgs g = {};
    g.bmode = B_TMA_K; g.M = M; g.J = N; g.R = K;
    g.A = x; g.lda = ldx; g.Bdense = Wd; g.ldb = ldw;
    if (lora) { g.r2 = lora->rank; g.A2 = t; g.lda2 = lora->rank; g.B2 = lora->B; g.ldb2 = lora->ldb; }
    g.out = y; g.ld_out = ldy; g.alpha = 1.0f;
    return launch_lut_gemm(g, s);
}

int32_t plz_soft_select(const plz_weight_t* w, const plz_logits_t* logits, const plz_noise_t* noise, float tau,
                        int32_t want_packed, void* w_soft, int64_t ws_n, int64_t ws_k, void* stream) {
    int rc = check_weight(w, want_packed != 0);
    if (rc) return rc;
    if (!logits || !logits->ptr) { set_last_error("null logits"); return PLZ_ERR_NULL; }
    if (!(tau > 0.f)) { set_last_error("tau must be positive"); return PLZ_ERR_BAD_SHAPE; }
    SelectParams p = {};
    p.logits = logits->ptr; p.ls_n = logits->s_n; p.ls_k = logits->s_k; p.ls_p = logits->s_p;
    if (noise) { p.noise = noise->ptr; p.ns_n = noise->s_n; p.ns_k = noise->s_k; p.ns_p = noise->s_p; p.noise_mode = noise->mode; p.seed = noise->seed; }
    p.inv_tau = 1.0f / tau;
    p.palette = (const __nv_bfloat16*)w->palette; p.gs_n = w->gs_n; p.gs_k = w->gs_k; p.n_kgroups = w->K / w->gs_k;
    p.N = w->N; p.K = w->K;
    p.packed = want_packed ? (uint8_t*)const_cast<void*>(w->packed) : nullptr; p.pitch = w->packed_pitch;
    p.w_soft = (__nv_bfloat16*)w_soft; p.ws_n = ws_n; p.ws_k = ws_k;
    if (!p.packed && !p.w_soft) return PLZ_OK;
    return launch_soft_select(p, logits->dtype == 1, (cudaStream_t)stream);
}

int32_t plz_bwd_dx(const plz_weight_t* w, const void* dY, int64_t lddy, int32_t M, const plz_lora_t* lora, void* dt,
                   void* dX, int64_t lddx, void* stream) {
    int rc = check_weight(w, true);
    if (rc) return rc;
    if (M < 0) { set_last_error("negative M"); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0) return PLZ_OK;
    if (w->N % 64) { set_last_error("bwd_dx needs N %% 64 == 0 (N=%d)", w->N); return PLZ_ERR_BAD_SHAPE; }
    if (!dY || !dX) { set_last_error("null gradient pointer"); return PLZ_ERR_NULL; }
    if ((rc = check_lora(lora, dt))) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (lora && (rc = lora_up_bwd(lora, dY, lddy, M, w->N, dt, s))) return rc;
    LutGemmArgs g = {};
    g.bmode = B_DECODE_MN; g.M = M; g.J = w->K; g.R = w->N;
    g.A = dY; g.lda = lddy;
    g.packed = w->packed; g.packed_pitch = w->packed_pitch; g.palette = w->palette;
    g.gs_n = w->gs_n; g.gs_k = w->gs_k; g.Wn = w->N; g.Wk = w->K;
    if (lora) { g.r2 = lora->rank; g.A2 = dt; g.lda2 = lora->rank; g.B2 = lora->A; g.ldb2 = lora->lda; }
    g.out = dX; g.ld_out = lddx; g.alpha = 1.0f; g.prof = g_prof_buffer;
    return launch_lut_gemm(g, s);
}

int32_t plz_lora_dt(const plz_lora_t* lora, const void* dY, int64_t lddy, int32_t M, int32_t N, void* dt, void* stream) {
    if (!lora) { set_last_error("null LoRA descriptor"); return PLZ_ERR_NULL; }
    if (M < 0 || N <= 0) { set_last_error("lora_dt: bad shape"); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0) return PLZ_OK;
    if (!dY) { set_last_error("null gradient pointer"); return PLZ_ERR_NULL; }
    int rc = check_lora(lora, dt);
    if (rc) return rc;
    return lora_up_bwd(lora, dY, lddy, M, N, dt, (cudaStream_t)stream);
}

int32_t plz_bwd_dx_with_dt(const plz_weight_t* w, const void* dY, int64_t lddy, int32_t M, const plz_lora_t* lora, const void* dt,
                           void* dX, int64_t lddx, void* stream) {
    int rc = check_weight(w, true);
    if (rc) return rc;
    if (M < 0) { set_last_error("negative M"); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0) return PLZ_OK;
    if (w->N % 64) { set_last_error("bwd_dx needs N %% 64 == 0 (N=%d)", w->N); return PLZ_ERR_BAD_SHAPE; }
    if (!dY || !dX) { set_last_error("null gradient pointer"); return PLZ_ERR_NULL; }
    if ((rc = check_lora(lora, dt))) return rc;
    LutGemmArgs g = {};
    g.bmode = B_DECODE_MN; g.M = M; g.J = w->K; g.R = w->N;
    g.A = dY; g.lda = lddy;
    g.packed = w->packed; g.packed_pitch = w->packed_pitch; g.palette = w->palette;
    g.gs_n = w->gs_n; g.gs_k = w->gs_k; g.Wn = w->N; g.Wk = w->K;
    if (lora) { g.r2 = lora->rank; g.A2 = dt; g.lda2 = lora->rank; g.B2 = lora->A; g.ldb2 = lora->lda; }
    g.out = dX; g.ld_out = lddx; g.alpha = 1.0f; g.prof = g_prof_buffer;
    return launch_lut_gemm(g, (cudaStream_t)stream);
}

int32_t plz_dense_bwd_dx(const void* Wd, int64_t ldw, int32_t N, int32_t K, const void* dY, int64_t lddy, int32_t M,
                         const plz_lora_t* lora, void* dt, void* dX, int64_t lddx, void* stream) {
    if (N <= 0 || K <= 0 || M < 0 || N % 64 || K % 8) { set_last_error("dense_bwd_dx: bad shape M=%d N=%d K=%d", M, N, K); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0) return PLZ_OK;
    if (!Wd || !dY || !dX) { set_last_error("null pointer"); return PLZ_ERR_NULL; }
    int rc;
    if ((rc = check_lora(lora, dt))) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (lora && (rc = lora_up_bwd(lora, dY, lddy, M, N, dt, s))) return rc;
    LutGemmArgs g = {};
    g.bmode = B_TMA_MN; g.M = M; g.J = K; g.R = N;
    g.A = dY; g.lda = lddy; g.Bdense = Wd; g.ldb = ldw;
    if (lora) { g.r2 = lora->rank; g.A2 = dt; g.lda2 = lora->rank; g.B2 = lora->A; g.ldb2 = lora->lda; }
    g.out = dX; g.ld_out = lddx; g.alpha = 1.0f;
    return launch_lut_gemm(g, s);
}

static int bwd_dw_common(int epi, const plz_weight_t* w, const void* x, int64_t ldx, const void* dY, int64_t lddy,
                         int32_t M, const plz_logits_t* logits, const plz_noise_t* noise, float tau, void* dlogits,
                         float* dpalette, void* stream, const void* t = nullptr, const void* dt = nullptr, int rank = 0,
                         float* dA = nullptr, float* dB = nullptr, float* const* peer_stage = nullptr, int world = 1,
                         int my_rank = 0, int scatter_add = 0) {
    int rc = check_weight(w, epi == EPI_HARD);
    if (rc) return rc;
    if (M < 0) { set_last_error("negative M"); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0) {
        // A rank without tokens contributes zeros. In the slot form of the fused reduce-scatter its slots would otherwise
        // keep the previous step's partials, which the owners' slot reduction would add again: clear them.
        if (world > 1 && !scatter_add) {
            if (w->N % world) { set_last_error("bwd_dw_soft_scatter: N=%d must be a multiple of world=%d", w->N, world); return PLZ_ERR_BAD_SHAPE; }
            const size_t shard_bytes = (size_t)(w->N / world) * (size_t)w->K * 16u;
            for (int r = 0; r < world; ++r) {
                if (!peer_stage[r]) { set_last_error("null peer staging pointer"); return PLZ_ERR_NULL; }
                PLZ_CUDA_CHECK(cudaMemsetAsync((char*)peer_stage[r] + (size_t)my_rank * shard_bytes, 0, shard_bytes, (cudaStream_t)stream));
            }
        }
        return PLZ_OK;
    }
    if (!x || !dY) { set_last_error("null activation pointer"); return PLZ_ERR_NULL; }
    TnArgs a = {};
    a.epi = epi; a.M = M;
    // Which of (n, k) runs along the TMEM lanes (threads of a warp) is chosen so that lanes walk the contiguous
    // axis of the logits: k for interleaved fp32 [N, K, 4] with a palette per weight row, n otherwise.
    bool rows_are_k = (w->gs_n == 1) && (w->gs_k % 128 == 0);
    if (epi == EPI_SOFT) {
        if (!logits || !logits->ptr) { set_last_error("null logits"); return PLZ_ERR_NULL; }
        rows_are_k = rows_are_k && logits->dtype == 0 && logits->s_p == 1 && logits->s_k < logits->s_n &&
                     (!noise || noise->mode != 1 || (noise->s_p == 1 && noise->s_k < noise->s_n));
    }
    a.rows_are_k = rows_are_k ? 1 : 0;
    if (rows_are_k) { a.I = w->K; a.J = w->N; a.P = x; a.ldp = ldx; a.Q = dY; a.ldq = lddy; }
    else { a.I = w->N; a.J = w->K; a.P = dY; a.ldp = lddy; a.Q = x; a.ldq = ldx; }
    if (epi == EPI_SOFT) {
        a.logits = logits->ptr; a.dlogits = dlogits; a.logits_f16 = logits->dtype == 1;
        a.ls_p = logits->s_p;
        a.ls_row = rows_are_k ? logits->s_k : logits->s_n;
        a.ls_col = rows_are_k ? logits->s_n : logits->s_k;
        if (noise) {
            a.noise_mode = noise->mode; a.noise = noise->ptr; a.seed = noise->seed; a.ns_p = noise->s_p;
            a.ns_row = rows_are_k ? noise->s_k : noise->s_n;
            a.ns_col = rows_are_k ? noise->s_n : noise->s_k;
        }
        a.hashN = w->N;
        a.tau = tau;
    } else {
        a.tau = 1.0f;
    }
    if (rank > 0) {
        // dB[n, r] += sum_m t[m, r] dY[m, n] and dA[r, k] += sum_m dt[m, r] x[m, k] ride as extra items of this launch
        const bool dy_is_p = !rows_are_k;  // P = dY when rows are n
        a.side_rank = rank;
        a.side_S[0] = dB ? t : nullptr; a.side_ld[0] = rank; a.side_q_is_p[0] = dy_is_p ? 1 : 0;
        a.side_out[0] = dB; a.side_si[0] = 1; a.side_sj[0] = rank;
        a.side_S[1] = dA ? dt : nullptr; a.side_ld[1] = rank; a.side_q_is_p[1] = dy_is_p ? 0 : 1;
        a.side_out[1] = dA; a.side_si[1] = w->K; a.side_sj[1] = 1;
    }
    a.palette = w->palette; a.dpalette = dpalette;
    a.gs_n = w->gs_n; a.gs_k = w->gs_k; a.n_kgroups = w->K / w->gs_k;
    a.packed = w->packed; a.packed_pitch = w->packed_pitch;
    int dev = 0, sms = 0;
    PLZ_CUDA_CHECK(cudaGetDevice(&dev));
    PLZ_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    a.sm_count = sms; a.prof = g_prof_buffer;
    if (world > 1) {
        a.world = world; a.rank = my_rank; a.scatter_add = scatter_add;
        for (int r = 0; r < world && r < 8; ++r) a.peer_stage[r] = peer_stage[r];
    }
    return launch_tn_gemm(a, (cudaStream_t)stream);
}

int32_t plz_bwd_dw_soft(const plz_weight_t* w, const void* x, int64_t ldx, const void* dY, int64_t lddy, int32_t M,
                        const plz_logits_t* logits, const plz_noise_t* noise, float tau, void* dlogits,
                        float* dpalette, void* stream) {
    if (!(tau > 0.f)) { set_last_error("tau must be positive"); return PLZ_ERR_BAD_SHAPE; }
    return bwd_dw_common(EPI_SOFT, w, x, ldx, dY, lddy, M, logits, noise, tau, dlogits, dpalette, stream);
}

int32_t plz_bwd_dw_soft_lora(const plz_weight_t* w, const void* x, int64_t ldx, const void* dY, int64_t lddy, int32_t M,
                             const plz_logits_t* logits, const plz_noise_t* noise, float tau, void* dlogits, float* dpalette,
                             const void* t, const void* dt, int32_t rank, float* dA, float* dB, void* stream) {
    if (!(tau > 0.f)) { set_last_error("tau must be positive"); return PLZ_ERR_BAD_SHAPE; }
    if (rank <= 0 || rank > 64 || rank % 8) { set_last_error("LoRA rank %d must be a multiple of 8 in [8, 64]", rank); return PLZ_ERR_BAD_SHAPE; }
    if ((dA && !dt) || (dB && !t)) { set_last_error("bwd_dw_soft_lora: dA needs dt and dB needs t"); return PLZ_ERR_NULL; }
    return bwd_dw_common(EPI_SOFT, w, x, ldx, dY, lddy, M, logits, noise, tau, dlogits, dpalette, stream, t, dt, rank, dA, dB);
}

int32_t plz_bwd_dw_soft_scatter(const plz_weight_t* w, const void* x, int64_t ldx, const void* dY, int64_t lddy, int32_t M,
                                const plz_logits_t* logits, const plz_noise_t* noise, float tau, float* const* stage,
                                int32_t world, int32_t my_rank, int32_t accumulate, float* dpalette, const void* t, const void* dt,
                                int32_t rank, float* dA, float* dB, void* stream) {
    if (!(tau > 0.f)) { set_last_error("tau must be positive"); return PLZ_ERR_BAD_SHAPE; }
    if (world < 2 || world > 8 || my_rank < 0 || my_rank >= world) { set_last_error("bwd_dw_soft_scatter: world must be in [2, 8] and 0 <= my_rank < world"); return PLZ_ERR_BAD_SHAPE; }
    if (!stage) { set_last_error("null staging pointer table"); return PLZ_ERR_NULL; }
    if (rank < 0 || rank > 64 || rank % 8) { set_last_error("LoRA rank %d must be 0 or a multiple of 8 in [8, 64]", rank); return PLZ_ERR_BAD_SHAPE; }
    if ((dA && !dt) || (dB && !t)) { set_last_error("bwd_dw_soft_scatter: dA needs dt and dB needs t"); return PLZ_ERR_NULL; }
    return bwd_dw_common(EPI_SOFT, w, x, ldx, dY, lddy, M, logits, noise, tau, nullptr, dpalette, stream, t, dt, rank, dA, dB,
                         stage, world, my_rank, accumulate ? 1 : 0);
}

// ---- peer-visible staging memory (CUDA IPC) ------------------------------------------------------------
int32_t plz_peer_alloc(int64_t bytes, void** ptr, uint8_t* handle64) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    if (bytes <= 0 || !ptr || !handle64) { set_last_error("peer_alloc: bad arguments"); return PLZ_ERR_NULL; }
    void* p = nullptr;
    PLZ_CUDA_CHECK(cudaMalloc(&p, (size_t)bytes));
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaMemset(p, 0, (size_t)bytes);
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) { cudaFree(p); set_last_error("peer_alloc: %s", cudaGetErrorString(e)); return PLZ_ERR_CUDA; }
    memcpy(handle64, &h, 64);
    *ptr = p;
    return PLZ_OK;
}
int32_t plz_peer_open(const uint8_t* handle64, void** ptr) {
    if (!handle64 || !ptr) { set_last_error("peer_open: null argument"); return PLZ_ERR_NULL; }
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    PLZ_CUDA_CHECK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return PLZ_OK;
}
int32_t plz_peer_copy(void* dst, const void* src, int64_t bytes, void* stream) {
    if (bytes < 0) { set_last_error("peer_copy: negative size"); return PLZ_ERR_BAD_SHAPE; }
    if (bytes == 0) return PLZ_OK;
    if (!dst || !src) { set_last_error("peer_copy: null pointer"); return PLZ_ERR_NULL; }
    PLZ_CUDA_CHECK(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDefault, (cudaStream_t)stream));
    return PLZ_OK;
}
int32_t plz_peer_zero(void* ptr, int64_t bytes, void* stream) {
    if (bytes < 0) { set_last_error("peer_zero: negative size"); return PLZ_ERR_BAD_SHAPE; }
    if (bytes == 0) return PLZ_OK;
    if (!ptr) { set_last_error("peer_zero: null pointer"); return PLZ_ERR_NULL; }
    PLZ_CUDA_CHECK(cudaMemsetAsync(ptr, 0, (size_t)bytes, (cudaStream_t)stream));
    return PLZ_OK;
}
int32_t plz_peer_close(void* ptr) { if (ptr) PLZ_CUDA_CHECK(cudaIpcCloseMemHandle(ptr)); return PLZ_OK; }
int32_t plz_peer_free(void* ptr) { if (ptr) PLZ_CUDA_CHECK(cudaFree(ptr)); return PLZ_OK; }

int32_t plz_reduce_slots(const float* stage, int32_t world, int64_t shard_elems, float* out, float scale, void* stream) {
    if (world < 1 || world > 8 || shard_elems < 0 || (shard_elems & 3)) { set_last_error("reduce_slots: world in [1, 8], shard_elems a non-negative multiple of 4"); return PLZ_ERR_BAD_SHAPE; }
    if (shard_elems == 0) return PLZ_OK;
    if (!stage || !out) { set_last_error("null pointer"); return PLZ_ERR_NULL; }
    if (((uintptr_t)stage | (uintptr_t)out) & 15) { set_last_error("reduce_slots: 16-byte alignment required"); return PLZ_ERR_BAD_ALIGN; }
    return launch_reduce_slots(stage, world, shard_elems, out, scale, (cudaStream_t)stream);
}

int32_t plz_bwd_dw_hard(const plz_weight_t* w, const void* x, int64_t ldx, const void* dY, int64_t lddy, int32_t M,
                        float* dpalette, void* stream) {
    if (!dpalette) { set_last_error("null dpalette"); return PLZ_ERR_NULL; }
    return bwd_dw_common(EPI_HARD, w, x, ldx, dY, lddy, M, nullptr, nullptr, 1.0f, nullptr, dpalette, stream);
}

int32_t plz_lora_bwd(const void* x, int64_t ldx, const void* dY, int64_t lddy, const void* t, const void* dt, int32_t M,
                     int32_t N, int32_t K, int32_t rank, float* dA, float* dB, void* stream) {
    if (M < 0 || N <= 0 || K <= 0 || rank <= 0 || rank > 64 || rank % 8) { set_last_error("lora_bwd: bad shape"); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0) return PLZ_OK;
    if (!x || !dY || !t || !dt) { set_last_error("null pointer"); return PLZ_ERR_NULL; }
    int dev = 0, sms = 0;
    PLZ_CUDA_CHECK(cudaGetDevice(&dev));
    PLZ_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    cudaStream_t s = (cudaStream_t)stream;
    int rc;
    if (dA) {
        // D[r, k] = sum_m dt[m, r] x[m, k]  -> dA[r * K + k]
        TnArgs a = {};
        a.epi = EPI_STORE; a.M = M; a.I = rank; a.J = K;
        a.P = dt; a.ldp = rank; a.Q = x; a.ldq = ldx;
        a.out = dA; a.out_si = K; a.out_sj = 1; a.alpha = 1.0f; a.out_I = rank; a.out_J = K;
        const int tiles = (K + 255) / 256;
        a.splits = (sms + tiles - 1) / tiles; a.sm_count = sms;
        if ((rc = launch_tn_gemm(a, s))) return rc;
    }
    if (dB) {
        // D[r, n] = sum_m t[m, r] dY[m, n] -> dB[n * rank + r]
        TnArgs a = {};
        a.epi = EPI_STORE; a.M = M; a.I = rank; a.J = N;
        a.P = t; a.ldp = rank; a.Q = dY; a.ldq = lddy;
        a.out = dB; a.out_si = 1; a.out_sj = rank; a.alpha = 1.0f; a.out_I = rank; a.out_J = N;
        const int tiles = (N + 255) / 256;
        a.splits = (sms + tiles - 1) / tiles; a.sm_count = sms;
        if ((rc = launch_tn_gemm(a, s))) return rc;
    }
    return PLZ_OK;
}

int32_t plz_rms_rstd(const void* x, int64_t ldx, int32_t M, int32_t K, float eps, float* rstd, void* stream) {
    if (M < 0 || K <= 0 || (K & 1)) { set_last_error("rms_rstd: K must be even and positive"); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0) return PLZ_OK;
    if (!x || !rstd) { set_last_error("null pointer"); return PLZ_ERR_NULL; }
    if (((uintptr_t)x & 3) || (ldx & 1)) { set_last_error("rms_rstd: rows must be 4-byte aligned"); return PLZ_ERR_BAD_ALIGN; }
    return launch_rms_rstd(x, ldx, M, K, eps, rstd, (cudaStream_t)stream);
}

static int fused_fwd(int fuse, const plz_weight_t* w, const plz_weight_t* w2, const void* x, int64_t ldx, int32_t M,
                     const float* row_scale, const void* col_scale, void* out, int64_t ldo, void* stream,
                     void* gate_out = nullptr, void* up_out = nullptr, int64_t ld_gu = 0) {
    int rc = check_weight(w, true);
    if (rc) return rc;
    if (fuse == 1) {
        if ((rc = check_weight(w2, true))) return rc;
        if (w2->N != w->N || w2->K != w->K || w2->gs_n != w->gs_n || w2->gs_k != w->gs_k || w2->packed_pitch != w->packed_pitch) {
            set_last_error("gate and up projections must have the same shape, grouping and packed pitch");
            return PLZ_ERR_BAD_SHAPE;
        }
        if (w->N % 128) { set_last_error("the fused gate/up forward needs N %% 128 == 0 (N=%d)", w->N); return PLZ_ERR_BAD_SHAPE; }
    }
    if (M < 0) { set_last_error("negative M"); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0) return PLZ_OK;
    if (!x || !out) { set_last_error("null activation pointer"); return PLZ_ERR_NULL; }
    if (col_scale && ((uintptr_t)col_scale & 15)) { set_last_error("norm weight must be 16-byte aligned"); return PLZ_ERR_BAD_ALIGN; }
    LutGemmArgs g = {};
    g.bmode = B_DECODE_K; g.M = M; g.J = (fuse == 1) ? 2 * w->N : w->N; g.R = w->K;
    g.A = x; g.lda = ldx;
    g.packed = w->packed; g.packed_pitch = w->packed_pitch; g.palette = w->palette;
    g.gs_n = w->gs_n; g.gs_k = w->gs_k; g.Wn = w->N; g.Wk = w->K;
    g.fuse = fuse; g.col_scale = col_scale; g.row_scale = row_scale;
    if (fuse == 1) { g.packed2 = w2->packed; g.palette2 = w2->palette; }
    if (gate_out || up_out) {
        if (!gate_out || !up_out) { set_last_error("gate and up outputs come together"); return PLZ_ERR_NULL; }
        if ((((uintptr_t)gate_out | (uintptr_t)up_out) & 15) || (ld_gu & 7) || ld_gu < w->N) {
            set_last_error("gate / up outputs: rows must be 16-byte aligned, pitch >= N"); return PLZ_ERR_BAD_ALIGN;
        }
        g.gate_out = gate_out; g.up_out = up_out; g.ld_gu = ld_gu;
    }
    g.out = out; g.ld_out = ldo; g.alpha = 1.0f;
    return launch_lut_gemm(g, (cudaStream_t)stream);
}

int32_t plz_swiglu_bwd(const void* gate, int64_t ldg, const void* up, int64_t ldu, const void* dact, int64_t ldd, int32_t M,
                       int32_t N, void* dgate, int64_t lddg, void* dup, int64_t lddu, void* stream) {
    if (M < 0 || N <= 0 || (N & 7)) { set_last_error("swiglu_bwd: N must be a positive multiple of 8"); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0) return PLZ_OK;
    if (!gate || !up || !dact || !dgate || !dup) { set_last_error("null pointer"); return PLZ_ERR_NULL; }
    if ((((uintptr_t)gate | (uintptr_t)up | (uintptr_t)dact | (uintptr_t)dgate | (uintptr_t)dup) & 15) ||
        ((ldg | ldu | ldd | lddg | lddu) & 7)) {
        set_last_error("swiglu_bwd: rows must be 16-byte aligned"); return PLZ_ERR_BAD_ALIGN;
    }
    return launch_swiglu_bwd(gate, ldg, up, ldu, dact, ldd, M, N, dgate, lddg, dup, lddu, (cudaStream_t)stream);
}

int32_t plz_rmsnorm_bwd(const void* x, int64_t ldx, const void* dh, int64_t lddh, const float* rstd, const void* g, int32_t M,
                        int32_t K, void* dx, int64_t lddx, float* dg, void* stream) {
    if (M < 0 || K <= 0 || (K & 1)) { set_last_error("rmsnorm_bwd: K must be even and positive"); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0) return PLZ_OK;
    if (!x || !dh || !rstd || !dx) { set_last_error("null pointer"); return PLZ_ERR_NULL; }
    if ((((uintptr_t)x | (uintptr_t)dh | (uintptr_t)dx | (uintptr_t)g) & 3) || ((ldx | lddh | lddx) & 1)) {
        set_last_error("rmsnorm_bwd: rows must be 4-byte aligned"); return PLZ_ERR_BAD_ALIGN;
    }
    return launch_rmsnorm_bwd(x, ldx, dh, lddh, rstd, g, M, K, dx, lddx, dg, (cudaStream_t)stream);
}

int32_t plz_hard_fwd_norm(const plz_weight_t* w, const void* x, int64_t ldx, int32_t M, const float* row_scale,
                          const void* col_scale, void* y, int64_t ldy, void* stream) {
    return fused_fwd(2, w, nullptr, x, ldx, M, row_scale, col_scale, y, ldy, stream);
}

int32_t plz_mlp_gate_up_fwd(const plz_weight_t* w_gate, const plz_weight_t* w_up, const void* x, int64_t ldx, int32_t M,
                            const float* row_scale, const void* col_scale, void* act, int64_t ldact, void* stream) {
    return fused_fwd(1, w_gate, w_up, x, ldx, M, row_scale, col_scale, act, ldact, stream);
}

int32_t plz_mlp_gate_up_fwd_keep(const plz_weight_t* w_gate, const plz_weight_t* w_up, const void* x, int64_t ldx, int32_t M,
                                 const float* row_scale, const void* col_scale, void* act, int64_t ldact, void* gate, void* up,
                                 int64_t ldgu, void* stream) {
    return fused_fwd(1, w_gate, w_up, x, ldx, M, row_scale, col_scale, act, ldact, stream, gate, up, ldgu);
}

int32_t plz_adamw_step(float* master, float* m, float* v, const void* grad, int32_t grad_dtype, float grad_scale, int64_t n,
                       float lr, float beta1, float beta2, float eps, float weight_decay, int32_t step, float clamp_lo,
                       float clamp_hi, int32_t clamp_master, void* param, int32_t param_dtype, void* stream) {
    if (n < 0 || step < 1) { set_last_error("adamw: n must be >= 0 and step >= 1"); return PLZ_ERR_BAD_SHAPE; }
    if (n == 0) return PLZ_OK;
    if (!master || !m || !v || !grad) { set_last_error("adamw: null state or gradient"); return PLZ_ERR_NULL; }
    if (grad_dtype < 0 || grad_dtype > 2 || param_dtype < 0 || param_dtype > 2) { set_last_error("adamw: dtype codes are 0 fp32, 1 fp16, 2 bf16"); return PLZ_ERR_UNSUPPORTED; }
    AdamParams p;
    p.master = master; p.m = m; p.v = v; p.grad = grad; p.param = param; p.n = n;
    p.grad_scale = grad_scale; p.lr = lr; p.beta1 = beta1; p.beta2 = beta2; p.eps = eps; p.weight_decay = weight_decay;
    p.bias_c1 = 1.0f - powf(beta1, (float)step);
    p.sqrt_bias_c2 = sqrtf(1.0f - powf(beta2, (float)step));
    p.clamp_lo = clamp_lo; p.clamp_hi = clamp_hi; p.clamp_master = clamp_master;
    return launch_adamw(p, grad_dtype, param_dtype, (cudaStream_t)stream);
}

int32_t plz_distill_loss(const void* s, int64_t lds, const void* t, int64_t ldt, int32_t M, int32_t H, float w_cos, float w_mse,
                         float upstream, float* ws, float* out4, void* ds, int64_t ldds, int32_t ds_dtype, void* stream) {
    if (M < 0 || H <= 0 || (H & 1)) { set_last_error("distill_loss: H must be even and positive (M=%d, H=%d)", M, H); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0) return PLZ_OK;
    if (!s || !t || !ws) { set_last_error("distill_loss: null input or workspace"); return PLZ_ERR_NULL; }
    if (((uintptr_t)ws & 15)) { set_last_error("distill_loss: the workspace must be 16-byte aligned"); return PLZ_ERR_BAD_ALIGN; }
    if (((uintptr_t)s & 3) || ((uintptr_t)t & 3) || (lds & 1) || (ldt & 1) || (ds && (ldds & 1))) { set_last_error("distill_loss: rows must be 4-byte aligned"); return PLZ_ERR_BAD_ALIGN; }
    if (ds_dtype != 0 && ds_dtype != 2) { set_last_error("distill_loss: gradient dtype must be 0 (fp32) or 2 (bf16)"); return PLZ_ERR_UNSUPPORTED; }
    return launch_distill_loss(s, lds, t, ldt, M, H, 1e-4f, w_cos, w_mse, upstream, ws, out4, ds, ldds, ds_dtype, (cudaStream_t)stream);
}

// ---- bias, and the soft path with its intermediates as tensors ------------------------------------------
int32_t plz_hard_fwd_bias(const plz_weight_t* w, const void* x, int64_t ldx, int32_t M, const void* bias, void* y, int64_t ldy,
                          void* stream) {
    int rc = check_weight(w, true);
    if (rc) return rc;
    if (M < 0) { set_last_error("negative M"); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0) return PLZ_OK;
    if (!x || !y) { set_last_error("null activation pointer"); return PLZ_ERR_NULL; }
    if (bias && ((uintptr_t)bias & 15)) { set_last_error("bias must be 16-byte aligned"); return PLZ_ERR_BAD_ALIGN; }
    LutGemmArgs g = {};
    g.bmode = B_DECODE_K; g.M = M; g.J = w->N; g.R = w->K;
    g.A = x; g.lda = ldx;
    g.packed = w->packed; g.packed_pitch = w->packed_pitch; g.palette = w->palette;
    g.gs_n = w->gs_n; g.gs_k = w->gs_k; g.Wn = w->N; g.Wk = w->K;
    g.fuse = 2; g.bias = bias;
    g.out = y; g.ld_out = ldy; g.alpha = 1.0f;
    return launch_lut_gemm(g, (cudaStream_t)stream);
}

int32_t plz_col_sum(const void* dY, int64_t lddy, int32_t M, int32_t N, float* out, void* stream) {
    if (M < 0 || N < 0 || (N & 1)) { set_last_error("col_sum: N must be even (M=%d, N=%d)", M, N); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0 || N == 0) return PLZ_OK;
    if (!dY || !out) { set_last_error("null pointer"); return PLZ_ERR_NULL; }
    if (((uintptr_t)dY & 3) || (lddy & 1)) { set_last_error("col_sum: rows must be 4-byte aligned"); return PLZ_ERR_BAD_ALIGN; }
    return launch_col_sum(dY, lddy, M, N, out, (cudaStream_t)stream);
}

int32_t plz_soft_weights(int32_t count, const plz_weight_t* const* ws, const plz_logits_t* const* logits,
                         const plz_noise_t* const* noise, float tau, int32_t hard_from_noisy, const plz_soft_out_t* const* outs,
                         void* stream) {
    if (count < 0 || count > 256) { set_last_error("soft_weights: 0 to 256 matrices per call"); return PLZ_ERR_BAD_SHAPE; }
    if (count == 0) return PLZ_OK;
    if (!ws || !logits || !outs) { set_last_error("soft_weights: null table"); return PLZ_ERR_NULL; }
    PwItem items[256];
    for (int i = 0; i < count; ++i) {
        int rc = check_weight(ws[i], false);
        if (rc) return rc;
        if (!logits[i] || !logits[i]->ptr || !outs[i]) { set_last_error("soft_weights: null logits or output descriptor %d", i); return PLZ_ERR_NULL; }
        if (logits[i]->dtype != 0 && logits[i]->dtype != 1) { set_last_error("soft_weights: logits dtype must be 0 (fp32) or 1 (fp16)"); return PLZ_ERR_UNSUPPORTED; }
        PwItem& d = items[i];
        d = PwItem{};
        d.logits = logits[i]->ptr; d.ls_n = logits[i]->s_n; d.ls_k = logits[i]->s_k; d.ls_p = logits[i]->s_p;
        d.logits_f16 = logits[i]->dtype == 1;
        const plz_noise_t* nz = noise ? noise[i] : nullptr;
        if (nz) { d.noise = nz->ptr; d.ns_n = nz->s_n; d.ns_k = nz->s_k; d.ns_p = nz->s_p; d.noise_mode = nz->mode; d.seed = nz->seed; }
        d.palette = (const __nv_bfloat16*)ws[i]->palette; d.gs_n = ws[i]->gs_n; d.gs_k = ws[i]->gs_k;
        d.n_kgroups = ws[i]->K / ws[i]->gs_k; d.N = ws[i]->N; d.K = ws[i]->K;
        d.n_fast = (logits[i]->s_n <= logits[i]->s_k) ? 1 : 0;
        d.P = outs[i]->P; d.p_n = outs[i]->p_n; d.p_k = outs[i]->p_k; d.p_p = outs[i]->p_p;
        d.w_soft = (__nv_bfloat16*)outs[i]->w_soft; d.ws_n = outs[i]->ws_n; d.ws_k = outs[i]->ws_k;
        d.w_hard = (__nv_bfloat16*)outs[i]->w_hard; d.wh_n = outs[i]->wh_n; d.wh_k = outs[i]->wh_k;
    }
    return launch_soft_weights(items, count, tau, hard_from_noisy ? 1 : 0, (cudaStream_t)stream);
}

int32_t plz_soft_bwd_elementwise(const plz_weight_t* w, const void* dW, int32_t dw_dtype, int64_t dw_n, int64_t dw_k, const void* P,
                                 int64_t p_n, int64_t p_k, int64_t p_p, const plz_logits_t* dlogits, float* dpalette, void* stream) {
    int rc = check_weight(w, false);
    if (rc) return rc;
    BwdElemArgs a = {};
    a.dW = dW; a.dw_dtype = dw_dtype; a.dw_n = dw_n; a.dw_k = dw_k;
    a.P = P; a.p_n = p_n; a.p_k = p_k; a.p_p = p_p;
    a.palette = w->palette; a.gs_n = w->gs_n; a.gs_k = w->gs_k; a.N = w->N; a.K = w->K;
    if (dlogits && dlogits->ptr) {
        if (dlogits->dtype != 0 && dlogits->dtype != 1) { set_last_error("soft_bwd_elementwise: dLogits dtype must be 0 or 1"); return PLZ_ERR_UNSUPPORTED; }
        a.dlogits = dlogits->ptr; a.dl_f16 = dlogits->dtype == 1; a.dl_n = dlogits->s_n; a.dl_k = dlogits->s_k; a.dl_p = dlogits->s_p;
    }
    a.dpalette = dpalette;
    return launch_soft_bwd_elementwise(a, (cudaStream_t)stream);
}

int32_t plz_weight_grad(const void* x, int64_t ldx, const void* dY, int64_t lddy, int32_t M, int32_t N, int32_t K, float* dW,
                        int64_t dw_n, int64_t dw_k, void* stream) {
    if (M < 0 || N <= 0 || K <= 0 || (N % 8) || (K % 8)) { set_last_error("weight_grad: bad shape M=%d N=%d K=%d", M, N, K); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0) return PLZ_OK;
    if (!x || !dY || !dW) { set_last_error("null pointer"); return PLZ_ERR_NULL; }
    int dev = 0, sms = 0;
    PLZ_CUDA_CHECK(cudaGetDevice(&dev));
    PLZ_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    TnArgs a = {};
    a.epi = EPI_STORE; a.M = M; a.alpha = 1.0f;
    // the 32 lanes of an epilogue warp are consecutive D rows: give them the axis along which dW is contiguous
    if (dw_n <= dw_k) { a.I = N; a.J = K; a.P = dY; a.ldp = lddy; a.Q = x; a.ldq = ldx; a.out_si = dw_n; a.out_sj = dw_k; }
    else { a.I = K; a.J = N; a.P = x; a.ldp = ldx; a.Q = dY; a.ldq = lddy; a.out_si = dw_k; a.out_sj = dw_n; }
    a.out = dW; a.out_I = a.I; a.out_J = a.J;
    const int tiles = ((a.I + 127) / 128) * ((a.J + 255) / 256);
    a.splits = tiles >= sms ? 1 : (sms + tiles - 1) / tiles;
    a.sm_count = sms;
    return launch_tn_gemm(a, (cudaStream_t)stream);
}

// ---- attention --------------------------------------------------------------------------------------------
int32_t plz_attn_fwd(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, int32_t B, int32_t S,
                     int32_t Hq, int32_t Hkv, int32_t head_dim, float scale, void* o, int64_t ldo, float* lse, void* stream) {
    AttnArgs a = {};
    a.B = B; a.S = S; a.Hq = Hq; a.Hkv = Hkv; a.head_dim = head_dim; a.scale = scale;
    a.q = q; a.ldq = ldq; a.k = k; a.ldk = ldk; a.v = v; a.ldv = ldv; a.o = o; a.ldo = ldo; a.lse = lse;
    return launch_attn_fwd(a, (cudaStream_t)stream);
}

int32_t plz_attn_bwd(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, const void* o, const void* d_o,
                     int64_t ldo, const float* lse, int32_t B, int32_t S, int32_t Hq, int32_t Hkv, int32_t head_dim, float scale,
                     float* dsum_ws, void* dq, void* dk, void* dv, void* stream) {
    AttnArgs a = {};
    a.B = B; a.S = S; a.Hq = Hq; a.Hkv = Hkv; a.head_dim = head_dim; a.scale = scale;
    a.q = q; a.ldq = ldq; a.k = k; a.ldk = ldk; a.v = v; a.ldv = ldv; a.o = const_cast<void*>(o); a.ldo = ldo;
    a.lse = const_cast<float*>(lse); a.d_o = d_o; a.dsum = dsum_ws; a.dq = dq; a.dk = dk; a.dv = dv;
    return launch_attn_bwd(a, (cudaStream_t)stream);
}

int64_t plz_attn_decode_ws_bytes(int32_t B, int32_t T, int32_t Hq, int32_t Hkv) {
    if (B <= 0 || T <= 0 || Hq <= 0 || Hkv <= 0) return 0;
    return attn_decode_ws_bytes(B, T, Hq, Hkv);
}

int32_t plz_attn_decode(const void* q, int64_t ldq, const void* k_cache, const void* v_cache, int64_t batch_stride, int64_t tok_stride,
                        int32_t B, int32_t T, int32_t Hq, int32_t Hkv, int32_t head_dim, float scale, void* out, int64_t ldo, void* ws,
                        int64_t ws_bytes, void* stream) {
    if (B < 0 || T <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || head_dim != 128) {
        set_last_error("attn_decode: needs T > 0, head_dim 128 and Hq a multiple of Hkv (B=%d T=%d Hq=%d Hkv=%d d=%d)", B, T, Hq, Hkv, head_dim);
        return PLZ_ERR_BAD_SHAPE;
    }
    if (B == 0) return PLZ_OK;
    if (!q || !k_cache || !v_cache || !out) { set_last_error("null pointer"); return PLZ_ERR_NULL; }
    if (((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || (ldq & 7) || (batch_stride & 7) || (tok_stride & 7) ||
        ((uintptr_t)ws & 15)) {
        set_last_error("attn_decode: rows must be 16-byte aligned"); return PLZ_ERR_BAD_ALIGN;
    }
    AttnDecodeArgs a = {};
    a.B = B; a.T = T; a.Hq = Hq; a.Hkv = Hkv; a.scale = scale; a.q = q; a.ldq = ldq; a.k = k_cache; a.v = v_cache;
    a.batch_stride = batch_stride; a.tok_stride = tok_stride; a.out = out; a.ldo = ldo; a.ws = ws; a.ws_bytes = ws ? ws_bytes : 0;
    return launch_attn_decode(a, (cudaStream_t)stream);
}

int32_t plz_embed_gather(const void* table, int64_t ldt, const int64_t* ids, int64_t n, int32_t width, int64_t vocab, void* out, int64_t ldo,
                         int32_t* bad, void* stream) {
    if (n < 0 || width <= 0 || (width & 7) || vocab <= 0) { set_last_error("embed_gather: width must be a positive multiple of 8"); return PLZ_ERR_BAD_SHAPE; }
    if (n == 0) return PLZ_OK;
    if (!table || !ids || !out) { set_last_error("null pointer"); return PLZ_ERR_NULL; }
    if (((uintptr_t)table & 15) || ((uintptr_t)out & 15) || (ldt & 7) || (ldo & 7)) { set_last_error("embed_gather: rows must be 16-byte aligned"); return PLZ_ERR_BAD_ALIGN; }
    return launch_embed_gather(table, ldt, (const long long*)ids, n, width, vocab, out, ldo, bad, (cudaStream_t)stream);
}

// ---- element-wise ops of a decoder layer ----------------------------------------------------------------
static bool rows16(const void* p, int64_t ld) { return (((uintptr_t)p & 15) == 0) && ((ld & 7) == 0); }

int32_t plz_rmsnorm_fwd(const void* x, int64_t ldx, const void* g, int32_t M, int32_t K, float eps, void* h, int64_t ldh, float* rstd,
                        void* stream) {
    if (M < 0 || K <= 0 || (K & 7)) { set_last_error("rmsnorm_fwd: K must be a positive multiple of 8"); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0) return PLZ_OK;
    if (!x || !h) { set_last_error("null pointer"); return PLZ_ERR_NULL; }
    if (!rows16(x, ldx) || !rows16(h, ldh) || (g && ((uintptr_t)g & 15))) { set_last_error("rmsnorm_fwd: rows must be 16-byte aligned"); return PLZ_ERR_BAD_ALIGN; }
    return launch_rmsnorm_fwd(x, ldx, g, M, K, eps, h, ldh, rstd, (cudaStream_t)stream);
}

int32_t plz_add_rmsnorm_fwd(const void* x, int64_t ldx, const void* addend, int64_t lda, void* sum_out, int64_t lds, const void* g, int32_t M,
                            int32_t K, float eps, void* h, int64_t ldh, float* rstd, void* stream) {
    if (M < 0 || K <= 0 || (K & 7)) { set_last_error("add_rmsnorm_fwd: K must be a positive multiple of 8"); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0) return PLZ_OK;
    if (!x || !addend || !sum_out || !h) { set_last_error("null pointer"); return PLZ_ERR_NULL; }
    if (!rows16(x, ldx) || !rows16(addend, lda) || !rows16(sum_out, lds) || !rows16(h, ldh) || (g && ((uintptr_t)g & 15))) {
        set_last_error("add_rmsnorm_fwd: rows must be 16-byte aligned"); return PLZ_ERR_BAD_ALIGN;
    }
    return launch_add_rmsnorm(x, ldx, addend, lda, sum_out, lds, g, M, K, eps, h, ldh, rstd, (cudaStream_t)stream);
}

int32_t plz_qknorm_rope_fwd2(const void* xq, int64_t ldxq, const void* wq, int32_t Hq, void* outq, int64_t ldoq, const void* xk, int64_t ldxk,
                             const void* wk, int32_t Hk, void* outk, int64_t ldok, const float* cos_tab, const float* sin_tab, int64_t tokens,
                             int32_t S, int32_t head_dim, float eps, void* stream) {
    if (tokens < 0 || Hq <= 0 || Hk <= 0 || S <= 0 || head_dim != 128) { set_last_error("qknorm_rope: head_dim must be 128 (Hq=%d Hk=%d S=%d)", Hq, Hk, S); return PLZ_ERR_BAD_SHAPE; }
    if (tokens == 0) return PLZ_OK;
    if (!xq || !xk || !outq || !outk || !cos_tab || !sin_tab) { set_last_error("null pointer"); return PLZ_ERR_NULL; }
    if (((uintptr_t)xq & 3) || ((uintptr_t)xk & 3) || ((uintptr_t)outq & 3) || ((uintptr_t)outk & 3) || (ldxq & 1) || (ldxk & 1) || (ldoq & 1) ||
        (ldok & 1) || ((uintptr_t)cos_tab & 7) || ((uintptr_t)sin_tab & 7)) {
        set_last_error("qknorm_rope: misaligned input"); return PLZ_ERR_BAD_ALIGN;
    }
    return launch_qknorm_rope2(xq, ldxq, wq, Hq, outq, ldoq, xk, ldxk, wk, Hk, outk, ldok, cos_tab, sin_tab, tokens, S, eps, (cudaStream_t)stream);
}

int32_t plz_qknorm_rope_fwd(const void* x, int64_t ldx, const void* w, const float* cos_tab, const float* sin_tab, int64_t tokens,
                            int32_t H, int32_t S, int32_t head_dim, float eps, void* out, int64_t ldo, void* stream) {
    if (tokens < 0 || H <= 0 || S <= 0 || head_dim != 128) { set_last_error("qknorm_rope: head_dim must be 128 (H=%d S=%d)", H, S); return PLZ_ERR_BAD_SHAPE; }
    if (tokens == 0) return PLZ_OK;
    if (!x || !cos_tab || !sin_tab || !out) { set_last_error("null pointer"); return PLZ_ERR_NULL; }
    if (((uintptr_t)x & 3) || ((uintptr_t)out & 3) || (ldx & 1) || (ldo & 1) || ((uintptr_t)cos_tab & 7) || ((uintptr_t)sin_tab & 7)) {
        set_last_error("qknorm_rope: misaligned input"); return PLZ_ERR_BAD_ALIGN;
    }
    return launch_qknorm_rope(0, x, ldx, w, cos_tab, sin_tab, nullptr, 0, tokens, H, S, eps, out, ldo, nullptr, (cudaStream_t)stream);
}

int32_t plz_qknorm_rope_bwd(const void* x, int64_t ldx, const void* w, const float* cos_tab, const float* sin_tab, const void* dy,
                            int64_t lddy, int64_t tokens, int32_t H, int32_t S, int32_t head_dim, float eps, void* dx, int64_t lddx,
                            float* dw, void* stream) {
    if (tokens < 0 || H <= 0 || S <= 0 || head_dim != 128) { set_last_error("qknorm_rope: head_dim must be 128 (H=%d S=%d)", H, S); return PLZ_ERR_BAD_SHAPE; }
    if (tokens == 0) return PLZ_OK;
    if (!x || !cos_tab || !sin_tab || !dy || !dx) { set_last_error("null pointer"); return PLZ_ERR_NULL; }
    if (((uintptr_t)x & 3) || ((uintptr_t)dy & 3) || ((uintptr_t)dx & 3) || (ldx & 1) || (lddy & 1) || (lddx & 1)) {
        set_last_error("qknorm_rope: misaligned input"); return PLZ_ERR_BAD_ALIGN;
    }
    return launch_qknorm_rope(1, x, ldx, w, cos_tab, sin_tab, dy, lddy, tokens, H, S, eps, dx, lddx, dw, (cudaStream_t)stream);
}

int32_t plz_swiglu_fwd(const void* gate, int64_t ldg, const void* up, int64_t ldu, int32_t M, int32_t N, void* act, int64_t lda, void* stream) {
    if (M < 0 || N <= 0 || (N & 7)) { set_last_error("swiglu_fwd: N must be a positive multiple of 8"); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0) return PLZ_OK;
    if (!gate || !up || !act) { set_last_error("null pointer"); return PLZ_ERR_NULL; }
    if (!rows16(gate, ldg) || !rows16(up, ldu) || !rows16(act, lda)) { set_last_error("swiglu_fwd: rows must be 16-byte aligned"); return PLZ_ERR_BAD_ALIGN; }
    return launch_swiglu_fwd(gate, ldg, up, ldu, M, N, act, lda, (cudaStream_t)stream);
}

int32_t plz_add(const void* a, int64_t lda, const void* b, int64_t ldb, const void* c, int64_t ldc, int32_t M, int32_t N, void* out,
                int64_t ldo, void* stream) {
    if (M < 0 || N <= 0 || (N & 7)) { set_last_error("add: N must be a positive multiple of 8"); return PLZ_ERR_BAD_SHAPE; }
    if (M == 0) return PLZ_OK;
    if (!a || !b || !out) { set_last_error("null pointer"); return PLZ_ERR_NULL; }
    if (!rows16(a, lda) || !rows16(b, ldb) || !rows16(out, ldo) || (c && !rows16(c, ldc))) { set_last_error("add: rows must be 16-byte aligned"); return PLZ_ERR_BAD_ALIGN; }
    return launch_add(a, lda, b, ldb, c, ldc, M, N, out, ldo, (cudaStream_t)stream);
}

int32_t plz_bwd_dw_hard_lora(const plz_weight_t* w, const void* x, int64_t ldx, const void* dY, int64_t lddy, int32_t M, float* dpalette,
                             const void* t, const void* dt, int32_t rank, float* dA, float* dB, void* stream) {
    if (!dpalette) { set_last_error("null dpalette"); return PLZ_ERR_NULL; }
    if (rank <= 0 || rank > 64 || rank % 8) { set_last_error("LoRA rank %d must be a multiple of 8 in [8, 64]", rank); return PLZ_ERR_BAD_SHAPE; }
    if ((dA && !dt) || (dB && !t)) { set_last_error("bwd_dw_hard_lora: dA needs dt and dB needs t"); return PLZ_ERR_NULL; }
    return bwd_dw_common(EPI_HARD, w, x, ldx, dY, lddy, M, nullptr, nullptr, 1.0f, nullptr, dpalette, stream, t, dt, rank, dA, dB);
}

}  // extern "C"
