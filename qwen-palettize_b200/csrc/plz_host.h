// Host-side helpers shared by the .cu files: error codes, tensor-map encoding, launch checks.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "plz_sm100.cuh"

// error codes returned through the C ABI (include/plz.h documents them)
#define PLZ_OK 0
#define PLZ_ERR_BAD_SHAPE 1
#define PLZ_ERR_BAD_ALIGN 2
#define PLZ_ERR_UNSUPPORTED 3
#define PLZ_ERR_CUDA 4
#define PLZ_ERR_WORKSPACE 5
#define PLZ_ERR_DEVICE_WAIT 6
#define PLZ_ERR_NULL 7
#define PLZ_ERR_TOO_LARGE 8

namespace plz {

void set_last_error(const char* fmt, ...);
StatusWord* device_status_ptr();  // address of the static device status word (per device)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_fn();

// 2-D bf16 row-major tensor [rows, cols] with row pitch `ld` elements; box = [box_cols, box_rows],
// 128-byte swizzle (box_cols * 2 bytes must be 128), out-of-range elements read as zero.
int make_tmap_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                   uint32_t box_cols, uint32_t box_rows);

#define PLZ_CUDA_CHECK(expr)                                                            \
    do {                                                                                \
        cudaError_t _e = (expr);                                                        \
        if (_e != cudaSuccess) {                                                        \
            plz::set_last_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                                __FILE__, __LINE__);                                    \
            return PLZ_ERR_CUDA;                                                        \
        }                                                                               \
    } while (0)

// Every kernel launch of the library is followed by this: the launch error check, and a process-wide launch counter
// (plz_launch_count) so that a caller can state how many kernels of this library a region of its program ran.
extern unsigned long long g_launch_count;
#define PLZ_LAUNCH_CHECK()                       \
    do {                                         \
        PLZ_CUDA_CHECK(cudaGetLastError());      \
        ++plz::g_launch_count;                   \
    } while (0)

// Launch of a small kernel of the token-decode chain. When plz_set_smallm_overlap is on, the launch carries the
// programmatic-stream-serialization attribute: the kernel may start while its predecessor in the stream is still running,
// so it must execute griddepcontrol.wait before it touches anything another kernel writes (pdl_wait below; a no-op
// without the attribute), and its griddepcontrol.launch_dependents lets the kernel after it (typically a small-M LUT
// kernel, which first streams its read-only weights) start early in turn.
extern int g_smallm_overlap;
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chain(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = g_smallm_overlap ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#define PLZ_LAUNCH_CHAIN(...)                        \
    do {                                             \
        PLZ_CUDA_CHECK(plz::launch_chain(__VA_ARGS__)); \
        ++plz::g_launch_count;                       \
    } while (0)

}  // namespace plz
