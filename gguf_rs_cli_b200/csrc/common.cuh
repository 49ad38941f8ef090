// Shared declarations of the sm_100a kernels: storage types, error reporting and the
// C entry points' conventions.  Every entry point is `extern "C"`, takes raw device
// pointers and the stream to launch on, and returns 0 or a non-zero code after
// leaving a message that gb_last_error() returns.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define GB_API extern "C" __attribute__((visibility("default")))

enum GbDtype { GB_F32 = 0, GB_BF16 = 1 };

// Positions per cache page; the host-side page pool uses the same constant.
constexpr int GB_PAGE = 64;
constexpr int GB_PAGE_SHIFT = 6;

int gb_fail(const char* fmt, ...);

#define GB_REQUIRE(cond, ...)                 \
    do {                                      \
        if (!(cond)) return gb_fail(__VA_ARGS__); \
    } while (0)

#define GB_LAUNCH_OK(name)                                                        \
    do {                                                                          \
        cudaError_t e__ = cudaGetLastError();                                     \
        if (e__ != cudaSuccess) return gb_fail("%s: launch failed: %s", name, cudaGetErrorString(e__)); \
    } while (0)

// Programmatic dependent launch: a kernel launched through gb_launch may start while the
// kernel before it on the stream is still running; it may touch nothing that kernel writes (or
// reads and this one writes) before gb_grid_wait() returns.  gb_grid_launch_dependents() lets the
// next kernel start its own prologue.  Both are no-ops for a kernel launched the ordinary way.
bool gb_pdl_enabled();
__device__ __forceinline__ void gb_grid_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void gb_grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// pdl false: an ordinary launch, which starts when everything before it on the stream has finished.
template <typename... KArgs, typename... Args>
static inline cudaError_t gb_launch_opt(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                        bool pdl, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    if (pdl && gb_pdl_enabled()) {
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
template <typename... KArgs, typename... Args>
static inline cudaError_t gb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args&&... args) {
    return gb_launch_opt(kernel, grid, block, smem, stream, true, static_cast<Args&&>(args)...);
}

static inline bool gb_is_dtype(int d) { return d == GB_F32 || d == GB_BF16; }
static inline size_t gb_dtype_size(int d) { return d == GB_F32 ? 4 : 2; }

__device__ __forceinline__ float gb_to_float(float v) { return v; }
__device__ __forceinline__ float gb_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T gb_from_float(float v);
template <> __device__ __forceinline__ float gb_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 gb_from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Loads/stores through a runtime dtype tag, for kernels whose cost is not in the
// conversion (norms, rotation, sampling).
__device__ __forceinline__ float gb_load(const void* p, int dtype, size_t i) {
    return dtype == GB_F32 ? reinterpret_cast<const float*>(p)[i]
                           : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void gb_store(void* p, int dtype, size_t i, float v) {
    if (dtype == GB_F32) reinterpret_cast<float*>(p)[i] = v;
    else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// Where position `pos` of the sequence with page-table row `row` lives: element offset
// of [kv head g][pos % PAGE][0] inside one run's K or V storage
// [pages][kv heads][PAGE][head_dim].
__device__ __forceinline__ size_t gb_kv_offset(const int* row, int ring_pages, int pos, int g, int nkv, int hd) {
    int page = row[(pos >> GB_PAGE_SHIFT) % ring_pages];
    return ((size_t(page) * nkv + g) * GB_PAGE + (pos & (GB_PAGE - 1))) * size_t(hd);
}

// Rotation of one pair by the angle whose sine and cosine are given.  Products and sums are rounded one by
// one (no fused multiply-add), so that every kernel that rotates gives the same bits.
__device__ __forceinline__ void gb_rotate(float x0, float x1, float cs, float sn, float& y0, float& y1) {
    y0 = __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
    y1 = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs));
}

__device__ __forceinline__ float gb_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float gb_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
