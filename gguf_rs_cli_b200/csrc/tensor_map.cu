// Host-side construction of TMA tensor maps (cuTensorMapEncodeTiled through the runtime's
// driver entry point; nothing links against libcuda).
#include <mutex>

#include "common.cuh"
#include "sm100.cuh"

namespace sm100 {

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn encode() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(f);
    });
    return fn;
}

int tensor_map_bf16_2d(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out) {
    EncodeFn fn = encode();
    if (!fn) return gb_fail("the driver gives no cuTensorMapEncodeTiled");
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || ld % 8 != 0)
        return gb_fail("a TMA operand must be 16-byte aligned with a pitch that is a multiple of 8 elements");
    cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
    cuuint64_t strides[1] = {cuuint64_t(ld) * 2};
    cuuint32_t box[2] = {64, cuuint32_t(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return gb_fail("cuTensorMapEncodeTiled failed with code %d", int(r));
    return 0;
}

}  // namespace sm100
