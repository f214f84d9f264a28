// Host side of the TMA path: tensor-map encoding through the driver entry point (no link-time
// dependency on libcuda) and the pinned error word that kernels with bounded waits report into.
#include <cuda.h>
#include <cuda_runtime.h>

#include "common.h"
#include "tma_utils.cuh"

namespace kutacc {
namespace dev {

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
        KUTACC_CHECK(e == cudaSuccess && q == cudaDriverEntryPointSuccess && p != nullptr,
                     "cuTensorMapEncodeTiled is not available from this driver");
        fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}
}  // namespace

bool make_tensor_map_bf16_3d(CUtensorMap *map, const void *base, uint64_t d0, uint64_t d1, uint64_t d2,
                             uint64_t stride1, uint64_t stride2, uint32_t box0, uint32_t box1, int swizzle_bytes,
                             uint32_t box2)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {stride1 * 2, stride2 * 2};  // bytes, dims 1 and 2
    cuuint32_t box[3] = {box0, box1, box2};
    cuuint32_t estr[3] = {1, 1, 1};
    CUtensorMapSwizzle sw = swizzle_bytes == 128  ? CU_TENSOR_MAP_SWIZZLE_128B
                            : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                            : swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                                  : CU_TENSOR_MAP_SWIZZLE_NONE;
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    KUTACC_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with ", (int)r, " dims ", d0, "x", d1, "x", d2,
                 " strides ", stride1, ",", stride2, " box ", box0, "x", box1);
    return r == CUDA_SUCCESS;
}

bool make_tensor_map_2d(CUtensorMap *map, const void *base, int elem_bytes, uint64_t d0, uint64_t d1, uint64_t stride1,
                        uint32_t box0, uint32_t box1, int swizzle_bytes)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn || (elem_bytes != 2 && elem_bytes != 4)) return false;
    cuuint64_t dims[2] = {d0, d1};
    cuuint64_t strides[1] = {stride1 * (cuuint64_t)elem_bytes};
    cuuint32_t box[2] = {box0, box1};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMapSwizzle sw = swizzle_bytes == 128  ? CU_TENSOR_MAP_SWIZZLE_128B
                            : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                            : swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                                  : CU_TENSOR_MAP_SWIZZLE_NONE;
    CUresult r = fn(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                    const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    KUTACC_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with ", (int)r, " dims ", d0, "x", d1, " stride ", stride1,
                 " box ", box0, "x", box1, " element bytes ", elem_bytes);
    return r == CUDA_SUCCESS;
}

KernelErrorWord &kernel_error_word()
{
    static KernelErrorWord w;
    if (w.host == nullptr) {
        void *h = nullptr;
        cudaError_t e = cudaHostAlloc(&h, sizeof(int), cudaHostAllocMapped);
        KUTACC_CHECK(e == cudaSuccess, "cannot allocate the kernel error word: ", cudaGetErrorString(e));
        if (e == cudaSuccess) {
            w.host = static_cast<int *>(h);
            *w.host = 0;
            void *d = nullptr;
            e = cudaHostGetDevicePointer(&d, h, 0);
            KUTACC_CHECK(e == cudaSuccess, "cannot map the kernel error word: ", cudaGetErrorString(e));
            w.device = static_cast<int *>(d);
        }
    }
    return w;
}

}  // namespace dev
}  // namespace kutacc
