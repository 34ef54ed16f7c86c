// Host helpers that encode the TMA tensor maps of the distance operands.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

namespace pinkb {

constexpr uint32_t kOperandSliceBytes = 128;   // bytes of K per pipeline stage = one 128-byte swizzle row

inline PFN_cuTensorMapEncodeTiled_v12000 encode_fn()
{
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess
            && qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    }
    return fn;
}

// rows x row_bytes matrix of bytes, K-contiguous; box = 128 bytes x box_rows, 128-byte swizzle.
inline bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows)
{
    auto fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = { row_bytes, rows };
    cuuint64_t strides[1] = { row_bytes };
    cuuint32_t box[2] = { kOperandSliceBytes, box_rows };
    cuuint32_t estr[2] = { 1, 1 };
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

} // namespace pinkb
