// Tiled bulk-tensor copies (TMA) over this GPU's own memory: host-side tensor-map encoding through the runtime's driver
// entry point query (the library does not link against libcuda), and the device-side copy instructions.  Every copy here
// is issued by one CTA for its own shared memory.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "tc05.cuh"

namespace hgq {
namespace tma {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_tiled_fn() {
    static const EncodeTiledFn fn = [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return (EncodeTiledFn) nullptr;
        }
        return (EncodeTiledFn)ptr;
    }();
    return fn;
}

// A map over a row-major fp32 matrix [rows, cols] (row stride ld floats): boxes of box_rows x box_cols floats, rows of a
// box contiguous in shared memory (no swizzle), zeros outside the matrix.  base 16-byte aligned, ld and box_cols
// multiples of 4, box_cols and box_rows <= 256.  swizzle128: box_cols = 32 (128-byte rows); the 16-byte chunk c of row r
// lands at chunk c ^ (r & 7) of its row, and the destination must start on a 1 KB boundary.
static inline bool make_map_2d(CUtensorMap *map, const float *base, int64_t rows, int64_t cols, int64_t ld, int box_cols,
                               int box_rows, bool swizzle128 = false) {
    const EncodeTiledFn enc = encode_tiled_fn();
    if (enc == nullptr || base == nullptr) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

#ifdef __CUDACC__
// this thread's arrival on `bar` plus the announcement of `bytes` bytes that copies will deliver
__device__ __forceinline__ void expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile(
        "{\n\t"
        ".reg .b64 st;\n\t"
        "mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t"
        "}\n" ::"r"(tc::smem_u32(bar)), "r"(bytes)
        : "memory");
}

// One tiled 2-D copy global -> this CTA's shared memory; c0 (the column) times 4 bytes must be a multiple of 16.
__device__ __forceinline__ void load_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(c0), "r"(c1), "r"(tc::smem_u32(bar))
                 : "memory");
}
#endif

}  // namespace tma
}  // namespace hgq
