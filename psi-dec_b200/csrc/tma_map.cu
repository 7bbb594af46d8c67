// Host side of the TMA path: the tensor map of a page arena.
#include <cuda_runtime.h>

#include "tma_common.cuh"

namespace psi {

namespace {

// The page arena as a TMA tensor [page][8-row group][element block][row in group][64 elements]: a page holds
// 2 * Hkv * tokens_per_page K and V rows of head_dim elements, a box is `box_rows / 8` consecutive groups with all their
// element blocks, written with the 128-byte swizzle in exactly the order the MMA descriptors read a tile in.
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
    static EncodeTiled fn = [] {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) != cudaSuccess ||
            result != cudaDriverEntryPointSuccess)
            entry = nullptr;
        return reinterpret_cast<EncodeTiled>(entry);
    }();
    return fn;
}

}  // namespace

bool make_kv_map(const AttendParams& p, uint32_t box_rows, CUtensorMap* map) {
    const EncodeTiled encode = encode_tiled();
    if (encode == nullptr) return false;
    const uint64_t page_bytes = p.geo.page_elems * 2;
    const uint64_t row_bytes = p.geo.head_dim * 2ull;
    const uint64_t rows_per_page = 2ull * p.geo.num_kv_heads * p.geo.tokens_per_page;
    if (reinterpret_cast<uintptr_t>(p.geo.pages) % 16 != 0 || page_bytes % 16 != 0 || p.geo.num_pages == 0 ||
        p.geo.num_pages > 0x7FFFFFFFull || rows_per_page * row_bytes > page_bytes || p.geo.tokens_per_page % 8 != 0)
        return false;
    const cuuint64_t dims[5] = {64, 8, p.geo.head_dim / 64, rows_per_page / 8, p.geo.num_pages};
    const cuuint64_t strides[4] = {row_bytes, 128, 8 * row_bytes, page_bytes};
    const cuuint32_t box[5] = {64, 8, p.geo.head_dim / 64, box_rows / 8, 1};
    const cuuint32_t elem_strides[5] = {1, 1, 1, 1, 1};
    const CUtensorMapDataType type = p.dtype == PSI_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    return encode(map, type, 5, const_cast<void*>(p.geo.pages), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}


}  // namespace psi
