// Tensor maps for the tiled bulk copies (cp.async.bulk.tensor) of the product and attention kernels.
#include "common.cuh"

namespace tsm {

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                               const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled from the driver that is already loaded (the library links the runtime only).
static EncodeTiled encode_tiled() {
    static EncodeTiled fn = [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult found;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &found) != cudaSuccess || found != cudaDriverEntryPointSuccess)
            ptr = nullptr;
        return (EncodeTiled)ptr;
    }();
    return fn;
}

// A rank-2 map over `rows` rows of `width` elements (pitch `pitch_bytes`), copied in boxes of box_w x box_h elements.
int make_tensor_map_2d(tsm_ctx* ctx, CUtensorMap* map, CUtensorMapDataType type, const void* base, uint64_t width, uint64_t rows, uint64_t pitch_bytes,
             uint32_t box_w, uint32_t box_h, CUtensorMapSwizzle swizzle) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return fail(ctx, TSM_ERR_UNSUPPORTED, "the driver does not export cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {width, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_w, box_h};
    cuuint32_t steps[2] = {1, 1};
    CUresult rc = encode(map, type, 2, const_cast<void*>(base), dims, strides, box, steps, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return fail(ctx, TSM_ERR_ARG, "cuTensorMapEncodeTiled refused a map (code " + std::to_string((int)rc) + ")");
    return TSM_OK;
}

bool tensor_maps_available() { return encode_tiled() != nullptr; }

}  // namespace tsm
