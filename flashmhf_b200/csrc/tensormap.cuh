// Host-side construction of TMA tensor maps for the operator's tensors.  The driver's encoder is
// fetched through the runtime (cudaGetDriverEntryPoint), so the library links against cudart only.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string.h>

#include "kernels.h"

namespace fmhf {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// bf16 tensor, innermost dim contiguous, 128-byte swizzle, out-of-range elements read as zero and
// are not written.  dims/box are innermost-first; stride_elems[i] is the element stride of dim i+1.
// A dim of extent 1 may carry any stride; it is replaced by a legal one.
//
// Encoded maps are kept in a small per-thread cache keyed by (base, rank, dims, strides, box): a map depends on
// nothing else, training and decode loops present the same tensors call after call, and the driver's encoder
// costs more host time than the rest of a call.  Per thread, so no lock; 64 entries, replaced round-robin.
struct MapKey {
    const void *base;
    int32_t rank;
    uint32_t box[4];
    uint64_t dims[4];
    int64_t strides[3];
};
struct MapCache {
    static constexpr int kEntries = 64;
    MapKey key[kEntries];
    CUtensorMap map[kEntries];
    int used = 0, next = 0;
};
inline MapCache &map_cache() {
    static thread_local MapCache c;
    return c;
}

inline int encode_bf16_map_uncached(CUtensorMap *out, const void *base, int rank, const uint64_t *dims,
                                    const int64_t *stride_elems, const uint32_t *box);

inline int encode_bf16_map(CUtensorMap *out, const void *base, int rank, const uint64_t *dims,
                           const int64_t *stride_elems, const uint32_t *box) {
    MapKey k;
    memset(&k, 0, sizeof(k));
    k.base = base;
    k.rank = rank;
    for (int i = 0; i < rank; ++i) { k.dims[i] = dims[i]; k.box[i] = box[i]; }
    for (int i = 0; i + 1 < rank; ++i) k.strides[i] = stride_elems[i];
    MapCache &c = map_cache();
    for (int i = 0; i < c.used; ++i)
        if (memcmp(&c.key[i], &k, sizeof(k)) == 0) {
            *out = c.map[i];
            return FLASHMHF_OK;
        }
    const int rc = encode_bf16_map_uncached(out, base, rank, dims, stride_elems, box);
    if (rc != FLASHMHF_OK) return rc;
    const int slot = c.used < MapCache::kEntries ? c.used++ : (c.next = (c.next + 1) % MapCache::kEntries);
    c.key[slot] = k;
    c.map[slot] = *out;
    return FLASHMHF_OK;
}

inline int encode_bf16_map_uncached(CUtensorMap *out, const void *base, int rank, const uint64_t *dims,
                                    const int64_t *stride_elems, const uint32_t *box) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) {
        set_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point not found");
        return FLASHMHF_ERR_CUDA;
    }
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return FLASHMHF_ERR_MISALIGNED;
    cuuint64_t gdim[5], gstr[4];
    cuuint32_t gbox[5], estr[5];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        gbox[i] = box[i];
        estr[i] = 1;
    }
    for (int i = 0; i + 1 < rank; ++i) {
        int64_t s = stride_elems[i];
        if (dims[i + 1] == 1) s = (int64_t)dims[0];  // never dereferenced beyond index 0
        if (s <= 0 || (s % 8) != 0 || (uint64_t)s * 2 >= (1ull << 40)) return FLASHMHF_ERR_BAD_STRIDE;
        gstr[i] = (cuuint64_t)s * 2;
    }
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void *>(base), gdim, gstr, gbox,
                    estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled rejected the tensor");
        return FLASHMHF_ERR_BAD_STRIDE;
    }
    return FLASHMHF_OK;
}

// [B,H,S,Dh] activation-like tensor -> 4-D map (Dh, S, H, B), box 64 x rows x 1 x 1.
inline int encode_act_map(CUtensorMap *out, const flashmhf_tensor &t, const flashmhf_dims &d, uint32_t box_rows) {
    uint64_t dims[4] = {(uint64_t)d.Dh, (uint64_t)d.S, (uint64_t)d.H, (uint64_t)d.B};
    int64_t str[3] = {t.stride[2], t.stride[1], t.stride[0]};
    uint32_t box[4] = {64, box_rows, 1, 1};
    return encode_bf16_map(out, t.ptr, 4, dims, str, box);
}
// [Hkuv,E,De,Dh] weight tensor -> 3-D map (Dh, E*De, Hkuv), box 64 x rows x 1.  Needs E and De to collapse.
inline int encode_weight_map(CUtensorMap *out, const flashmhf_tensor &t, const flashmhf_dims &d, uint32_t box_rows) {
    if (d.E > 1 && t.stride[1] != (int64_t)d.De * t.stride[2]) return FLASHMHF_ERR_BAD_STRIDE;
    uint64_t dims[3] = {(uint64_t)d.Dh, (uint64_t)d.E * d.De, (uint64_t)d.Hkuv};
    int64_t str[2] = {t.stride[2], t.stride[0]};
    uint32_t box[3] = {64, box_rows, 1};
    return encode_bf16_map(out, t.ptr, 3, dims, str, box);
}

}  // namespace fmhf
