// Device helpers for writing the staged activation image (see layout.cuh: three bf16 limbs per value in MMA
// feed order, plus 32-column sums), shared by the staging kernel and by producer kernels that emit it directly.
#pragma once
#include <cuda_bf16.h>

#include "layout.cuh"

namespace juno {

// Splits v into three bf16 limbs with hi + mid + lo == v.
__device__ __forceinline__ void split3(float v, unsigned short &hi, unsigned short &mid, unsigned short &lo) {
    __nv_bfloat16 h = __float2bfloat16_rn(v);
    float r1 = v - __bfloat162float(h);
    __nv_bfloat16 m = __float2bfloat16_rn(r1);
    float r2 = r1 - __bfloat162float(m);
    __nv_bfloat16 l = __float2bfloat16_rn(r2);
    hi = __bfloat16_as_ushort(h);
    mid = __bfloat16_as_ushort(m);
    lo = __bfloat16_as_ushort(l);
}

// Where batch row b of a K-column activation lives inside an image made of chunks of `bc` rows
// (chunk = [K/16][3*rows][4][4] bf16; a short last chunk has fewer limb columns).
struct StageImage {
    uint8_t *img = nullptr;
    int K = 0, batch = 0, bc = 1, b0 = 0;  // b0: offset added to the caller's row index
    size_t chunk_stride = 0;
    __device__ __forceinline__ void locate(int b, unsigned short *&xb, int &NC, int &col0) const {
        const int bb = b + b0, chunk = bb / bc, nbc = min(bc, batch - chunk * bc);
        NC = 3 * nbc;
        col0 = 3 * (bb - chunk * bc);
        xb = reinterpret_cast<unsigned short *>(img + (size_t)chunk * chunk_stride);
    }
};

// One value (column i of batch row b).
__device__ __forceinline__ void stage_store1(unsigned short *xb, int NC, int col0, int i, float v) {
    unsigned short l0, l1, l2;
    split3(v, l0, l1, l2);
    unsigned short *dst = xb + xb_index(i, NC, col0);
    dst[0] = l0;
    dst[16] = l1;  // next limb column: +4*4 elements
    dst[32] = l2;
}

}  // namespace juno
