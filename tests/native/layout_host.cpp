// Test-only host build of the tile-layout index maps (repack.cuh, dequant.cuh): the same code the device kernels run,
// compiled with the C++ compiler so that the layout tests need no GPU.  Not part of the product library.
#include <stdint.h>

#include "../../juno_b200/csrc/dequant.cuh"
#include "../../juno_b200/csrc/layout.cuh"
#include "../../juno_b200/csrc/repack.cuh"

using namespace juno;

extern "C" int64_t layout_tiled_bytes(int type, int64_t rows, int64_t cols) {
    if (cols % 256 || !tile_bytes(type)) return -1;
    return ((rows + 15) / 16) * (cols / 256) * (int64_t)tile_bytes(type);
}

extern "C" int layout_repack(int type, const uint8_t *raw, int64_t rows, int64_t cols, uint8_t *out) {
    if (cols % 256 || rows < 1 || !tile_bytes(type)) return -1;
    const int nsb = (int)(cols / 256), RT = (int)((rows + 15) / 16);
    const size_t rrb = (size_t)nsb * (type == 12 ? 144 : type == 14 ? 210 : 8 * 34);
    const int wpt = tile_bytes(type) / 4;
    uint32_t *o = reinterpret_cast<uint32_t *>(out);
    for (int R = 0; R < RT; R++)
        for (int b = 0; b < nsb; b++)
            for (int w = 0; w < wpt; w++)
                o[((size_t)R * nsb + b) * wpt + w] = type == 12   ? q4k_out_word(raw, rrb, (int)rows, b, R, w)
                                                     : type == 14 ? q6k_out_word(raw, rrb, (int)rows, b, R, w)
                                                                  : q80_out_word(raw, rrb, (int)rows, b, R, w);
    return 0;
}

extern "C" int layout_dequant_tiled(int type, const uint8_t *tiles, int64_t rows, int64_t cols, float *out) {
    if (cols % 256 || !tile_bytes(type)) return -1;
    const int64_t nb = cols / 256;
    for (int64_t r = 0; r < rows; r++)
        for (int64_t c = 0; c < cols; c++)
            out[r * cols + c] = tile_elem_value(type, tiles + ((r >> 4) * nb + (c >> 8)) * (int64_t)tile_bytes(type), (int)(r & 15), (int)(c & 255));
    return 0;
}
