// Host-side construction of TMA tensor maps (cached by address and shape).
#pragma once

#include <cuda.h>

// A [rows, cols] bfloat16 matrix with row stride `ld` elements, fetched in boxes of box_rows x box_cols elements
// with the 128-byte swizzle (box_cols * 2 bytes must be 128).  Returns 0, or a negative code after fb_fail().
int fb_tensor_map_bf16(CUtensorMap* out, const void* ptr, long rows, long cols, long ld, int box_cols, int box_rows);

// As above, but nothing is cached and no host memory is taken.
int fb_tensor_map_bf16_uncached(CUtensorMap* out, const void* ptr, long rows, long cols, long ld, int box_cols,
                                int box_rows);

// The output of a product, [slabs][rows][cols] of float32 (elem_bytes 4) or bfloat16 (2), for stores of boxes of
// box_rows x box_cols elements of one slab from shared memory (no swizzle).  0: made; 1: these strides or this
// address do not allow one (store without it); negative: refused by the driver, after fb_fail().
int fb_tensor_map_out(CUtensorMap* out, void* ptr, int elem_bytes, long rows, long cols, long ld, long slabs,
                      long slab_stride, int box_cols, int box_rows);
