// Tensor maps for the tensor memory accelerator (TMA): descriptors of 2-D bfloat16 tensors in global memory,
// from which a kernel copies [box_rows x box_cols] tiles into shared memory with one instruction.
// The driver's encoder is looked up at run time, so the library links against the CUDA runtime only.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

namespace bt {

// A map of `rows` x `cols` bfloat16 elements, rows `row_stride` elements apart (a multiple of 8), copied in tiles
// of box_rows x 64 columns (128 bytes) with the 128-byte swizzle.  Maps are cached by their arguments.
// Returns 0 and fills *map, or sets the library's error text and returns non-zero.
int tensor_map_2d_bf16(CUtensorMap* map, const void* base, unsigned long long rows, unsigned long long cols,
                       unsigned long long row_stride, unsigned box_rows);

}  // namespace bt
