// Tensor maps over row-major bfloat16 matrices, shared by the kernels that stream weights with TMA.
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace akv {

// Map over a row-major bfloat16 matrix [rows, cols]: boxes of 64 columns by `box_rows` rows, 128-byte swizzle, zeros
// outside the matrix.  Maps are cached by (base, rows, cols, box_rows).  False when the driver entry point is missing
// or refuses the shape.
bool weight_tensor_map(const void* base, int64_t rows, int64_t cols, int box_rows, CUtensorMap* out);

}  // namespace akv
