// Tensor maps (TMA descriptors) of row-major bfloat16 matrices, shared by the kernels that load
// tiles with cp.async.bulk.tensor.
#pragma once
#include "common.cuh"
#include <cuda.h>

// A map of the matrix [rows, cols] at ptr with a row stride of ld elements, read in boxes of
// box_rows rows x 64 columns (128 bytes) that land in shared memory with the 128-byte swizzle.
// Maps are cached by (ptr, rows, cols, ld, box_rows): encoding one costs microseconds, and the
// engine's buffers keep their addresses.  ptr and ld * 2 must be multiples of 16 bytes.
// `who` names the caller in the error message.  Returns CE_OK or a negative code.
int ce_tensor_map_bf16(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out,
                       const char* who);
