// Host-side helper that encodes 2-D/3-D TMA tensor maps through the driver entry point
// (looked up at run time, so the library links without libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace z2h {

enum TmaSwizzle { kSwizzleNone = 0, kSwizzle128 = 1 };

// Row-major matrix [rows, cols] of 2-byte elements with row pitch ld (elements).
// Box = box_cols (innermost) x box_rows. Returns false on failure.
bool make_tma_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows, uint32_t box_cols, TmaSwizzle swz);

// Generic version: dims/strides given innermost first; strides in bytes for dims 1..rank-1.
bool make_tma_nd(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                 const uint64_t* strides_bytes, const uint32_t* box, int elem_bytes, TmaSwizzle swz);

}  // namespace z2h
