// Host-side tensor-map construction shared by the kernels that use TMA.
#pragma once
#include <cuda.h>
#include <cstdint>

namespace b200 {

// bf16 tensor of up to 3 dims (d0 innermost; d2 = 0 for a 2-D tensor), strides in bytes (multiples of 16),
// box {b0, b1, 1}, 128-byte swizzle, zero fill outside the tensor.  Encoded maps are cached by key.
// Returns 0, or a negative code (-1 no driver entry point, -2 misaligned, -3 encode failed).
int make_map(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1_bytes,
             uint64_t s2_bytes, uint32_t b0, uint32_t b1);

// CUresult of the last encode that failed (0 if none has): part of the error text of the entry points
int tma_last_encode_result();

}  // namespace b200
