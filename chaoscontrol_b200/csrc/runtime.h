// Host-side runtime shared by all launchers: error text, launch counter,
// status word, SM count and TMA tensor-map construction.  The driver entry
// point cuTensorMapEncodeTiled is resolved through the CUDA runtime at first
// use, so the library carries no link-time dependency on libcuda.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ccb {

int set_error(const char* fmt, ...);   // records the message, returns -1
void count_launch(int n = 1);

// bf16 tensor, up to three dimensions: d0 contiguous, d1 rows with stride ld
// (elements), d2 batches with stride bstride (elements).  128-byte swizzle;
// box0 * 2 bytes must equal 128.
int make_tmap_bf16_3d(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                      uint64_t ld, uint64_t bstride, uint32_t box0, uint32_t box1);
// Same for 1-byte (fp8) elements: box0 must be 128.
int make_tmap_u8_3d(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                    uint64_t ld, uint64_t bstride, uint32_t box0, uint32_t box1);

}  // namespace ccb
