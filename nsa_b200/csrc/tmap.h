// Host-side creation of TMA tensor maps.  cuTensorMapEncodeTiled is resolved through the runtime's
// driver-entry-point query, so the library has no link-time dependency on libcuda.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nsa {

// bf16 tensor [N0][N1][H][D] (D contiguous).  Box = 64 columns x 1 head x `box_rows` rows of N1,
// 128-byte swizzle, out-of-range rows read as zero.  Returns 0 or a negative library error.
int make_tmap_rows4d(CUtensorMap* out, const void* base, int D, int H, long long N1, long long N0, int box_rows);

// bf16 matrix [rows][D] (D contiguous).  Box = 64 columns x `box_rows` rows, 128-byte swizzle.
int make_tmap_rows2d(CUtensorMap* out, const void* base, int D, long long rows, int box_rows);

// Generic bf16 tensor map: `rank` dims (innermost first, dim 0 contiguous), byte strides for dims 1.., box extents.
int make_tmap_generic(CUtensorMap* out, const void* base, int rank, const unsigned long long* dims,
                      const unsigned long long* strides, const unsigned* box);

void set_error(const char* fmt, ...);

// Process-wide count of kernels this library has launched (read through nsa_kernel_launch_count()).
void note_launches(int n);
long long launch_count();

}  // namespace nsa
