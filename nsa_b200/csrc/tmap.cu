#include "tmap.h"

#include <cudaTypedefs.h>
#include <atomic>
#include <mutex>

namespace nsa {

static std::atomic<long long> g_launches{0};
void note_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launch_count() { return g_launches.load(std::memory_order_relaxed); }

static PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
static std::once_flag g_once;

static void resolve() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
      q == cudaDriverEntryPointSuccess)
    g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
}

static int encode(CUtensorMap* out, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                  const cuuint32_t* box) {
  std::call_once(g_once, resolve);
  // cuTensorMapEncodeTiled is a driver-API call and needs a context current on the calling thread.  PyTorch runs
  // backward passes on worker threads that may not have touched the runtime yet when this is the first thing an entry
  // point does, so the primary context of the thread's current device is bound here (a no-op afterwards).
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  if (!g_encode) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return -20;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) {
    set_error("tensor base address must be 16-byte aligned for TMA");
    return -21;
  }
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return -22;
  }
  return 0;
}

int make_tmap_generic(CUtensorMap* out, const void* base, int rank, const unsigned long long* dims,
                      const unsigned long long* strides, const unsigned* box) {
  cuuint64_t d[5], st[4];
  cuuint32_t bx[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    bx[i] = box[i];
    if (i) st[i - 1] = strides[i - 1];
  }
  return encode(out, base, rank, d, st, bx);
}

int make_tmap_rows4d(CUtensorMap* out, const void* base, int D, int H, long long N1, long long N0, int box_rows) {
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)N1, (cuuint64_t)N0};
  cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)H * D * 2, (cuuint64_t)N1 * H * D * 2};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  return encode(out, base, 4, dims, strides, box);
}

int make_tmap_rows2d(CUtensorMap* out, const void* base, int D, long long rows, int box_rows) {
  cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)D * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  return encode(out, base, 2, dims, strides, box);
}

}  // namespace nsa
