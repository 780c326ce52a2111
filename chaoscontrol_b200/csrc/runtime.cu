#include "runtime.h"
#include "ccb_api.h"
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include <atomic>
#include <mutex>

namespace ccb {

static thread_local char g_err[512] = "";
static std::atomic<int> g_launches{0};
static int* g_status[16] = {nullptr};
static int g_sms[16] = {0};
static std::mutex g_mu;

int set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return -1;
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

static int resolve_encode() {
  if (g_encode) return 0;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_encode) return 0;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || fn == nullptr || qres != cudaDriverEntryPointSuccess)
    return set_error("cuTensorMapEncodeTiled not available: %s", cudaGetErrorString(e));
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return 0;
}

static int make_tmap(CUtensorMap* out, CUtensorMapDataType dt, int esize, const void* base,
                     uint64_t d0, uint64_t d1, uint64_t d2, uint64_t ld, uint64_t bstride,
                     uint32_t box0, uint32_t box1) {
  if (resolve_encode()) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0)
    return set_error("tensor map base %p is not 16-byte aligned", base);
  if ((ld * esize) % 16 != 0) return set_error("tensor map row stride %llu not 16B aligned", (unsigned long long)ld);
  if (d2 <= 1 || bstride == 0) bstride = ld * d1;   // any legal value for a size-1 dimension
  if ((bstride * esize) % 16 != 0) return set_error("tensor map batch stride not 16B aligned");
  cuuint64_t dims[3] = {d0, d1, d2 < 1 ? 1 : d2};
  cuuint64_t strides[2] = {ld * (uint64_t)esize, bstride * (uint64_t)esize};
  cuuint32_t box[3] = {box0, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error("cuTensorMapEncodeTiled failed (%d) dims=%llu,%llu,%llu ld=%llu box=%u,%u", (int)r,
                     (unsigned long long)d0, (unsigned long long)d1, (unsigned long long)d2,
                     (unsigned long long)ld, box0, box1);
  return 0;
}

int make_tmap_bf16_3d(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                      uint64_t ld, uint64_t bstride, uint32_t box0, uint32_t box1) {
  return make_tmap(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, d0, d1, d2, ld, bstride, box0, box1);
}
int make_tmap_u8_3d(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                    uint64_t ld, uint64_t bstride, uint32_t box0, uint32_t box1) {
  return make_tmap(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, base, d0, d1, d2, ld, bstride, box0, box1);
}

}  // namespace ccb

using namespace ccb;

extern "C" int ccb_init(void) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return set_error("cudaGetDevice: %s", cudaGetErrorString(e));
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_status[dev & 15] == nullptr) {
    int* p = nullptr;
    e = cudaMalloc(&p, 64);
    if (e != cudaSuccess) return set_error("cudaMalloc(status): %s", cudaGetErrorString(e));
    cudaMemset(p, 0, 64);
    g_status[dev & 15] = p;
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    g_sms[dev & 15] = sms;
  }
  return 0;
}
extern "C" int* ccb_status_ptr(void) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (g_status[dev & 15] == nullptr) ccb_init();
  return g_status[dev & 15];
}
extern "C" int ccb_read_status(int reset) {
  int* p = ccb_status_ptr();
  if (!p) return -1;
  int v = 0;
  cudaError_t e = cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) { set_error("read status: %s", cudaGetErrorString(e)); return -2; }
  if (reset && v != 0) cudaMemset(p, 0, sizeof(int));
  return v;
}
extern "C" int ccb_num_sms(void) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (g_sms[dev & 15] == 0) ccb_init();
  return g_sms[dev & 15];
}
extern "C" int ccb_launch_count(void) { return g_launches.load(); }
extern "C" const char* ccb_last_error(void) { return g_err; }
