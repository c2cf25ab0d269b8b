// Host-side runtime shared by all entry points of libdlblas_b200:
// error message storage, cached device properties, tensor-map encoding.
// The library never allocates or frees device memory.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>

#include "common.cuh"

namespace dlb {

static thread_local char g_last_error[512] = {0};

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

// DLBLAS_B200_WAIT_BUDGET_MS in the environment sets the limit at load time (1..60000 ms); dlb_set_wait_budget_ms
// changes it later
static uint64_t initial_wait_budget_ns() {
  const char* v = getenv("DLBLAS_B200_WAIT_BUDGET_MS");
  if (v != nullptr) {
    const long ms = strtol(v, nullptr, 10);
    if (ms >= 1 && ms <= 60000) return (uint64_t)ms * 1000000ull;
  }
  return DLB_WAIT_BUDGET_NS;
}
static std::atomic<uint64_t> g_wait_budget_ns{initial_wait_budget_ns()};

uint64_t wait_budget_ns() { return g_wait_budget_ns.load(std::memory_order_relaxed); }

int current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return dev;
}

int sm_count(int device) {
  static int cache[64];
  static std::once_flag once[64];
  if (device < 0 || device >= 64) return 148;
  std::call_once(once[device], [device]() {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
    cache[device] = n;
  });
  return cache[device];
}

PFN_encodeTiled get_encode_tiled() {
  static PFN_encodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = (PFN_encodeTiled)p;
    }
  });
  return fn;
}

int make_tmap_2d_16b(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                     uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
  PFN_encodeTiled enc = get_encode_tiled();
  DLB_CHECK_ARG(enc != nullptr, DLB_ERR_DRIVER, "cuTensorMapEncodeTiled is not available from the driver");
  DLB_CHECK_ARG(((uintptr_t)base & 15) == 0, DLB_ERR_ALIGNMENT, "tensor base %p is not 16-byte aligned", base);
  DLB_CHECK_ARG((row_stride_bytes & 15) == 0, DLB_ERR_ALIGNMENT, "row stride %llu B is not a multiple of 16",
                (unsigned long long)row_stride_bytes);
  DLB_CHECK_ARG(box_inner * 2 == 128, DLB_ERR_BAD_ARG, "128-byte swizzle needs a 128-byte inner box");
  DLB_CHECK_ARG(box_outer >= 1 && box_outer <= 256, DLB_ERR_BAD_ARG, "box_outer %u out of range", box_outer);
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  DLB_CHECK_ARG(r == CUDA_SUCCESS, DLB_ERR_DRIVER, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return DLB_OK;
}

// Encode a 4-D tensor map over a paged cache [pages, slots, heads, d] (element
// strides given), box = 64 x 1 x box_slots x 1, 128-byte swizzle.
int make_tmap_cache(CUtensorMap* out, const void* base, int64_t d, int64_t heads, int64_t slots,
                           int64_t pages, int64_t stride_page, int64_t stride_slot, int64_t stride_head,
                           int box_slots) {
  PFN_encodeTiled enc = get_encode_tiled();
  DLB_CHECK_ARG(enc != nullptr, DLB_ERR_DRIVER, "cuTensorMapEncodeTiled is not available from the driver");
  DLB_CHECK_ARG(((uintptr_t)base & 15) == 0, DLB_ERR_ALIGNMENT, "cache base is not 16-byte aligned");
  DLB_CHECK_ARG((stride_page * 2) % 16 == 0 && (stride_slot * 2) % 16 == 0 && (stride_head * 2) % 16 == 0,
                DLB_ERR_ALIGNMENT, "cache strides must be multiples of 16 bytes");
  cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)heads, (cuuint64_t)slots, (cuuint64_t)pages};
  cuuint64_t strides[3] = {(cuuint64_t)stride_head * 2, (cuuint64_t)stride_slot * 2, (cuuint64_t)stride_page * 2};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_slots, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  DLB_CHECK_ARG(r == CUDA_SUCCESS, DLB_ERR_DRIVER, "cuTensorMapEncodeTiled(cache) failed with CUresult %d", (int)r);
  return DLB_OK;
}


}  // namespace dlb

extern "C" {

int dlb_version(void) { return 100; }

const char* dlb_last_error(void) { return dlb::g_last_error; }

int dlb_set_wait_budget_ms(int64_t ms) {
  DLB_CHECK_ARG(ms >= 1 && ms <= 60000, DLB_ERR_BAD_ARG, "wait budget %lld ms not in [1, 60000]", (long long)ms);
  dlb::g_wait_budget_ns.store((uint64_t)ms * 1000000ull, std::memory_order_relaxed);
  return DLB_OK;
}

}  // extern "C"
