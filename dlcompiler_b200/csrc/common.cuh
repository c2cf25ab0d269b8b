// Shared device/host helpers for the sm_100a kernels of libdlblas_b200.
//
// Everything here is header-only.  The PTX wrappers cover the Blackwell
// execution model pieces the tensor-core kernels use: mbarrier, TMA
// (cp.async.bulk.tensor), tcgen05 (TMEM allocation, MMA, commit, ld/st).
// Every wait on an mbarrier is bounded: after a wall-clock budget the waiter
// raises a CTA-wide abort flag, records where it gave up in a device status
// word and returns false, so a protocol bug can never hang the GPU.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <nvtx3/nvToolsExt.h>

// NVTX range around the host side of an entry point (argument checks, tensor-map encoding, launches): a
// timeline tool shows each library call under its own name; without a tool attached the calls cost a
// pointer test each.
namespace dlb {
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};
}  // namespace dlb
#define DLB_NVTX(name) ::dlb::NvtxRange dlb_nvtx_range_(name)

// ----------------------------------------------------------------------------
// Status codes returned by every extern "C" entry point.
//   0        ok
//   < 0      argument / support error (see dlb_last_error())
//   > 0      cudaError_t of the failing runtime call
// ----------------------------------------------------------------------------
#define DLB_OK 0
#define DLB_ERR_BAD_ARG (-1)
#define DLB_ERR_UNSUPPORTED (-2)
#define DLB_ERR_ALIGNMENT (-3)
#define DLB_ERR_DRIVER (-4)
#define DLB_ERR_TOO_LARGE (-5)

// The public prototypes: every translation unit that defines an entry point sees its declaration, so
// a definition whose arguments drift from the header fails to compile.  The element type codes
// (DLB_DTYPE_*) and the flag values of the boundary come from there.
#include "dlblas_b200.h"

// Layout of the device status word array (int32[4]) that kernels with bounded
// waits write when they give up:  [0] = error code (0 = none), [1] = wait site,
// [2] = blockIdx.x, [3] = auxiliary value (tile / iteration).
#define DLB_DEV_OK 0
#define DLB_DEV_WAIT_TIMEOUT 1

namespace dlb {

void set_last_error(const char* fmt, ...);

#define DLB_CHECK_ARG(cond, code, ...)      \
  do {                                      \
    if (!(cond)) {                          \
      ::dlb::set_last_error(__VA_ARGS__);   \
      return (code);                        \
    }                                       \
  } while (0)

#define DLB_CUDA_LAUNCH_CHECK()                                             \
  do {                                                                      \
    cudaError_t e__ = cudaGetLastError();                                   \
    if (e__ != cudaSuccess) {                                               \
      ::dlb::set_last_error("CUDA launch failed: %s", cudaGetErrorString(e__)); \
      return (int)e__;                                                      \
    }                                                                       \
  } while (0)

// Wall-clock limit of a wait on another GPU's flag (dlb_set_wait_budget_ms; 2 s unless changed).
uint64_t wait_budget_ns();

// Cached per-device properties (immutable after first query).
int sm_count(int device);
int current_device();

// Driver entry point for tensor-map encoding, resolved through the runtime so
// the library does not link against libcuda directly.
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
PFN_encodeTiled get_encode_tiled();

// Encode a 2-D row-major tensor map (inner dimension contiguous) for 16-bit
// elements with the 128-byte swizzle; box = box_inner x box_outer elements.
// Returns DLB_OK or a negative status with the message set.
// 4-D tensor map over a paged cache [pages, slots, heads, d] (element strides), box = 64 x 1 x box_slots x 1,
// 128-byte swizzle.
int make_tmap_cache(CUtensorMap* out, const void* base, int64_t d, int64_t heads, int64_t slots, int64_t pages,
                    int64_t stride_page, int64_t stride_slot, int64_t stride_head, int box_slots);
int make_tmap_2d_16b(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                     uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer);

#ifdef __CUDACC__

// ----------------------------------------------------------------------------
// Small numeric helpers
// ----------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<__nv_bfloat16> {
  using T2 = __nv_bfloat162;
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float2 to_f2(__nv_bfloat162 v) { return __bfloat1622float2(v); }
  static __device__ __forceinline__ __nv_bfloat162 from_f2(float a, float b) { return __floats2bfloat162_rn(a, b); }
};
template <> struct Elem<__half> {
  using T2 = __half2;
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ float2 to_f2(__half2 v) { return __half22float2(v); }
  static __device__ __forceinline__ __half2 from_f2(float a, float b) { return __floats2half2_rn(a, b); }
};
template <> struct Elem<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};

// Rotate-half rotary embedding of one (lower, upper) element pair, arithmetic in the tensors' 16-bit type:
// each product and the sum round to T, as separate operations in T would (the reference evaluates
// x * cos + rotate_half(x) * sin in the tensor dtype, apply_rotary_pos_emb.py:50-54,70-71).
template <typename T> __device__ __forceinline__ T rot_lo(T lo, T hi, T c, T s) {
  const float a = Elem<T>::to_f(Elem<T>::from_f(Elem<T>::to_f(lo) * Elem<T>::to_f(c)));
  const float b = Elem<T>::to_f(Elem<T>::from_f(Elem<T>::to_f(hi) * Elem<T>::to_f(s)));
  return Elem<T>::from_f(a - b);
}
template <typename T> __device__ __forceinline__ T rot_hi(T lo, T hi, T c, T s) {
  const float a = Elem<T>::to_f(Elem<T>::from_f(Elem<T>::to_f(hi) * Elem<T>::to_f(c)));
  const float b = Elem<T>::to_f(Elem<T>::from_f(Elem<T>::to_f(lo) * Elem<T>::to_f(s)));
  return Elem<T>::from_f(a + b);
}
// the same on 8 pairs held in two 16-byte vectors, with packed two-element arithmetic: a packed multiply,
// add or subtract rounds each lane once to T, which is what the scalar form above does (the fp32
// product of two 16-bit values is exact, and so is the fp32 sum whenever it could round differently)
template <typename T>
__device__ __forceinline__ void rot_vec8(const uint4& lo, const uint4& hi, const uint4& cl, const uint4& ch,
                                         const uint4& sl, const uint4& sh, uint4& olo, uint4& ohi) {
  using T2 = typename Elem<T>::T2;
  const T2* l2 = reinterpret_cast<const T2*>(&lo);
  const T2* h2 = reinterpret_cast<const T2*>(&hi);
  const T2* cl2 = reinterpret_cast<const T2*>(&cl);
  const T2* ch2 = reinterpret_cast<const T2*>(&ch);
  const T2* sl2 = reinterpret_cast<const T2*>(&sl);
  const T2* sh2 = reinterpret_cast<const T2*>(&sh);
  T2* ol2 = reinterpret_cast<T2*>(&olo);
  T2* oh2 = reinterpret_cast<T2*>(&ohi);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    ol2[j] = __hsub2_rn(__hmul2_rn(l2[j], cl2[j]), __hmul2_rn(h2[j], sl2[j]));
    oh2[j] = __hadd2_rn(__hmul2_rn(h2[j], ch2[j]), __hmul2_rn(l2[j], sh2[j]));
  }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ----------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Make generic-proxy writes to shared memory visible to the async proxy
// (TMA, tcgen05.mma operand reads).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Wall-clock budget of one wait before the CTA aborts (nanoseconds).
#ifndef DLB_WAIT_BUDGET_NS
#define DLB_WAIT_BUDGET_NS 2000000000ull
#endif

// Bounded wait.  `abort_flag` lives in shared memory and is shared by every
// role of the CTA; `status` is the global int32[4] status word (may be null).
// Returns false if the CTA is aborting.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int site, int aux) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 0xff) == 0) {
      if (*abort_flag) return false;
      uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > DLB_WAIT_BUDGET_NS) {
        *abort_flag = 1;
        if (status != nullptr && atomicCAS(status, DLB_DEV_OK, DLB_DEV_WAIT_TIMEOUT) == DLB_DEV_OK) {
          status[1] = site;
          status[2] = (int)blockIdx.x;
          status[3] = aux;
        }
        return false;
      }
    }
  }
}

// ----------------------------------------------------------------------------
// TMA (tiled bulk tensor copies, no multicast anywhere in this library)
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
// x = element coordinate along the contiguous dimension (x * elemsize must be a
// multiple of 16 bytes), y = row coordinate.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int x,
                                            int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// ----------------------------------------------------------------------------
// tcgen05: tensor memory + 5th-generation tensor-core MMA (cta_group::1)
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// tcgen05.mma, issued by ONE thread.  D[tmem] (+)= A * B with A from a shared-memory descriptor (ss) or
// from TMEM (ts: A occupies lanes 0..127, one row each; a 32-bit TMEM column holds two K-consecutive
// 16-bit elements, so one K16 step spans 8 columns), B from a shared-memory descriptor.
// The forms are deliberately lean.  A single thread issues every MMA of a CTA, so the instructions
// AROUND each tcgen05.mma bound the tensor pipe at small N: measured on B200 with back-to-back MMAs
// from one thread, 64-bit descriptors built or added per MMA with the accumulate flag through setp
// sustain 99 / 107 / 171 clocks per M128 K16 MMA at N = 64 / 128 / 256; the forms below (descriptor
// as two 32-bit halves of which only the low one moves, accumulate flag as a literal) 48 / 64 / 128,
// i.e. the math rate at N >= 128.  ACC = 0 overwrites the accumulator, 1 adds to it.
template <int ACC>
__device__ __forceinline__ void umma_ss_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                             uint32_t b_hi, uint32_t idesc) {
  if constexpr (ACC != 0) {
    asm volatile(
        "{\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, 1;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, 0;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc) : "memory");
  }
}
template <int ACC>
__device__ __forceinline__ void umma_ts_lohi(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                             uint32_t idesc) {
  if constexpr (ACC != 0) {
    asm volatile(
        "{\n\t.reg .b64 db;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, 1;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .b64 db;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, 0;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc) : "memory");
  }
}
// mbarrier arrives once every previously issued MMA of this thread retired.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Warp-collective load of 32 consecutive fp32 columns for this thread's lane
// (TMEM lane = 32 * (warp_id % 4) + lane_id).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
      "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
      "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// Shared-memory matrix descriptor (64 bit) for tcgen05.mma operands:
//   [0,14)  start address >> 4        [16,30) leading byte offset >> 4
//   [32,46) stride byte offset >> 4   [46,48) version = 1 (sm_100)
//   [61,64) swizzle: 0 none, 2 = 128 B, 4 = 64 B, 6 = 32 B
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t swizzle_code) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)(swizzle_code & 7) << 61;
  return d;
}

// Instruction descriptor (32 bit) for kind::f16 with fp32 accumulation.
//   ab_format: 0 = f16, 1 = bf16;  *_mn_major: 0 = K-major operand, 1 = MN-major.
__host__ __device__ constexpr uint32_t make_idesc_f16(uint32_t m, uint32_t n, uint32_t ab_format,
                                                      uint32_t a_mn_major, uint32_t b_mn_major) {
  return (1u << 4)                     // D format: f32
         | (ab_format << 7)            // A format
         | (ab_format << 10)           // B format
         | (a_mn_major << 15)          // A major
         | (b_mn_major << 16)          // B major
         | ((n >> 3) << 17)            // N / 8
         | ((m >> 4) << 24);           // M / 16
}

#endif  // __CUDACC__

}  // namespace dlb
