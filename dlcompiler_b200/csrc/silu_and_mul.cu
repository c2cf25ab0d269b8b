// silu_and_mul: out[t, i] = silu(x[t, i]) * x[t, N + i]
//
// Mirrors dlblas/kernels/activation.py:17-85 (reference Triton kernels): the
// gate is the first half of each row, the math runs in fp32
// (g / (1 + exp(-g)) * u) and the result is rounded once on store.
//
// HBM-bound streaming kernel: 3 * N * elemsize bytes per row.  Each thread
// moves 128-bit vectors (8 x 16-bit elements) with streaming cache hints; a
// thread owns UNROLL vectors spaced one block apart so that a warp's accesses
// stay fully coalesced and several loads are in flight per thread.
#include "common.cuh"

namespace dlb {

__device__ __forceinline__ float silu_mul_f32(float g, float u) {
  return __fdividef(g, 1.0f + __expf(-g)) * u;
}

template <typename T, int UNROLL>
__global__ void __launch_bounds__(512) silu_and_mul_vec_kernel(const T* __restrict__ x, T* __restrict__ out,
                                                               int nvec /* N / 8 */, int64_t x_row_stride,
                                                               int64_t out_row_stride, int n) {
  using T2 = typename Elem<T>::T2;
  // blockIdx.x = row, blockIdx.y = segment of the row: no integer division anywhere
  const int64_t r = blockIdx.x;
  const int bd = blockDim.x;
  const int c0 = blockIdx.y * (bd * UNROLL) + threadIdx.x;
  const uint4* gp = reinterpret_cast<const uint4*>(x + r * x_row_stride);
  const uint4* up = reinterpret_cast<const uint4*>(x + r * x_row_stride + n);
  uint4* op = reinterpret_cast<uint4*>(out + r * out_row_stride);

  uint4 g[UNROLL], u[UNROLL];
#pragma unroll
  for (int i = 0; i < UNROLL; ++i) {
    const int c = c0 + i * bd;
    if (c < nvec) {
      g[i] = __ldcs(gp + c);
      u[i] = __ldcs(up + c);
    }
  }
#pragma unroll
  for (int i = 0; i < UNROLL; ++i) {
    const int c = c0 + i * bd;
    if (c >= nvec) continue;
    uint4 o;
    const T2* g2 = reinterpret_cast<const T2*>(&g[i]);
    const T2* u2 = reinterpret_cast<const T2*>(&u[i]);
    T2* o2 = reinterpret_cast<T2*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 gf = Elem<T>::to_f2(g2[j]);
      const float2 uf = Elem<T>::to_f2(u2[j]);
      o2[j] = Elem<T>::from_f2(silu_mul_f32(gf.x, uf.x), silu_mul_f32(gf.y, uf.y));
    }
    __stcs(op + c, o);
  }
}

// Generic fallback for shapes/strides that do not allow 128-bit accesses
// (N not a multiple of the vector width, unaligned rows, fp32 data).
template <typename T>
__global__ void __launch_bounds__(256) silu_and_mul_scalar_kernel(const T* __restrict__ x, T* __restrict__ out,
                                                                  int64_t rows, int n, int64_t x_row_stride,
                                                                  int64_t out_row_stride) {
  const int64_t total = rows * (int64_t)n;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / n;
    const int c = (int)(idx - r * n);
    const float g = Elem<T>::to_f(x[r * x_row_stride + c]);
    const float u = Elem<T>::to_f(x[r * x_row_stride + n + c]);
    out[r * out_row_stride + c] = Elem<T>::from_f(silu_mul_f32(g, u));
  }
}

template <typename T>
static int launch_silu(const void* x, void* out, int64_t rows, int n, int64_t xs, int64_t os, cudaStream_t stream) {
  constexpr int VEC = 16 / sizeof(T);
  const bool vec_ok = (sizeof(T) == 2) && (n % VEC == 0) && (xs % VEC == 0) && (os % VEC == 0) &&
                      (((uintptr_t)x & 15) == 0) && (((uintptr_t)out & 15) == 0);
  if (vec_ok) {
    if constexpr (sizeof(T) == 2) {
      const int nvec = n / VEC;
      // block size (whole warps) and vectors per thread: the pair that leaves the fewest idle vector slots in
      // a row's last block.  N = 11008 has 1376 vectors per row: 352 threads x 4 cover a row with 32 idle
      // slots, where 256 threads x 2 leave 160 of 1536 idle.
      constexpr int kPreferredUnroll = 4;   // measured at N = 11008: 4 and 2 are equal (0.955 / 0.95 of HBM), 8 is 0.91
      int best_u = 1, best_bd = 256;
      int64_t best_cost = -1;
      for (int bd = 128; bd <= 512; bd += 32) {
        for (int u : {1, 2, 4, 8}) {
          const int per_block = bd * u;
          const int64_t waste = (int64_t)((nvec + per_block - 1) / per_block) * per_block - nvec;
          // ties: the preferred unroll, then the block size nearest 256
          const int64_t cost = waste * 4096 + (u == kPreferredUnroll ? 0 : 1024) + (bd > 256 ? bd - 256 : 256 - bd);
          if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best_u = u;
            best_bd = bd;
          }
        }
      }
      const int segs = (nvec + best_bd * best_u - 1) / (best_bd * best_u);
      DLB_CHECK_ARG(rows <= 0x7fffffffLL && segs <= 65535, DLB_ERR_TOO_LARGE, "silu_and_mul: grid too large");
      const dim3 grid((unsigned)rows, (unsigned)segs);
      const T* xp = (const T*)x;
      T* op = (T*)out;
      switch (best_u) {
        case 1: silu_and_mul_vec_kernel<T, 1><<<grid, best_bd, 0, stream>>>(xp, op, nvec, xs, os, n); break;
        case 2: silu_and_mul_vec_kernel<T, 2><<<grid, best_bd, 0, stream>>>(xp, op, nvec, xs, os, n); break;
        case 4: silu_and_mul_vec_kernel<T, 4><<<grid, best_bd, 0, stream>>>(xp, op, nvec, xs, os, n); break;
        default: silu_and_mul_vec_kernel<T, 8><<<grid, best_bd, 0, stream>>>(xp, op, nvec, xs, os, n); break;
      }
    }
  } else {
    const int64_t total = rows * (int64_t)n;
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = (int64_t)sm_count(current_device()) * 32;
    if (blocks > cap) blocks = cap;
    silu_and_mul_scalar_kernel<T><<<(unsigned)blocks, 256, 0, stream>>>((const T*)x, (T*)out, rows, n, xs, os);
  }
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}

}  // namespace dlb

extern "C" int dlb_silu_and_mul(const void* gate_up, void* out, int64_t rows, int64_t n,
                                int64_t gate_up_row_stride, int64_t out_row_stride, int dtype,
                                void* stream) {
  DLB_NVTX("dlb_silu_and_mul");
  using namespace dlb;
  DLB_CHECK_ARG(rows >= 0 && n >= 0, DLB_ERR_BAD_ARG, "silu_and_mul: negative size");
  DLB_CHECK_ARG(n <= 0x3fffffff, DLB_ERR_TOO_LARGE, "silu_and_mul: N=%lld too large", (long long)n);
  if (rows == 0 || n == 0) return DLB_OK;
  DLB_CHECK_ARG(gate_up != nullptr && out != nullptr, DLB_ERR_BAD_ARG, "silu_and_mul: null pointer");
  DLB_CHECK_ARG(gate_up_row_stride >= 2 * n && out_row_stride >= n, DLB_ERR_BAD_ARG,
                "silu_and_mul: row strides (%lld, %lld) smaller than the row", (long long)gate_up_row_stride,
                (long long)out_row_stride);
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case DLB_DTYPE_BF16:
      return launch_silu<__nv_bfloat16>(gate_up, out, rows, (int)n, gate_up_row_stride, out_row_stride, s);
    case DLB_DTYPE_F16:
      return launch_silu<__half>(gate_up, out, rows, (int)n, gate_up_row_stride, out_row_stride, s);
    case DLB_DTYPE_F32:
      return launch_silu<float>(gate_up, out, rows, (int)n, gate_up_row_stride, out_row_stride, s);
    default:
      set_last_error("silu_and_mul: unsupported dtype %d", dtype);
      return DLB_ERR_UNSUPPORTED;
  }
}
