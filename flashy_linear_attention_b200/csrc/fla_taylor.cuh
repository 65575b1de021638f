// Second-order Taylor feature map for linear attention and its gradient, for sm_100a:
//     phi(x) = [1, x / d^(1/4), vec(x x^T) / (sqrt(2) sqrt(d))]        (1 + d + d^2 features)
// so that phi(q) . phi(k) = 1 + s + s^2 / 2 with s = q . k / sqrt(d). The reference has no such code
// (its README only links the idea); benchmark configuration 4 feeds these features, d = 16 -> 273,
// to LinearAttentionSmallVHD. The forward kernel writes the features straight into rows padded to
// a multiple of 8 elements, i.e. in the layout the attention kernels address with TMA, so no pad
// pass is needed; the backward kernel contracts the feature gradients back to d raw dimensions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fla {

template <int D>
struct TaylorDims {
  static constexpr int F = 1 + D + D * D;        // features
  static constexpr int FP = (F + 7) / 8 * 8;     // padded row length (elements)
  static constexpr int PIECES = FP / 8;          // 16-byte pieces per row
};

__device__ __forceinline__ float taylor_c1(int d) { return rsqrtf(sqrtf(static_cast<float>(d))); }
__device__ __forceinline__ float taylor_c2(int d) { return rsqrtf(2.f * static_cast<float>(d)); }

constexpr int kTaylorRows = 128;  // rows per block tile (one thread per row) in both kernels
template <int D>
__host__ __device__ constexpr int taylor_tile_smem_bytes() {
  // row stride FP/2 + 1 words: odd, so that one thread per row touches 32 different banks
  return kTaylorRows * (TaylorDims<D>::FP / 2 + 1) * 4;
}

// x: [rows][D] bf16 contiguous; phi: [rows][FP] bf16 (FP - F zero columns at the end).
// Thread t computes the features of row t from registers (all indices are compile-time) into a
// shared-memory tile; the block then writes the tile out in coalesced 16-byte pieces.
template <int D>
__global__ void __launch_bounds__(kTaylorRows)
fla_taylor_fwd_kernel(const __nv_bfloat16* __restrict__ x, uint4* __restrict__ phi, long long rows) {
  using dims = TaylorDims<D>;
  static_assert(D % 8 == 0, "raw rows are moved as 16-byte pieces");
  constexpr int WSTRIDE = dims::FP / 2 + 1;
  extern __shared__ uint32_t taylor_smem[];
  const float c1 = taylor_c1(D), c2 = taylor_c2(D);
  for (long long row0 = static_cast<long long>(blockIdx.x) * kTaylorRows; row0 < rows;
       row0 += static_cast<long long>(gridDim.x) * kTaylorRows) {
    const int nrows = static_cast<int>(min(static_cast<long long>(kTaylorRows), rows - row0));
    __syncthreads();  // the previous tile has been written out
    const int r = threadIdx.x;
    if (r < nrows) {
      float xv[D];
      const uint4* xrow = reinterpret_cast<const uint4*>(x + (row0 + r) * D);
#pragma unroll
      for (int pc = 0; pc < D / 8; ++pc) {
        const uint4 v = xrow[pc];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          xv[pc * 8 + 2 * j] = __uint_as_float(w[j] << 16);
          xv[pc * 8 + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
        }
      }
      uint32_t* out = taylor_smem + r * WSTRIDE;
      auto feature = [&](int f) -> float {  // f is a compile-time constant after unrolling
        if (f == 0) return 1.f;
        if (f <= D) return c1 * xv[f - 1];
        if (f < dims::F) return c2 * xv[(f - 1 - D) / D] * xv[(f - 1 - D) % D];
        return 0.f;
      };
#pragma unroll
      for (int w = 0; w < dims::FP / 2; ++w) {
        const __nv_bfloat162 pr = __floats2bfloat162_rn(feature(2 * w), feature(2 * w + 1));
        out[w] = *reinterpret_cast<const uint32_t*>(&pr);
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nrows * dims::PIECES; idx += kTaylorRows) {
      const int rr = idx / dims::PIECES, pc = idx - rr * dims::PIECES;
      const uint32_t* src = taylor_smem + rr * WSTRIDE + pc * 4;
      phi[(row0 + rr) * dims::PIECES + pc] = make_uint4(src[0], src[1], src[2], src[3]);
    }
  }
}

// dx[r][a] = c1 dphi[r][1 + a] + c2 sum_b (dphi[r][1 + D + a D + b] + dphi[r][1 + D + b D + a]) x[r][b]
// dphi: [rows][FP] bf16 (row stride FP), x: [rows][D] bf16, dx: [rows][D] bf16.
// A block stages kTaylorRows rows of dphi in shared memory (coalesced 16-byte loads, row stride
// FP/2 + 1 words so that one thread per row reads without bank conflicts), then thread t contracts
// row t.
template <int D>
__global__ void __launch_bounds__(kTaylorRows)
fla_taylor_bwd_kernel(const uint4* __restrict__ dphi, const __nv_bfloat16* __restrict__ x,
                      __nv_bfloat16* __restrict__ dx, long long rows) {
  using dims = TaylorDims<D>;
  constexpr int WSTRIDE = dims::FP / 2 + 1;  // words per staged row
  extern __shared__ uint32_t taylor_smem[];
  const float c1 = taylor_c1(D), c2 = taylor_c2(D);
  for (long long row0 = static_cast<long long>(blockIdx.x) * kTaylorRows; row0 < rows;
       row0 += static_cast<long long>(gridDim.x) * kTaylorRows) {
    const int nrows = static_cast<int>(min(static_cast<long long>(kTaylorRows), rows - row0));
    __syncthreads();  // the previous tile has been consumed
    for (int idx = threadIdx.x; idx < nrows * dims::PIECES; idx += kTaylorRows) {
      const int r = idx / dims::PIECES, pc = idx - r * dims::PIECES;
      const uint4 v = dphi[(row0 + r) * dims::PIECES + pc];
      uint32_t* dst = taylor_smem + r * WSTRIDE + pc * 4;
      dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
    }
    __syncthreads();
    const int r = threadIdx.x;
    if (r < nrows) {
      const uint32_t* g = taylor_smem + r * WSTRIDE;
      auto gval = [&](int f) {
        const uint32_t w = g[f >> 1];
        return __uint_as_float((f & 1) ? (w & 0xFFFF0000u) : (w << 16));
      };
      static_assert(D % 8 == 0, "raw rows are moved as 16-byte pieces");
      float xv[D], acc[D];
      const uint4* xrow = reinterpret_cast<const uint4*>(x + (row0 + r) * D);
#pragma unroll
      for (int pc = 0; pc < D / 8; ++pc) {
        const uint4 v = xrow[pc];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          xv[pc * 8 + 2 * j] = __uint_as_float(w[j] << 16);
          xv[pc * 8 + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
        }
      }
#pragma unroll
      for (int a = 0; a < D; ++a) acc[a] = c1 * gval(1 + a);
#pragma unroll
      for (int a = 0; a < D; ++a) {
#pragma unroll
        for (int b = 0; b < D; ++b) {
          const float gv = c2 * gval(1 + D + a * D + b);
          acc[a] += gv * xv[b];
          acc[b] += gv * xv[a];
        }
      }
      uint4* orow = reinterpret_cast<uint4*>(dx + (row0 + r) * D);
#pragma unroll
      for (int pc = 0; pc < D / 8; ++pc) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const __nv_bfloat162 pr = __floats2bfloat162_rn(acc[pc * 8 + 2 * j], acc[pc * 8 + 2 * j + 1]);
          w[j] = *reinterpret_cast<const uint32_t*>(&pr);
        }
        orow[pc] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
}

}  // namespace fla
