// Denominator of causal linear attention and its gradients, as streaming kernels for sm_100a.
//
// The reference leaves the normalisation to PyTorch (README.md:27-30):
//     denom = (q * k.cumsum(-2)).sum(-1, keepdim=True) + eps;   out = num / denom
// which materialises the cumulative sum and the product as full tensors. Here
//   fla_normalize_fwd_kernel     one sweep over q, k, num per head: running z = sum_j k_j (fp32,
//                                one thread per column), den_i = q_i . z_i + eps, out_i = num_i / den_i
//   fla_normalize_bwd_prepare    per row: dnum = g / den (what the product's backward consumes) and
//                                dden = -(g . out) / den
//   fla_normalize_bwd_sweep      dQ_i += dden_i z_i (ascending sweep over k) and
//                                dK_j += sum_{i>=j} dden_i q_i (descending sweep over q)
//   fla_colsum_kernel            per (head, segment): column sums of k (or of dden_i q_i), so that
//                                the sweeps above can start every segment of a sequence from its
//                                prefix (suffix) and many CTAs share one head
// All are bound by HBM; token tiles are staged in shared memory with cp.async.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fla {

struct NormTensor {
  void* ptr;
  long long sb, sh, sn;  // element strides (batch, head, token); innermost stride 1
};

struct NormParams {
  NormTensor q, k;      // [B, H, N, dk] bf16
  NormTensor x;         // fwd: num in / out (normalised in place); prepare: g; sweep: unused
  NormTensor y;         // prepare: normalised output (in); sweep: unused
  NormTensor z;         // prepare: dnum (out)
  NormTensor dq, dk_;   // sweep: gradients updated in place
  float* den;           // [B*H, N] fp32: fwd out, prepare in
  float* dden;          // [B*H, N] fp32: prepare out, sweep in
  int heads, n, dk, dv;
  float eps;
  int seg_len;          // tokens per segment (a multiple of the token tile); grid x = segment
  int nseg;
  const float* sums;    // [B*H][nseg][dk] fp32 column sums per segment (ascending sweeps: of k)
  const float* rsums;   // same for the descending sweep: sums of dden_i q_i
  float* sums_out;      // colsum kernel: output
  int weighted;         // colsum kernel: weight row i by dden_i
};

constexpr int kNormTile = 64;      // tokens per tile (32 for head dims above 128)
constexpr int kNormThreads = 256;
constexpr int kNormStages = 2;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint32_t norm_smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ const __nv_bfloat16* norm_row(const NormTensor& t, int b, int h, long long tok) {
  return static_cast<const __nv_bfloat16*>(t.ptr) + b * t.sb + h * t.sh + tok * t.sn;
}

// Copies rows [tok0, tok0 + T) x [0, dpad) of `t` into a [T][dpad] bf16 tile (dpad a multiple of 8);
// rows past the sequence are zero-filled.
template <int T>
__device__ __forceinline__ void norm_load_tile(__nv_bfloat16* tile, const NormTensor& t, int b, int h,
                                               int tok0, int n, int dpad) {
  const int pieces = dpad >> 3;
  for (int idx = threadIdx.x; idx < T * pieces; idx += kNormThreads) {
    const int r = idx / pieces;
    const int c = (idx - r * pieces) << 3;
    __nv_bfloat16* dst = tile + r * dpad + c;
    if (tok0 + r < n) {
      cp_async16(norm_smem_u32(dst), norm_row(t, b, h, tok0 + r) + c);
    } else {
      *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

// Thread layout of the column scans: a thread owns one PAIR of columns (one 32-bit bf16x2 word) and
// one group of consecutive tokens of the tile; the groups' totals are exchanged through shared
// memory (two-level scan), so that all 256 threads work and the dependent chain is T / groups long.
struct ScanLayout {
  int pairs;    // column pairs = dkp / 2
  int groups;   // token groups (power of two)
  int gt;       // tokens per group
  int cp, grp;  // this thread's pair and group; active if grp < groups
};
template <int T>
__device__ __forceinline__ ScanLayout scan_layout(int dkp) {
  ScanLayout L;
  L.pairs = dkp >> 1;
  int g = kNormThreads / L.pairs;
  int groups = 1;
  while (groups * 2 <= g && groups * 2 <= T / 4) groups *= 2;
  L.groups = groups;
  L.gt = T / groups;
  L.cp = threadIdx.x % L.pairs;
  L.grp = threadIdx.x / L.pairs;
  return L;
}
// Lanes that share one row in the row-wise phases (8 columns per lane and step): a power of two.
__device__ __forceinline__ int lanes_per_row(int dpad) {
  const int need = dpad >> 3;
  int l = 1;
  while (l < need && l < 32) l *= 2;
  return l;
}
__device__ __forceinline__ float2 bf2_to_f2(uint32_t w) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
}
__device__ __forceinline__ uint32_t f2_to_bf2(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// Column sums of one segment of p.k (weighted = 0) or of dden_i * p.q rows (weighted = 1):
// sums_out[bh][segment][c]. Thread t owns the 8 columns of 16-byte piece (t % pieces) and every
// (256 / pieces)-th row; the row groups are combined through shared memory.
__global__ void __launch_bounds__(kNormThreads)
fla_colsum_kernel(const NormParams p) {
  __shared__ float part[kNormThreads * 8];
  const int seg = blockIdx.x, bh = blockIdx.y;
  const int b = bh / p.heads, h = bh % p.heads;
  const int dkp = (p.dk + 7) / 8 * 8;
  const int pieces = dkp >> 3;
  const NormTensor& src = p.weighted ? p.q : p.k;
  const int tok0 = seg * p.seg_len;
  const int tok1 = min(p.n, tok0 + p.seg_len);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const int rows_per_pass = kNormThreads / pieces;  // >= 1 for head dims up to 2048
  const int piece = threadIdx.x % pieces;
  const int rgrp = threadIdx.x / pieces;
  if (rgrp < rows_per_pass) {
    for (int tok = tok0 + rgrp; tok < tok1; tok += rows_per_pass) {
      const uint4 v = *reinterpret_cast<const uint4*>(norm_row(src, b, h, tok) + piece * 8);
      const float w = p.weighted ? p.dden[static_cast<size_t>(bh) * p.n + tok] : 1.f;
      const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&words[j]));
        acc[2 * j] += w * f.x;
        acc[2 * j + 1] += w * f.y;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) part[threadIdx.x * 8 + j] = (rgrp < rows_per_pass) ? acc[j] : 0.f;
  __syncthreads();
  for (int c = threadIdx.x; c < p.dk; c += kNormThreads) {
    float tot = 0.f;
    const int pc = c >> 3, j = c & 7;
    for (int g = 0; g < rows_per_pass; ++g) tot += part[(g * pieces + pc) * 8 + j];
    p.sums_out[(static_cast<size_t>(bh) * p.nseg + seg) * p.dk + c] = tot;
  }
}

// Shared memory: kNormStages x (q tile, k tile, x tile) + Z [T][dkp] fp32
__host__ __device__ inline size_t norm_fwd_smem_bytes(int dk, int dv, int tile) {
  const size_t dkp = (dk + 7) / 8 * 8, dvp = (dv + 7) / 8 * 8;
  return kNormStages * tile * (2 * dkp + dvp) * 2 + tile * dkp * 4 + kNormThreads * 8;  // + group totals
}

// D: compile-time head dim when dk == dv == D (strides, divisions and loop counts then fold to
// constants), 0: head dims taken from the parameters at run time.
template <int T, int D>
__global__ void __launch_bounds__(kNormThreads)
fla_normalize_fwd_kernel(const NormParams p_in) {
  constexpr int kNormTile = T;  // shadows the default tile size inside this kernel
  NormParams p = p_in;
  if (D != 0) p.dk = p.dv = D;
  extern __shared__ __align__(16) uint8_t norm_smem[];
  const int seg = blockIdx.x, bh = blockIdx.y;
  const int b = bh / p.heads, h = bh % p.heads;
  const int dkp = (p.dk + 7) / 8 * 8, dvp = (p.dv + 7) / 8 * 8;
  const int stage_elems = kNormTile * (2 * dkp + dvp);
  __nv_bfloat16* stages = reinterpret_cast<__nv_bfloat16*>(norm_smem);
  float* Z = reinterpret_cast<float*>(norm_smem + static_cast<size_t>(kNormStages) * stage_elems * 2);
  const int seg_tok0 = seg * p.seg_len;
  const int seg_tokens = min(p.seg_len, p.n - seg_tok0);
  const int ntiles = (seg_tokens + kNormTile - 1) / kNormTile;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  auto issue = [&](int t) {
    if (t < ntiles) {
      __nv_bfloat16* st = stages + (t % kNormStages) * stage_elems;
      const int tok0 = seg_tok0 + t * kNormTile;
      norm_load_tile<T>(st, p.q, b, h, tok0, p.n, dkp);
      norm_load_tile<T>(st + kNormTile * dkp, p.k, b, h, tok0, p.n, dkp);
      norm_load_tile<T>(st + 2 * kNormTile * dkp, p.x, b, h, tok0, p.n, dvp);
    }
    cp_async_commit();
  };
  issue(0);
  // Running column sums of k, one column pair per thread (see ScanLayout); a segment starts from
  // the sums of the segments before it.
  const ScanLayout L = scan_layout<T>(dkp);
  const bool scan_active = L.grp < L.groups;
  const bool valid0 = 2 * L.cp < p.dk, valid1 = 2 * L.cp + 1 < p.dk;
  float2 zrun = make_float2(0.f, 0.f);
  if (p.sums != nullptr && scan_active) {
    for (int s2 = 0; s2 < seg; ++s2) {
      const float* sp = p.sums + (static_cast<size_t>(bh) * p.nseg + s2) * p.dk;
      if (valid0) zrun.x += sp[2 * L.cp];
      if (valid1) zrun.y += sp[2 * L.cp + 1];
    }
  }
  float2* totals = reinterpret_cast<float2*>(Z + kNormTile * dkp);  // [groups][pairs]
  const int lpr_k = lanes_per_row(dkp), lpr_v = lanes_per_row(dvp);
  const int lpr = lpr_k > lpr_v ? lpr_k : lpr_v;  // lanes per row of the row-wise phase
  const int rpw = 32 / lpr;                        // rows per warp and step
  const int sub = lane % lpr, rsel = lane / lpr;
  for (int t = 0; t < ntiles; ++t) {
    issue(t + 1);
    cp_async_wait<1>();
    __syncthreads();
    const __nv_bfloat16* qt = stages + (t % kNormStages) * stage_elems;
    const __nv_bfloat16* kt = qt + kNormTile * dkp;
    const __nv_bfloat16* xt = kt + kNormTile * dkp;
    // ---- inclusive column scan of the k tile -> Z (fp32): group-local sums, then the offsets
    if (scan_active) {
      float2 z = make_float2(0.f, 0.f);
      for (int ii = 0; ii < L.gt; ++ii) {
        const int i = L.grp * L.gt + ii;
        const float2 kv = bf2_to_f2(*reinterpret_cast<const uint32_t*>(kt + i * dkp + 2 * L.cp));
        z.x += valid0 ? kv.x : 0.f;
        z.y += valid1 ? kv.y : 0.f;
        *reinterpret_cast<float2*>(Z + i * dkp + 2 * L.cp) = z;
      }
      totals[L.grp * L.pairs + L.cp] = z;
    }
    __syncthreads();
    if (scan_active) {
      float2 off = zrun;
      float2 all = zrun;
      for (int g = 0; g < L.groups; ++g) {
        const float2 tg = totals[g * L.pairs + L.cp];
        if (g < L.grp) { off.x += tg.x; off.y += tg.y; }
        all.x += tg.x; all.y += tg.y;
      }
      for (int ii = 0; ii < L.gt; ++ii) {
        float2* zp = reinterpret_cast<float2*>(Z + (L.grp * L.gt + ii) * dkp + 2 * L.cp);
        float2 z = *zp;
        z.x += off.x; z.y += off.y;
        *zp = z;
      }
      zrun = all;
    }
    __syncthreads();
    // ---- den_i = q_i . z_i + eps, out_i = num_i / den_i: `lpr` lanes per token row, 8 columns per
    //      lane and step
    for (int i0 = warp * rpw; i0 < kNormTile; i0 += (kNormThreads / 32) * rpw) {
      const int i = i0 + rsel;
      const int tok = seg_tok0 + t * kNormTile + i;
      float acc = 0.f;
      for (int c = sub * 8; c < dkp; c += lpr * 8) {
        const float4 z0 = *reinterpret_cast<const float4*>(Z + i * dkp + c);
        const float4 z1 = *reinterpret_cast<const float4*>(Z + i * dkp + c + 4);
        const uint4 qv = *reinterpret_cast<const uint4*>(qt + i * dkp + c);
        const float2 q01 = bf2_to_f2(qv.x), q23 = bf2_to_f2(qv.y), q45 = bf2_to_f2(qv.z), q67 = bf2_to_f2(qv.w);
        if (c + 7 < p.dk) {
          acc += z0.x * q01.x + z0.y * q01.y + z0.z * q23.x + z0.w * q23.y +
                 z1.x * q45.x + z1.y * q45.y + z1.z * q67.x + z1.w * q67.y;
        } else {  // the row's padding columns may hold anything
          const float zz[8] = {z0.x, z0.y, z0.z, z0.w, z1.x, z1.y, z1.z, z1.w};
          const float qq[8] = {q01.x, q01.y, q23.x, q23.y, q45.x, q45.y, q67.x, q67.y};
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (c + j < p.dk) acc += zz[j] * qq[j];
        }
      }
      for (int o = lpr >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      const float den = acc + p.eps;
      if (tok < p.n) {
        if (sub == 0) p.den[static_cast<size_t>(bh) * p.n + tok] = den;
        const float inv = 1.f / den;
        __nv_bfloat16* orow = const_cast<__nv_bfloat16*>(norm_row(p.x, b, h, tok));
        for (int c = sub * 8; c < dvp; c += lpr * 8) {
          const uint4 xv = *reinterpret_cast<const uint4*>(xt + i * dvp + c);
          const float2 x01 = bf2_to_f2(xv.x), x23 = bf2_to_f2(xv.y), x45 = bf2_to_f2(xv.z), x67 = bf2_to_f2(xv.w);
          uint4 ov;
          ov.x = f2_to_bf2(x01.x * inv, x01.y * inv);
          ov.y = f2_to_bf2(x23.x * inv, x23.y * inv);
          ov.z = f2_to_bf2(x45.x * inv, x45.y * inv);
          ov.w = f2_to_bf2(x67.x * inv, x67.y * inv);
          if (c + 7 < p.dv) {
            *reinterpret_cast<uint4*>(orow + c) = ov;
          } else {
            const __nv_bfloat16* vals = reinterpret_cast<const __nv_bfloat16*>(&ov);
            for (int j = 0; j < 8; ++j)
              if (c + j < p.dv) orow[c + j] = vals[j];
          }
        }
      }
    }
    __syncthreads();  // Z and this stage are rewritten by the next iterations
  }
  cp_async_wait<0>();
}

// Per row: dnum = g / den, dden = -(g . out) / den. Grid (blocks, batch*heads); `lpr` lanes share
// a row (8 columns per lane and step), the warps of a head's blocks stride over its tokens.
template <int D>
__global__ void __launch_bounds__(kNormThreads)
fla_normalize_bwd_prepare_kernel(const NormParams p_in) {
  NormParams p = p_in;
  if (D != 0) p.dk = p.dv = D;
  const int lane = threadIdx.x & 31;
  const int bh = blockIdx.y;
  const int b = bh / p.heads, h = bh % p.heads;
  const int dvp = (p.dv + 7) / 8 * 8;
  const int lpr = lanes_per_row(dvp);
  const int rpw = 32 / lpr;
  const int sub = lane % lpr, rsel = lane / lpr;
  const int warp0 = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const float* den = p.den + static_cast<size_t>(bh) * p.n;
  float* dden = p.dden + static_cast<size_t>(bh) * p.n;
  for (int tok0 = warp0 * rpw; tok0 < p.n; tok0 += nwarps * rpw) {
    const int tok = tok0 + rsel;
    const bool live = tok < p.n;
    const int tokc = live ? tok : p.n - 1;  // keep the whole warp in the shuffles
    const __nv_bfloat16* g = norm_row(p.x, b, h, tokc);
    const __nv_bfloat16* o = norm_row(p.y, b, h, tokc);
    __nv_bfloat16* dn = const_cast<__nv_bfloat16*>(norm_row(p.z, b, h, tokc));
    const float inv = 1.f / den[tokc];
    float acc = 0.f;
    for (int c = sub * 8; c < dvp; c += lpr * 8) {
      const uint4 gv = *reinterpret_cast<const uint4*>(g + c);
      const uint4 ov = *reinterpret_cast<const uint4*>(o + c);
      const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
      const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w};
      uint32_t res[4];
      if (c + 7 < p.dv) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 gg = bf2_to_f2(gw[j]), oo = bf2_to_f2(ow[j]);
          acc += gg.x * oo.x + gg.y * oo.y;
          res[j] = f2_to_bf2(gg.x * inv, gg.y * inv);
        }
        if (live) *reinterpret_cast<uint4*>(dn + c) = make_uint4(res[0], res[1], res[2], res[3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 gg = bf2_to_f2(gw[j]), oo = bf2_to_f2(ow[j]);
          const bool v0 = c + 2 * j < p.dv, v1 = c + 2 * j + 1 < p.dv;
          acc += (v0 ? gg.x * oo.x : 0.f) + (v1 ? gg.y * oo.y : 0.f);
          const __nv_bfloat162 r = __floats2bfloat162_rn(gg.x * inv, gg.y * inv);
          if (live && v0) dn[c + 2 * j] = r.x;
          if (live && v1) dn[c + 2 * j + 1] = r.y;
        }
      }
    }
    for (int o2 = lpr >> 1; o2 > 0; o2 >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o2);
    if (live && sub == 0) dden[tok] = -acc * inv;
  }
}

// Shared memory: kNormStages x ((src tile, dst tile) bf16 + T floats of dden)
__host__ __device__ inline size_t norm_sweep_smem_bytes(int dk, int tile) {
  const size_t dkp = (dk + 7) / 8 * 8;
  return kNormStages * (tile * 2 * dkp * 2 + tile * 4) + kNormThreads * 8;  // + group totals
}

// blockIdx.z = 0: ascending sweep, z += k_i, dQ_i += dden_i z   (z includes token i)
// blockIdx.z = 1: descending sweep, w += dden_i q_i, dK_i += w  (w includes token i)
template <int T, int D>
__global__ void __launch_bounds__(kNormThreads)
fla_normalize_bwd_sweep_kernel(const NormParams p_in) {
  constexpr int kNormTile = T;
  NormParams p = p_in;
  if (D != 0) p.dk = p.dv = D;
  extern __shared__ __align__(16) uint8_t norm_smem[];
  const int seg = blockIdx.x, bh = blockIdx.y;
  const bool rev = blockIdx.z == 1;
  const int b = bh / p.heads, h = bh % p.heads;
  const int dkp = (p.dk + 7) / 8 * 8;
  const NormTensor& src = rev ? p.q : p.k;
  const NormTensor& dst = rev ? p.dk_ : p.dq;
  const int stage_bytes = kNormTile * 2 * dkp * 2 + kNormTile * 4;
  const int seg_tok0 = seg * p.seg_len;
  const int seg_tokens = min(p.seg_len, p.n - seg_tok0);
  const int ntiles = (seg_tokens + kNormTile - 1) / kNormTile;
  auto tile_of = [&](int t) { return rev ? ntiles - 1 - t : t; };
  auto stage_ptr = [&](int t) { return norm_smem + static_cast<size_t>(t % kNormStages) * stage_bytes; };

  auto issue = [&](int t) {
    if (t < ntiles) {
      uint8_t* st = stage_ptr(t);
      __nv_bfloat16* s_src = reinterpret_cast<__nv_bfloat16*>(st);
      __nv_bfloat16* s_dst = s_src + kNormTile * dkp;
      float* s_dd = reinterpret_cast<float*>(st + kNormTile * 2 * dkp * 2);
      const int tok0 = seg_tok0 + tile_of(t) * kNormTile;
      norm_load_tile<T>(s_src, src, b, h, tok0, p.n, dkp);
      norm_load_tile<T>(s_dst, dst, b, h, tok0, p.n, dkp);
      if (threadIdx.x < kNormTile) {
        const int tok = tok0 + threadIdx.x;
        s_dd[threadIdx.x] = tok < p.n ? p.dden[static_cast<size_t>(bh) * p.n + tok] : 0.f;
      }
    }
    cp_async_commit();
  };
  issue(0);
  // One column pair per thread and one token group per thread (see ScanLayout). The running sums
  // start from the segments before (ascending) or after (descending) this one.
  const ScanLayout L = scan_layout<T>(dkp);
  const bool scan_active = L.grp < L.groups;
  const bool valid0 = 2 * L.cp < p.dk, valid1 = 2 * L.cp + 1 < p.dk;
  float2 run = make_float2(0.f, 0.f);
  const float* seg_sums = rev ? p.rsums : p.sums;
  if (seg_sums != nullptr && scan_active) {
    const int s_lo = rev ? seg + 1 : 0, s_hi = rev ? p.nseg : seg;
    for (int s2 = s_lo; s2 < s_hi; ++s2) {
      const float* sp = seg_sums + (static_cast<size_t>(bh) * p.nseg + s2) * p.dk;
      if (valid0) run.x += sp[2 * L.cp];
      if (valid1) run.y += sp[2 * L.cp + 1];
    }
  }
  float2* totals = reinterpret_cast<float2*>(norm_smem + static_cast<size_t>(kNormStages) * stage_bytes);
  for (int t = 0; t < ntiles; ++t) {
    issue(t + 1);
    cp_async_wait<1>();
    __syncthreads();
    uint8_t* st = stage_ptr(t);
    __nv_bfloat16* s_src = reinterpret_cast<__nv_bfloat16*>(st);
    __nv_bfloat16* s_dst = s_src + kNormTile * dkp;
    const float* s_dd = reinterpret_cast<const float*>(st + kNormTile * 2 * dkp * 2);
    // ---- group totals: sum of s (ascending) or of dden_i * s_i (descending) over the group
    if (scan_active) {
      float2 tot = make_float2(0.f, 0.f);
      for (int ii = 0; ii < L.gt; ++ii) {
        const int i = L.grp * L.gt + ii;
        const float2 sv = bf2_to_f2(*reinterpret_cast<const uint32_t*>(s_src + i * dkp + 2 * L.cp));
        const float w = rev ? s_dd[i] : 1.f;
        tot.x += valid0 ? w * sv.x : 0.f;
        tot.y += valid1 ? w * sv.y : 0.f;
      }
      totals[L.grp * L.pairs + L.cp] = tot;
    }
    __syncthreads();
    // ---- offsets of the groups processed earlier, then the group's own tokens in sweep order
    if (scan_active) {
      float2 acc = run, all = run;
      for (int g = 0; g < L.groups; ++g) {
        const float2 tg = totals[g * L.pairs + L.cp];
        const bool earlier = rev ? (g > L.grp) : (g < L.grp);
        if (earlier) { acc.x += tg.x; acc.y += tg.y; }
        all.x += tg.x; all.y += tg.y;
      }
      for (int ii = 0; ii < L.gt; ++ii) {
        const int i = L.grp * L.gt + (rev ? L.gt - 1 - ii : ii);
        const float2 sv = bf2_to_f2(*reinterpret_cast<const uint32_t*>(s_src + i * dkp + 2 * L.cp));
        const float dd = s_dd[i];
        float2 add;
        if (rev) {
          acc.x += valid0 ? dd * sv.x : 0.f;
          acc.y += valid1 ? dd * sv.y : 0.f;
          add = acc;
        } else {
          acc.x += valid0 ? sv.x : 0.f;
          acc.y += valid1 ? sv.y : 0.f;
          add = make_float2(dd * acc.x, dd * acc.y);
        }
        uint32_t* dp = reinterpret_cast<uint32_t*>(s_dst + i * dkp + 2 * L.cp);
        const float2 dv2 = bf2_to_f2(*dp);
        *dp = f2_to_bf2(dv2.x + add.x, dv2.y + add.y);
      }
      run = all;
    }
    __syncthreads();
    // write the updated tile back (16-byte pieces; the ragged last piece element by element)
    const int tok0 = seg_tok0 + tile_of(t) * kNormTile;
    const int pieces = dkp >> 3;
    for (int idx = threadIdx.x; idx < kNormTile * pieces; idx += kNormThreads) {
      const int r = idx / pieces;
      const int c = (idx - r * pieces) << 3;
      if (tok0 + r >= p.n) continue;
      __nv_bfloat16* grow = const_cast<__nv_bfloat16*>(norm_row(dst, b, h, tok0 + r)) + c;
      const __nv_bfloat16* srow = s_dst + r * dkp + c;
      if (c + 8 <= p.dk) {
        *reinterpret_cast<uint4*>(grow) = *reinterpret_cast<const uint4*>(srow);
      } else {
        for (int j = 0; c + j < p.dk; ++j) grow[j] = srow[j];
      }
    }
    __syncthreads();  // the stage is refilled by the next iteration's loads
  }
  cp_async_wait<0>();
}

}  // namespace fla
