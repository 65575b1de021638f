// C ABI of libflashlinear_sm100.so (declared in include/flashlinear_sm100.h).
//
// Forward and backward of causal linear attention are expressed with ONE device kernel,
// fla_chunk_kernel (fla_kernel.cuh), which computes  out_i = sum_{j<=i} (a_i . b_j) c_j  (or the
// anti-causal sum j>=i). With a=q, b=k, c=v this is the forward output
// (flashlinear/kernels/linear_attn_kernels.py:74-82); the gradients of
// flashlinear/kernels/linear_attn_kernels.py:179-197 and :291-299 are the same product with
// permuted operands:
//     dQ_i = sum_{j<=i} (dO_i . v_j) k_j      causal      (a=dO, b=v,  c=k)
//     dV_j = sum_{i>=j} (k_j . q_i) dO_i      anti-causal (a=k,  b=q,  c=dO)
//     dK_j = sum_{i>=j} (v_j . dO_i) q_i      anti-causal (a=v,  b=dO, c=q)
// dV and dK run side by side in one grid so that their shared reads of q and dO hit in L2.
#include "../../include/flashlinear_sm100.h"
#include "fla_kernel.cuh"
#include "fla_wide_kernel.cuh"
#include "fla_normalize.cuh"
#include "fla_taylor.cuh"

#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace {

using fla::KernelParams;
using fla::Problem;

#ifndef FLA_L2_PROMOTION
#define FLA_L2_PROMOTION CU_TENSOR_MAP_L2_PROMOTION_L2_256B
#endif

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static std::atomic<EncodeTiledFn> cached{nullptr};
  EncodeTiledFn fn = cached.load(std::memory_order_acquire);
  if (fn) return fn;
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) !=
          cudaSuccess ||
      qres != cudaDriverEntryPointSuccess || sym == nullptr) {
    return nullptr;
  }
  fn = reinterpret_cast<EncodeTiledFn>(sym);
  cached.store(fn, std::memory_order_release);
  return fn;
}

thread_local int g_last_launches = 0;
// Bounded-wait limit (units of 1024 SM cycles, 0 = default) and the wait-timeout test hook of the
// call in progress on this thread; check_common() sets them from FlaArgs.
thread_local unsigned g_wait_limit_us = 0;
thread_local int g_debug_withhold = 0;
thread_local int g_no_fused = 0;  // FLA_DEBUG_NO_FUSED_SEGMENTS: keep the three-launch segmented path
thread_local int g_force_single_sweep = 0;  // FLA_DEBUG_FORCE_SINGLE_SWEEP
thread_local int g_half = 0;  // FlaArgs::dtype == FLA_DTYPE_F16

// The single-sweep backward computes dQ as "total minus suffix": every chunk's own share comes out
// as the difference of two sums over the whole chunk, which costs the early rows of a chunk a few
// bf16 roundings of accuracy. Over a long sequence that vanishes against the prefix term; over a
// short one it can push dQ to the reference tests' bound (Frobenius 1e-2 against a bf16 naive
// path, flashlinear/test_attn.py:17,117). Sequences of at most this many 128-token chunks
// (the reference's tests stop at 1984 tokens, test_attn.py:69) therefore keep the two-direction form.
constexpr int kSingleSweepMinChunks = 17;
bool single_sweep_allowed(int nchunks) { return g_force_single_sweep || nchunks >= kSingleSweepMinChunks; }

// FLA_DEBUG=1 in the environment: failed CUDA calls are described on stderr.
bool debug_enabled() {
  static const bool on = [] {
    const char* e = getenv("FLA_DEBUG");
    return e != nullptr && e[0] == '1';
  }();
  return on;
}
#define FLA_LOG_FAILURE(...)                  \
  do {                                        \
    if (debug_enabled()) {                    \
      fprintf(stderr, "[flashlinear_sm100] "); \
      fprintf(stderr, __VA_ARGS__);           \
      fprintf(stderr, "\n");                  \
    }                                         \
  } while (0)

struct Operand {
  const void* ptr;
  int64_t sb, sh, sn;  // element strides
  int dim;             // valid head dim (columns beyond it read as zero / are not written)
};

Operand operand(const FlaTensor& t, int dim) {
  Operand o;
  o.ptr = t.ptr;
  o.sb = t.stride_b;
  o.sh = t.stride_h;
  o.sn = t.stride_n;
  o.dim = dim;
  return o;
}

int check_operand(const Operand& o, int B, int H) {
  if (o.ptr == nullptr) return FLA_ERR_INVALID;
  if (reinterpret_cast<uintptr_t>(o.ptr) % 16 != 0) return FLA_ERR_ALIGNMENT;
  if ((o.sn * 2) % 16 != 0 || o.sn < (o.dim + 7) / 8 * 8) return FLA_ERR_ALIGNMENT;
  if (H > 1 && (o.sh * 2) % 16 != 0) return FLA_ERR_ALIGNMENT;
  if (B > 1 && (o.sb * 2) % 16 != 0) return FLA_ERR_ALIGNMENT;
  return FLA_OK;
}

// 4-D tensor map (dim, token, head, batch); box = 64 columns x box_rows tokens, 128-byte swizzle.
// Columns >= dim and tokens >= N are out of bounds: loads fill zeros, stores skip them.
int encode_map(CUtensorMap* m, const Operand& o, int B, int H, int N, int box_rows = fla::kChunk) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return FLA_ERR_CUDA;
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(o.sn) * 2;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(o.dim), static_cast<cuuint64_t>(N),
                        static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(B)};
  // Strides of size-1 dimensions are never used for addressing but must still be valid.
  cuuint64_t sh = (H > 1) ? static_cast<cuuint64_t>(o.sh) * 2 : row_bytes * N;
  cuuint64_t sb = (B > 1) ? static_cast<cuuint64_t>(o.sb) * 2 : sh * H;
  cuuint64_t strides[3] = {row_bytes, sh, sb};
  cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(o.ptr), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  FLA_L2_PROMOTION, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    FLA_LOG_FAILURE("cuTensorMapEncodeTiled failed (%d): ptr %p dims %llu %llu %llu %llu strides %llu %llu %llu box %u",
                    static_cast<int>(r), o.ptr, (unsigned long long)dims[0], (unsigned long long)dims[1],
                    (unsigned long long)dims[2], (unsigned long long)dims[3], (unsigned long long)strides[0],
                    (unsigned long long)strides[1], (unsigned long long)strides[2], box[1]);
  return r == CUDA_SUCCESS ? FLA_OK : FLA_ERR_CUDA;
}

// One product out_i = sum (a_i . b_j) c_j; a, b have dim `da`, c and out have dim `dc`.
struct Product {
  Operand a, b, c, out;
  int flags;  // fla::kFlag* bits
  const float* ext_init;  // caller's running state, or null
  float* ext_final;
  int ext_trans;  // the caller's state arrays hold the transpose of the product's [da][dc] state
  // Fused segmented launch only. With bound_base set, segment 0 starts from ext_init and segment
  // g >= 1 from the stored boundary state (bound_slot0 - g * bound_step) of bound_base
  // ([bh][bound_stride][da*dc], layout flag bound_trans relative to this product's state) instead
  // of from the partial sums of the launch. bound_out: segments g >= 1 store the state they start
  // from ([bh][segments - 1][da*dc], scratch layout) for a later call to use as bound_base.
  const float* bound_base = nullptr;
  int bound_stride = 0, bound_slot0 = 0, bound_step = 0, bound_trans = 0;
  float* bound_out = nullptr;
};

// ---------------------------------------------------------------- segment state scan
// ws: [prob][bh][seg][cols][rows] holds per-segment sums on entry and, on exit, the exclusive
// prefix (in scan order) including the caller's initial state. The scratch keeps every state
// TRANSPOSED (column index slowest): the chunk kernel reads and writes states with one thread per
// row, so consecutive lanes then touch consecutive addresses.
struct ScanProblem {
  float* ws;
  const float* ext_init;
  float* ext_final;
  int ext_trans;
};
struct ScanParams {
  ScanProblem prob[3];
  int nseg, rows, cols, bh_count;
  int have_last;  // the last segment's sum is present (needed only for ext_final)
};

// Block = 32 x 32 threads on a 32 x 32 tile of the state: thread (tx, ty) scans element
// (row = row0 + tx, col = col0 + ty), so the scratch ([col][row]) is read and written along tx.
// The caller-layout arrays ([row][col], or the scratch layout when ext_trans) are touched through
// a shared-memory transpose, along tx as well: whole 128-byte segments instead of one word per line.
__global__ void __launch_bounds__(1024) fla_state_scan_kernel(const ScanParams sp) {
  __shared__ float tile[32][33];
  const ScanProblem pr = sp.prob[blockIdx.z];
  const int bh = blockIdx.y;
  const int elems = sp.rows * sp.cols;
  const int tiles_r = (sp.rows + 31) / 32;
  const int row0 = (blockIdx.x % tiles_r) * 32, col0 = (blockIdx.x / tiles_r) * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int row = row0 + tx, col = col0 + ty;
  const bool valid = row < sp.rows && col < sp.cols;
  const size_t ext_base = static_cast<size_t>(bh) * elems;
  // element this thread moves for the caller-layout arrays: (row0 + ty, col0 + tx)
  const int trow = row0 + ty, tcol = col0 + tx;
  const bool tvalid = trow < sp.rows && tcol < sp.cols;
  float run = 0.f;
  if (pr.ext_init != nullptr) {
    if (pr.ext_trans) {
      if (valid) run = pr.ext_init[ext_base + static_cast<size_t>(col) * sp.rows + row];
    } else {
      tile[ty][tx] = tvalid ? pr.ext_init[ext_base + static_cast<size_t>(trow) * sp.cols + tcol] : 0.f;
      __syncthreads();
      run = tile[tx][ty];
      __syncthreads();
    }
  }
  if (valid) {
    float* __restrict__ base = pr.ws + static_cast<size_t>(bh) * sp.nseg * elems +
                               static_cast<size_t>(col) * sp.rows + row;
    const int npresent = sp.have_last ? sp.nseg : sp.nseg - 1;  // segments whose sum was written
    // Batches of 8 segments: all loads of a batch are issued before the dependent stores.
    for (int g0 = 0; g0 < sp.nseg; g0 += 8) {
      float local[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int g = g0 + j;
        local[j] = (g < npresent) ? __ldcg(base + static_cast<size_t>(g) * elems) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int g = g0 + j;
        if (g < sp.nseg) {
          base[static_cast<size_t>(g) * elems] = run;
          run += local[j];
        }
      }
    }
  }
  if (pr.ext_final != nullptr) {
    if (pr.ext_trans) {
      if (valid) pr.ext_final[ext_base + static_cast<size_t>(col) * sp.rows + row] = run;
    } else {
      tile[ty][tx] = run;
      __syncthreads();
      if (tvalid) pr.ext_final[ext_base + static_cast<size_t>(trow) * sp.cols + tcol] = tile[tx][ty];
    }
  }
}

// ---------------------------------------------------------------- scan fused with the exchange
// Sequence sharding: the segment scan of one rank, the transfer of its total to every peer GPU
// (stores into peer-mapped memory over NVLink), the bounded wait for the peers' totals and the
// addition of the ones that precede (follow) this rank, all in one kernel. See FlaExchange in the
// header. Inbox layout: [parity][source rank][bh][elems] (scratch layout), flags
// [parity][source rank][block]; parity = epoch & 1.
struct ExchangeParams {
  float* ws;
  int nseg, rows, cols, bh_count;
  int rank, world, reverse;
  unsigned epoch;
  float* inbox[FLA_MAX_RANKS];
  unsigned* flags[FLA_MAX_RANKS];
  float* remote_out;
  float* inclusive_out;
  int* status;
  const unsigned* epoch_counter;  // device-side count (epoch = *epoch_counter + 1), or null
  unsigned long long wait_limit_ns;  // how long a block waits for a peer's flag
};

// Stores the epoch an exchange kernel just used back into its device-side counter.
__global__ void fla_exchange_bump_kernel(unsigned* counter) { *counter = *counter + 1u; }

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Every thread handles the elements e0, e0 + stride, ... of one head (stride = threads of the
// head's blocks), so that a few hundred blocks cover the state and each pays the system-scope
// fence and the flag round trip once.
__global__ void fla_state_exchange_kernel(const ExchangeParams xp) {
  const int bh = blockIdx.y;
  const int elems = xp.rows * xp.cols;
  const int e0 = blockIdx.x * blockDim.x + threadIdx.x;
  const int stride = gridDim.x * blockDim.x;
  // every block reads the same count: it only changes in the one-thread kernel behind this one
  const unsigned epoch = xp.epoch_counter != nullptr ? __ldcg(xp.epoch_counter) + 1u : xp.epoch;
  const unsigned parity = epoch & 1u;
  const size_t nblocks = static_cast<size_t>(gridDim.x) * gridDim.y;
  const size_t block_id = static_cast<size_t>(bh) * gridDim.x + blockIdx.x;
  const size_t state_elems = static_cast<size_t>(xp.bh_count) * elems;
  float* head_ws = xp.ws + static_cast<size_t>(bh) * xp.nseg * elems;

  // 1. this rank's total over its segments, 2. published with one store per peer into that peer's
  //    inbox slot for this rank
  for (int e = e0; e < elems; e += stride) {
    float total = 0.f;
    for (int g = 0; g < xp.nseg; ++g) total += __ldcg(head_ws + static_cast<size_t>(g) * elems + e);
    const size_t slot = (static_cast<size_t>(parity) * xp.world + xp.rank) * state_elems +
                        static_cast<size_t>(bh) * elems + e;
    for (int d = 0; d < xp.world; ++d)
      if (d != xp.rank) xp.inbox[d][slot] = total;
  }
  // Every thread waits for its own stores to be performed at system scope (so that the waits for
  // the NVLink acknowledgements run side by side, not one after the other in the flag writers);
  // then thread d raises this block's flag in peer d's inbox with a RELEASE store: the barrier
  // puts the whole block's stores before it, and the release is what carries them to the peer's
  // acquire load (a fence that thread d executed before the barrier would not cover the other
  // threads' stores). The flag stores of all peers are in flight together.
  __threadfence_system();
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < xp.world && static_cast<int>(threadIdx.x) != xp.rank) {
    const size_t f = (static_cast<size_t>(parity) * xp.world + xp.rank) * nblocks + block_id;
    st_release_sys(xp.flags[threadIdx.x] + f, epoch);
  }
  // 3. wait (bounded) for the same block of every other rank. Waiting for all of them, not only the
  //    ones whose totals are needed, keeps any rank from running two exchanges ahead of another,
  //    which is what makes two parity buffers enough.
  __shared__ int timed_out;
  if (threadIdx.x == 0) timed_out = 0;
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < xp.world && static_cast<int>(threadIdx.x) != xp.rank) {
    const unsigned* f = xp.flags[xp.rank] +
                        (static_cast<size_t>(parity) * xp.world + threadIdx.x) * nblocks + block_id;
    const unsigned long long t0 = globaltimer_ns();
    unsigned spins = 0;
    while (ld_acquire_sys(f) != epoch) {
      if ((++spins & 15u) == 0u && globaltimer_ns() - t0 > xp.wait_limit_ns) {
        timed_out = 1;
        break;
      }
    }
  }
  __syncthreads();
  const bool failed = timed_out != 0;
  if (failed && threadIdx.x == 0 && xp.status != nullptr) atomicOr(xp.status, 2);
  // A wait that ran out must not leave plausible numbers behind: everything this block would have
  // produced becomes NaN, so the outputs of the passes built on it are NaN too and the failure shows
  // even where nobody reads the status word.
  const float poison = __int_as_float(0x7fc00000);
  const int lo = xp.reverse ? xp.rank + 1 : 0;
  const int hi = xp.reverse ? xp.world : xp.rank;
  for (int e = e0; e < elems; e += stride) {
    // 4. totals of the ranks before (after) this one, from this GPU's own inbox
    float remote = failed ? poison : 0.f;
    if (!failed) {
      for (int s = lo; s < hi; ++s)
        remote += __ldcg(xp.inbox[xp.rank] + (static_cast<size_t>(parity) * xp.world + s) * state_elems +
                         static_cast<size_t>(bh) * elems + e);
    }
    // 5. segment prefixes on top of it
    float run = remote;
    for (int g = 0; g < xp.nseg; ++g) {
      float* p = head_ws + static_cast<size_t>(g) * elems + e;
      const float local = __ldcg(p);
      *p = run;
      run += local;
    }
    const int col = e / xp.rows, row = e % xp.rows;  // scratch layout [col][row] -> caller [row][col]
    const size_t ext_idx = static_cast<size_t>(bh) * elems + static_cast<size_t>(row) * xp.cols + col;
    if (xp.remote_out) xp.remote_out[ext_idx] = remote;
    if (xp.inclusive_out) xp.inclusive_out[ext_idx] = run;
  }
}

// ---------------------------------------------------------------- row padding
// TMA needs 16-byte row strides, which a contiguous bf16 tensor with an odd head dim (273-dim
// Taylor features) does not have. These two kernels copy between rows of d elements and rows of
// dpad elements (dpad a multiple of 8); both sides contiguous.
//
// Both kernels give every block a run of kPadRowsPerBlock rows, so that all index arithmetic
// inside a block is 32-bit.
constexpr int kPadRowsPerBlock = 32;

// Pad: one thread per 16-byte piece of the destination; the (up to) 8 source elements start at an
// arbitrary 2-byte offset, so they are fetched as aligned 32-bit words and shifted.
__global__ void fla_pad_rows_kernel(const uint32_t* __restrict__ src, uint4* __restrict__ dst,
                                    long long rows, int d, int dpad) {
  const int pieces = dpad >> 3;
  for (long long blk = blockIdx.x; blk * kPadRowsPerBlock < rows; blk += gridDim.x) {
    const long long row0 = blk * kPadRowsPerBlock;
    const int nrows = static_cast<int>(min(static_cast<long long>(kPadRowsPerBlock), rows - row0));
    // the block's source elements start at element row0 * d (an even number: 32 rows per block)
    const uint32_t* bsrc = src + ((row0 * d) >> 1);
    uint4* bdst = dst + row0 * pieces;
    const int total = nrows * pieces;
    for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
      const int r = idx / pieces;
      const int c0 = (idx - r * pieces) * 8;
      const int valid = min(8, d - c0);  // <= 0: the piece is all padding
      uint32_t w[5] = {0u, 0u, 0u, 0u, 0u};
      uint32_t out[4] = {0u, 0u, 0u, 0u};
      if (valid > 0) {
        const int e0 = r * d + c0;  // first source element, relative to the block
        const int w0 = e0 >> 1;
        const int odd = e0 & 1;
        const int nwords = (odd + valid + 1) >> 1;
#pragma unroll
        for (int j = 0; j < 5; ++j)
          if (j < nwords) w[j] = bsrc[w0 + j];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t x = odd ? __funnelshift_r(w[j], w[j + 1], 16) : w[j];
          const int left = valid - 2 * j;  // elements of this word that are inside the row
          if (left <= 0) x = 0u;
          else if (left == 1) x &= 0xFFFFu;
          out[j] = x;
        }
      }
      bdst[idx] = make_uint4(out[0], out[1], out[2], out[3]);
    }
  }
}

// Unpad: one thread per 32-bit word of the destination (two elements, possibly of two rows).
__global__ void fla_unpad_rows_kernel(const unsigned short* __restrict__ src,
                                      unsigned short* __restrict__ dst, long long rows, int d,
                                      int dpad) {
  for (long long blk = blockIdx.x; blk * kPadRowsPerBlock < rows; blk += gridDim.x) {
    const long long row0 = blk * kPadRowsPerBlock;
    const int nrows = static_cast<int>(min(static_cast<long long>(kPadRowsPerBlock), rows - row0));
    const unsigned short* bsrc = src + row0 * dpad;
    unsigned short* bdst = dst + row0 * d;  // 4-byte aligned: 32 rows per block
    const int total_elems = nrows * d;
    const int total = (total_elems + 1) >> 1;
    for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
      const int e0 = idx * 2;
      const int r0 = e0 / d;
      const int c0 = e0 - r0 * d;
      const uint32_t lo = bsrc[r0 * dpad + c0];
      if (e0 + 1 < total_elems) {
        const int r1 = (c0 + 1 < d) ? r0 : r0 + 1;
        const int c1 = (c0 + 1 < d) ? c0 + 1 : 0;
        const uint32_t hi = bsrc[r1 * dpad + c1];
        reinterpret_cast<uint32_t*>(bdst)[idx] = lo | (hi << 16);
      } else {
        bdst[e0] = static_cast<unsigned short>(lo);
      }
    }
  }
}

// ---------------------------------------------------------------- launch plumbing
struct DeviceInfo {
  int sm_count;
  int cc_major;
  int clock_khz;  // nominal SM clock, converts FlaArgs::wait_limit_us to cycles
  bool attr_set[2];
};

int device_info(DeviceInfo** out) {
  static DeviceInfo infos[64];
  static std::atomic<int> ready[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    FLA_LOG_FAILURE("cudaGetDevice failed or device index %d out of range", dev);
    return FLA_ERR_CUDA;
  }
  // Bind the device's primary context to THIS thread: cuTensorMapEncodeTiled is a driver call and
  // needs a current context, which a thread that has only inherited the device index (an
  // autograd worker, for one) does not have yet.
  if (cudaSetDevice(dev) != cudaSuccess) {
    FLA_LOG_FAILURE("cudaSetDevice(%d) failed", dev);
    return FLA_ERR_CUDA;
  }
  if (ready[dev].load(std::memory_order_acquire) != 2) {
    int expected = 0;
    if (ready[dev].compare_exchange_strong(expected, 1)) {
      DeviceInfo& d = infos[dev];
      d.sm_count = 148;
      d.cc_major = 0;
      d.clock_khz = 1965000;
      cudaDeviceGetAttribute(&d.clock_khz, cudaDevAttrClockRate, dev);
      cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
      cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
      bool ok = true;
      ok &= cudaFuncSetAttribute(fla::fla_chunk_kernel<64, 64>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 fla::Cfg<64, 64>::SMEM_BYTES) == cudaSuccess;
      ok &= cudaFuncSetAttribute(fla::fla_chunk_kernel<128, 128>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 fla::Cfg<128, 128>::SMEM_BYTES) == cudaSuccess;
      ok &= cudaFuncSetAttribute(fla::fla_chunk_kernel<64, 64, true>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 fla::Cfg<64, 64>::SMEM_BYTES) == cudaSuccess;
      ok &= cudaFuncSetAttribute(fla::fla_chunk_kernel<128, 128, true>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 fla::Cfg<128, 128>::SMEM_BYTES) == cudaSuccess;
      ok &= cudaFuncSetAttribute(fla::fla_wide_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 fla::WideCfg<2>::SMEM_BYTES) == cudaSuccess;
      ok &= cudaFuncSetAttribute(fla::fla_wide_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 fla::WideCfg<3>::SMEM_BYTES) == cudaSuccess;
      constexpr int kMaxSmem = 232448;
      auto big_smem = [&](const void* fn) {
        ok &= cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem) == cudaSuccess;
      };
      big_smem(reinterpret_cast<const void*>(fla::fla_normalize_fwd_kernel<32, 0>));
      big_smem(reinterpret_cast<const void*>(fla::fla_normalize_fwd_kernel<32, 64>));
      big_smem(reinterpret_cast<const void*>(fla::fla_normalize_fwd_kernel<32, 128>));
      big_smem(reinterpret_cast<const void*>(fla::fla_normalize_fwd_kernel<16, 0>));
      big_smem(reinterpret_cast<const void*>(fla::fla_normalize_bwd_sweep_kernel<32, 0>));
      big_smem(reinterpret_cast<const void*>(fla::fla_normalize_bwd_sweep_kernel<32, 64>));
      big_smem(reinterpret_cast<const void*>(fla::fla_normalize_bwd_sweep_kernel<32, 128>));
      big_smem(reinterpret_cast<const void*>(fla::fla_normalize_bwd_sweep_kernel<16, 0>));
      d.attr_set[0] = d.attr_set[1] = ok;
      ready[dev].store(2, std::memory_order_release);
    } else {
      while (ready[dev].load(std::memory_order_acquire) != 2) {
      }
    }
  }
  *out = &infos[dev];
  return FLA_OK;
}

int pick_template(int da, int dc) {
  const int m = da > dc ? da : dc;
  if (m <= 64) return 64;
  if (m <= 128) return 128;
  return 0;
}

int current_sm_count_early() {
  int sm = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev);
  return sm;
}

int auto_segments(int nprob, int bh, int nchunks, int sm_count) {
  const long ctas = static_cast<long>(nprob) * bh;
  if (ctas * 4 >= static_cast<long>(sm_count) * 3) return 1;  // already >= 75 % of the SMs
  // One wave: as many segments as fit the SMs once (every CTA pays a fixed start-up cost, and the
  // state pass re-reads b and c, so more, shorter segments do not pay).
  int want = static_cast<int>(sm_count / ctas);
  int max_seg = nchunks / 2;  // at least two chunks per segment
  if (max_seg < 1) max_seg = 1;
  if (want > max_seg) want = max_seg;
  if (want < 1) want = 1;
  // make segments equal: seg_chunks = ceil(nchunks / want), then recompute the count
  const int seg_chunks = (nchunks + want - 1) / want;
  return (nchunks + seg_chunks - 1) / seg_chunks;
}

// Floats one state takes in the scratch of a segmented call: the fused form stores states padded
// to the kernel's tile (64 x 64 or 128 x 128), whatever the head dims are.
size_t scratch_state_elems(int rows, int cols) {
  const int t = pick_template(rows, cols);
  return t > 0 ? static_cast<size_t>(t) * t : static_cast<size_t>(rows) * cols;
}

size_t segment_ws_bytes(int nprob, int bh, int nseg, int rows, int cols) {
  if (nseg <= 1) return 0;
  return static_cast<size_t>(nprob) * bh * nseg * scratch_state_elems(rows, cols) * sizeof(float);
}

struct SegPlan {
  int nseg;
  int seg_chunks;
};

SegPlan make_plan(int want, int nchunks) {
  if (want > nchunks) want = nchunks;
  if (want < 1) want = 1;
  SegPlan p;
  p.seg_chunks = (nchunks + want - 1) / want;
  p.nseg = (nchunks + p.seg_chunks - 1) / p.seg_chunks;
  return p;
}

// Segments of a forward call (one product per head).
SegPlan forward_plan(const FlaArgs* a, int sm_count) {
  const int nchunks = (a->seqlen + fla::kChunk - 1) / fla::kChunk;
  const int want = a->segments > 0 ? a->segments : auto_segments(1, a->batch * a->heads, nchunks, sm_count);
  SegPlan p = make_plan(want, nchunks);
  if (a->segments <= 0 && p.nseg > 1 && nchunks % p.seg_chunks != 0) {
    // An automatic split prefers equal segments (up to a quarter longer than the even share): the
    // backward can then be cut at a subset of the forward's boundaries and start from its states.
    for (int d = p.seg_chunks + 1; d <= p.seg_chunks + p.seg_chunks / 4; ++d) {
      if (nchunks % d == 0) {
        p.seg_chunks = d;
        p.nseg = nchunks / d;
        break;
      }
    }
  }
  return p;
}

// Segments of a backward call (three products per head) whose boundaries are boundaries of the
// forward plan `f`, so that the states the forward stored at its boundaries can start dQ's
// segments. nseg = 1 when no such plan exists or the backward would not be split anyway.
SegPlan backward_aligned_plan(const FlaArgs* a, int sm_count, const SegPlan& f) {
  const int nchunks = (a->seqlen + fla::kChunk - 1) / fla::kChunk;
  const int bh = a->batch * a->heads;
  const SegPlan none = {1, nchunks};
  const SegPlan base = make_plan(auto_segments(3, bh, nchunks, sm_count), nchunks);
  if (base.nseg <= 1 || f.nseg <= 1 || nchunks % f.seg_chunks != 0) return none;
  SegPlan b;
  b.seg_chunks = (base.seg_chunks + f.seg_chunks - 1) / f.seg_chunks * f.seg_chunks;
  b.nseg = (nchunks + b.seg_chunks - 1) / b.seg_chunks;
  if (b.nseg <= 1 || 3l * b.nseg * bh > sm_count) return none;
  return b;
}

// Bytes of the boundary states a fused forward stores for a fused backward, or 0 when the pair of
// calls does not run that way for these shapes.
size_t seg_states_bytes(const FlaArgs* a, int sm_count, SegPlan* fwd_out, SegPlan* bwd_out) {
  if (a->dk != a->dv || a->dk > 128 || g_no_fused) return 0;
  if (!single_sweep_allowed((a->seqlen + fla::kChunk - 1) / fla::kChunk)) return 0;
  const int bh = a->batch * a->heads;
  const SegPlan f = forward_plan(a, sm_count);
  if (f.nseg <= 1 || static_cast<long>(f.nseg) * bh > sm_count || bh > fla::kBarHeads) return 0;
  const SegPlan b = backward_aligned_plan(a, sm_count, f);
  if (b.nseg <= 1) return 0;
  if (fwd_out) *fwd_out = f;
  if (bwd_out) *bwd_out = b;
  return static_cast<size_t>(f.nseg - 1) * bh * scratch_state_elems(a->dk, a->dv) * sizeof(float);
}

template <int D>
int launch_kernel(const KernelParams& kp_in, dim3 grid, cudaStream_t stream) {
  KernelParams kp = kp_in;
  kp.wait_limit_us = g_wait_limit_us;
  kp.debug_withhold = g_debug_withhold;
  if (g_half)
    fla::fla_chunk_kernel<D, D, true><<<grid, fla::kThreads, fla::Cfg<D, D>::SMEM_BYTES, stream>>>(kp);
  else
    fla::fla_chunk_kernel<D, D><<<grid, fla::kThreads, fla::Cfg<D, D>::SMEM_BYTES, stream>>>(kp);
  ++g_last_launches;
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    FLA_LOG_FAILURE("launch of fla_chunk_kernel<%d> grid (%u,%u,%u) failed: %s", D, grid.x, grid.y,
                    grid.z, cudaGetErrorString(e));
  return e == cudaSuccess ? FLA_OK : FLA_ERR_CUDA;
}

int launch_template(int tmpl, const KernelParams& kp, dim3 grid, cudaStream_t stream) {
  if (tmpl == 64) return launch_kernel<64>(kp, grid, stream);
  if (tmpl == 128) return launch_kernel<128>(kp, grid, stream);
  return FLA_ERR_UNSUPPORTED;
}

// Which set of barrier words the next fused launch of this process gets (round-robin).
std::atomic<unsigned> g_next_barrier_slot{0};

// Cooperative launch (all CTAs resident at once, or the launch fails) of the fused segmented form.
template <int D>
int launch_fused_kernel(const KernelParams& kp_in, dim3 grid, cudaStream_t stream) {
  KernelParams kp = kp_in;
  kp.wait_limit_us = g_wait_limit_us;
  kp.debug_withhold = g_debug_withhold;
  kp.bar_slot = g_next_barrier_slot.fetch_add(1, std::memory_order_relaxed) % fla::kGridBarSlots;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = dim3(fla::kThreads, 1, 1);
  cfg.dynamicSmemBytes = fla::Cfg<D, D>::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  memset(&attr, 0, sizeof(attr));
  attr.id = cudaLaunchAttributeCooperative;
  attr.val.cooperative = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  const cudaError_t e = g_half ? cudaLaunchKernelEx(&cfg, fla::fla_chunk_kernel<D, D, true>, kp)
                               : cudaLaunchKernelEx(&cfg, fla::fla_chunk_kernel<D, D, false>, kp);
  ++g_last_launches;
  if (e != cudaSuccess) {
    FLA_LOG_FAILURE("cooperative launch of fla_chunk_kernel<%d> grid (%u,%u,%u) failed: %s", D, grid.x,
                    grid.y, grid.z, cudaGetErrorString(e));
    (void)cudaGetLastError();
  }
  return e == cudaSuccess ? FLA_OK : FLA_ERR_CUDA;
}

int launch_fused(int tmpl, const KernelParams& kp, dim3 grid, cudaStream_t stream) {
  if (tmpl == 64) return launch_fused_kernel<64>(kp, grid, stream);
  if (tmpl == 128) return launch_fused_kernel<128>(kp, grid, stream);
  return FLA_ERR_UNSUPPORTED;
}

// Runs `nprob` products that share shapes (da, dc) in one grid (plus, with segments, a state pass
// and a scan before it).
// `seg_chunks_in` > 0 fixes the segment length (in chunks) instead of deriving it from `segments`.
int run_products(const Product* prods, int nprob, int B, int H, int N, int da, int dc,
                 int segments, void* workspace, size_t workspace_bytes, int32_t* status,
                 cudaStream_t stream, const DeviceInfo& dev, bool states_ready = false,
                 int seg_chunks_in = 0) {
  const int tmpl = pick_template(da, dc);
  if (tmpl == 0) return FLA_ERR_UNSUPPORTED;
  const int bh = B * H;
  const int nchunks = (N + fla::kChunk - 1) / fla::kChunk;
  int nseg = segments;
  if (nseg <= 0) nseg = auto_segments(nprob, bh, nchunks, dev.sm_count);
  if (nseg > nchunks) nseg = nchunks;
  const int seg_chunks = seg_chunks_in > 0 ? seg_chunks_in : (nchunks + nseg - 1) / nseg;
  nseg = (nchunks + seg_chunks - 1) / seg_chunks;
  const size_t ws_per_prob = static_cast<size_t>(bh) * nseg * da * dc;
  if (nseg > 1) {
    if (workspace == nullptr || workspace_bytes < segment_ws_bytes(nprob, bh, nseg, da, dc))
      return FLA_ERR_WORKSPACE;
  }

  KernelParams kp;
  memset(&kp, 0, sizeof(kp));
  kp.heads = H;
  kp.nchunks = nchunks;
  kp.seg_chunks = seg_chunks;
  kp.st_rows = da;
  kp.st_cols = dc;
  kp.status = status;
  bool want_final = false;
  for (int i = 0; i < nprob; ++i) {
    const Product& pd = prods[i];
    int rc;
    if ((rc = check_operand(pd.a, B, H)) || (rc = check_operand(pd.b, B, H)) ||
        (rc = check_operand(pd.c, B, H)) || (rc = check_operand(pd.out, B, H)))
      return rc;
    Problem& pr = kp.prob[i];
    if ((rc = encode_map(&pr.q, pd.a, B, H, N)) || (rc = encode_map(&pr.k, pd.b, B, H, N)) ||
        (rc = encode_map(&pr.v, pd.c, B, H, N)) || (rc = encode_map(&pr.o, pd.out, B, H, N, 32)))
      return rc;
    pr.flags = pd.flags;
    pr.n_tokens = N;
    want_final |= (pd.ext_final != nullptr);
  }

  if (states_ready) {
    // The caller ran the state pass already (fla_sm100_state / fla_sm100_state_exchange): the
    // workspace holds the segment prefixes of these tokens, in the scratch layout; the caller's
    // initial state, if any, is added for every segment.
    if (nprob != 1 || prods[0].ext_final != nullptr) return FLA_ERR_INVALID;
    if (workspace == nullptr ||
        workspace_bytes < static_cast<size_t>(bh) * nseg * da * dc * sizeof(float))
      return FLA_ERR_WORKSPACE;
    kp.prob[0].s_init = static_cast<float*>(workspace);
    kp.prob[0].s_final = nullptr;
    kp.prob[0].st_trans = 1;
    kp.prob[0].s_add = prods[0].ext_init;
    kp.prob[0].add_trans = prods[0].ext_trans;
    kp.mode = 0;
    return launch_template(tmpl, kp, dim3(1, nseg, bh), stream);
  }

  if (nseg == 1) {
    for (int i = 0; i < nprob; ++i) {
      kp.prob[i].s_init = prods[i].ext_init;
      kp.prob[i].s_final = prods[i].ext_final;
      kp.prob[i].st_trans = prods[i].ext_trans;
    }
    kp.mode = 0;
    return launch_template(tmpl, kp, dim3(nprob, 1, bh), stream);
  }

  float* ws = static_cast<float*>(workspace);
  // The fused form sums ONE state per (head, segment). Products that start from the partial sums
  // must therefore all carry that state or its transpose (dV and dK: q^T dO and dO^T q) and walk
  // the sequence in the same direction; a product with another state (dQ: v^T k) can only ride
  // along when its starting states come from stored boundary states.
  bool fusable = !g_no_fused && static_cast<long>(nprob) * nseg * bh <= dev.sm_count && bh <= fla::kBarHeads;
  {
    const Product* first = nullptr;
    for (int i = 0; i < nprob && fusable; ++i) {
      const Product& pd = prods[i];
      if (pd.bound_base != nullptr) continue;
      if (first == nullptr) {
        first = &pd;
        continue;
      }
      const bool same = pd.b.ptr == first->b.ptr && pd.c.ptr == first->c.ptr && pd.ext_trans == first->ext_trans;
      const bool swapped = pd.b.ptr == first->c.ptr && pd.c.ptr == first->b.ptr && pd.ext_trans != first->ext_trans;
      const bool same_dir = ((pd.flags ^ first->flags) & fla::kFlagDescending) == 0;
      if (!(same || swapped) || !same_dir || da != dc) fusable = false;
    }
    if (first == nullptr) fusable = false;
  }
  if (fusable) {
    // Everything fits the GPU at once: ONE cooperative launch in which every CTA sums its share of
    // its segment (phase A), all CTAs meet at a grid barrier, and each then starts the attention
    // loop from the sum of the partials of the earlier segments. The three-launch form below pays
    // the pipeline fill and drain of a launch three times and reads b, c once more from HBM.
    int pre = 0;
    for (int i = 0; i < nprob; ++i) {
      Problem& pr = kp.prob[i];
      const Product& pd = prods[i];
      pr.s_init = nullptr;
      pr.s_add = pd.ext_init;
      pr.add_trans = pd.ext_trans;
      pr.s_final = pd.ext_final;   // written by the last segment's CTA
      pr.st_trans = pd.ext_trans;
      if (pd.bound_base != nullptr) {
        pr.init_kind = fla::kInitBound;
        pr.init_base = pd.bound_base;
        pr.init_trans = pd.bound_trans;
        pr.init_stride = pd.bound_stride;
        pr.bound_slot0 = pd.bound_slot0;
        pr.bound_step = pd.bound_step;
      } else {
        pr.init_kind = fla::kInitParts;
        pr.init_base = ws;
        // The partials hold the state of problem `pre` in the scratch layout; a problem whose own
        // state is the transpose of that one (dK beside dV) reads them the other way round.
        pre = i;
      }
      pr.bound_out = pd.bound_out;
    }
    // `pre`: the (last) problem that starts from partial sums; its b, c operands and direction
    // define phase A. Problems with the transposed state read the partials transposed.
    for (int i = 0; i < nprob; ++i)
      if (kp.prob[i].init_kind == fla::kInitParts)
        kp.prob[i].init_trans = (prods[i].ext_trans == prods[pre].ext_trans) ? 1 : 0;
    kp.mode = 0;
    kp.fused = 1;
    kp.pre_prob = pre;
    kp.part_out = ws;
    return launch_fused(tmpl, kp, dim3(nprob, nseg, bh), stream);
  }
  // Pass A: per-segment sums of b^T c into the workspace (the last segment only when a final
  // state is wanted), exclusive scan over segments, then pass B with per-segment initial states.
  ScanParams sp;
  memset(&sp, 0, sizeof(sp));
  for (int i = 0; i < nprob; ++i) {
    kp.prob[i].s_init = nullptr;
    kp.prob[i].s_final = ws + i * ws_per_prob;
    kp.prob[i].st_trans = 1;  // scratch layout, see fla_state_scan_kernel
    sp.prob[i].ws = ws + i * ws_per_prob;
    sp.prob[i].ext_init = prods[i].ext_init;
    sp.prob[i].ext_final = prods[i].ext_final;
    sp.prob[i].ext_trans = prods[i].ext_trans;
  }
  kp.mode = 1;
  kp.skip_last_segment = want_final ? 0 : 1;
  int rc = launch_template(tmpl, kp, dim3(nprob, nseg, bh), stream);
  if (rc) return rc;
  sp.nseg = nseg;
  sp.rows = da;
  sp.cols = dc;
  sp.bh_count = bh;
  sp.have_last = want_final ? 1 : 0;
  {
    dim3 grid(((da + 31) / 32) * ((dc + 31) / 32), bh, nprob);
    fla_state_scan_kernel<<<grid, dim3(32, 32, 1), 0, stream>>>(sp);
    ++g_last_launches;
    if (cudaGetLastError() != cudaSuccess) return FLA_ERR_CUDA;
  }
  for (int i = 0; i < nprob; ++i) {
    kp.prob[i].s_init = ws + i * ws_per_prob;
    kp.prob[i].s_final = nullptr;
  }
  kp.mode = 0;
  kp.skip_last_segment = 0;
  return launch_template(tmpl, kp, dim3(nprob, nseg, bh), stream);
}

// Sum over all tokens of b^T c (fp32, [bh][da][dc]) into `final`: the per-shard state that
// sequence-sharded callers exchange between GPUs. Uses segments to fill the GPU when bh is small.
int run_state(const Operand& bop, const Operand& cop, int B, int H, int N, int da, int dc,
              int segments, float* final, void* workspace, size_t workspace_bytes,
              int32_t* status, cudaStream_t stream, const DeviceInfo& dev) {
  const int tmpl = pick_template(da, dc);
  if (tmpl == 0) return FLA_ERR_UNSUPPORTED;
  if (final == nullptr) return FLA_ERR_INVALID;
  const int bh = B * H;
  const int nchunks = (N + fla::kChunk - 1) / fla::kChunk;
  int nseg = segments;
  if (nseg <= 0) nseg = auto_segments(1, bh, nchunks, dev.sm_count);
  if (nseg > nchunks) nseg = nchunks;
  const int seg_chunks = (nchunks + nseg - 1) / nseg;
  nseg = (nchunks + seg_chunks - 1) / seg_chunks;
  if (nseg > 1 &&
      (workspace == nullptr || workspace_bytes < segment_ws_bytes(1, bh, nseg, da, dc)))
    return FLA_ERR_WORKSPACE;
  int rc;
  if ((rc = check_operand(bop, B, H)) || (rc = check_operand(cop, B, H))) return rc;
  KernelParams kp;
  memset(&kp, 0, sizeof(kp));
  kp.heads = H;
  kp.nchunks = nchunks;
  kp.seg_chunks = seg_chunks;
  kp.st_rows = da;
  kp.st_cols = dc;
  kp.status = status;
  kp.mode = 1;
  if ((rc = encode_map(&kp.prob[0].k, bop, B, H, N)) || (rc = encode_map(&kp.prob[0].v, cop, B, H, N)))
    return rc;
  kp.prob[0].s_final = (nseg == 1) ? final : static_cast<float*>(workspace);
  kp.prob[0].st_trans = (nseg == 1) ? 0 : 1;  // the scratch keeps states transposed
  rc = launch_template(tmpl, kp, dim3(1, nseg, bh), stream);
  if (rc || nseg == 1) return rc;
  ScanParams sp;
  memset(&sp, 0, sizeof(sp));
  sp.prob[0].ws = static_cast<float*>(workspace);
  sp.prob[0].ext_final = final;
  sp.nseg = nseg;
  sp.rows = da;
  sp.cols = dc;
  sp.bh_count = bh;
  sp.have_last = 1;
  fla_state_scan_kernel<<<dim3(((da + 31) / 32) * ((dc + 31) / 32), bh, 1), dim3(32, 32, 1), 0, stream>>>(sp);
  ++g_last_launches;
  return cudaGetLastError() == cudaSuccess ? FLA_OK : FLA_ERR_CUDA;
}

// Head dims above the 128-wide tiles of fla_chunk_kernel.
constexpr int kWideMaxDim = 384;   // widest a/b (wide-a) or c/out (wide-c) head dim
constexpr int kWideNarrowDim = 64; // c/out columns one CTA of the wide-a kernel computes

bool is_wide_a(int da, int dc) { return da > 128 && da <= kWideMaxDim && dc <= kWideMaxDim; }
bool is_wide_c(int da, int dc) { return da <= 128 && dc > 128 && dc <= kWideMaxDim; }

// a, b wider than 128 columns: fla_wide_kernel, one CTA per (64-column slice of c/out, batch, head).
// It accumulates the whole a/b width in fp32 on chip; c/out may be as wide as a/b (LinearAttention
// with head dims up to 256 on both sides, flashlinear/kernels/linear_attn_kernels.py:316-322).
int run_wide_a(const Product& pd, int B, int H, int N, int da, int dc, int32_t* status,
               cudaStream_t stream) {
  if (!is_wide_a(da, dc)) return FLA_ERR_UNSUPPORTED;
  if (g_half) return FLA_ERR_UNSUPPORTED;  // the wide-head kernel exists for bf16 only
  if (pd.ext_init != nullptr || pd.ext_final != nullptr) return FLA_ERR_UNSUPPORTED;
  int rc;
  if ((rc = check_operand(pd.a, B, H)) || (rc = check_operand(pd.b, B, H)) ||
      (rc = check_operand(pd.c, B, H)) || (rc = check_operand(pd.out, B, H)))
    return rc;
  fla::WideParams wp;
  memset(&wp, 0, sizeof(wp));
  if ((rc = encode_map(&wp.a, pd.a, B, H, N)) || (rc = encode_map(&wp.b, pd.b, B, H, N)) ||
      (rc = encode_map(&wp.c, pd.c, B, H, N)) || (rc = encode_map(&wp.o, pd.out, B, H, N, 32)))
    return rc;
  wp.flags = pd.flags;
  wp.n_tokens = N;
  wp.heads = H;
  wp.nchunks = (N + fla::kWideChunk - 1) / fla::kWideChunk;
  wp.da = da;
  wp.status = status;
  wp.wait_limit_us = g_wait_limit_us;
  wp.debug_withhold = g_debug_withhold;
  // one CTA per (64-column slice of c/out, batch, head)
  const dim3 grid((dc + kWideNarrowDim - 1) / kWideNarrowDim, 1, B * H);
  if (da <= 256)
    fla::fla_wide_kernel<2><<<grid, fla::kWideThreads, fla::WideCfg<2>::SMEM_BYTES, stream>>>(wp);
  else
    fla::fla_wide_kernel<3><<<grid, fla::kWideThreads, fla::WideCfg<3>::SMEM_BYTES, stream>>>(wp);
  ++g_last_launches;
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    FLA_LOG_FAILURE("launch of fla_wide_kernel (da %d) failed: %s", da, cudaGetErrorString(e));
  return e == cudaSuccess ? FLA_OK : FLA_ERR_CUDA;
}

// c and out wider than 128 columns, a and b at most 128: the output columns are independent, so
// every 128-column slice of c/out is one problem of fla_chunk_kernel<128,128>; the slices of a
// head run side by side in one grid and share their a and b reads in L2.
int run_wide_c(const Product& pd, int B, int H, int N, int da, int dc, int32_t* status,
               cudaStream_t stream, const DeviceInfo& dev) {
  if (!is_wide_c(da, dc)) return FLA_ERR_UNSUPPORTED;
  if (pd.ext_init != nullptr || pd.ext_final != nullptr) return FLA_ERR_UNSUPPORTED;
  // Equal slices (rounded up to 16 columns, which keeps every slice 16-byte aligned): CTAs of a
  // narrow last slice would cost a full CTA slot for little traffic.
  Product slices[3];
  const int nslices = (dc + 127) / 128;
  const int width = ((dc + nslices - 1) / nslices + 15) / 16 * 16;
  int n = 0;
  for (int c0 = 0; c0 < dc; c0 += width, ++n) {
    Product& sl = slices[n];
    sl = pd;
    sl.c.ptr = static_cast<const char*>(pd.c.ptr) + static_cast<size_t>(c0) * 2;
    sl.out.ptr = static_cast<const char*>(pd.out.ptr) + static_cast<size_t>(c0) * 2;
    sl.c.dim = sl.out.dim = (dc - c0 < width) ? dc - c0 : width;
  }
  // check_operand wants sn >= round-up of dim; a slice's row stride covers the whole row
  return run_products(slices, n, B, H, N, da, 128, /*segments=*/1, nullptr, 0, status, stream, dev);
}

// One product of any supported head-dim pair without running-state arguments.
int run_wide_any(const Product& pd, int B, int H, int N, int da, int dc, int32_t* status,
                 cudaStream_t stream, const DeviceInfo& dev) {
  if (is_wide_a(da, dc)) return run_wide_a(pd, B, H, N, da, dc, status, stream);
  if (is_wide_c(da, dc)) return run_wide_c(pd, B, H, N, da, dc, status, stream, dev);
  return FLA_ERR_UNSUPPORTED;
}

int check_common(const FlaArgs* a, DeviceInfo** dev) {
  if (a == nullptr) return FLA_ERR_INVALID;
  // The launch checks below read the thread's last-error slot; drop whatever an earlier,
  // unrelated call of this thread (another library's probe, for one) may have left in it.
  (void)cudaGetLastError();
  if (a->batch <= 0 || a->heads <= 0 || a->seqlen <= 0 || a->dk <= 0 || a->dv <= 0)
    return FLA_ERR_INVALID;
  if (static_cast<long>(a->batch) * a->heads > 65535) return FLA_ERR_UNSUPPORTED;
  int rc = device_info(dev);
  if (rc) return rc;
  if ((*dev)->cc_major != 10) return FLA_ERR_DEVICE;
  if (!(*dev)->attr_set[0]) return FLA_ERR_CUDA;
  g_wait_limit_us = a->wait_limit_us > 0x7fffffffu ? 0x7fffffffu : a->wait_limit_us;
  g_debug_withhold = (a->debug_flags & FLA_DEBUG_WITHHOLD_FIRST_TILE) ? 1 : 0;
  g_no_fused = (a->debug_flags & FLA_DEBUG_NO_FUSED_SEGMENTS) ? 1 : 0;
  g_force_single_sweep = (a->debug_flags & FLA_DEBUG_FORCE_SINGLE_SWEEP) ? 1 : 0;
  if (a->dtype != FLA_DTYPE_BF16 && a->dtype != FLA_DTYPE_F16) return FLA_ERR_INVALID;
  g_half = a->dtype == FLA_DTYPE_F16 ? 1 : 0;
  return FLA_OK;
}

// ---------------------------------------------------------------- scratch that nobody allocates
// Scratch for fla_sm100_fwd_static_scratch(): a fixed array that is part of the loaded module, so
// that a caller who is not in a position to allocate device memory can still run the segmented
// forward. Every GPU that loads the library carries these bytes until the process exits.
// NOTE for host code: the NAME of this array is only a host-side handle. Its device address is
// obtained with cudaGetSymbolAddress() (static_scratch_address() below) and that pointer is what
// the kernels receive.
static __device__ __align__(256) unsigned char g_static_scratch[FLA_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch on the current device, looked up once per device.
int static_scratch_address(void** out) {
  static void* addr[64];
  static std::atomic<int> ready[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FLA_ERR_CUDA;
  if (ready[dev].load(std::memory_order_acquire) != 2) {
    int expected = 0;
    if (ready[dev].compare_exchange_strong(expected, 1)) {
      void* p = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);  // device `dev` is current
      if (e != cudaSuccess || p == nullptr) {
        ready[dev].store(0, std::memory_order_release);
        return FLA_ERR_CUDA;
      }
      addr[dev] = p;
      ready[dev].store(2, std::memory_order_release);
    } else {
      while (ready[dev].load(std::memory_order_acquire) == 1) {
      }
      if (ready[dev].load(std::memory_order_acquire) != 2) return FLA_ERR_CUDA;
    }
  }
  *out = addr[dev];
  return FLA_OK;
}

}  // namespace

extern "C" {

int fla_sm100_abi_version(void) { return FLA_ABI_VERSION; }

int fla_sm100_timeout_records(unsigned* out, int max_records) {
  if (out == nullptr || max_records <= 0) return FLA_ERR_INVALID;
  if (cudaDeviceSynchronize() != cudaSuccess) return FLA_ERR_CUDA;
  unsigned n = 0;
  static unsigned host_copy[fla::ptx::kTimeoutRecords * 8];
  if (cudaMemcpyFromSymbol(&n, fla::ptx::g_timeout_count, sizeof(n)) != cudaSuccess ||
      cudaMemcpyFromSymbol(host_copy, fla::ptx::g_timeout_records, sizeof(host_copy)) != cudaSuccess)
    return FLA_ERR_CUDA;
  const unsigned zero = 0;
  if (cudaMemcpyToSymbol(fla::ptx::g_timeout_count, &zero, sizeof(zero)) != cudaSuccess) return FLA_ERR_CUDA;
  int got = static_cast<int>(n < static_cast<unsigned>(fla::ptx::kTimeoutRecords) ? n : fla::ptx::kTimeoutRecords);
  if (got > max_records) got = max_records;
  memcpy(out, host_copy, static_cast<size_t>(got) * 8 * sizeof(unsigned));
  return got;
}

const char* fla_sm100_strerror(int code) {
  switch (code) {
    case FLA_OK: return "ok";
    case FLA_ERR_INVALID: return "invalid argument (null pointer or non-positive size)";
    case FLA_ERR_UNSUPPORTED: return "unsupported head dimension or batch*heads for the sm_100a kernels";
    case FLA_ERR_ALIGNMENT: return "pointer or byte stride is not a multiple of 16";
    case FLA_ERR_CUDA: return "a CUDA call failed";
    case FLA_ERR_WORKSPACE: return "workspace missing or too small";
    case FLA_ERR_DEVICE: return "current device is not an sm_100 GPU";
    case FLA_ERR_SCRATCH_LIMIT:
      return "shape needs more scratch than the built-in array of fla_sm100_fwd_static_scratch holds";
    default: return "unknown error";
  }
}

int fla_sm100_last_launch_count(void) { return g_last_launches; }

int fla_sm100_auto_segments(const FlaArgs* a, int pass) {
  if (a == nullptr) return 1;
  if (a->dk > 128 || a->dv > 128) return 1;  // the wide paths never split the sequence
  if (a->segments > 0) return a->segments;
  int sm = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess)
    cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev);
  const int nchunks = (a->seqlen + fla::kChunk - 1) / fla::kChunk;
  return auto_segments(pass == 1 ? 3 : 1, a->batch * a->heads, nchunks, sm);
}

size_t fla_sm100_workspace_bytes(const FlaArgs* a, int pass) {
  if (a == nullptr) return 0;
  const int nchunks = (a->seqlen + fla::kChunk - 1) / fla::kChunk;
  int nseg = fla_sm100_auto_segments(a, pass);
  if (nseg > nchunks) nseg = nchunks;
  if (nseg <= 1) return 0;
  const int seg_chunks = (nchunks + nseg - 1) / nseg;
  nseg = (nchunks + seg_chunks - 1) / seg_chunks;
  return segment_ws_bytes(pass == 1 ? 3 : 1, a->batch * a->heads, nseg, a->dk, a->dv) + 1024;
}

size_t fla_sm100_seg_states_bytes(const FlaArgs* a) {
  if (a == nullptr || a->batch <= 0 || a->heads <= 0 || a->seqlen <= 0) return 0;
  if (a->segment_states_ready) return 0;
  const int saved = g_no_fused, saved_force = g_force_single_sweep;
  g_no_fused = (a->debug_flags & FLA_DEBUG_NO_FUSED_SEGMENTS) ? 1 : 0;
  g_force_single_sweep = (a->debug_flags & FLA_DEBUG_FORCE_SINGLE_SWEEP) ? 1 : 0;
  const size_t n = seg_states_bytes(a, current_sm_count_early(), nullptr, nullptr);
  g_no_fused = saved;
  g_force_single_sweep = saved_force;
  return n;
}

int fla_sm100_bwd_uses_final_state(const FlaArgs* a) {
  if (a == nullptr || a->batch <= 0 || a->heads <= 0 || a->seqlen <= 0) return 0;
  if (a->dk > 128 || a->dv > 128) return 0;
  const int nchunks = (a->seqlen + fla::kChunk - 1) / fla::kChunk;
  if (!(nchunks >= kSingleSweepMinChunks || (a->debug_flags & FLA_DEBUG_FORCE_SINGLE_SWEEP))) return 0;
  if (fla_sm100_seg_states_bytes(a) > 0) return 1;
  int nseg = a->segments > 0 ? a->segments
                             : auto_segments(3, a->batch * a->heads, nchunks, current_sm_count_early());
  return nseg <= 1 ? 1 : 0;
}

int fla_sm100_fwd(const FlaArgs* a) {
  DeviceInfo* dev = nullptr;
  g_last_launches = 0;
  int rc = check_common(a, &dev);
  if (rc) return rc;
  Product p;
  p.a = operand(a->q, a->dk);
  p.b = operand(a->k, a->dk);
  p.c = operand(a->v, a->dv);
  p.out = operand(a->o, a->dv);
  p.flags = 0;
  p.ext_init = a->s_init;
  p.ext_final = a->s_final;
  p.ext_trans = 0;
  if (a->dk > 128 || a->dv > 128)
    return run_wide_any(p, a->batch, a->heads, a->seqlen, a->dk, a->dv, a->status,
                        static_cast<cudaStream_t>(a->stream), *dev);
  if (a->seg_states != nullptr && a->segment_states_ready == 0) {
    SegPlan f, b;
    const size_t need = seg_states_bytes(a, dev->sm_count, &f, &b);
    if (need > 0) {
      if (a->seg_states_bytes < need) return FLA_ERR_WORKSPACE;
      p.bound_out = static_cast<float*>(a->seg_states);
      // the segments the backward's plan was made for
      return run_products(&p, 1, a->batch, a->heads, a->seqlen, a->dk, a->dv, f.nseg, a->workspace,
                          a->workspace_bytes, a->status, static_cast<cudaStream_t>(a->stream), *dev,
                          false, f.seg_chunks);
    }
  }
  return run_products(&p, 1, a->batch, a->heads, a->seqlen, a->dk, a->dv, a->segments,
                      a->workspace, a->workspace_bytes, a->status,
                      static_cast<cudaStream_t>(a->stream), *dev, a->segment_states_ready != 0);
}

int fla_sm100_bwd(const FlaArgs* a) {
  DeviceInfo* dev = nullptr;
  g_last_launches = 0;
  int rc = check_common(a, &dev);
  if (rc) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  // dQ: causal, state sum v^T k = S^T (dv x dk)
  Product pq;
  pq.a = operand(a->d_o, a->dv);
  pq.b = operand(a->v, a->dv);
  pq.c = operand(a->k, a->dk);
  pq.out = operand(a->d_q, a->dk);
  pq.flags = 0;
  pq.ext_init = a->s_init;
  pq.ext_final = nullptr;
  pq.ext_trans = 1;
  // dV: anti-causal, state sum q^T dO = R (dk x dv)
  Product pv;
  pv.a = operand(a->k, a->dk);
  pv.b = operand(a->q, a->dk);
  pv.c = operand(a->d_o, a->dv);
  pv.out = operand(a->d_v, a->dv);
  pv.flags = fla::kFlagDescending | fla::kFlagUpperMask;
  pv.ext_init = a->r_init;
  pv.ext_final = a->r_final;
  pv.ext_trans = 0;
  // dK: anti-causal, state sum dO^T q = R^T (dv x dk)
  Product pk;
  pk.a = operand(a->v, a->dv);
  pk.b = operand(a->d_o, a->dv);
  pk.c = operand(a->q, a->dk);
  pk.out = operand(a->d_k, a->dk);
  pk.flags = fla::kFlagDescending | fla::kFlagUpperMask;
  pk.ext_init = a->r_init;
  pk.ext_final = nullptr;
  pk.ext_trans = 1;

  if (a->dk > 128 || a->dv > 128) {
    // Head dims above the 128-wide tiles (SmallVHD shapes: dQ and dK have the wide head dim on the
    // output side, dV on the a/b side; both sides wide: all three through the wide-a kernel).
    if (a->s_init || a->r_init || a->r_final || a->s_last) return FLA_ERR_UNSUPPORTED;
    auto any = [&](const Product& pd, int da, int dc) {
      if (da <= 128 && dc <= 128)
        return run_products(&pd, 1, a->batch, a->heads, a->seqlen, da, dc, a->segments, a->workspace,
                            a->workspace_bytes, a->status, stream, *dev);
      return run_wide_any(pd, a->batch, a->heads, a->seqlen, da, dc, a->status, stream, *dev);
    };
    if ((rc = any(pq, a->dv, a->dk))) return rc;
    if ((rc = any(pk, a->dv, a->dk))) return rc;
    return any(pv, a->dk, a->dv);
  }
  const int nchunks = (a->seqlen + fla::kChunk - 1) / fla::kChunk;
  if (a->seg_states != nullptr && a->s_last != nullptr && single_sweep_allowed(nchunks)) {
    // Few heads: the forward ran as one fused segmented launch and stored the state at each of
    // its segment boundaries. The backward is split at a subset of those boundaries; dQ walks every
    // segment end-to-start from the stored state at the segment's end (total minus suffix, as in
    // the unsegmented case), dV and dK start from the partial sums of q^T dO that the same launch
    // forms first. One launch, and the three products of a (head, segment) stream the same chunks.
    SegPlan f, bp;
    const size_t need = seg_states_bytes(a, dev->sm_count, &f, &bp);
    if (need > 0) {
      if (a->seg_states_bytes < need) return FLA_ERR_WORKSPACE;
      pq.flags = fla::kFlagDescending | fla::kFlagTotalMinusSuffix;
      if (a->s_init == nullptr) pq.flags |= fla::kFlagFirstChunkExact;
      pq.ext_init = a->s_last;  // segment 0 of the descending walk: the end of the sequence
      pq.bound_base = static_cast<const float*>(a->seg_states);
      pq.bound_trans = 1;       // the forward stored S^T, which is this product's own state
      pq.bound_stride = f.nseg - 1;
      pq.bound_slot0 = nchunks / f.seg_chunks - 1;
      pq.bound_step = bp.seg_chunks / f.seg_chunks;
      Product all[3] = {pq, pv, pk};
      return run_products(all, 3, a->batch, a->heads, a->seqlen, a->dk, a->dv, bp.nseg, a->workspace,
                          a->workspace_bytes, a->status, stream, *dev, false, bp.seg_chunks);
    }
  }
  int nseg = a->segments > 0 ? a->segments
                             : auto_segments(3, a->batch * a->heads, nchunks, dev->sm_count);
  if (nseg > nchunks) nseg = nchunks;
  if (a->s_last != nullptr && nseg <= 1 && single_sweep_allowed(nchunks)) {
    // The forward state after this call's tokens is known: dQ can walk the sequence in the same
    // descending order as dV and dK (state = total minus suffix), so the three products of a
    // head stream the same chunks at the same time and share their q, k, v, dO reads in L2.
    pq.flags = fla::kFlagDescending | fla::kFlagTotalMinusSuffix;
    if (a->s_init == nullptr) pq.flags |= fla::kFlagFirstChunkExact;  // nothing precedes token 0
    pq.ext_init = a->s_last;
  }
  if (a->dk == a->dv) {
    // Same shapes: one grid. Block x = product; dV and dK of a head are neighbours in launch order.
    Product all[3] = {pq, pv, pk};
    return run_products(all, 3, a->batch, a->heads, a->seqlen, a->dk, a->dv, nseg, a->workspace,
                        a->workspace_bytes, a->status, stream, *dev);
  }
  // dk != dv: dQ and dK have (da, dc) = (dv, dk); dV has (dk, dv). The caller's scratch is split
  // two thirds / one third.
  Product two[2] = {pq, pk};
  const size_t third = (a->workspace_bytes / 3) & ~static_cast<size_t>(255);
  char* ws = static_cast<char*>(a->workspace);
  rc = run_products(two, 2, a->batch, a->heads, a->seqlen, a->dv, a->dk, nseg, ws,
                    ws ? 2 * third : 0, a->status, stream, *dev);
  if (rc) return rc;
  return run_products(&pv, 1, a->batch, a->heads, a->seqlen, a->dk, a->dv, nseg,
                      ws ? ws + 2 * third : nullptr, ws ? third : 0, a->status, stream, *dev);
}

int fla_sm100_state(const FlaArgs* a, int which) {
  DeviceInfo* dev = nullptr;
  g_last_launches = 0;
  int rc = check_common(a, &dev);
  if (rc) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  if (which == 0)
    return run_state(operand(a->k, a->dk), operand(a->v, a->dv), a->batch, a->heads, a->seqlen,
                     a->dk, a->dv, a->segments, a->s_final, a->workspace, a->workspace_bytes,
                     a->status, stream, *dev);
  if (which == 1)
    return run_state(operand(a->q, a->dk), operand(a->d_o, a->dv), a->batch, a->heads, a->seqlen,
                     a->dk, a->dv, a->segments, a->r_final, a->workspace, a->workspace_bytes,
                     a->status, stream, *dev);
  return FLA_ERR_INVALID;
}

int fla_sm100_fwd_static_scratch(const FlaArgs* a) {
  DeviceInfo* dev = nullptr;
  g_last_launches = 0;
  int rc = check_common(a, &dev);
  if (rc) return rc;
  Product p;
  p.a = operand(a->q, a->dk);
  p.b = operand(a->k, a->dk);
  p.c = operand(a->v, a->dv);
  p.out = operand(a->o, a->dv);
  p.flags = 0;
  p.ext_init = a->s_init;
  p.ext_final = a->s_final;
  p.ext_trans = 0;
  // head dims above 128: those kernels never split the sequence and use no scratch
  if (a->dk > 128 || a->dv > 128)
    return run_wide_any(p, a->batch, a->heads, a->seqlen, a->dk, a->dv, a->status,
                        static_cast<cudaStream_t>(a->stream), *dev);
  // How much scratch this shape needs with the segment count the call will use.
  const int nchunks = (a->seqlen + fla::kChunk - 1) / fla::kChunk;
  int nseg = a->segments > 0 ? a->segments
                             : auto_segments(1, a->batch * a->heads, nchunks, dev->sm_count);
  if (nseg > nchunks) nseg = nchunks;
  if (nseg > 1) {
    const int seg_chunks = (nchunks + nseg - 1) / nseg;
    nseg = (nchunks + seg_chunks - 1) / seg_chunks;
  }
  const size_t need = segment_ws_bytes(1, a->batch * a->heads, nseg, a->dk, a->dv);
  if (need > static_cast<size_t>(FLA_STATIC_SCRATCH_BYTES)) return FLA_ERR_SCRATCH_LIMIT;
  // The array's address is looked up only by calls that use it, so an unsegmented call never
  // makes the symbol query (which is not allowed while a stream is being captured).
  void* scratch = nullptr;
  if (nseg > 1 && (rc = static_scratch_address(&scratch)) != FLA_OK) return rc;
  // Nothing in the scratch has to start at zero: every per-segment sum that the scan reads is
  // written by the state pass of this same call first.
  return run_products(&p, 1, a->batch, a->heads, a->seqlen, a->dk, a->dv, nseg, scratch,
                      nseg > 1 ? FLA_STATIC_SCRATCH_BYTES : 0, a->status,
                      static_cast<cudaStream_t>(a->stream), *dev);
}

int fla_sm100_taylor_dims(int d, int* features, int* padded) {
  if (d != 8 && d != 16) return FLA_ERR_UNSUPPORTED;
  const int f = 1 + d + d * d;
  if (features) *features = f;
  if (padded) *padded = (f + 7) / 8 * 8;
  return FLA_OK;
}

int fla_sm100_taylor_features(const void* x, void* phi, long long rows, int d, void* stream) {
  (void)cudaGetLastError();
  g_last_launches = 0;
  if (x == nullptr || phi == nullptr || rows <= 0) return FLA_ERR_INVALID;
  if (d != 8 && d != 16) return FLA_ERR_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(x) % 16 != 0 || reinterpret_cast<uintptr_t>(phi) % 16 != 0)
    return FLA_ERR_ALIGNMENT;
  const int blocks = static_cast<int>(
      std::min<long long>((rows + fla::kTaylorRows - 1) / fla::kTaylorRows, 148 * 16));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (d == 16) {
    constexpr int smem = fla::taylor_tile_smem_bytes<16>();
    if (cudaFuncSetAttribute(fla::fla_taylor_fwd_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             smem) != cudaSuccess)
      return FLA_ERR_CUDA;
    fla::fla_taylor_fwd_kernel<16><<<blocks, fla::kTaylorRows, smem, st>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<uint4*>(phi), rows);
  } else {
    constexpr int smem = fla::taylor_tile_smem_bytes<8>();
    fla::fla_taylor_fwd_kernel<8><<<blocks, fla::kTaylorRows, smem, st>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<uint4*>(phi), rows);
  }
  ++g_last_launches;
  return cudaGetLastError() == cudaSuccess ? FLA_OK : FLA_ERR_CUDA;
}

int fla_sm100_taylor_features_bwd(const void* dphi, const void* x, void* dx, long long rows, int d,
                                  void* stream) {
  (void)cudaGetLastError();
  g_last_launches = 0;
  if (dphi == nullptr || x == nullptr || dx == nullptr || rows <= 0) return FLA_ERR_INVALID;
  if (d != 8 && d != 16) return FLA_ERR_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(x) % 16 != 0 || reinterpret_cast<uintptr_t>(dphi) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(dx) % 16 != 0)
    return FLA_ERR_ALIGNMENT;
  const int blocks = static_cast<int>(
      std::min<long long>((rows + fla::kTaylorRows - 1) / fla::kTaylorRows, 148 * 16));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (d == 16) {
    constexpr int smem = fla::taylor_tile_smem_bytes<16>();
    e = cudaFuncSetAttribute(fla::fla_taylor_bwd_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return FLA_ERR_CUDA;
    fla::fla_taylor_bwd_kernel<16><<<blocks, fla::kTaylorRows, smem, st>>>(
        static_cast<const uint4*>(dphi), static_cast<const __nv_bfloat16*>(x),
        static_cast<__nv_bfloat16*>(dx), rows);
  } else {
    constexpr int smem = fla::taylor_tile_smem_bytes<8>();
    fla::fla_taylor_bwd_kernel<8><<<blocks, fla::kTaylorRows, smem, st>>>(
        static_cast<const uint4*>(dphi), static_cast<const __nv_bfloat16*>(x),
        static_cast<__nv_bfloat16*>(dx), rows);
  }
  ++g_last_launches;
  return cudaGetLastError() == cudaSuccess ? FLA_OK : FLA_ERR_CUDA;
}

int fla_sm100_pad_rows(const void* src, void* dst, long long rows, int d, int dpad, void* stream) {
  (void)cudaGetLastError();
  g_last_launches = 0;
  if (src == nullptr || dst == nullptr || rows <= 0 || d <= 0 || dpad < d) return FLA_ERR_INVALID;
  if (dpad % 8 != 0 || reinterpret_cast<uintptr_t>(dst) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(src) % 4 != 0)
    return FLA_ERR_ALIGNMENT;
  const int blocks = static_cast<int>(
      std::min<long long>((rows + kPadRowsPerBlock - 1) / kPadRowsPerBlock, 148 * 32));
  fla_pad_rows_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(src), static_cast<uint4*>(dst), rows, d, dpad);
  ++g_last_launches;
  return cudaGetLastError() == cudaSuccess ? FLA_OK : FLA_ERR_CUDA;
}

int fla_sm100_unpad_rows(const void* src, void* dst, long long rows, int d, int dpad, void* stream) {
  (void)cudaGetLastError();
  g_last_launches = 0;
  if (src == nullptr || dst == nullptr || rows <= 0 || d <= 0 || dpad < d) return FLA_ERR_INVALID;
  if (reinterpret_cast<uintptr_t>(dst) % 4 != 0 || reinterpret_cast<uintptr_t>(src) % 2 != 0)
    return FLA_ERR_ALIGNMENT;
  const int blocks = static_cast<int>(
      std::min<long long>((rows + kPadRowsPerBlock - 1) / kPadRowsPerBlock, 148 * 32));
  fla_unpad_rows_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned short*>(src), static_cast<unsigned short*>(dst), rows, d, dpad);
  ++g_last_launches;
  return cudaGetLastError() == cudaSuccess ? FLA_OK : FLA_ERR_CUDA;
}

namespace {
fla::NormTensor norm_tensor(const FlaTensor& t) {
  fla::NormTensor n;
  n.ptr = t.ptr;
  n.sb = t.stride_b;
  n.sh = t.stride_h;
  n.sn = t.stride_n;
  return n;
}
// token tile of the normalisation kernels: small tiles keep three CTAs resident per SM
int norm_tile(int dk, int dv) { return (dk <= 128 && dv <= 128) ? 32 : 16; }
constexpr size_t kNormSmemLimit = 232448;

// Sequence segments of the normalisation kernels: about three CTAs (heads x segments) per SM;
// segments a multiple of 64 tokens and at least 256 tokens long. The forward kernel (three CTAs
// resident per SM) gets no more CTAs than fit at once (round_up = false); the sweep kernel (six
// resident, two sweeps) measured faster with the count rounded up.
void norm_segments(const FlaArgs* a, int sm_count, bool round_up, int* seg_len, int* nseg) {
  const int bh = a->batch * a->heads;
  int want = round_up ? (3 * sm_count + bh - 1) / bh : (3 * sm_count) / bh;
  const int max_seg = (a->seqlen + 255) / 256;
  if (want > max_seg) want = max_seg;
  if (want < 1) want = 1;
  int len = (a->seqlen + want - 1) / want;
  len = (len + 63) / 64 * 64;
  *seg_len = len;
  *nseg = (a->seqlen + len - 1) / len;
}

// Fills the geometry fields and launches the column-sum kernel for k (weighted = 0) or for
// dden_i q_i (weighted = 1) into `out`.
int launch_colsum(fla::NormParams p, int weighted, float* out, int bh, cudaStream_t stream) {
  p.weighted = weighted;
  p.sums_out = out;
  fla::fla_colsum_kernel<<<dim3(p.nseg, bh, 1), fla::kNormThreads, 0, stream>>>(p);
  ++g_last_launches;
  return cudaGetLastError() == cudaSuccess ? FLA_OK : FLA_ERR_CUDA;
}
}  // namespace

size_t fla_sm100_normalize_workspace_bytes(const FlaArgs* a) {
  if (a == nullptr || a->batch <= 0 || a->heads <= 0 || a->seqlen <= 0 || a->dk <= 0) return 0;
  int sm = 148, dev = 0, seg_len = 0, nseg = 1;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev);
  norm_segments(a, sm, true, &seg_len, &nseg);
  return 2 * static_cast<size_t>(a->batch) * a->heads * nseg * a->dk * sizeof(float);
}

int fla_sm100_normalize_fwd(const FlaArgs* a, float eps, float* den) {
  DeviceInfo* dev = nullptr;
  g_last_launches = 0;
  int rc = check_common(a, &dev);
  if (rc) return rc;
  if (den == nullptr) return FLA_ERR_INVALID;
  if ((rc = check_operand(operand(a->q, a->dk), a->batch, a->heads)) ||
      (rc = check_operand(operand(a->k, a->dk), a->batch, a->heads)) ||
      (rc = check_operand(operand(a->o, a->dv), a->batch, a->heads)))
    return rc;
  const int tile = norm_tile(a->dk, a->dv);
  const size_t smem = fla::norm_fwd_smem_bytes(a->dk, a->dv, tile);
  if (smem > kNormSmemLimit || a->dk > 512) return FLA_ERR_UNSUPPORTED;
  fla::NormParams p;
  memset(&p, 0, sizeof(p));
  norm_segments(a, dev->sm_count, false, &p.seg_len, &p.nseg);
  const int bh = a->batch * a->heads;
  const size_t sums_bytes = static_cast<size_t>(bh) * p.nseg * a->dk * sizeof(float);
  if (p.nseg > 1 && (a->workspace == nullptr || a->workspace_bytes < sums_bytes)) return FLA_ERR_WORKSPACE;
  p.q = norm_tensor(a->q);
  p.k = norm_tensor(a->k);
  p.x = norm_tensor(a->o);
  p.den = den;
  p.heads = a->heads;
  p.n = a->seqlen;
  p.dk = a->dk;
  p.dv = a->dv;
  p.eps = eps;
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  if (p.nseg > 1) {
    float* sums = static_cast<float*>(a->workspace);
    if ((rc = launch_colsum(p, 0, sums, bh, stream))) return rc;
    p.sums = sums;
  }
  const dim3 grid(p.nseg, bh, 1);
  const int fixed = (a->dk == a->dv && (a->dk == 64 || a->dk == 128)) ? a->dk : 0;
  if (fixed == 128)
    fla::fla_normalize_fwd_kernel<32, 128><<<grid, fla::kNormThreads, smem, stream>>>(p);
  else if (fixed == 64)
    fla::fla_normalize_fwd_kernel<32, 64><<<grid, fla::kNormThreads, smem, stream>>>(p);
  else if (tile == 32)
    fla::fla_normalize_fwd_kernel<32, 0><<<grid, fla::kNormThreads, smem, stream>>>(p);
  else
    fla::fla_normalize_fwd_kernel<16, 0><<<grid, fla::kNormThreads, smem, stream>>>(p);
  ++g_last_launches;
  return cudaGetLastError() == cudaSuccess ? FLA_OK : FLA_ERR_CUDA;
}

int fla_sm100_normalize_bwd_prepare(const FlaArgs* a, const float* den, float* dden) {
  DeviceInfo* dev = nullptr;
  g_last_launches = 0;
  int rc = check_common(a, &dev);
  if (rc) return rc;
  if (den == nullptr || dden == nullptr) return FLA_ERR_INVALID;
  if ((rc = check_operand(operand(a->d_o, a->dv), a->batch, a->heads)) ||
      (rc = check_operand(operand(a->o, a->dv), a->batch, a->heads)) ||
      (rc = check_operand(operand(a->d_v, a->dv), a->batch, a->heads)))
    return rc;
  fla::NormParams p;
  memset(&p, 0, sizeof(p));
  p.x = norm_tensor(a->d_o);
  p.y = norm_tensor(a->o);
  p.z = norm_tensor(a->d_v);
  p.den = const_cast<float*>(den);
  p.dden = dden;
  p.heads = a->heads;
  p.n = a->seqlen;
  p.dk = a->dk;
  p.dv = a->dv;
  // blocks per head: enough warps for about eight blocks per SM, at most one warp step per block
  const int bh = a->batch * a->heads;
  int bx = std::max(1, (148 * 8 + bh - 1) / bh);
  bx = std::min(bx, std::max(1, (a->seqlen + 7) / 8));
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  if (a->dv == 128)
    fla::fla_normalize_bwd_prepare_kernel<128><<<dim3(bx, bh, 1), fla::kNormThreads, 0, stream>>>(p);
  else if (a->dv == 64)
    fla::fla_normalize_bwd_prepare_kernel<64><<<dim3(bx, bh, 1), fla::kNormThreads, 0, stream>>>(p);
  else
    fla::fla_normalize_bwd_prepare_kernel<0><<<dim3(bx, bh, 1), fla::kNormThreads, 0, stream>>>(p);
  ++g_last_launches;
  return cudaGetLastError() == cudaSuccess ? FLA_OK : FLA_ERR_CUDA;
}

int fla_sm100_normalize_bwd_sweep(const FlaArgs* a, const float* dden) {
  DeviceInfo* dev = nullptr;
  g_last_launches = 0;
  int rc = check_common(a, &dev);
  if (rc) return rc;
  if (dden == nullptr) return FLA_ERR_INVALID;
  if ((rc = check_operand(operand(a->q, a->dk), a->batch, a->heads)) ||
      (rc = check_operand(operand(a->k, a->dk), a->batch, a->heads)) ||
      (rc = check_operand(operand(a->d_q, a->dk), a->batch, a->heads)) ||
      (rc = check_operand(operand(a->d_k, a->dk), a->batch, a->heads)))
    return rc;
  const int tile = norm_tile(a->dk, a->dv);
  const size_t smem = fla::norm_sweep_smem_bytes(a->dk, tile);
  if (smem > kNormSmemLimit || a->dk > 512) return FLA_ERR_UNSUPPORTED;
  fla::NormParams p;
  memset(&p, 0, sizeof(p));
  norm_segments(a, dev->sm_count, true, &p.seg_len, &p.nseg);
  const int bh = a->batch * a->heads;
  const size_t sums_elems = static_cast<size_t>(bh) * p.nseg * a->dk;
  if (p.nseg > 1 && (a->workspace == nullptr || a->workspace_bytes < 2 * sums_elems * sizeof(float)))
    return FLA_ERR_WORKSPACE;
  p.q = norm_tensor(a->q);
  p.k = norm_tensor(a->k);
  p.dq = norm_tensor(a->d_q);
  p.dk_ = norm_tensor(a->d_k);
  p.dden = const_cast<float*>(dden);
  p.heads = a->heads;
  p.n = a->seqlen;
  p.dk = a->dk;
  p.dv = a->dv;
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  if (p.nseg > 1) {
    float* sums = static_cast<float*>(a->workspace);
    if ((rc = launch_colsum(p, 0, sums, bh, stream))) return rc;
    if ((rc = launch_colsum(p, 1, sums + sums_elems, bh, stream))) return rc;
    p.sums = sums;
    p.rsums = sums + sums_elems;
  }
  const dim3 grid(p.nseg, bh, 2);
  const int fixed = (a->dk == 64 || a->dk == 128) ? a->dk : 0;  // only dk matters to the sweep
  if (fixed == 128 && tile == 32)
    fla::fla_normalize_bwd_sweep_kernel<32, 128><<<grid, fla::kNormThreads, smem, stream>>>(p);
  else if (fixed == 64 && tile == 32)
    fla::fla_normalize_bwd_sweep_kernel<32, 64><<<grid, fla::kNormThreads, smem, stream>>>(p);
  else if (tile == 32)
    fla::fla_normalize_bwd_sweep_kernel<32, 0><<<grid, fla::kNormThreads, smem, stream>>>(p);
  else
    fla::fla_normalize_bwd_sweep_kernel<16, 0><<<grid, fla::kNormThreads, smem, stream>>>(p);
  ++g_last_launches;
  return cudaGetLastError() == cudaSuccess ? FLA_OK : FLA_ERR_CUDA;
}

int fla_sm100_product(const FlaArgs* a, int anticausal) {
  DeviceInfo* dev = nullptr;
  g_last_launches = 0;
  int rc = check_common(a, &dev);
  if (rc) return rc;
  Product p;
  p.a = operand(a->q, a->dk);
  p.b = operand(a->k, a->dk);
  p.c = operand(a->v, a->dv);
  p.out = operand(a->o, a->dv);
  p.flags = anticausal ? (fla::kFlagDescending | fla::kFlagUpperMask) : 0;
  p.ext_init = a->s_init;
  p.ext_final = a->s_final;
  p.ext_trans = 0;
  if (a->dk > 128 || a->dv > 128)
    return run_wide_any(p, a->batch, a->heads, a->seqlen, a->dk, a->dv, a->status,
                        static_cast<cudaStream_t>(a->stream), *dev);
  return run_products(&p, 1, a->batch, a->heads, a->seqlen, a->dk, a->dv, a->segments,
                      a->workspace, a->workspace_bytes, a->status,
                      static_cast<cudaStream_t>(a->stream), *dev);
}

namespace {
// Segment count and scratch size of the exchange path (scratch is needed even for one segment).
int exchange_segments(const FlaArgs* a, int sm_count) {
  const int nchunks = (a->seqlen + fla::kChunk - 1) / fla::kChunk;
  int nseg = a->segments > 0 ? a->segments : auto_segments(1, a->batch * a->heads, nchunks, sm_count);
  if (nseg > nchunks) nseg = nchunks;
  if (nseg < 1) nseg = 1;
  const int seg_chunks = (nchunks + nseg - 1) / nseg;
  return (nchunks + seg_chunks - 1) / seg_chunks;
}
int current_sm_count() {
  int sm = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev);
  return sm;
}
}  // namespace

size_t fla_sm100_exchange_workspace_bytes(const FlaArgs* a) {
  if (a == nullptr) return 0;
  const int nseg = exchange_segments(a, current_sm_count());
  // (the slack matches fla_sm100_workspace_bytes, so that one buffer serves both calls)
  return static_cast<size_t>(a->batch) * a->heads * nseg * a->dk * a->dv * sizeof(float) + 1024;
}

int fla_sm100_enable_peer_access(int peer_device) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return FLA_ERR_CUDA;
  if (peer_device == dev) return FLA_OK;
  int can = 0;
  if (cudaDeviceCanAccessPeer(&can, dev, peer_device) != cudaSuccess || !can) {
    FLA_LOG_FAILURE("device %d cannot access peer %d", dev, peer_device);
    return FLA_ERR_DEVICE;
  }
  const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    (void)cudaGetLastError();
    return FLA_OK;
  }
  if (e != cudaSuccess) FLA_LOG_FAILURE("cudaDeviceEnablePeerAccess(%d) failed: %s", peer_device, cudaGetErrorString(e));
  return e == cudaSuccess ? FLA_OK : FLA_ERR_CUDA;
}

// Exchange buffers are allocated by the library itself (plain cudaMalloc, zero-filled) so that
// their CUDA IPC handles refer to whole allocations, and a peer opens them with ITS OWN device
// current: an import made under another device's context is not reachable from this device's
// kernels, peer access or not.
int fla_sm100_exchange_alloc(size_t bytes, void** ptr, unsigned char* handle64) {
  if (ptr == nullptr || handle64 == nullptr || bytes == 0) return FLA_ERR_INVALID;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    FLA_LOG_FAILURE("exchange_alloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    if (p) cudaFree(p);
    return FLA_ERR_CUDA;
  }
  memcpy(handle64, &h, 64);
  *ptr = p;
  return FLA_OK;
}

int fla_sm100_exchange_open(const unsigned char* handle64, void** ptr) {
  if (ptr == nullptr || handle64 == nullptr) return FLA_ERR_INVALID;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    FLA_LOG_FAILURE("cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    return FLA_ERR_CUDA;
  }
  // Check the mapping with a runtime copy (an error code, not a device fault, if it is unusable).
  unsigned probe = 0;
  e = cudaMemcpy(&probe, p, sizeof(probe), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) e = cudaMemcpy(p, &probe, sizeof(probe), cudaMemcpyHostToDevice);  // same value back
  if (e != cudaSuccess) {
    FLA_LOG_FAILURE("peer mapping is not readable / writable: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    cudaIpcCloseMemHandle(p);
    return FLA_ERR_CUDA;
  }
  *ptr = p;
  return FLA_OK;
}

int fla_sm100_exchange_close(void* ptr) {
  return (ptr != nullptr && cudaIpcCloseMemHandle(ptr) == cudaSuccess) ? FLA_OK : FLA_ERR_CUDA;
}

int fla_sm100_exchange_free(void* ptr) {
  return (ptr != nullptr && cudaFree(ptr) == cudaSuccess) ? FLA_OK : FLA_ERR_CUDA;
}

int fla_sm100_exchange_bytes(const FlaArgs* a, int world, size_t* inbox_bytes, size_t* flag_bytes) {
  if (a == nullptr || world < 1 || world > FLA_MAX_RANKS) return FLA_ERR_INVALID;
  const size_t bh = static_cast<size_t>(a->batch) * a->heads;
  const size_t elems = static_cast<size_t>(a->dk) * a->dv;
  const size_t nblocks = bh * ((elems + 255) / 256);
  if (inbox_bytes) *inbox_bytes = 2 * static_cast<size_t>(world) * bh * elems * sizeof(float);
  if (flag_bytes) *flag_bytes = 2 * static_cast<size_t>(world) * nblocks * sizeof(unsigned);
  return FLA_OK;
}

int fla_sm100_state_exchange(const FlaArgs* a, int which, const FlaExchange* x) {
  DeviceInfo* dev = nullptr;
  g_last_launches = 0;
  int rc = check_common(a, &dev);
  if (rc) return rc;
  if (x == nullptr || x->world < 1 || x->world > FLA_MAX_RANKS || x->rank < 0 ||
      x->rank >= x->world || (x->epoch == 0 && x->epoch_counter == nullptr) ||
      (which != 0 && which != 1))
    return FLA_ERR_INVALID;
  for (int d = 0; d < x->world; ++d)
    if (x->inbox[d] == nullptr || x->flags[d] == nullptr) return FLA_ERR_INVALID;
  const Operand bop = which == 0 ? operand(a->k, a->dk) : operand(a->q, a->dk);
  const Operand cop = which == 0 ? operand(a->v, a->dv) : operand(a->d_o, a->dv);
  const int da = a->dk, dc = a->dv;
  const int tmpl = pick_template(da, dc);
  if (tmpl == 0) return FLA_ERR_UNSUPPORTED;
  if ((rc = check_operand(bop, a->batch, a->heads)) || (rc = check_operand(cop, a->batch, a->heads)))
    return rc;
  const int bh = a->batch * a->heads;
  const int nchunks = (a->seqlen + fla::kChunk - 1) / fla::kChunk;
  const int nseg = exchange_segments(a, dev->sm_count);
  const int seg_chunks = (nchunks + nseg - 1) / nseg;
  const size_t need = static_cast<size_t>(bh) * nseg * da * dc * sizeof(float);
  if (a->workspace == nullptr || a->workspace_bytes < need) return FLA_ERR_WORKSPACE;
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);

  // state pass: every segment's sum of b^T c into the scratch (scratch layout)
  KernelParams kp;
  memset(&kp, 0, sizeof(kp));
  kp.heads = a->heads;
  kp.nchunks = nchunks;
  kp.seg_chunks = seg_chunks;
  kp.st_rows = da;
  kp.st_cols = dc;
  kp.status = a->status;
  kp.mode = 1;
  if ((rc = encode_map(&kp.prob[0].k, bop, a->batch, a->heads, a->seqlen)) ||
      (rc = encode_map(&kp.prob[0].v, cop, a->batch, a->heads, a->seqlen)))
    return rc;
  kp.prob[0].s_final = static_cast<float*>(a->workspace);
  kp.prob[0].st_trans = 1;
  kp.prob[0].flags = x->reverse ? (fla::kFlagDescending | fla::kFlagUpperMask) : 0;
  if ((rc = launch_template(tmpl, kp, dim3(1, nseg, bh), stream))) return rc;

  // scan + publish to the peers + bounded wait + add the peers' totals
  ExchangeParams xp;
  memset(&xp, 0, sizeof(xp));
  xp.ws = static_cast<float*>(a->workspace);
  xp.nseg = nseg;
  xp.rows = da;
  xp.cols = dc;
  xp.bh_count = bh;
  xp.rank = x->rank;
  xp.world = x->world;
  xp.reverse = x->reverse;
  xp.epoch = x->epoch;
  for (int d = 0; d < x->world; ++d) {
    xp.inbox[d] = x->inbox[d];
    xp.flags[d] = x->flags[d];
  }
  xp.remote_out = x->remote_out;
  xp.inclusive_out = x->inclusive_out;
  xp.status = a->status;
  xp.epoch_counter = x->epoch_counter;
  xp.wait_limit_ns = (x->wait_limit_us ? static_cast<unsigned long long>(x->wait_limit_us) : 400000ull) * 1000ull;
  // Blocks per head: every block waits for its twin on the other GPUs, so all blocks of all heads
  // must be resident together. At most four blocks per SM are used (others may share the GPU);
  // threads loop over the elements their blocks do not cover. The count depends on the shapes
  // only, so it is the same on every rank (it indexes the flags).
  const int elems = da * dc;
  const int full = (elems + 255) / 256;
  const int resident = 4 * 148;
  if (bh > resident) return FLA_ERR_UNSUPPORTED;
  const int bx = std::min(full, std::max(1, resident / bh));
  fla_state_exchange_kernel<<<dim3(bx, bh, 1), 256, 0, stream>>>(xp);
  ++g_last_launches;
  if (x->epoch_counter != nullptr) {
    fla_exchange_bump_kernel<<<1, 1, 0, stream>>>(x->epoch_counter);
    ++g_last_launches;
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) FLA_LOG_FAILURE("launch of fla_state_exchange_kernel failed: %s", cudaGetErrorString(e));
  return e == cudaSuccess ? FLA_OK : FLA_ERR_CUDA;
}

}  // extern "C"
