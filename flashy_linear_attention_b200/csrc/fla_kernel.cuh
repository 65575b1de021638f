// Chunked causal linear attention for sm_100a.
//
// One generic kernel computes, for one head and one run of 128-token chunks,
//     o_i = sum_{j <= i} (q_i . k_j) v_j            (causal)
//     o_i = sum_{j >= i} (q_i . k_j) v_j            (anti-causal: descending walk, upper mask)
// as  P = (Q K^T) (.) mask,  O = P V + Q S,  S += K^T V   per chunk, where S (dk x dv, fp32) is the
// running state carried in tensor memory. The forward pass and all three gradients are this same
// product with the operands permuted (see fla_api.cu), which replaces the quadratic tile loops of
// flashlinear/kernels/linear_attn_kernels.py:63-85 (fwd), :171-200 and :283-302 (bwd).
//
// CTA layout (480 threads, one CTA per SM):
//   warp 0        TMA producer: Q, K, V chunk tiles -> a ring of shared-memory slots (128B swizzle)
//   warp 1        MMA issuer X (one elected lane) and TMEM owner: S += K^T V, P = Q K^T
//   warp 14       MMA issuer Y (one elected lane): O = Q Sb, O += Pb V
//   warps 2-5     converter group A  } P fp32 (TMEM) -> mask -> bf16 (TMEM, A operand of P V)
//   warps 6-9     converter group B  } S fp32 (TMEM) -> bf16 (shared memory, B operand of Q S);
//                                      each group owns one half of the columns
//   warps 10-13   epilogue group: O fp32 (TMEM) -> bf16 -> staging buffer -> TMA store
//
// Two warps issue MMAs so that the waits of one overlap the issue of the other: X produces the
// intermediates (state S, score tile P of the NEXT chunk), Y consumes their bf16 forms into the
// output accumulator. Orderings that a single issuing thread would get for free are explicit
// mbarrier edges here (see the role comments).
#pragma once
#include "ptx.cuh"

#include <type_traits>

namespace fla {

constexpr int kChunk = 128;                // tokens per chunk (= MMA M)
constexpr int kThreads = 480;              // 15 warps
constexpr int kGroupBytes = kChunk * 128;  // one 64-column group of a chunk tile: 128 rows x 128 B

struct Problem {
  CUtensorMap q, k, v;     // 4-D maps (dim, token, head, batch), box 64 x 128 x 1 x 1, 128B swizzle
  CUtensorMap o;           // output map with a 64 x 32 box: every epilogue warp stores its own rows
  const float* s_init;     // [bh * segments + g][st_rows][st_cols] fp32, or null
  float* s_final;          // same indexing, or null
  int flags;               // kFlag* bits below
  int st_trans;            // state arrays are stored transposed: element (row, col) at [col][row]
  int n_tokens;            // sequence length
  int add_trans;           // layout of s_add: transposed like st_trans
  const float* s_add;      // optional [bh][st_rows][st_cols] fp32 added to s_init for every segment
  // ---- fused segments only (KernelParams::fused): where the state a segment starts from comes from
  int init_kind;           // kInitParts: s_add + the partial sums of all earlier segments;
                           // kInitBound: segment 0 starts from s_add, segment g >= 1 from ONE stored
                           // boundary state, slot bound_slot0 - g * bound_step of init_base
  int init_trans;          // layout of the init_base arrays relative to this product's state
  const float* init_base;  // kInitParts: [bh][segments * splits][rows*cols] (KernelParams::part_out);
                           // kInitBound: [bh][init_stride][rows*cols]
  int init_stride;         // kInitBound: boundary states per head
  int bound_slot0, bound_step;
  float* bound_out;        // optional: segment g >= 1 stores the state it starts from at slot g - 1 of
                           // [bh][segments - 1][rows*cols], scratch layout (a later pass reads it back
                           // through kInitBound)
};
constexpr int kInitParts = 0;
constexpr int kInitBound = 1;

// Problem::flags
constexpr int kFlagDescending = 1;  // walk the chunks from the last token to the first
constexpr int kFlagUpperMask = 2;   // keep (a_i . b_j) for j >= i instead of j <= i
// "Total minus suffix" form of the causal (j <= i) sum for a descending walk: the state starts as
// the sum over ALL tokens (s_init), every chunk SUBTRACTS its b^T c after using the state, and the
// intra-chunk tile contributes -(a_i . b_j) for j > i, because the state a chunk sees still
// contains that chunk's own tokens:  sum_{j<=i} = sum_{j in chunks <= this one} - sum_{j>i, same chunk}.
constexpr int kFlagTotalMinusSuffix = 4;
// With kFlagTotalMinusSuffix: the sequence has no tokens before token 0 of this call, so the state
// seen by the first chunk is exactly that chunk's own sum. That chunk is then computed from its
// score tile alone (ordinary lower mask, no state term); otherwise its first rows would be the
// small difference of two 128-term sums and lose accuracy.
constexpr int kFlagFirstChunkExact = 8;

struct KernelParams {
  Problem prob[3];
  int heads;       // heads per batch entry (block z = b * heads + h; block x = problem)
  int nchunks;     // ceil(seqlen / 128)
  int seg_chunks;  // chunks per segment (block y = segment index in scan order)
  int mode;        // 0: attention, 1: state only (sum of K^T V over the segment -> s_final)
  int st_rows;     // valid rows / cols of the state arrays in global memory
  int st_cols;
  int skip_last_segment;  // mode 1: the last segment's sum is not needed
  int* status;     // device word, bit 0 set when a bounded wait ran out; may be null
  unsigned wait_limit_us;  // limit of one bounded wait in microseconds of the global timer; 0 = default
  int debug_withhold;  // test hook: the producer skips the load of its first tile, so that the
                       // consumers' bounded wait runs out and the status path is exercised
  // ---- fused segments: ONE launch does what mode 1 + the scan kernel + mode 0 do in three.
  // Phase A: the sums of b^T c over segments 0 .. segments - 2 are needed (operands and walking
  // direction of problem `pre_prob`); all gridDim.x * gridDim.y CTAs of a head share that work,
  // CTA number c (= segment * gridDim.x + blockIdx.x) summing share c % shares of segment
  // c / shares, and store their sums as slot c of the head in part_out. The CTAs of a head then meet
  // at a barrier (the launch must be cooperative: every CTA resident), turn the partials into
  // per-segment prefixes together (each CTA scans some of the state's elements over all slots, in
  // place: the prefix of segment s lands in slot s * shares - 1), meet again, and each CTA takes
  // the prefix of its segment as its starting state and runs the attention loop.
  int fused;
  int pre_prob;
  float* part_out;
  unsigned bar_slot;   // which pair of g_grid_barriers this launch uses
};

// Barrier words of the fused form. Only the CTAs of one head exchange data, so every head has its
// own two barriers (after the partial sums, after the scan): [launch slot][head][barrier] pairs of
// (arrival count, generation), zero when the module is loaded and left consistent by every launch
// (see ptx::grid_barrier). The host hands out the launch slots round-robin, so launches that may
// overlap on the GPU use different words.
constexpr int kGridBarSlots = 64;
constexpr int kBarHeads = 80;  // the fused form needs heads * segments * products <= SM count anyway
static __device__ unsigned g_grid_barriers[kGridBarSlots * kBarHeads * 2 * 2];

template <int DK, int DV>
struct Cfg {
  static_assert(DK == DV, "tile ring assumes equally sized q/k and v tiles");
  static_assert(DK % 64 == 0 && DK <= 128, "unsupported head dims");
  static constexpr int GK = DK / 64;
  static constexpr int GV = DV / 64;
  static constexpr int TILE_BYTES = GK * kGroupBytes;  // one chunk tile of q, k or v
  static constexpr int SB_BYTES = GV * DK * 128;       // bf16 state as MMA B operand
  static constexpr int OST_BYTES = GV * kGroupBytes;   // output staging for the TMA store
  static constexpr int BAR_BYTES = 512;
  static constexpr int SMEM_LIMIT = 232448;  // 227 KB
  static constexpr int NSLOT_RAW =
      (SMEM_LIMIT - 1024 - BAR_BYTES - SB_BYTES - OST_BYTES) / TILE_BYTES;
  static constexpr int NSLOT = NSLOT_RAW > 9 ? 9 : NSLOT_RAW;
  static_assert(NSLOT >= 5, "need at least five tile slots");
  static constexpr int SMEM_BYTES = 1024 + NSLOT * TILE_BYTES + SB_BYTES + OST_BYTES + BAR_BYTES;
  static_assert(SMEM_BYTES <= SMEM_LIMIT, "shared memory budget");
  static_assert((2 * NSLOT + 12) * 8 + 16 <= BAR_BYTES, "barrier area");
  // TMEM columns (32-bit each, 128 lanes)
  static constexpr int P_COL = 0;         // P fp32: 128 columns
  static constexpr int PB_COL = 128;      // P bf16 (two per column): two buffers of 64 columns
  // O fp32: DV columns per buffer. With DV <= 64 there is room for two accumulators, so issuer Y
  // starts chunk i + 1 while the epilogue still reads chunk i; with DV = 128 tensor memory is full
  // and the accumulator is single.
  static constexpr int O_BUFS = (DV <= 64) ? 2 : 1;
  static constexpr int O_COL = 256;
  static constexpr int S_COL = 256 + O_BUFS * DV;  // S fp32: DV columns, lane = dk index
  static constexpr int TMEM_COLS = 512;
  static_assert(S_COL + DV <= TMEM_COLS, "TMEM budget");
};

// Arguments of converter_prologue(): where the CTA is and where its buffers and barriers are.
struct PrologueArgs {
  int prob_idx, g, nseg, bh, a_iter;
  uint32_t tmem_base, sb_addr, ost_addr;
  uint32_t s_full, part_done, grid_done, sb_ready;  // mbarrier addresses
  volatile int* abort_flag;
};

// What the converter warps (2..9) do before the chunk loop. Fused form: store the partial sum of
// phase A, meet the head's other CTAs, scan, meet again. Then, whenever the CTA starts from a
// state: fetch it, write it to TMEM (fp32) and to the operand buffer (16-bit) and release the MMA
// issuers. Returns false when a bounded wait gave up.
template <int DK, int DV, bool HALF>
__device__ __noinline__ bool converter_prologue(const KernelParams& p, const PrologueArgs pa) {
  using cfg = Cfg<DK, DV>;
  const int warp = static_cast<int>(threadIdx.x >> 5);
  const int lane = static_cast<int>(threadIdx.x & 31);
  const int g = pa.g, nseg = pa.nseg, bh = pa.bh, a_iter = pa.a_iter;
  // Copies of the parameters this function reads inside its loops: `p` is a generic reference here,
  // and the L2 loads below are volatile with memory clobbers, so a p.x in a loop would be fetched
  // again after every one of them.
  const Problem& pr = p.prob[pa.prob_idx];
  const int st_rows = p.st_rows, st_cols = p.st_cols, seg_chunks = p.seg_chunks;
  float* const part_out = p.part_out;
  const unsigned bar_slot = p.bar_slot % kGridBarSlots;
  float* const bound_out = pr.bound_out;
  const bool fused = p.fused != 0;
  const bool has_init = fused || pr.s_init != nullptr;
  const uint32_t sb_addr = pa.sb_addr, ost_addr = pa.ost_addr;
  const uint32_t s_full = pa.s_full, part_done = pa.part_done, grid_done = pa.grid_done, sb_ready = pa.sb_ready;
  volatile int* abort_flag = pa.abort_flag;
  const size_t st_elems = static_cast<size_t>(st_rows) * st_cols;
  const size_t st_index = (fused ? static_cast<size_t>(bh) : static_cast<size_t>(bh) * nseg + g) * st_elems;
  const bool st_trans = pr.st_trans != 0;
  const int half = (warp - 2) >> 2;
  const int quad = warp & 3;
  const int row = quad * 32 + lane;
  const uint32_t lane_base = pa.tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
  const uint32_t sb_row = sb_addr + row * 128;
  const uint32_t swz = static_cast<uint32_t>(row & 7);
  constexpr int SBLK = DV / 64;
  constexpr bool kStagedStateIO = (DK == 128);
  const uint32_t xpose_off = static_cast<uint32_t>(warp - 2) * 4096u;
  uint32_t ra[32], rb[32];
  auto wait_uniform = [&](uint32_t bar, uint32_t parity) {
    const int ok = ptx::mbar_wait(bar, parity, abort_flag) ? 1 : 0;
    return __all_sync(0xffffffffu, ok) != 0;
  };
  auto xpose_addr = [&](uint32_t base, int j, int r) {
    return base + xpose_off + static_cast<uint32_t>((j * 32 + (r ^ j)) * 4);
  };
  auto store_sb = [&](int cb, const uint32_t (&r)[32]) {
    const uint32_t grp = sb_row + (cb >> 1) * (DK * 128);
    const uint32_t j0 = (cb & 1) * 4;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const uint32_t a0 = ptx::pack16x2<HALF>(__uint_as_float(r[jj * 8 + 0]), __uint_as_float(r[jj * 8 + 1]));
      const uint32_t a1 = ptx::pack16x2<HALF>(__uint_as_float(r[jj * 8 + 2]), __uint_as_float(r[jj * 8 + 3]));
      const uint32_t a2 = ptx::pack16x2<HALF>(__uint_as_float(r[jj * 8 + 4]), __uint_as_float(r[jj * 8 + 5]));
      const uint32_t a3 = ptx::pack16x2<HALF>(__uint_as_float(r[jj * 8 + 6]), __uint_as_float(r[jj * 8 + 7]));
      ptx::st_shared_v4(grp + (((j0 + jj) ^ swz) << 4), a0, a1, a2, a3);
    }
  };

  // Scratch of the fused form (partial sums, scanned prefixes, stored boundary states): one state
  // is DK x DV floats whatever the real head dims are (the rows and columns beyond them hold the
  // zeros the MMAs produce from zero-filled tiles), in "fragment order": element (r, c) sits at
  // ((c / 4) * DK + r) * 4 + c % 4. A thread owns a row, so its 32 columns of a block are eight
  // 16-byte vectors DK * 16 bytes apart, and a warp's vector access covers 512 contiguous bytes.
  // All strides are compile-time constants: the code that moves a block is 8 (or, for the
  // transposed read, 32) instructions with immediate offsets. That matters more than the byte
  // count: this code runs once per CTA, straight from a cold instruction cache.
  constexpr size_t kFragElems = static_cast<size_t>(DK) * DV;
  constexpr int kFragVecStride = DK * 16;  // bytes between consecutive 4-column groups of a row
  auto store_frag = [&](float* state, int cb, const uint32_t (&r)[32]) {
    float* ptr = state + (static_cast<size_t>(cb) * 8 * DK + row) * 4;
    ptx::static_for<8>([&](auto i) {
      constexpr int I = decltype(i)::value;
      ptx::st_global_cg_v4<I * kFragVecStride>(ptr, r[4 * I], r[4 * I + 1], r[4 * I + 2], r[4 * I + 3]);
    });
  };
  auto load_frag = [&](const float* state, int cb, uint32_t (&r)[32]) {
    const float* ptr = state + (static_cast<size_t>(cb) * 8 * DK + row) * 4;
    ptx::static_for<8>([&](auto i) {
      constexpr int I = decltype(i)::value;
      ptx::ld_global_cg_v4<I * kFragVecStride>(ptr, r[4 * I], r[4 * I + 1], r[4 * I + 2], r[4 * I + 3]);
    });
    ptx::keep_together(r);
  };
  // Stores the transpose: element (row, col) of the product goes to position (r = col, c = row).
  // Stores are not waited for, so the 32 scalar instructions cost issue slots only; the reader
  // (the dQ product of a later backward call, whose state is the transpose) then loads vectors.
  auto store_frag_transposed = [&](float* state, int cb, const uint32_t (&r)[32]) {
    float* ptr = state + (static_cast<size_t>(row >> 2) * DK + cb * 32) * 4 + (row & 3);
    ptx::static_for<32>([&](auto j) {
      constexpr int J = decltype(j)::value;
      ptx::st_global_cg_b32_at<J * 16>(ptr, r[J]);
    });
  };
  // The stored state is the transpose of this product's state: element (row, col) of the product
  // is stored element (r = col, c = row).
  auto load_frag_transposed = [&](const float* state, int cb, uint32_t (&r)[32]) {
    const float* ptr = state + (static_cast<size_t>(row >> 2) * DK + cb * 32) * 4 + (row & 3);
    ptx::static_for<32>([&](auto j) {
      constexpr int J = decltype(j)::value;
      r[J] = ptx::ld_global_cg_b32_at<J * 16>(ptr);
    });
    ptx::keep_together(r);
  };

  bool conv_ok = true;
  unsigned gen0 = 0, gen1 = 0;  // barrier generations, fetched while phase A still runs
  if (fused && warp == 2 && lane == 0) {
    gen0 = ptx::barrier_generation(&g_grid_barriers[((bar_slot * kBarHeads + bh) * 2 + 0) * 2]);
    gen1 = ptx::barrier_generation(&g_grid_barriers[((bar_slot * kBarHeads + bh) * 2 + 1) * 2]);
  }
  if (fused) {
    // ---------------- phase A read-out: this CTA's partial sum -> part_out (scratch layout,
    // one thread per state row), then the barrier of the head's CTAs. Every CTA takes part in
    // the barriers, whether it had chunks to sum or not.
    if (a_iter > 0) {
      int ok = ptx::mbar_wait(s_full, 0, abort_flag) ? 1 : 0;
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        ptx::tc_fence_after();
        const size_t slot = static_cast<size_t>(bh) * (static_cast<size_t>(nseg) * gridDim.x) +
                            static_cast<size_t>(g) * gridDim.x + blockIdx.x;  // CTA number within the head
        float* dst = part_out + slot * kFragElems;
#pragma unroll 1
        for (int jb = 0; jb < SBLK; ++jb) {
          const int cb = half * SBLK + jb;
          ptx::tmem_ld32(lane_base + cfg::S_COL + cb * 32, ra);
          if (row < DK) store_frag(dst, cb, ra);
        }
        ptx::tc_fence_before();
      }
      conv_ok = ok != 0;
    }
    // Barrier of this head's CTAs: every converter thread fences its stores and reports on an
    // mbarrier; one warp then arrives at the head's barrier word, waits for the other CTAs of
    // the head and releases the group. Used twice (after the partials, after the scan).
    const unsigned head_ctas = gridDim.x * gridDim.y;
    auto head_bar_words = [&](int which) {
      return &g_grid_barriers[((bar_slot * kBarHeads + bh) * 2 + which) * 2];
    };
    auto head_barrier = [&](int which, unsigned gen_before) {
      __threadfence();
      if (conv_ok) ptx::mbar_arrive(part_done);
      if (warp == 2) {
        bool ok = wait_uniform(part_done, which);
        if (ok) {
          int passed = 1;
          if (lane == 0)
            passed = ptx::grid_barrier(head_bar_words(which), head_ctas, gen_before, abort_flag) ? 1 : 0;
          ok = __shfl_sync(0xffffffffu, passed, 0) != 0;
        }
        if (ok && lane == 0) ptx::mbar_arrive(grid_done);
      }
      if (conv_ok) {
        const int ok = ptx::mbar_wait(grid_done, which, abort_flag) ? 1 : 0;
        conv_ok = __all_sync(0xffffffffu, ok) != 0;
      }
    };
    head_barrier(0, gen0);
    if (conv_ok && nseg > 1) {
      // ---------------- scan: partial sums -> exclusive prefixes per segment, in place. The
      // head's CTAs share the state's 16-byte vectors (units of 256, one vector per thread); a
      // thread walks ALL slots of its vector in order (slot j = share j % shares of segment
      // j / shares): after the last share of segment s the running sum is the prefix of segment
      // s + 1 and overwrites that last share's slot, (s + 1) * shares - 1, whose partial has just
      // been consumed. kScanSlots slots are loaded at a time, all loads before the first use.
      constexpr int kScanSlots = 8;
      constexpr int kUnits = static_cast<int>(kFragElems / 4 / 256);
      const int nsplit = static_cast<int>(gridDim.x);
      const int shares = static_cast<int>(head_ctas) / (nseg - 1);
      const int tid = (warp - 2) * 32 + lane;
      float* hb = part_out + static_cast<size_t>(bh) * head_ctas * kFragElems;
      const int nslots = (nseg - 1) * shares;                // slots that can hold a partial
      const int last_slot = static_cast<int>(head_ctas) - 1;  // last slot of this head's scratch
      // bit x: share x of a segment is not empty (a CTA with an empty share stored nothing)
      unsigned stored_mask = 0;
      for (int x = 0; x < shares; ++x)
        if (seg_chunks * (x + 1) / shares - seg_chunks * x / shares > 0) stored_mask |= 1u << x;
#pragma unroll 1
      for (int unit = g * nsplit + static_cast<int>(blockIdx.x); unit < kUnits;
           unit += static_cast<int>(head_ctas)) {
        float* vec = hb + (static_cast<size_t>(unit) * 256 + tid) * 4;
        float run[4] = {0.f, 0.f, 0.f, 0.f};
        int x0 = 0;  // share index of slot j0
#pragma unroll 1
        for (int j0 = 0; j0 < nslots; j0 += kScanSlots) {
          uint32_t val[4 * kScanSlots];
          static_assert(4 * kScanSlots == 32, "one keep_together() per batch");
#pragma unroll
          for (int jj = 0; jj < kScanSlots; ++jj) {
            const float* src = vec + static_cast<size_t>(min(j0 + jj, last_slot)) * kFragElems;
            ptx::ld_global_cg_v4<0>(src, val[4 * jj], val[4 * jj + 1], val[4 * jj + 2], val[4 * jj + 3]);
          }
          ptx::keep_together(val);  // all loads of the batch before any store
          int x = x0;
#pragma unroll
          for (int jj = 0; jj < kScanSlots; ++jj) {
            const int j = j0 + jj;
            if (j < nslots) {
              if ((stored_mask >> x) & 1u) {
#pragma unroll
                for (int u = 0; u < 4; ++u) run[u] += __uint_as_float(val[4 * jj + u]);
              }
              if (x + 1 == shares) {
                ptx::st_global_cg_v4<0>(vec + static_cast<size_t>(j) * kFragElems, __float_as_uint(run[0]),
                                        __float_as_uint(run[1]), __float_as_uint(run[2]),
                                        __float_as_uint(run[3]));
                x = 0;
              } else {
                ++x;
              }
            }
          }
          x0 = x;
        }
      }
    }
    head_barrier(1, gen1);
  }

  if (has_init && conv_ok) {
    // ---------------- phase B: the state this CTA starts from -> TMEM (fp32) and the bf16
    // operand buffer: an optional array of the caller plus `nsrc` arrays `stride` elements apart
    // (the segment's stored state; partial sums of earlier segments; one stored boundary state).
    //
    // fetch(): one 32-column block of a [st_rows][st_cols] array (transposed storage if `trans`)
    // into a register array, zero outside the valid part. All 32 loads are issued before their
    // first use (volatile loads keep their order), so every thread has 32 requests in flight:
    // the arrays sit in L2 (loads bypass L1: in the fused form other CTAs of the same launch wrote
    // them) and the step is pure latency otherwise. Row-major arrays are fetched along rows by
    // the lanes (whole 128-byte segments per warp instruction) and settle() then exchanges them
    // through the output staging buffer, which is idle before chunk 0.
    const bool full_tile = st_rows == DK && st_cols == DV;  // no element of a block is padding
    auto fetch = [&](int cb, const float* base, bool trans, uint32_t (&r)[32]) {
      if (full_tile) {
        // same access patterns as below with every offset an immediate and no bounds tests: a
        // quarter of the instructions, which is what this once-per-CTA code costs in
        if (trans) {
          // rows beyond the state (DK = 64: the upper two warp quadrants) load row 0 and are zeroed below
          const float* ptr = base + static_cast<size_t>(cb) * 32 * DK + (row < DK ? row : 0);
          ptx::static_for<32>([&](auto j) {
            constexpr int J = decltype(j)::value;
            r[J] = ptx::ld_global_cg_b32_at<J * DK * 4>(ptr);
          });
        } else if (kStagedStateIO) {
          const float* ptr = base + static_cast<size_t>(quad) * 32 * DV + cb * 32 + lane;
          ptx::static_for<32>([&](auto j) {
            constexpr int J = decltype(j)::value;
            r[J] = ptx::ld_global_cg_b32_at<J * DV * 4>(ptr);
          });
        } else {
          const float* ptr = base + static_cast<size_t>(row < DK ? row : 0) * DV + cb * 32;
          ptx::static_for<8>([&](auto j) {
            constexpr int J = decltype(j)::value;
            ptx::ld_global_cg_v4<J * 16>(ptr, r[4 * J], r[4 * J + 1], r[4 * J + 2], r[4 * J + 3]);
          });
        }
        ptx::keep_together(r);
        if (!kStagedStateIO || trans) {
          if (row >= DK) {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0u;
          }
        }
        return;
      }
      if (kStagedStateIO && !trans) {
        const int col = cb * 32 + lane;
#pragma unroll
        for (int rr = 0; rr < 32; ++rr) {
          const int grow = quad * 32 + rr;
          const bool valid = col < st_cols && grow < st_rows;
          r[rr] = ptx::ld_global_cg_b32(base + (valid ? static_cast<size_t>(grow) * st_cols + col : 0));
        }
        ptx::keep_together(r);
#pragma unroll
        for (int rr = 0; rr < 32; ++rr)
          if (!(col < st_cols && quad * 32 + rr < st_rows)) r[rr] = 0u;
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = cb * 32 + j;
          const bool valid = row < st_rows && col < st_cols;
          const size_t off = trans ? static_cast<size_t>(col) * st_rows + row
                                   : static_cast<size_t>(row) * st_cols + col;
          r[j] = ptx::ld_global_cg_b32(base + (valid ? off : 0));
        }
        ptx::keep_together(r);
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (!(row < st_rows && cb * 32 + j < st_cols)) r[j] = 0u;
      }
    };
    auto settle = [&](bool trans, uint32_t (&r)[32]) {
      if (kStagedStateIO && !trans) {
        const uint32_t base = ost_addr;
#pragma unroll
        for (int rr = 0; rr < 32; ++rr) ptx::st_shared_b32(xpose_addr(base, lane, rr), r[rr]);
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = ptx::ld_shared_b32(xpose_addr(base, j, lane));
        __syncwarp();
      }
    };
    const bool add_trans = pr.add_trans != 0;
    const size_t head_index = static_cast<size_t>(bh) * st_elems;
    if (!fused) {
      // one array in the layout the state pass / the caller wrote, plus the caller's state
      const float* src = pr.s_init + st_index;
      const float* add = pr.s_add != nullptr ? pr.s_add + head_index : nullptr;
#pragma unroll 1
      for (int jb = 0; jb < SBLK; ++jb) {
        const int cb = half * SBLK + jb;
        fetch(cb, src, st_trans, ra);
        settle(st_trans, ra);
        if (add != nullptr) {
          fetch(cb, add, add_trans, rb);
          settle(add_trans, rb);
#pragma unroll
          for (int c = 0; c < 32; ++c)
            ra[c] = __float_as_uint(__uint_as_float(ra[c]) + __uint_as_float(rb[c]));
        }
        ptx::tmem_st32(lane_base + cfg::S_COL + cb * 32, ra);
        if (row < DK) store_sb(cb, ra);
      }
    } else {
      static_assert(DK == DV, "the transposed read of a stored state assumes square scratch states");
      // Fused form. Segment g >= 1 starts from ONE scratch state: the scanned prefix of its
      // segment (slot g * nsplit of the head) or a boundary state an earlier call stored; the
      // caller's state is added for every segment (partial sums) or is all segment 0 has (boundary
      // states). `own`: the scratch state has this product's orientation.
      const bool bound = pr.init_kind == kInitBound;
      const float* add = (pr.s_add != nullptr && (!bound || g == 0)) ? pr.s_add + head_index : nullptr;
      const bool own = pr.init_trans != 0;
      const float* src = nullptr;
      if (g > 0) {
        // the scanned prefix of segment g sits in the last share slot of segment g - 1
        const size_t head_ctas = static_cast<size_t>(nseg) * gridDim.x;
        const size_t slot = bound ? static_cast<size_t>(bh) * pr.init_stride + (pr.bound_slot0 - g * pr.bound_step)
                                  : static_cast<size_t>(bh) * head_ctas + g * (head_ctas / (nseg - 1)) - 1;
        src = pr.init_base + slot * kFragElems;
      }
      float* keep = (bound_out != nullptr && g > 0)
                        ? bound_out + (static_cast<size_t>(bh) * (nseg - 1) + (g - 1)) * kFragElems
                        : nullptr;
#pragma unroll 1
      for (int jb = 0; jb < SBLK; ++jb) {
        const int cb = half * SBLK + jb;
        if (src != nullptr && row < DK) {
          if (own) load_frag(src, cb, ra);
          else load_frag_transposed(src, cb, ra);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) ra[j] = 0u;
        }
        if (add != nullptr) {
          fetch(cb, add, add_trans, rb);
          settle(add_trans, rb);
#pragma unroll
          for (int c = 0; c < 32; ++c)
            ra[c] = __float_as_uint(__uint_as_float(ra[c]) + __uint_as_float(rb[c]));
        }
        if (keep != nullptr && row < DK) store_frag_transposed(keep, cb, ra);
        ptx::tmem_st32(lane_base + cfg::S_COL + cb * 32, ra);
        if (row < DK) store_sb(cb, ra);
      }
    }
    ptx::tc_wait_st();
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before();
    ptx::mbar_arrive(sb_ready);
  }

  return conv_ok;
}

// HALF: operands and outputs are fp16 instead of bf16 (same tiles, same pipeline; only the MMA
// operand format and the fp32 -> 16-bit roundings differ).
template <int DK, int DV, bool HALF = false>
__global__ void __launch_bounds__(kThreads, 1)
fla_chunk_kernel(const __grid_constant__ KernelParams p) {
  using cfg = Cfg<DK, DV>;
  constexpr int NSLOT = cfg::NSLOT;
  extern __shared__ uint8_t smem_raw[];

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // provably warp-uniform
  const int lane = threadIdx.x & 31;
  const int prob_idx = blockIdx.x;
  const int g = blockIdx.y;
  const int nseg = gridDim.y;
  const int bh = blockIdx.z;
  const int mode = p.mode;
  if (mode == 1 && p.skip_last_segment && g == nseg - 1) return;  // whole CTA, before any setup

  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - raw_addr);

  const uint32_t sb_addr = smem_base + NSLOT * cfg::TILE_BYTES;
  const uint32_t ost_addr = sb_addr + cfg::SB_BYTES;
  const uint32_t bar_base = ost_addr + cfg::OST_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (NSLOT + s); };
  const uint32_t p_full = bar_base + 8u * (2 * NSLOT + 0);
  const uint32_t pb_ready = bar_base + 8u * (2 * NSLOT + 1);
  // One o_full barrier per bf16-P buffer (chunk parity): a waiter that needs "chunk i-1 is done"
  // must not be overtaken by the completion for chunk i, which a shared barrier would allow.
  const uint32_t o_full0 = bar_base + 8u * (2 * NSLOT + 2);
  const uint32_t o_full1 = bar_base + 8u * (2 * NSLOT + 7);
  const uint32_t qs_done = bar_base + 8u * (2 * NSLOT + 6);
  const uint32_t p_read = bar_base + 8u * (2 * NSLOT + 8);
  const uint32_t sb_ready = bar_base + 8u * (2 * NSLOT + 3);
  // one o_free barrier per accumulator buffer (both names denote the same barrier when there is one)
  const uint32_t o_free0 = bar_base + 8u * (2 * NSLOT + 5);
  const uint32_t o_free1 = cfg::O_BUFS == 2 ? bar_base + 8u * (2 * NSLOT + 9) : o_free0;
  const uint32_t s_full = bar_base + 8u * (2 * NSLOT + 4);
  const uint32_t part_done = bar_base + 8u * (2 * NSLOT + 10);  // fused: partial sum stored (256 arrivals)
  const uint32_t grid_done = bar_base + 8u * (2 * NSLOT + 11);  // fused: the grid barrier was passed
  const uint32_t holder_off =
      NSLOT * cfg::TILE_BYTES + cfg::SB_BYTES + cfg::OST_BYTES + 8u * (2 * NSLOT + 12);
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem_gen + holder_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + holder_off + 4);

  const Problem& pr = p.prob[prob_idx];
  const int h = bh % p.heads;
  const int b = bh / p.heads;
  const int chunk0 = g * p.seg_chunks;
  const int n_iter = min(p.seg_chunks, p.nchunks - chunk0);
  const bool descending = (pr.flags & kFlagDescending) != 0;
  const bool tms = (pr.flags & kFlagTotalMinusSuffix) != 0;
  const bool upper_flag = (pr.flags & kFlagUpperMask) != 0;
  const bool exact0 = tms && (pr.flags & kFlagFirstChunkExact) != 0;
  // Fused segments: every CTA loads a starting state (possibly all zeros), see phase B below.
  const bool fused = (mode == 0) && (p.fused != 0);
  const bool has_init = (mode == 0) && (fused || pr.s_init != nullptr);
  // Phase A of the fused form: this CTA's share of its segment's chunks, in the scan order of the
  // problem whose state is being summed. The last segment's sum is not needed by anyone.
  const Problem& pre = p.prob[fused ? p.pre_prob : prob_idx];
  const bool pre_desc = (pre.flags & kFlagDescending) != 0;
  int a_lo = 0, a_iter = 0, a_chunk0 = 0;
  if (fused && nseg > 1) {
    // The nseg - 1 segments whose sums are needed are shared by ALL CTAs of the head, `shares` per
    // segment (the CTA that later walks the last segment sums too): CTA number c of the head takes
    // share c % shares of segment c / shares. Partial c goes to slot c of the head's scratch.
    const int head_ctas = nseg * static_cast<int>(gridDim.x);
    const int c = g * static_cast<int>(gridDim.x) + static_cast<int>(blockIdx.x);
    const int shares = head_ctas / (nseg - 1);
    if (c < shares * (nseg - 1)) {
      const int sa = c / shares, xa = c - sa * shares;
      a_chunk0 = sa * p.seg_chunks;
      a_lo = p.seg_chunks * xa / shares;
      a_iter = p.seg_chunks * (xa + 1) / shares - a_lo;
    }
  }
  const int t0 = 2 * a_iter;  // the tiles of phase A come first in the ring numbering
  const size_t st_elems = static_cast<size_t>(p.st_rows) * p.st_cols;
  // state arrays are indexed per (head, segment), except in the fused form, whose only such array
  // is the caller's final state (one per head)
  const size_t st_index = (p.fused ? static_cast<size_t>(bh)
                                   : static_cast<size_t>(bh) * nseg + g) * st_elems;
  const bool st_trans = pr.st_trans != 0;
  auto st_off = [&](int row, int col) {
    return st_index + (st_trans ? static_cast<size_t>(col) * p.st_rows + row
                                : static_cast<size_t>(row) * p.st_cols + col);
  };
  // Tiles are numbered in load order: chunk i holds tiles t0 + tpc*i + {0: q, 1: k, 2: v} (mode 0)
  // or 2*i + {0: k, 1: v} (mode 1, and phase A of the fused form); tile t lives in slot t % NSLOT
  // during ring pass t / NSLOT.
  const int tpc = (mode == 0) ? 3 : 2;

  // ------------------------------------------------------------------ setup
  if (threadIdx.x == 0) {
    abort_flag[0] = 0;
    abort_flag[1] = static_cast<int>(p.wait_limit_us);
    for (int s = 0; s < NSLOT; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      // mode 0: every tile is read by two MMA groups, each followed by a tcgen05.commit arrival
      ptx::mbar_init(empty_bar(s), mode == 0 ? 2 : 1);
    }
    ptx::mbar_init(p_full, 1);
    ptx::mbar_init(pb_ready, 256);
    ptx::mbar_init(o_full0, 1);
    ptx::mbar_init(o_full1, 1);
    ptx::mbar_init(qs_done, 1);
    ptx::mbar_init(p_read, 256);
    ptx::mbar_init(sb_ready, 256);
    ptx::mbar_init(o_free0, 128);
    if (cfg::O_BUFS == 2) ptx::mbar_init(o_free1, 128);
    ptx::mbar_init(s_full, 1);
    ptx::mbar_init(part_done, 256);
    ptx::mbar_init(grid_done, 1);
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_holder)), cfg::TMEM_COLS);
    ptx::tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    if (mode == 0) {
      ptx::prefetch_tensormap(&pr.q);
      ptx::prefetch_tensormap(&pr.o);
    }
    ptx::prefetch_tensormap(&pr.k);
    ptx::prefetch_tensormap(&pr.v);
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  // Wait executed by a whole warp; the outcome is made uniform so that the warp never diverges
  // around .sync.aligned instructions.
  auto wait_uniform = [&](uint32_t bar, uint32_t parity) {
    const int ok = ptx::mbar_wait(bar, parity, abort_flag) ? 1 : 0;
    return __all_sync(0xffffffffu, ok) != 0;
  };
  auto mem_chunk = [&](int i) {
    return descending ? (p.nchunks - 1 - (chunk0 + i)) : (chunk0 + i);
  };
  // chunk i is computed without the state (see kFlagFirstChunkExact)
  auto plain_chunk = [&](int i) { return exact0 && mem_chunk(i) == 0; };
  auto pre_mem_chunk = [&](int i) {
    const int c = a_chunk0 + a_lo + i;
    return pre_desc ? (p.nchunks - 1 - c) : c;
  };
  auto slot_addr = [&](int t) {
    return smem_base + static_cast<uint32_t>(t % NSLOT) * cfg::TILE_BYTES;
  };

  if (warp == 0) {
    // ================================================================ TMA producer
    // The whole warp runs the loop (so that addresses and coordinates stay warp-uniform); one
    // elected lane issues. In mode 0 the q and k tiles of a chunk complete on the q tile's barrier.
    const bool leader = ptx::elect_one();
    const int n_tiles = t0 + n_iter * tpc;
    for (int t = 0; t < n_tiles; ++t) {
      const int s = t % NSLOT;
      const uint32_t ph = (t / NSLOT) & 1;
      if (!wait_uniform(empty_bar(s), ph ^ 1u)) break;
      const bool phase_a = t < t0;  // k, v tiles of the summed problem, each on its own barrier
      const int tt = phase_a ? t : t - t0;
      const int i = phase_a ? (tt >> 1) : tt / tpc;
      const int which = phase_a ? 1 + (tt & 1) : tt - i * tpc + (mode == 0 ? 0 : 1);  // 0 q, 1 k, 2 v
      const Problem& src = phase_a ? pre : pr;
      const CUtensorMap* map = (which == 0) ? &src.q : (which == 1 ? &src.k : &src.v);
      const uint32_t dst = slot_addr(t);
      const int tok = (phase_a ? pre_mem_chunk(i) : mem_chunk(i)) * kChunk;
      const bool paired = mode == 0 && !phase_a;  // q and k of a chunk complete on q's barrier
      // barrier that the tile's bytes complete on, and the bytes armed on it at this point
      const uint32_t bar = (paired && which == 1) ? full_bar((t - 1) % NSLOT) : full_bar(s);
      if (leader) {
        if (paired && which == 0) ptx::mbar_expect_tx(bar, 2 * cfg::TILE_BYTES);
        if (!paired || which == 2) ptx::mbar_expect_tx(bar, cfg::TILE_BYTES);
        // The k slot's own barrier is not waited on; complete its phase so that the parity of
        // later ring passes stays in step.
        if (paired && which == 1) ptx::mbar_arrive(full_bar(s));
        if (!(p.debug_withhold && t == 0)) {
#pragma unroll
          for (int gg = 0; gg < cfg::GK; ++gg)
            ptx::tma_load_4d(dst + gg * kGroupBytes, map, bar, gg * 64, tok, h, b);
        }
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer X
    // S += K_i^T V_i, then P = Q_{i+1} K_{i+1}^T. The whole warp runs the loop with warp-uniform
    // operands; one elected lane issues the tcgen05.mma / tcgen05.commit instructions.
    // Edges it waits on besides tile arrival:
    //   sb_ready(i-1)  the converters have read S of chunk i-1 out of TMEM      (before S += ..)
    //   p_read(i)      the converters have read P of chunk i out of TMEM        (before P = ..)
    //   o_full(i-1)    issuer Y's P V of chunk i-1 is done: that bf16 P buffer is reused by
    //                  the conversion of the tile written here
    constexpr uint32_t IDESC_QK = ptx::make_idesc(128, kChunk, false, false, HALF);  // P  = Q K^T
    constexpr uint32_t IDESC_KV_ADD = ptx::make_idesc(128, DV, true, true, HALF);    // S += K^T V
    constexpr uint32_t IDESC_KV_SUB = IDESC_KV_ADD | (1u << 13);               // S -= K^T V (A negated)
    const uint32_t IDESC_KV = tms ? IDESC_KV_SUB : IDESC_KV_ADD;
    const uint32_t tP = tmem_base + cfg::P_COL;
    const uint32_t tS = tmem_base + cfg::S_COL;
    const bool leader = ptx::elect_one();
    auto wait_tile = [&](int t) { return wait_uniform(full_bar(t % NSLOT), (t / NSLOT) & 1); };
    auto release_tile = [&](int t) {
      if (leader) ptx::tc_commit(empty_bar(t % NSLOT));
    };
    // P = Q K^T of chunk i (both operands K-major, 16 columns of dk per instruction)
    auto issue_qk = [&](int i) {
      if (!wait_tile(t0 + 3 * i)) return false;  // covers the k tile too
      const uint32_t q_lo = ptx::desc_lo(slot_addr(t0 + 3 * i), 16);
      const uint32_t k_lo = ptx::desc_lo(slot_addr(t0 + 3 * i + 1), 16);
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk) {
          const uint32_t off = ((kk >> 2) * kGroupBytes + (kk & 3) * 32) >> 4;
          ptx::mma_ss(tP, q_lo + off, k_lo + off, ptx::kDescHi, IDESC_QK, kk > 0 ? 1u : 0u);
        }
        ptx::tc_commit(p_full);
      }
      release_tile(t0 + 3 * i);      // first of two arrivals on q (the other: issuer Y after Q Sb)
      release_tile(t0 + 3 * i + 1);  // first of two arrivals on k (the other: below, after K^T V)
      __syncwarp();
      return true;
    };
    if (mode == 0) {
      uint32_t sb_waits = 0;
      bool ok = true;
      // ---- phase A of the fused form: plain sum of b^T c over this CTA's share of the segment
      // (always added, whatever sign the CTA's own product uses), read out by the converters
      for (int i = 0; ok && i < a_iter; ++i) {
        if (!wait_tile(2 * i) || !wait_tile(2 * i + 1)) { ok = false; break; }
        const uint32_t k_lo = ptx::desc_lo(slot_addr(2 * i), kGroupBytes);
        const uint32_t v_lo = ptx::desc_lo(slot_addr(2 * i + 1), kGroupBytes);
        ptx::tc_fence_after();
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < kChunk / 16; ++kk) {
            ptx::mma_ss(tS, k_lo + kk * (2048 >> 4), v_lo + kk * (2048 >> 4), ptx::kDescHi,
                        IDESC_KV_ADD, (i > 0 || kk > 0) ? 1u : 0u);
          }
          // the ring's barriers expect two consumers per tile in mode 0
          ptx::tc_commit(empty_bar((2 * i) % NSLOT));
          ptx::tc_commit(empty_bar((2 * i) % NSLOT));
          ptx::tc_commit(empty_bar((2 * i + 1) % NSLOT));
          ptx::tc_commit(empty_bar((2 * i + 1) % NSLOT));
          if (i == a_iter - 1) ptx::tc_commit(s_full);
        }
        __syncwarp();
      }
      ok = ok && issue_qk(0);
      for (int i = 0; ok && i < n_iter; ++i) {
        // k, v MN-major: 64-column groups kGroupBytes apart
        const uint32_t k_lo = ptx::desc_lo(slot_addr(t0 + 3 * i + 1), kGroupBytes);
        const uint32_t v_lo = ptx::desc_lo(slot_addr(t0 + 3 * i + 2), kGroupBytes);
        const bool have_state = (i > 0) || has_init;
        // ---- S += K^T V  (both operands MN-major: the token index is the MMA K dimension).
        // For DK = 64 the instruction still spans 128 rows; the upper 64 read whatever follows
        // the K tile in shared memory and land in TMEM lanes nobody reads.
        if (have_state) {
          if (!wait_uniform(sb_ready, sb_waits & 1)) break;
          ++sb_waits;
        }
        if (!wait_tile(t0 + 3 * i + 2)) break;
        ptx::tc_fence_after();
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < kChunk / 16; ++kk) {
            ptx::mma_ss(tS, k_lo + kk * (2048 >> 4), v_lo + kk * (2048 >> 4), ptx::kDescHi,
                        IDESC_KV, kk > 0 ? 1u : (have_state ? 1u : 0u));
          }
          ptx::tc_commit(s_full);
        }
        release_tile(t0 + 3 * i + 1);
        release_tile(t0 + 3 * i + 2);  // first of two arrivals on v (the other: issuer Y after P V)
        // ---- score tile of the next chunk
        if (i + 1 < n_iter) {
          if (!wait_uniform(p_read, i & 1)) break;
          if (i >= 1 && !wait_uniform(((i - 1) & 1) ? o_full1 : o_full0, ((i - 1) >> 1) & 1)) break;
          ptx::tc_fence_after();
          ok = issue_qk(i + 1);
        }
      }
    } else {
      for (int i = 0; i < n_iter; ++i) {
        if (!wait_tile(2 * i) || !wait_tile(2 * i + 1)) break;
        const uint32_t k_lo = ptx::desc_lo(slot_addr(2 * i), kGroupBytes);
        const uint32_t v_lo = ptx::desc_lo(slot_addr(2 * i + 1), kGroupBytes);
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < kChunk / 16; ++kk) {
            ptx::mma_ss(tS, k_lo + kk * (2048 >> 4), v_lo + kk * (2048 >> 4), ptx::kDescHi,
                        IDESC_KV, (i > 0 || kk > 0) ? 1u : 0u);
          }
        }
        release_tile(2 * i);
        release_tile(2 * i + 1);
        if (leader && i == n_iter - 1) ptx::tc_commit(s_full);
        __syncwarp();
      }
    }
  } else if (warp == 14) {
    // ================================================================ MMA issuer Y
    // O = Q_i Sb_{i-1}, then O += Pb_i V_i. Edges besides tile arrival:
    //   o_free(i-1)   the epilogue has drained the accumulator of chunk i-1 (of chunk i-2 when
    //                 there are two accumulators)
    //   sb_ready(i-1) the bf16 state of chunk i-1 is in shared memory
    //   pb_ready(i)   the bf16 score tile of chunk i is in TMEM
    // and it signals qs_done(i) (the state buffer may be overwritten) and o_full(i).
    if (mode == 0) {
      constexpr uint32_t IDESC_PV = ptx::make_idesc(128, DV, false, true, HALF);  // O += Pb V
      constexpr uint32_t IDESC_QS = ptx::make_idesc(128, DV, false, true, HALF);  // O  = Q Sb
      const uint32_t tO0 = tmem_base + cfg::O_COL;
      const uint32_t sb_lo = ptx::desc_lo(sb_addr, DK * 128);  // MN-major, groups DK*128 B apart
      const bool leader = ptx::elect_one();
      auto wait_tile = [&](int t) { return wait_uniform(full_bar(t % NSLOT), (t / NSLOT) & 1); };
      uint32_t sb_waits = 0;
      for (int i = 0; i < n_iter; ++i) {
        const uint32_t q_lo = ptx::desc_lo(slot_addr(t0 + 3 * i), 16);                // K-major
        const uint32_t v_lo = ptx::desc_lo(slot_addr(t0 + 3 * i + 2), kGroupBytes);  // MN-major
        const bool have_state = (i > 0) || has_init;
        const bool use_state = have_state && !plain_chunk(i);
        const uint32_t tPb = tmem_base + cfg::PB_COL + (i & 1) * 64;
        const uint32_t tO = tO0 + (cfg::O_BUFS == 2 ? (i & 1) * DV : 0);
        if (cfg::O_BUFS == 2) {
          if (i >= 2 && !wait_uniform((i & 1) ? o_free1 : o_free0, ((i - 2) >> 1) & 1)) break;
        } else {
          if (i >= 1 && !wait_uniform(o_free0, (i - 1) & 1)) break;
        }
        if (have_state) {
          if (!wait_uniform(sb_ready, sb_waits & 1)) break;
          ++sb_waits;
        }
        if (!wait_tile(t0 + 3 * i)) break;
        ptx::tc_fence_after();
        if (leader) {
          if (use_state) {
#pragma unroll
            for (int kk = 0; kk < DK / 16; ++kk) {
              const uint32_t off = ((kk >> 2) * kGroupBytes + (kk & 3) * 32) >> 4;
              ptx::mma_ss(tO, q_lo + off, sb_lo + kk * (2048 >> 4), ptx::kDescHi, IDESC_QS,
                          kk > 0 ? 1u : 0u);
            }
          }
          ptx::tc_commit(qs_done);
          ptx::tc_commit(empty_bar((t0 + 3 * i) % NSLOT));  // second arrival on q
        }
        if (!wait_uniform(pb_ready, i & 1)) break;
        if (!wait_tile(t0 + 3 * i + 2)) break;
        ptx::tc_fence_after();
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < kChunk / 16; ++kk) {
            ptx::mma_ts(tO, tPb + kk * 8, v_lo + kk * (2048 >> 4), ptx::kDescHi, IDESC_PV,
                        kk > 0 ? 1u : (use_state ? 1u : 0u));
          }
          ptx::tc_commit((i & 1) ? o_full1 : o_full0);
          ptx::tc_commit(empty_bar((t0 + 3 * i + 2) % NSLOT));  // second arrival on v
        }
        __syncwarp();
      }
    }
  } else if (warp < 10) {
    // ================================================================ converter groups A, B
    const int half = (warp - 2) >> 2;  // column half this group owns
    const int quad = warp & 3;         // TMEM lane quadrant this warp may access
    const int row = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const uint32_t sb_row = sb_addr + row * 128;
    const uint32_t swz = static_cast<uint32_t>(row & 7);
    constexpr int SBLK = DV / 64;  // 32-column state blocks per group
    uint32_t ra[32], rb[32];

    // Packs 32 fp32 state values (columns cb*32 ..) to bf16 and writes them to the B-operand
    // buffer: [dv group of 64][dk row][128 B], 16-byte pieces XOR-swizzled by (row % 8).
    auto store_sb = [&](int cb, const uint32_t (&r)[32]) {
      const uint32_t grp = sb_row + (cb >> 1) * (DK * 128);
      const uint32_t j0 = (cb & 1) * 4;
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const uint32_t a0 = ptx::pack16x2<HALF>(__uint_as_float(r[jj * 8 + 0]), __uint_as_float(r[jj * 8 + 1]));
        const uint32_t a1 = ptx::pack16x2<HALF>(__uint_as_float(r[jj * 8 + 2]), __uint_as_float(r[jj * 8 + 3]));
        const uint32_t a2 = ptx::pack16x2<HALF>(__uint_as_float(r[jj * 8 + 4]), __uint_as_float(r[jj * 8 + 5]));
        const uint32_t a3 = ptx::pack16x2<HALF>(__uint_as_float(r[jj * 8 + 6]), __uint_as_float(r[jj * 8 + 7]));
        ptx::st_shared_v4(grp + (((j0 + jj) ^ swz) << 4), a0, a1, a2, a3);
      }
    };
    // State arrays in the caller's layout ([row][col], col contiguous) are read and written
    // through a per-warp 32x32 transpose in shared memory, so that global accesses are whole
    // 128-byte row segments instead of one word per lane per line. (The transposed layout, used
    // by the scratch, is coalesced as it is: consecutive lanes = consecutive rows.)
    constexpr bool kStagedStateIO = (DK == 128);  // needs 8 x 4 KB of free shared memory
    const uint32_t xpose_off = static_cast<uint32_t>(warp - 2) * 4096u;
    auto xpose_addr = [&](uint32_t base, int j, int r) {  // element (col j, row r), XOR-swizzled
      return base + xpose_off + static_cast<uint32_t>((j * 32 + (r ^ j)) * 4);
    };
    auto write_final = [&](int cb, const uint32_t (&r)[32]) {
      if (kStagedStateIO && !st_trans) {
        const uint32_t base = sb_addr;  // the operand buffer is idle when a final state is written
#pragma unroll
        for (int j = 0; j < 32; ++j) ptx::st_shared_b32(xpose_addr(base, j, lane), r[j]);
        __syncwarp();
        const int col = cb * 32 + lane;
#pragma unroll 4
        for (int rr = 0; rr < 32; ++rr) {
          const int grow = quad * 32 + rr;
          const uint32_t x = ptx::ld_shared_b32(xpose_addr(base, lane, rr));
          if (grow < p.st_rows && col < p.st_cols)
            pr.s_final[st_index + static_cast<size_t>(grow) * p.st_cols + col] = __uint_as_float(x);
        }
        __syncwarp();
        return;
      }
      if (row < p.st_rows) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (cb * 32 + j < p.st_cols) pr.s_final[st_off(row, cb * 32 + j)] = __uint_as_float(r[j]);
      }
    };
    // Reads this group's share of S from TMEM and routes it to the operand buffer and/or s_final.
    auto convert_state = [&](bool to_sb, bool to_final) {
      if (SBLK == 2) {
        ptx::tmem_ld32x2(lane_base + cfg::S_COL + (half * 2) * 32, ra,
                         lane_base + cfg::S_COL + (half * 2 + 1) * 32, rb);
        if (to_final) { write_final(half * 2, ra); write_final(half * 2 + 1, rb); }
        if (to_sb && row < DK) { store_sb(half * 2, ra); store_sb(half * 2 + 1, rb); }
      } else {
        ptx::tmem_ld32(lane_base + cfg::S_COL + half * 32, ra);
        if (to_final) write_final(half, ra);
        if (to_sb && row < DK) store_sb(half, ra);
      }
    };

    // Everything a converter thread does before the chunk loop (fused form: partial sum, barriers,
    // scan; then the starting state into TMEM and the operand buffer) lives in a function of its
    // own, so that its register needs stay out of the allocation of the loops below.
    PrologueArgs pa;
    pa.prob_idx = prob_idx;
    pa.g = g;
    pa.nseg = nseg;
    pa.bh = bh;
    pa.a_iter = a_iter;
    pa.tmem_base = tmem_base;
    pa.sb_addr = sb_addr;
    pa.ost_addr = ost_addr;
    pa.s_full = s_full;
    pa.part_done = part_done;
    pa.grid_done = grid_done;
    pa.sb_ready = sb_ready;
    pa.abort_flag = abort_flag;
    const bool conv_ok = converter_prologue<DK, DV, HALF>(p, pa);

    // phase A, if it ran, used the first phase of s_full
    const uint32_t s_off = a_iter > 0 ? 1u : 0u;
    if (mode == 0) {
      for (int i = 0; conv_ok && i < n_iter; ++i) {
        // ---------------- P: fp32 -> causal mask -> bf16 A operand (this group's 64 columns)
        int ok = ptx::mbar_wait(p_full, i & 1, abort_flag) ? 1 : 0;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ptx::tc_fence_after();
        // Column blocks of 32: relative to this warp's 32 rows a block is entirely kept, entirely
        // masked, or (block index == quadrant) the diagonal block that needs per-element tests.
        // The three mask modes are compiled separately (MODE 0: keep col <= row; 1: keep
        // col >= row; 2: keep col > row and negate) and selected by a warp-uniform branch.
        auto p_convert = [&](auto mode_c) {
          constexpr int MODE = decltype(mode_c)::value;
          constexpr bool kUpper = MODE != 0;
          uint32_t pk[16];
          const int cb0 = half * 2, cb1 = half * 2 + 1;
          const bool masked0 = kUpper ? (cb0 < quad) : (cb0 > quad);  // warp-uniform
          const bool masked1 = kUpper ? (cb1 < quad) : (cb1 > quad);
          // both blocks are fetched before either is converted: the two TMEM loads are in flight
          // together
          if (!masked0 && !masked1) {
            ptx::tmem_ld32x2(lane_base + cfg::P_COL + cb0 * 32, ra, lane_base + cfg::P_COL + cb1 * 32, rb);
          } else if (!masked0) {
            ptx::tmem_ld32(lane_base + cfg::P_COL + cb0 * 32, ra);
          } else if (!masked1) {
            ptx::tmem_ld32(lane_base + cfg::P_COL + cb1 * 32, rb);
          }
          auto convert_block = [&](int cb, bool masked, const uint32_t (&r)[32]) {
            if (masked) {
#pragma unroll
              for (int j = 0; j < 16; ++j) pk[j] = 0u;
            } else {
              if (cb == quad) {
                // first kept column (upper modes) resp. last kept column (lower) of this row
                const int edge = (MODE == 2) ? lane + 1 : lane;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  const bool k0 = kUpper ? (2 * j >= edge) : (2 * j <= edge);
                  const bool k1 = kUpper ? (2 * j + 1 >= edge) : (2 * j + 1 <= edge);
                  pk[j] = ptx::pack16x2<HALF>(k0 ? __uint_as_float(r[2 * j]) : 0.f,
                                              k1 ? __uint_as_float(r[2 * j + 1]) : 0.f);
                }
              } else {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  pk[j] = ptx::pack16x2<HALF>(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
              }
              if (MODE == 2) {
#pragma unroll
                for (int j = 0; j < 16; ++j) pk[j] ^= 0x80008000u;  // negate both halves
              }
            }
            ptx::tmem_st16(lane_base + cfg::PB_COL + (i & 1) * 64 + cb * 16, pk);
          };
          convert_block(cb0, masked0, ra);
          convert_block(cb1, masked1, rb);
          // Issuer X may overwrite the fp32 tile now. The arrival comes AFTER the conversions, which
          // consume every loaded register: placed directly behind the load (and its
          // tcgen05.wait::ld) it was observed to let X's next score MMA overwrite columns that the
          // second of the two loads had not delivered yet -- rarely, when X was already polling
          // this barrier (first chunk of a CTA), and the block then held a mix of this chunk's and
          // the next chunk's scores.
          ptx::tc_fence_before();
          ptx::mbar_arrive(p_read);
        };
        if (tms && !plain_chunk(i)) {
          p_convert(std::integral_constant<int, 2>{});
        } else if (upper_flag) {
          p_convert(std::integral_constant<int, 1>{});
        } else {
          p_convert(std::integral_constant<int, 0>{});
        }
        ptx::tc_wait_st();
        ptx::tc_fence_before();
        ptx::mbar_arrive(pb_ready);

        // ---------------- S: fp32 -> bf16 B operand for the next chunk (or -> s_final)
        const bool last = (i == n_iter - 1);
        const bool to_final = last && (pr.s_final != nullptr) && (g == nseg - 1);
        if (!last || to_final) {
          ok = ptx::mbar_wait(s_full, (i + s_off) & 1, abort_flag) ? 1 : 0;
          // the state buffer is still the B operand of issuer Y's Q Sb of this chunk
          // (also before a final-state write, which borrows that buffer as transpose scratch)
          if (ok) ok = ptx::mbar_wait(qs_done, i & 1, abort_flag) ? 1 : 0;
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          ptx::tc_fence_after();
          convert_state(!last, to_final);
          if (!last) {
            ptx::fence_proxy_async_smem();
            ptx::tc_fence_before();
            ptx::mbar_arrive(sb_ready);
          }
        }
      }
    } else {
      // state only: one read-out after the last chunk
      int ok = ptx::mbar_wait(s_full, 0, abort_flag) ? 1 : 0;
      ok = __all_sync(0xffffffffu, ok);
      if (ok && pr.s_final != nullptr) {
        ptx::tc_fence_after();
        convert_state(false, true);
      }
    }
  } else {
    // ================================================================ epilogue group
    if (mode == 0) {
      const int quad = warp & 3;
      const int row = quad * 32 + lane;
      const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
      const uint32_t swz = static_cast<uint32_t>(row & 7);
      uint32_t ra[32], rb[32];
      for (int i = 0; i < n_iter; ++i) {
        int ok = ptx::mbar_wait((i & 1) ? o_full1 : o_full0, (i >> 1) & 1, abort_flag) ? 1 : 0;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ptx::tc_fence_after();
        // Every warp stages and stores its own 32 rows (a 64 x 32 box per column group), so no
        // barrier spans the group and nobody waits for a store except the warp that issued it:
        // before overwriting its rows, lane 0 checks that the previous store has read them.
        if (lane == 0) ptx::bulk_wait_group_read0();
        __syncwarp();
        const uint32_t obuf = ost_addr + row * 128;
        // One 64-column group at a time: two TMEM loads in flight, rounded and written to the
        // staging rows straight away (16-byte pieces XOR-swizzled by row % 8), so that only 64
        // accumulator values are ever held in registers.
#pragma unroll
        for (int gg = 0; gg < cfg::GV; ++gg) {
          const uint32_t o_col = cfg::O_COL + (cfg::O_BUFS == 2 ? (i & 1) * DV : 0) + gg * 64;
          ptx::tmem_ld32x2(lane_base + o_col, ra, lane_base + o_col + 32, rb);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            ptx::st_shared_v4(
                obuf + gg * kGroupBytes + ((static_cast<uint32_t>(j) ^ swz) << 4),
                ptx::pack16x2<HALF>(__uint_as_float(ra[8 * j + 0]), __uint_as_float(ra[8 * j + 1])),
                ptx::pack16x2<HALF>(__uint_as_float(ra[8 * j + 2]), __uint_as_float(ra[8 * j + 3])),
                ptx::pack16x2<HALF>(__uint_as_float(ra[8 * j + 4]), __uint_as_float(ra[8 * j + 5])),
                ptx::pack16x2<HALF>(__uint_as_float(ra[8 * j + 6]), __uint_as_float(ra[8 * j + 7])));
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            ptx::st_shared_v4(
                obuf + gg * kGroupBytes + ((static_cast<uint32_t>(j + 4) ^ swz) << 4),
                ptx::pack16x2<HALF>(__uint_as_float(rb[8 * j + 0]), __uint_as_float(rb[8 * j + 1])),
                ptx::pack16x2<HALF>(__uint_as_float(rb[8 * j + 2]), __uint_as_float(rb[8 * j + 3])),
                ptx::pack16x2<HALF>(__uint_as_float(rb[8 * j + 4]), __uint_as_float(rb[8 * j + 5])),
                ptx::pack16x2<HALF>(__uint_as_float(rb[8 * j + 6]), __uint_as_float(rb[8 * j + 7])));
          }
        }
        ptx::tc_fence_before();
        // the accumulator has been read: issuer Y may reuse it
        ptx::mbar_arrive((cfg::O_BUFS == 2 && (i & 1)) ? o_free1 : o_free0);
        ptx::fence_proxy_async_smem();
        __syncwarp();
        const int tok = mem_chunk(i) * kChunk + quad * 32;
        if (lane == 0 && tok < pr.n_tokens) {
#pragma unroll
          for (int gg = 0; gg < cfg::GV; ++gg)
            ptx::tma_store_4d(&pr.o, ost_addr + gg * kGroupBytes + quad * (32 * 128), gg * 64, tok,
                              h, b);
          ptx::bulk_commit_group();
        }
      }
      if (lane == 0) ptx::bulk_wait_group0();

    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_flag) {
    // A wait gave up: let copies in flight land before the shared memory is released.
    __nanosleep(100000);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status != nullptr) atomicOr(p.status, 1);
}

}  // namespace fla
