// Causal linear attention product with a wide q/k head dim and a narrow v head dim, for sm_100a:
//     o_i = sum_{j <= i} (a_i . b_j) c_j     (or j >= i: descending walk, upper mask)
// with a, b of up to 128 * NT columns and c, o of up to 64 columns. This is the forward and the dV
// product of the reference's SmallVHD kernels (flashlinear/kernels/linear_attn_kernels_smallv_hd.py
// :12-108 and :160-227), e.g. 273-dimensional second-order Taylor features against 64-dimensional
// values.
//
// Per 128-token chunk the a and b tiles are streamed through shared memory in NT pairs of 128
// columns; each pair feeds three tensor-core products while it is resident,
//     P   += A_t B_t^T          (score tile, accumulates over the pairs)
//     O   += A_t Sb_t           (inter-chunk term, Sb = bf16 copy of the state rows of pair t)
//     S_t += B_t^T C            (state rows of pair t, fp32 in tensor memory)
// and the chunk ends with O += mask(P) C. The state S (128*NT x 64 fp32) never leaves tensor memory.
//
// CTA layout (448 threads, one CTA per (batch, head)):
//   warp 0       TMA producer: c tile of the chunk (own double buffer), then the a/b tile pairs
//                into a ring of eight 16 KB slots (one 64-column group each; a tile takes the one
//                or two groups that hold valid columns, so padding costs no ring space)
//   warp 1       MMA issuer (one elected lane) and TMEM owner
//   warps 2-9    converters: P fp32 -> mask -> bf16 (TMEM), S fp32 -> bf16 (shared memory)
//   warps 10-13  epilogue: O fp32 -> bf16 -> staging -> TMA store (each warp its own 32 rows)
// The kernel is bound by HBM (1.3 KB per token-head against ~3.3k tensor cycles per chunk), so one
// issuing warp in program order is enough; its tcgen05.commit arrivals order everything else.
#pragma once
#include "ptx.cuh"

#include <type_traits>

namespace fla {

struct WideParams {
  CUtensorMap a, b;  // 4-D maps (dim, token, head, batch), box 64 x 128, 128B swizzle
  CUtensorMap c;     // same box; at most 64 columns
  CUtensorMap o;     // box 64 x 32
  int flags;         // kFlagDescending | kFlagUpperMask for the anti-causal product, else 0
  int n_tokens;
  int heads;
  int nchunks;
  int da;            // valid columns of a and b
  int* status;       // device word, bit 0 set when a bounded wait ran out; may be null
  unsigned wait_limit_us;  // limit of one bounded wait in microseconds of the global timer; 0 = default
  int debug_withhold;  // test hook: the first c tile is never loaded, so the waits on it run out
};

constexpr int kWideThreads = 448;
constexpr int kWideChunk = 128;
constexpr int kWideGroupBytes = kWideChunk * 128;   // 64 columns x 128 rows
constexpr int kWideSlots = 8;  // ring slots of one 64-column group (16 KB) each

template <int NT>
struct WideCfg {
  static_assert(NT >= 2 && NT <= 3, "state of 128*NT x 64 must fit tensor memory next to P and O");
  static constexpr int RING_BYTES = kWideSlots * kWideGroupBytes;
  static constexpr int C_BYTES = 2 * kWideGroupBytes;
  static constexpr int SB_BYTES = NT * 128 * 128;  // bf16 state, one 128-byte row per state row
  // one more group after the ring: the state update of a one-group tile in the last slot reads
  // 128 rows and so runs into the following 16 KB (the c buffers), which must exist
  static constexpr int OST_BYTES = kWideGroupBytes;
  static constexpr int BAR_BYTES = 512;
  static constexpr int SMEM_BYTES = 1024 + RING_BYTES + C_BYTES + SB_BYTES + OST_BYTES + BAR_BYTES;
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
  static constexpr int P_COL = 0;     // P fp32, 128 columns
  static constexpr int PB_COL = 128;  // P bf16, 64 columns
  static constexpr int O_COL = 192;   // O fp32, 64 columns
  static constexpr int S_COL = 256;   // S fp32, NT blocks of 64 columns (lane = state row % 128)
  static constexpr int TMEM_COLS = 512;
  static_assert(S_COL + NT * 64 <= TMEM_COLS, "TMEM budget");
};

template <int NT>
__global__ void __launch_bounds__(kWideThreads, 1)
fla_wide_kernel(const __grid_constant__ WideParams p) {
  using cfg = WideCfg<NT>;
  extern __shared__ uint8_t smem_raw[];

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
  const int lane = threadIdx.x & 31;
  const int bh = blockIdx.z;
  const int h = bh % p.heads;
  const int b = bh / p.heads;
  // c and out wider than 64 columns: block x takes columns [64 x, 64 x + 64). The slices of a head
  // are neighbours in launch order, stream the same a, b tiles at the same time and share them in
  // L2; columns beyond the tensors' width are zero-filled on load and dropped on store by the TMA.
  const int c_col0 = static_cast<int>(blockIdx.x) * 64;

  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - raw_addr);
  const uint32_t c_addr = smem_base + cfg::RING_BYTES;
  const uint32_t sb_addr = c_addr + cfg::C_BYTES;
  const uint32_t ost_addr = sb_addr + cfg::SB_BYTES;
  const uint32_t bar_base = ost_addr + cfg::OST_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kWideSlots + s); };
  auto cfull_bar = [&](int s) { return bar_base + 8u * (2 * kWideSlots + s); };
  auto cempty_bar = [&](int s) { return bar_base + 8u * (2 * kWideSlots + 2 + s); };
  const uint32_t p_full = bar_base + 8u * (2 * kWideSlots + 4);
  const uint32_t pb_ready = bar_base + 8u * (2 * kWideSlots + 5);
  const uint32_t s_full = bar_base + 8u * (2 * kWideSlots + 6);
  const uint32_t sb_ready = bar_base + 8u * (2 * kWideSlots + 7);
  const uint32_t o_full = bar_base + 8u * (2 * kWideSlots + 8);
  const uint32_t o_free = bar_base + 8u * (2 * kWideSlots + 9);
  const uint32_t holder_off = cfg::RING_BYTES + cfg::C_BYTES + cfg::SB_BYTES + cfg::OST_BYTES +
                              8u * (2 * kWideSlots + 10);
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem_gen + holder_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + holder_off + 4);

  const bool descending = (p.flags & kFlagDescending) != 0;
  const bool upper_flag = (p.flags & kFlagUpperMask) != 0;
  const int n_iter = p.nchunks;
  // columns of a/b that pair t holds, and the 16-column MMA steps / 64-column groups they span
  auto pair_cols = [&](int t) { return max(0, min(128, p.da - 128 * t)); };

  if (threadIdx.x == 0) {
    abort_flag[0] = 0;
    abort_flag[1] = static_cast<int>(p.wait_limit_us);
    for (int s = 0; s < kWideSlots; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(cfull_bar(s), 1);
      ptx::mbar_init(cempty_bar(s), 1);
    }
    ptx::mbar_init(p_full, 1);
    ptx::mbar_init(pb_ready, 256);
    ptx::mbar_init(s_full, 1);
    ptx::mbar_init(sb_ready, 256);
    ptx::mbar_init(o_full, 1);
    ptx::mbar_init(o_free, 128);
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_holder)), cfg::TMEM_COLS);
    ptx::tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tensormap(&p.a);
    ptx::prefetch_tensormap(&p.b);
    ptx::prefetch_tensormap(&p.c);
    ptx::prefetch_tensormap(&p.o);
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  auto wait_uniform = [&](uint32_t bar, uint32_t parity) {
    const int ok = ptx::mbar_wait(bar, parity, abort_flag) ? 1 : 0;
    return __all_sync(0xffffffffu, ok) != 0;
  };
  auto mem_chunk = [&](int i) { return descending ? (p.nchunks - 1 - i) : i; };
  // The ring is counted in 64-column groups, in load order: per chunk a_0, b_0, a_1, b_1, ...,
  // each tile taking pair_groups(t) consecutive slots. Every pair takes an even number of groups
  // and only the last pair can have one-group tiles, so a two-group tile always starts on an even
  // slot: its groups are adjacent in memory and never straddle the end of the ring.
  auto pair_groups = [&](int t) { return pair_cols(t) > 64 ? 2 : 1; };
  int groups_per_chunk = 0;
  for (int t = 0; t < NT; ++t) groups_per_chunk += 2 * pair_groups(t);
  // index of the first group of tile (chunk i, pair t, w = 0: a, 1: b)
  auto tile_group = [&](int i, int t, int w) {
    int g = i * groups_per_chunk;
    for (int tt = 0; tt < t; ++tt) g += 2 * pair_groups(tt);
    return g + w * pair_groups(t);
  };
  auto group_addr = [&](int g) {
    return smem_base + static_cast<uint32_t>(g % kWideSlots) * kWideGroupBytes;
  };

  if (warp == 0) {
    // ================================================================ TMA producer
    const bool leader = ptx::elect_one();
    bool ok = true;
    for (int i = 0; ok && i < n_iter; ++i) {
      const int tok = mem_chunk(i) * kWideChunk;
      const int cs = i & 1;
      if (!wait_uniform(cempty_bar(cs), ((i >> 1) & 1) ^ 1u)) break;
      if (leader) {
        ptx::mbar_expect_tx(cfull_bar(cs), kWideGroupBytes);
        if (!(p.debug_withhold && i == 0))
          ptx::tma_load_4d(c_addr + cs * kWideGroupBytes, &p.c, cfull_bar(cs), c_col0, tok, h, b);
      }
      for (int t = 0; t < NT; ++t) {
        const int groups = pair_groups(t);  // a group that is all padding is not loaded
        for (int w = 0; w < 2; ++w) {
          for (int gg = 0; gg < groups; ++gg) {
            const int g = tile_group(i, t, w) + gg;
            const int s = g % kWideSlots;
            if (!wait_uniform(empty_bar(s), ((g / kWideSlots) & 1) ^ 1u)) { ok = false; break; }
            if (leader) {
              ptx::mbar_expect_tx(full_bar(s), kWideGroupBytes);
              ptx::tma_load_4d(group_addr(g), w == 0 ? &p.a : &p.b, full_bar(s), t * 128 + gg * 64,
                               tok, h, b);
            }
          }
          if (!ok) break;
        }
        if (!ok) break;
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer
    constexpr uint32_t IDESC_P = ptx::make_idesc(128, 128, false, false);  // P   += A_t B_t^T
    constexpr uint32_t IDESC_AS = ptx::make_idesc(128, 64, false, true);   // O   += A_t Sb_t
    constexpr uint32_t IDESC_S = ptx::make_idesc(128, 64, true, true);     // S_t += B_t^T C
    constexpr uint32_t IDESC_PC = ptx::make_idesc(128, 64, false, true);   // O   += Pb C
    const uint32_t tP = tmem_base + cfg::P_COL;
    const uint32_t tPb = tmem_base + cfg::PB_COL;
    const uint32_t tO = tmem_base + cfg::O_COL;
    const uint32_t tS = tmem_base + cfg::S_COL;
    const bool leader = ptx::elect_one();
    const uint32_t sb_lo = ptx::desc_lo(sb_addr, kWideGroupBytes);
    bool ok = true;
    for (int i = 0; ok && i < n_iter; ++i) {
      const bool have_state = i > 0;
      const int cs = i & 1;
      const uint32_t c_lo = ptx::desc_lo(c_addr + cs * kWideGroupBytes, kWideGroupBytes);  // MN-major
      if (!wait_uniform(cfull_bar(cs), (i >> 1) & 1)) break;
      if (i > 0) {
        // the epilogue has drained O of chunk i-1; the converters have read S of chunk i-1 out of
        // tensor memory and its bf16 copy is in shared memory
        if (!wait_uniform(o_free, (i - 1) & 1)) break;
        if (!wait_uniform(sb_ready, (i - 1) & 1)) break;
      }
      for (int t = 0; t < NT; ++t) {
        const int groups = pair_groups(t);
        const int ga = tile_group(i, t, 0);
        const int gb = tile_group(i, t, 1);
        for (int gg = 0; ok && gg < groups; ++gg) {
          ok = wait_uniform(full_bar((ga + gg) % kWideSlots), ((ga + gg) / kWideSlots) & 1) &&
               wait_uniform(full_bar((gb + gg) % kWideSlots), ((gb + gg) / kWideSlots) & 1);
        }
        if (!ok) break;
        ptx::tc_fence_after();
        const int ksteps = (pair_cols(t) + 15) >> 4;
        const uint32_t a_lo = ptx::desc_lo(group_addr(ga), 16);                // K-major
        const uint32_t b_lo = ptx::desc_lo(group_addr(gb), 16);                // K-major
        const uint32_t bt_lo = ptx::desc_lo(group_addr(gb), kWideGroupBytes);  // MN-major
        if (leader) {
          for (int kk = 0; kk < ksteps; ++kk) {
            const uint32_t off = ((kk >> 2) * kWideGroupBytes + (kk & 3) * 32) >> 4;
            ptx::mma_ss(tP, a_lo + off, b_lo + off, ptx::kDescHi, IDESC_P, (t > 0 || kk > 0) ? 1u : 0u);
          }
          if (t == NT - 1) ptx::tc_commit(p_full);
          if (have_state) {
            for (int kk = 0; kk < ksteps; ++kk) {
              const uint32_t off = ((kk >> 2) * kWideGroupBytes + (kk & 3) * 32) >> 4;
              ptx::mma_ss(tO, a_lo + off, sb_lo + (t * 8 + kk) * (2048 >> 4), ptx::kDescHi, IDESC_AS,
                          (t > 0 || kk > 0) ? 1u : 0u);
            }
          }
          // The instruction spans 128 state rows; rows past the loaded columns of b read whatever
          // the slot holds and land in tensor-memory lanes nobody reads.
#pragma unroll
          for (int kk = 0; kk < kWideChunk / 16; ++kk) {
            ptx::mma_ss(tS + t * 64, bt_lo + kk * (2048 >> 4), c_lo + kk * (2048 >> 4), ptx::kDescHi,
                        IDESC_S, (have_state || kk > 0) ? 1u : 0u);
          }
          for (int gg = 0; gg < groups; ++gg) {
            ptx::tc_commit(empty_bar((ga + gg) % kWideSlots));
            ptx::tc_commit(empty_bar((gb + gg) % kWideSlots));
          }
        }
        __syncwarp();
      }
      if (!ok) break;
      if (leader) ptx::tc_commit(s_full);  // S of chunk i complete, Sb no longer read
      __syncwarp();
      if (!wait_uniform(pb_ready, i & 1)) break;
      ptx::tc_fence_after();
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < kWideChunk / 16; ++kk) {
          ptx::mma_ts(tO, tPb + kk * 8, c_lo + kk * (2048 >> 4), ptx::kDescHi, IDESC_PC,
                      (have_state || kk > 0) ? 1u : 0u);
        }
        ptx::tc_commit(o_full);
        ptx::tc_commit(cempty_bar(cs));
      }
      __syncwarp();
    }
  } else if (warp < 10) {
    // ================================================================ converters
    const int half = (warp - 2) >> 2;  // column half this group owns
    const int quad = warp & 3;         // TMEM lane quadrant this warp may access
    const int row = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const uint32_t swz = static_cast<uint32_t>(row & 7);
    uint32_t ra[32], rb[32];
    for (int i = 0; i < n_iter; ++i) {
      int ok = ptx::mbar_wait(p_full, i & 1, abort_flag) ? 1 : 0;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tc_fence_after();
      // Column blocks of 32 are, relative to this warp's 32 rows, entirely kept, entirely masked,
      // or the diagonal block (block index == quadrant) with per-element tests.
      auto p_convert = [&](auto upper_c) {
        constexpr bool kUpper = decltype(upper_c)::value;
        uint32_t pk[16];
        const int cb0 = half * 2, cb1 = half * 2 + 1;
        const bool masked0 = kUpper ? (cb0 < quad) : (cb0 > quad);  // warp-uniform
        const bool masked1 = kUpper ? (cb1 < quad) : (cb1 > quad);
        // both blocks are fetched before either is converted (two TMEM loads in flight together)
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
          } else if (cb == quad) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const bool k0 = kUpper ? (2 * j >= lane) : (2 * j <= lane);
              const bool k1 = kUpper ? (2 * j + 1 >= lane) : (2 * j + 1 <= lane);
              pk[j] = ptx::pack_bf16x2(k0 ? __uint_as_float(r[2 * j]) : 0.f,
                                       k1 ? __uint_as_float(r[2 * j + 1]) : 0.f);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              pk[j] = ptx::pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
          }
          ptx::tmem_st16(lane_base + cfg::PB_COL + cb * 16, pk);
        };
        convert_block(cb0, masked0, ra);
        convert_block(cb1, masked1, rb);
      };
      if (upper_flag) {
        p_convert(std::true_type{});
      } else {
        p_convert(std::false_type{});
      }
      ptx::tc_wait_st();
      ptx::tc_fence_before();
      ptx::mbar_arrive(pb_ready);

      if (i + 1 < n_iter) {
        // S fp32 -> bf16 rows of the B operand of the next chunk's A_t Sb_t: state row r at
        // sb + r * 128 B, 16-byte pieces XOR-swizzled by (r % 8); this group's 32 columns.
        ok = ptx::mbar_wait(s_full, i & 1, abort_flag) ? 1 : 0;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ptx::tc_fence_after();
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          if (quad * 32 < (((pair_cols(t) + 15) >> 4) << 4)) {  // warp-uniform: rows the MMAs read
            ptx::tmem_ld32(lane_base + cfg::S_COL + t * 64 + half * 32, ra);
            const uint32_t dst = sb_addr + static_cast<uint32_t>(t * 128 + row) * 128;
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              const uint32_t a0 = ptx::pack_bf16x2(__uint_as_float(ra[jj * 8 + 0]), __uint_as_float(ra[jj * 8 + 1]));
              const uint32_t a1 = ptx::pack_bf16x2(__uint_as_float(ra[jj * 8 + 2]), __uint_as_float(ra[jj * 8 + 3]));
              const uint32_t a2 = ptx::pack_bf16x2(__uint_as_float(ra[jj * 8 + 4]), __uint_as_float(ra[jj * 8 + 5]));
              const uint32_t a3 = ptx::pack_bf16x2(__uint_as_float(ra[jj * 8 + 6]), __uint_as_float(ra[jj * 8 + 7]));
              ptx::st_shared_v4(dst + (((half * 4 + jj) ^ swz) << 4), a0, a1, a2, a3);
            }
          }
        }
        ptx::fence_proxy_async_smem();
        ptx::tc_fence_before();
        ptx::mbar_arrive(sb_ready);
      }
    }
  } else {
    // ================================================================ epilogue
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const uint32_t swz = static_cast<uint32_t>(row & 7);
    uint32_t ra[32], rb[32];
    uint32_t pk[32];
    for (int i = 0; i < n_iter; ++i) {
      int ok = ptx::mbar_wait(o_full, i & 1, abort_flag) ? 1 : 0;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tc_fence_after();
      ptx::tmem_ld32x2(lane_base + cfg::O_COL, ra,
                       lane_base + cfg::O_COL + 32, rb);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        pk[j] = ptx::pack_bf16x2(__uint_as_float(ra[2 * j]), __uint_as_float(ra[2 * j + 1]));
        pk[16 + j] = ptx::pack_bf16x2(__uint_as_float(rb[2 * j]), __uint_as_float(rb[2 * j + 1]));
      }
      if (lane == 0) ptx::bulk_wait_group_read0();  // the previous store has read these rows
      __syncwarp();
      const uint32_t obuf = ost_addr + row * 128;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        ptx::st_shared_v4(obuf + ((static_cast<uint32_t>(j) ^ swz) << 4), pk[j * 4], pk[j * 4 + 1],
                          pk[j * 4 + 2], pk[j * 4 + 3]);
      // the accumulator may be overwritten: signalled after the stores that consume every loaded
      // register (an arrival directly behind a TMEM load does not reliably wait for its data)
      ptx::tc_fence_before();
      ptx::mbar_arrive(o_free);
      ptx::fence_proxy_async_smem();
      __syncwarp();
      const int tok = mem_chunk(i) * kWideChunk + quad * 32;
      if (lane == 0 && tok < p.n_tokens) {
        ptx::tma_store_4d(&p.o, ost_addr + quad * (32 * 128), c_col0, tok, h, b);
        ptx::bulk_commit_group();
      }
    }
    if (lane == 0) ptx::bulk_wait_group0();
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_flag) __nanosleep(100000);  // a wait gave up: let copies in flight land
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status != nullptr) atomicOr(p.status, 1);
}

}  // namespace fla
