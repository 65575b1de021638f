// Chunked causal linear attention for sm_100a.
//
// One generic kernel computes, for one head and one run of 128-token chunks,
//     o_i = sum_{j <= i} (q_i . k_j) v_j            (reverse = 0)
//     o_i = sum_{j >= i} (q_i . k_j) v_j            (reverse = 1)
// as  P = (Q K^T) (.) mask,  O = P V + Q S,  S += K^T V   per chunk, where S (dk x dv, fp32) is the
// running state carried in tensor memory. The forward pass and all three gradients are this same
// product with the operands permuted (see fla_api.cu), which replaces the quadratic tile loops of
// flashlinear/kernels/linear_attn_kernels.py:63-85 (fwd), :171-200 and :283-302 (bwd).
//
// CTA layout (320 threads, one CTA per SM):
//   warp 0      TMA producer: Q, K, V chunk tiles -> shared memory (128-byte swizzle), mbarrier ring
//   warp 1      tcgen05.mma issuer (one thread) and TMEM owner
//   warps 2-5   converter group: P fp32 (TMEM) -> mask -> bf16 (TMEM, A operand);
//               S fp32 (TMEM) -> bf16 (shared memory, B operand)
//   warps 6-9   epilogue group: O fp32 (TMEM) -> bf16 -> shared memory -> TMA store
#pragma once
#include "ptx.cuh"

namespace fla {

constexpr int kChunk = 128;    // tokens per chunk (= MMA M)
constexpr int kThreads = 320;  // 10 warps
constexpr int kGroupBytes = kChunk * 128;  // one 64-column group of a chunk tile: 128 rows x 128 B

struct Problem {
  CUtensorMap q, k, v, o;  // 4-D maps (dim, token, head, batch), box 64 x 128 x 1 x 1, 128B swizzle
  const float* s_init;     // [bh * segments + g][st_rows][st_cols] fp32, or null
  float* s_final;          // same indexing, or null
  int reverse;
  int st_trans;            // state arrays are stored transposed: element (row, col) at [col][row]
};

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
};

template <int DK, int DV>
struct Cfg {
  static_assert(DK % 64 == 0 && DV % 64 == 0 && DK <= 128 && DV <= 128, "unsupported head dims");
  static constexpr int GK = DK / 64;
  static constexpr int GV = DV / 64;
  static constexpr int Q_BYTES = GK * kGroupBytes;
  static constexpr int K_BYTES = GK * kGroupBytes;
  static constexpr int V_BYTES = GV * kGroupBytes;
  static constexpr int STAGE_BYTES = Q_BYTES + K_BYTES + V_BYTES;
  static constexpr int SB_BYTES = GV * DK * 128;  // bf16 state as MMA B operand
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_LIMIT = 232448;  // 227 KB
  static constexpr int NSTAGES_RAW = (SMEM_LIMIT - 1024 - BAR_BYTES - SB_BYTES) / STAGE_BYTES;
  static constexpr int NSTAGES = NSTAGES_RAW > 4 ? 4 : NSTAGES_RAW;
  static_assert(NSTAGES >= 2, "need at least two stages");
  static constexpr int SMEM_BYTES = 1024 + NSTAGES * STAGE_BYTES + SB_BYTES + BAR_BYTES;
  // The epilogue stages O in the Q buffer of the chunk it belongs to.
  static_assert(V_BYTES <= Q_BYTES, "O staging needs dv <= dk tiles");
  // TMEM columns (32-bit each, 128 lanes)
  static constexpr int P_COL = 0;            // P fp32: 128 columns
  static constexpr int PB_COL = 128;         // P bf16 (two per column): 64 columns
  static constexpr int O_COL = 192;          // O fp32: DV columns
  static constexpr int S_COL = 192 + DV;     // S fp32: DV columns, lane = dk index
  static constexpr int TMEM_COLS = 512;
  static_assert(S_COL + DV <= TMEM_COLS, "TMEM budget");
};

template <int DK, int DV>
__global__ void __launch_bounds__(kThreads, 1)
fla_chunk_kernel(const __grid_constant__ KernelParams p) {
  using cfg = Cfg<DK, DV>;
  constexpr int NS = cfg::NSTAGES;
  extern __shared__ uint8_t smem_raw[];

  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - raw_addr);

  const uint32_t sb_addr = smem_base + NS * cfg::STAGE_BYTES;
  const uint32_t bar_base = sb_addr + cfg::SB_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (NS + s); };
  const uint32_t p_full = bar_base + 8u * (2 * NS + 0);
  const uint32_t pb_ready = bar_base + 8u * (2 * NS + 1);
  const uint32_t o_full = bar_base + 8u * (2 * NS + 2);
  const uint32_t o_free = bar_base + 8u * (2 * NS + 3);
  const uint32_t s_full = bar_base + 8u * (2 * NS + 4);
  const uint32_t sb_ready = bar_base + 8u * (2 * NS + 5);
  const uint32_t o_staged = bar_base + 8u * (2 * NS + 6);
  const uint32_t holder_off = NS * cfg::STAGE_BYTES + cfg::SB_BYTES + 8u * (2 * NS + 7);
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem_gen + holder_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + holder_off + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int prob_idx = blockIdx.x;
  const int g = blockIdx.y;
  const int nseg = gridDim.y;
  const int bh = blockIdx.z;
  const Problem& pr = p.prob[prob_idx];
  const int h = bh % p.heads;
  const int b = bh / p.heads;
  const int chunk0 = g * p.seg_chunks;
  const int n_iter = min(p.seg_chunks, p.nchunks - chunk0);
  const bool reverse = pr.reverse != 0;
  const int mode = p.mode;
  const bool has_init = (mode == 0) && (pr.s_init != nullptr);
  const size_t st_elems = static_cast<size_t>(p.st_rows) * p.st_cols;
  const size_t st_index = (static_cast<size_t>(bh) * nseg + g) * st_elems;
  const bool st_trans = pr.st_trans != 0;
  auto st_off = [&](int row, int col) {
    return st_index + (st_trans ? static_cast<size_t>(col) * p.st_rows + row
                                : static_cast<size_t>(row) * p.st_cols + col);
  };
  if (mode == 1 && p.skip_last_segment && g == nseg - 1) return;  // whole CTA, before any setup

  // ------------------------------------------------------------------ setup
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < NS; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), mode == 0 ? 2 : 1);
    }
    ptx::mbar_init(p_full, 1);
    ptx::mbar_init(pb_ready, 128);
    ptx::mbar_init(o_full, 1);
    ptx::mbar_init(o_free, 128);
    ptx::mbar_init(s_full, 1);
    ptx::mbar_init(sb_ready, 128);
    ptx::mbar_init(o_staged, 128);
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

  auto mem_chunk = [&](int i) { return reverse ? (p.nchunks - 1 - (chunk0 + i)) : (chunk0 + i); };
  auto stage_addr = [&](int s) { return smem_base + static_cast<uint32_t>(s) * cfg::STAGE_BYTES; };

  if (warp == 0) {
    // ================================================================ TMA producer
    for (int i = 0; i < n_iter; ++i) {
      int ok = 1;
      if (lane == 0) {
        const int s = i % NS;
        const uint32_t ph = (i / NS) & 1;
        ok = ptx::mbar_wait(empty_bar(s), ph ^ 1u, abort_flag) ? 1 : 0;
        if (ok) {
          const uint32_t st = stage_addr(s);
          const int tok = mem_chunk(i) * kChunk;
          const uint32_t bytes = (mode == 0 ? cfg::Q_BYTES : 0) + cfg::K_BYTES + cfg::V_BYTES;
          ptx::mbar_expect_tx(full_bar(s), bytes);
          if (mode == 0) {
#pragma unroll
            for (int gg = 0; gg < cfg::GK; ++gg)
              ptx::tma_load_4d(st + gg * kGroupBytes, &pr.q, full_bar(s), gg * 64, tok, h, b);
          }
#pragma unroll
          for (int gg = 0; gg < cfg::GK; ++gg)
            ptx::tma_load_4d(st + cfg::Q_BYTES + gg * kGroupBytes, &pr.k, full_bar(s), gg * 64, tok,
                             h, b);
#pragma unroll
          for (int gg = 0; gg < cfg::GV; ++gg)
            ptx::tma_load_4d(st + cfg::Q_BYTES + cfg::K_BYTES + gg * kGroupBytes, &pr.v,
                             full_bar(s), gg * 64, tok, h, b);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer
    constexpr uint32_t IDESC_QK = ptx::make_idesc(128, kChunk, false, false);  // P  = Q K^T
    constexpr uint32_t IDESC_PV = ptx::make_idesc(128, DV, false, true);       // O += Pb V
    constexpr uint32_t IDESC_QS = ptx::make_idesc(128, DV, false, true);       // O  = Q Sb
    constexpr uint32_t IDESC_KV = ptx::make_idesc(128, DV, true, true);        // S += K^T V
    const uint32_t tP = tmem_base + cfg::P_COL;
    const uint32_t tPb = tmem_base + cfg::PB_COL;
    const uint32_t tO = tmem_base + cfg::O_COL;
    const uint32_t tS = tmem_base + cfg::S_COL;
    uint32_t sb_waits = 0;
    for (int i = 0; i < n_iter; ++i) {
      int ok = 1;
      if (lane == 0) {
        const int s = i % NS;
        const uint32_t ph = (i / NS) & 1;
        const uint32_t q_addr = stage_addr(s);
        const uint32_t k_addr = q_addr + cfg::Q_BYTES;
        const uint32_t v_addr = k_addr + cfg::K_BYTES;
        const bool have_state = (i > 0) || has_init;
        do {
          if (!ptx::mbar_wait(full_bar(s), ph, abort_flag)) { ok = 0; break; }
          ptx::tc_fence_after();
          if (mode == 0) {
            // ---- P = Q K^T  (both operands K-major, 16 columns of dk per instruction)
#pragma unroll
            for (int kk = 0; kk < DK / 16; ++kk) {
              const uint32_t off = (kk >> 2) * kGroupBytes + (kk & 3) * 32;
              ptx::mma_ss(tP, ptx::make_smem_desc(q_addr + off, 16, 1024),
                          ptx::make_smem_desc(k_addr + off, 16, 1024), IDESC_QK, kk > 0);
            }
            ptx::tc_commit(p_full);
            // ---- O = Q Sb  (inter-chunk part; Sb is dk x dv, dv contiguous: MN-major B)
            if (i > 0) {
              if (!ptx::mbar_wait(o_free, (i - 1) & 1, abort_flag)) { ok = 0; break; }
            }
            if (have_state) {
              if (!ptx::mbar_wait(sb_ready, sb_waits & 1, abort_flag)) { ok = 0; break; }
              ++sb_waits;
              ptx::tc_fence_after();
#pragma unroll
              for (int kk = 0; kk < DK / 16; ++kk) {
                const uint32_t off = (kk >> 2) * kGroupBytes + (kk & 3) * 32;
                ptx::mma_ss(tO, ptx::make_smem_desc(q_addr + off, 16, 1024),
                            ptx::make_smem_desc(sb_addr + kk * 2048, DK * 128, 1024), IDESC_QS,
                            kk > 0);
              }
            }
            // ---- O += Pb V  (A from TMEM: 16 bf16 = 8 columns per instruction; V MN-major)
            if (!ptx::mbar_wait(pb_ready, i & 1, abort_flag)) { ok = 0; break; }
            ptx::tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < kChunk / 16; ++kk) {
              ptx::mma_ts(tO, tPb + kk * 8,
                          ptx::make_smem_desc(v_addr + kk * 2048, kGroupBytes, 1024), IDESC_PV,
                          (have_state || kk > 0) ? 1u : 0u);
            }
            ptx::tc_commit(o_full);
          }
          // ---- S += K^T V  (both operands MN-major: the token index is the MMA K dimension).
          // For DK = 64 the instruction still spans 128 rows; the upper 64 read whatever follows
          // the K tile in shared memory and land in TMEM lanes nobody reads.
#pragma unroll
          for (int kk = 0; kk < kChunk / 16; ++kk) {
            ptx::mma_ss(tS, ptx::make_smem_desc(k_addr + kk * 2048, kGroupBytes, 1024),
                        ptx::make_smem_desc(v_addr + kk * 2048, kGroupBytes, 1024), IDESC_KV,
                        (have_state || kk > 0) ? 1u : 0u);
          }
          if (mode == 0 || i == n_iter - 1) ptx::tc_commit(s_full);
          ptx::tc_commit(empty_bar(s));
        } while (false);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
    }
  } else if (warp < 6) {
    // ================================================================ converter group
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    const int row = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const uint32_t sb_row = sb_addr + row * 128;
    const uint32_t swz = static_cast<uint32_t>(row & 7);
    uint32_t r[32];

    // Packs 32 fp32 state values (columns cb*32 ..) to bf16 and writes them to the B-operand
    // buffer: [dv group of 64][dk row][128 B], 16-byte pieces XOR-swizzled by (row % 8).
    auto store_sb = [&](int cb) {
      const uint32_t grp = sb_row + (cb >> 1) * (DK * 128);
      const uint32_t j0 = (cb & 1) * 4;
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const uint32_t a0 = ptx::pack_bf16x2(__uint_as_float(r[jj * 8 + 0]), __uint_as_float(r[jj * 8 + 1]));
        const uint32_t a1 = ptx::pack_bf16x2(__uint_as_float(r[jj * 8 + 2]), __uint_as_float(r[jj * 8 + 3]));
        const uint32_t a2 = ptx::pack_bf16x2(__uint_as_float(r[jj * 8 + 4]), __uint_as_float(r[jj * 8 + 5]));
        const uint32_t a3 = ptx::pack_bf16x2(__uint_as_float(r[jj * 8 + 6]), __uint_as_float(r[jj * 8 + 7]));
        ptx::st_shared_v4(grp + (((j0 + jj) ^ swz) << 4), a0, a1, a2, a3);
      }
    };

    if (has_init) {
      const float* src = pr.s_init;
#pragma unroll 1
      for (int cb = 0; cb < DV / 32; ++cb) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = cb * 32 + j;
          float x = 0.f;
          if (row < p.st_rows && col < p.st_cols) x = src[st_off(row, col)];
          r[j] = __float_as_uint(x);
        }
        ptx::tmem_st32(lane_base + cfg::S_COL + cb * 32, r);
        if (row < DK) store_sb(cb);
      }
      ptx::tc_wait_st();
      ptx::fence_proxy_async_smem();
      ptx::tc_fence_before();
      ptx::mbar_arrive(sb_ready);
    }

    if (mode == 0) {
      for (int i = 0; i < n_iter; ++i) {
        // ---------------- P: fp32 -> causal mask -> bf16 A operand
        int ok = ptx::mbar_wait(p_full, i & 1, abort_flag) ? 1 : 0;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ptx::tc_fence_after();
#pragma unroll
        for (int cb = 0; cb < 4; ++cb) {
          uint32_t pk[16];
          const bool all_masked = reverse ? (cb < quad) : (cb > quad);  // warp-uniform
          if (!all_masked) {
            ptx::tmem_ld32(lane_base + cfg::P_COL + cb * 32, r);
            ptx::tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int c0 = cb * 32 + 2 * j;
              const bool k0 = reverse ? (c0 >= row) : (c0 <= row);
              const bool k1 = reverse ? (c0 + 1 >= row) : (c0 + 1 <= row);
              pk[j] = ptx::pack_bf16x2(k0 ? __uint_as_float(r[2 * j]) : 0.f,
                                       k1 ? __uint_as_float(r[2 * j + 1]) : 0.f);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) pk[j] = 0u;
          }
          ptx::tmem_st16(lane_base + cfg::PB_COL + cb * 16, pk);
        }
        ptx::tc_wait_st();
        ptx::tc_fence_before();
        ptx::mbar_arrive(pb_ready);

        // ---------------- S: fp32 -> bf16 B operand for the next chunk (or -> s_final)
        const bool last = (i == n_iter - 1);
        const bool write_final = last && (pr.s_final != nullptr) && (g == nseg - 1);
        if (!last || write_final) {
          ok = ptx::mbar_wait(s_full, i & 1, abort_flag) ? 1 : 0;
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          ptx::tc_fence_after();
#pragma unroll 1
          for (int cb = 0; cb < DV / 32; ++cb) {
            ptx::tmem_ld32(lane_base + cfg::S_COL + cb * 32, r);
            ptx::tc_wait_ld();
            if (write_final && row < p.st_rows) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (cb * 32 + j < p.st_cols)
                  pr.s_final[st_off(row, cb * 32 + j)] = __uint_as_float(r[j]);
            }
            if (!last && row < DK) store_sb(cb);
          }
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
#pragma unroll 1
        for (int cb = 0; cb < DV / 32; ++cb) {
          ptx::tmem_ld32(lane_base + cfg::S_COL + cb * 32, r);
          ptx::tc_wait_ld();
          if (row < p.st_rows) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (cb * 32 + j < p.st_cols)
                pr.s_final[st_off(row, cb * 32 + j)] = __uint_as_float(r[j]);
          }
        }
      }
    }
  } else {
    // ================================================================ epilogue group
    if (mode == 0) {
      const int quad = warp & 3;
      const int row = quad * 32 + lane;
      const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
      const uint32_t swz = static_cast<uint32_t>(row & 7);
      uint32_t r[32];
      uint32_t pk[DV / 2];
      for (int i = 0; i < n_iter; ++i) {
        const int s = i % NS;
        int ok = ptx::mbar_wait(o_full, i & 1, abort_flag) ? 1 : 0;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ptx::tc_fence_after();
#pragma unroll
        for (int cb = 0; cb < DV / 32; ++cb) {
          ptx::tmem_ld32(lane_base + cfg::O_COL + cb * 32, r);
          ptx::tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j)
            pk[cb * 16 + j] =
                ptx::pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
        }
        ptx::tc_fence_before();
        ptx::mbar_arrive(o_free);
        // Stage O in this chunk's Q buffer (every MMA that read it has completed), same
        // swizzled layout as the loads, and hand it to the TMA store.
        const uint32_t obuf = stage_addr(s) + row * 128;
#pragma unroll
        for (int gg = 0; gg < cfg::GV; ++gg) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int base = gg * 32 + j * 4;
            ptx::st_shared_v4(obuf + gg * kGroupBytes + ((static_cast<uint32_t>(j) ^ swz) << 4),
                              pk[base], pk[base + 1], pk[base + 2], pk[base + 3]);
          }
        }
        ptx::fence_proxy_async_smem();
        ptx::mbar_arrive(o_staged);
        // One thread waits (bounded) until all 128 rows are staged, then issues the store.
        if (threadIdx.x == 6 * 32 && ptx::mbar_wait(o_staged, i & 1, abort_flag)) {
          const int tok = mem_chunk(i) * kChunk;
#pragma unroll
          for (int gg = 0; gg < cfg::GV; ++gg)
            ptx::tma_store_4d(&pr.o, stage_addr(s) + gg * kGroupBytes, gg * 64, tok, h, b);
          ptx::bulk_commit_group();
          ptx::bulk_wait_group_read0();
          ptx::mbar_arrive(empty_bar(s));
        }
      }
      if (threadIdx.x == 6 * 32) ptx::bulk_wait_group0();
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
