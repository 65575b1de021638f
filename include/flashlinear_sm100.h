/*
 * C ABI of libflashlinear_sm100.so: causal, unnormalised linear attention
 *     O = (Q K^T (.) M) V          (M = lower-triangular ones, diagonal included)
 * forward and backward on NVIDIA B200 (sm_100a), bf16 operands, fp32 accumulation.
 *
 * These entry points are what the launch wrappers of the reference library
 * (flashlinear/kernels/linear_attn_kernels.py:310-341 `linear_flash_wrapper_fwd`,
 *  :345-384 `linear_flash_wrapper_bwd`, and
 *  flashlinear/kernels/linear_attn_kernels_smallv_hd.py:320-359 / :363-405, the
 *  `_smallv_hd` pair for dk != dv) bind instead of launching their Triton kernels.
 *
 * Conventions
 *  - plain C types only; all tensor pointers are device pointers on the CURRENT device;
 *  - tensors are [batch, heads, seqlen, dim] bf16 with arbitrary (batch, head, token) element
 *    strides and an innermost stride of 1; base addresses and byte strides must be multiples
 *    of 16 (return FLA_ERR_ALIGNMENT otherwise; the Python wrapper then repacks); outputs are
 *    stored in 16-byte units, so the row pitch must cover dim rounded up to a multiple of 8 and,
 *    when dim is not such a multiple, the elements between a row's last column and the next
 *    16-byte boundary are overwritten with zeros;
 *  - every call is asynchronous on `stream`, never synchronises, never allocates or frees
 *    device memory; scratch memory (when fla_sm100_workspace_bytes() > 0) is the caller's;
 *  - returns 0 or a negative FLA_ERR_* code for argument errors, synchronously;
 *  - device-side waits are bounded; a wait that runs out sets bit 0 of *status (optional device
 *    word the caller zero-initialises and reads after synchronising).
 */
#ifndef FLASHLINEAR_SM100_H_
#define FLASHLINEAR_SM100_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FLA_ABI_VERSION 9
#define FLA_DTYPE_BF16 0
#define FLA_DTYPE_F16 1

enum {
  FLA_OK = 0,
  FLA_ERR_INVALID = -1,     /* null pointer, non-positive size, bad struct */
  FLA_ERR_UNSUPPORTED = -2, /* head dims outside what the kernels are built for */
  FLA_ERR_ALIGNMENT = -3,   /* pointer or byte stride not a multiple of 16 */
  FLA_ERR_CUDA = -4,        /* a CUDA runtime / driver call failed */
  FLA_ERR_WORKSPACE = -5,   /* workspace missing or too small */
  FLA_ERR_DEVICE = -6,      /* current device is not compute capability 10.x */
  FLA_ERR_SCRATCH_LIMIT = -7 /* fla_sm100_fwd_static_scratch: shape exceeds the built-in scratch */
};

/* Size of the built-in scratch array used by fla_sm100_fwd_static_scratch(). */
#define FLA_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)

/* One [batch, heads, seqlen, dim] bf16 tensor: device pointer and element strides of the three
 * outer dimensions (the innermost stride is 1). */
typedef struct FlaTensor {
  void* ptr;
  int64_t stride_b;
  int64_t stride_h;
  int64_t stride_n;
} FlaTensor;

typedef struct FlaArgs {
  int32_t batch, heads, seqlen;
  int32_t dk; /* head dim of q, k (and dQ, dK) */
  int32_t dv; /* head dim of v, o (and dO, dV) */

  FlaTensor q, k, v; /* inputs of both passes */
  FlaTensor o;       /* forward output          [.., dv] */
  FlaTensor d_o;     /* backward input          [.., dv] */
  FlaTensor d_q;     /* backward outputs        [.., dk] */
  FlaTensor d_k;     /*                         [.., dk] */
  FlaTensor d_v;     /*                         [.., dv] */

  /* Optional running state, fp32 [batch*heads, dk, dv], contiguous. Forward: s_init is
   * S = sum_j k_j^T v_j over the tokens that precede this call's tokens, s_final receives the
   * state after them. Backward: s_init as in the forward (needed for dQ), r_init is
   * R = sum_i q_i^T dO_i over the tokens that FOLLOW this call's tokens, r_final receives the
   * state including them. NULL = zero / not wanted. */
  const float* s_init;
  float* s_final;
  const float* r_init;
  float* r_final;
  /* Backward only, optional: the forward state AFTER this call's tokens (what the forward call
   * wrote to s_final). When given (and fla_sm100_bwd_uses_final_state() says so: the call is not
   * split into segments or comes with seg_states, and the sequence is longer than 2048 tokens) dQ
   * is computed in the same end-to-start sweep as dK and dV, which lets the three share every read
   * of q, k, v, dO; s_init is then not needed. */
  const float* s_last;

  /* Sequence segments per head (intra-GPU sequence split). 0 = pick automatically, 1 = none.
   * With more than one segment the call needs fla_sm100_workspace_bytes() of scratch. */
  int32_t segments;
  /* Forward / product calls only, with more than one segment: non-zero means that `workspace`
   * already holds the per-segment prefix states of these tokens, exactly as fla_sm100_state()
   * left them there for the same k, v, shapes and `segments`. The call then skips its own state
   * pass and scan, and s_init (if any) is added on top for every segment. This is how a
   * sequence-sharded forward avoids reading k, v a third time: state pass -> exchange of the
   * per-GPU totals -> this call. */
  int32_t segment_states_ready;

  void* workspace;
  size_t workspace_bytes;

  int32_t* status; /* optional device word, see above */
  void* stream;    /* cudaStream_t */

  /* Optional, few heads per GPU: boundary states that a segmented forward stores for the backward.
   * fla_sm100_seg_states_bytes() says how many bytes the pair of calls wants for these shapes (0:
   * not used). Give the same buffer, the same `segments` and s_final / s_last to fla_sm100_fwd and
   * fla_sm100_bwd: the backward then runs as one launch, split at the forward's segment boundaries,
   * instead of a state pass, a scan and the product pass. The contents are private to the library. */
  void* seg_states;
  size_t seg_states_bytes;

  /* Element type of every [batch, heads, seqlen, dim] tensor of the call: FLA_DTYPE_BF16 (0, what
   * the reference computes in, flashlinear/kernels/linear_attn_kernels.py:82,98) or FLA_DTYPE_F16.
   * fp16 runs the same kernels with fp16 tensor-core operands and fp16 outputs, for head dims up
   * to 128 (fla_sm100_fwd / _bwd / _state / _product); accumulation and the running states stay
   * fp32. Mind the range: the unnormalised product grows with the sequence and fp16 ends at 65504. */
  int32_t dtype;

  /* Limit of one device-side wait in microseconds of the GPU's global timer; 0 = the default of
   * 2 s. Legitimate waits of these kernels last microseconds; the default leaves room for a kernel
   * that is switched out for another context's time slice on a shared GPU. */
  uint32_t wait_limit_us;
  /* FLA_DEBUG_* bits, 0 in production. */
  uint32_t debug_flags;
} FlaArgs;

/* Test hook for the status path: the kernel never loads its first tile, so the waits that depend
 * on it run out after wait_limit_us, bit 0 of *status is set and the CTAs return normally (the
 * outputs of the call are garbage). Nothing faults or hangs. */
#define FLA_DEBUG_WITHHOLD_FIRST_TILE 1u
/* Segmented calls normally run as ONE cooperative launch when all their CTAs fit the GPU at once
 * (see fla_sm100_seg_states_bytes). This bit keeps the older three-launch form (state pass, scan,
 * product pass), for comparisons.
 * The CTAs of such a launch meet at barriers whose words come from a pool of 64 sets inside the
 * library, handed out round-robin per launch (a captured launch keeps the set it was captured
 * with). Launches in one stream never overlap; launches that do run at the same time on one GPU
 * (several streams) must not hold the same set, i.e. must not be 64 or a multiple of 64 fused
 * launches apart. A process that replays many captured graphs on concurrent streams should set
 * this bit for all but one of the streams. */
#define FLA_DEBUG_NO_FUSED_SEGMENTS 2u
/* The backward uses s_last (dQ in the same end-to-start sweep as dK and dV) only for sequences
 * longer than 2048 tokens; on shorter ones that form is a little less accurate than the
 * two-direction form and saves nothing worth having. This bit lifts the length rule, for tests. */
#define FLA_DEBUG_FORCE_SINGLE_SWEEP 4u

/* Diagnostics for bit 0 of the status word: copies up to max_records records (8 words each) of the
 * first waits that ran out on the current device since the last call, and clears them. Words:
 * shared-memory address of the mbarrier, parity waited for, thread index, block x / y / z,
 * shared-memory address of the CTA's abort flag (which locates the barrier area), clock >> 10.
 * Synchronises the device. Returns the number of records, or a negative error code. */
int fla_sm100_timeout_records(unsigned* out, int max_records);

/* pass: 0 = forward, 1 = backward, 2 = fla_sm100_state */
int fla_sm100_abi_version(void);
const char* fla_sm100_strerror(int code);
size_t fla_sm100_workspace_bytes(const FlaArgs* args, int pass);
/* Number of segments the call will use for args->segments == 0. */
int fla_sm100_auto_segments(const FlaArgs* args, int pass);
/* Bytes for FlaArgs::seg_states, or 0 when forward + backward of these shapes do not use them (many
 * heads: nothing is segmented; dk != dv; head dims above 128). The reference has no counterpart: its
 * grid is (sequence blocks, batch*heads) with quadratic work per block
 * (flashlinear/kernels/linear_attn_kernels.py:329-331) and needs no state. */
size_t fla_sm100_seg_states_bytes(const FlaArgs* args);
/* 1 when fla_sm100_bwd for these shapes makes use of s_last (so that the forward should be asked
 * for s_final), 0 when it would ignore it: segmented backward without seg_states, sequences of at
 * most 2048 tokens, head dims above 128. */
int fla_sm100_bwd_uses_final_state(const FlaArgs* args);

/* replaces linear_flash_wrapper_fwd / linear_flash_wrapper_fwd_smallv_hd
 * (flashlinear/kernels/linear_attn_kernels.py:310, linear_attn_kernels_smallv_hd.py:320) */
int fla_sm100_fwd(const FlaArgs* args);
/* replaces linear_flash_wrapper_bwd / linear_flash_wrapper_bwd_smallv_hd
 * (flashlinear/kernels/linear_attn_kernels.py:345, linear_attn_kernels_smallv_hd.py:363) */
int fla_sm100_bwd(const FlaArgs* args);

/* State of this call's tokens only, without an output: which = 0 writes
 * s_final = sum_j k_j^T v_j (reads k, v), which = 1 writes r_final = sum_i q_i^T dO_i (reads q, d_o).
 * Sequence-sharded callers exchange these [batch*heads, dk, dv] fp32 states between GPUs before
 * calling fla_sm100_fwd / fla_sm100_bwd with s_init / r_init. The reference has no counterpart:
 * its kernels are quadratic and keep no state (flashlinear/kernels/linear_attn_kernels.py:63). */
int fla_sm100_state(const FlaArgs* args, int which);

/* ---- sequence sharding: state pass fused with the exchange between the GPUs of one node ----
 * Every rank holds N/W consecutive tokens of every head. fla_sm100_state_exchange() computes the
 * per-segment states of this rank's tokens (which = 0: sum k^T v, reads k, v; which = 1: sum q^T dO,
 * reads q, d_o) and then, in ONE kernel, (1) scans them, (2) stores this rank's total straight into
 * the inbox of every peer GPU over NVLink (plain stores to peer-mapped memory) and raises a flag
 * there, (3) waits -- bounded -- for the peers' flags in its own inbox, (4) adds the totals of the
 * ranks before it (after it when `reverse`) to every segment prefix. Afterwards
 *   - args->workspace holds the per-segment prefixes including the other GPUs' contribution: call
 *     fla_sm100_fwd / fla_sm100_product with segment_states_ready = 1 and no s_init;
 *   - remote_out (optional) holds the other GPUs' contribution alone, inclusive_out (optional) that
 *     plus this rank's total: the s_init / r_init / s_last of the backward call.
 * No NCCL call is involved. The reference has no counterpart (it has no multi-GPU code).
 *
 * inbox[d] / flags[d] are the base addresses of rank d's inbox and flag array AS MAPPED INTO THIS
 * PROCESS (peer-mapped device memory, e.g. opened from CUDA IPC handles); inbox[rank] / flags[rank]
 * are this rank's own. Sizes: fla_sm100_exchange_bytes(). Both must be zero before the first use.
 * `epoch` starts at 1 and increases by 1 with every exchange on these buffers, on all ranks alike.
 * Alternatively the count lives on the device: with `epoch_counter` set (a zero-initialised device
 * word per buffer set, the same on every rank) the kernel uses *epoch_counter + 1 and a one-thread
 * kernel behind it stores that value back; `epoch` is then ignored and the call has no argument
 * that changes between launches, so it can be captured in a CUDA graph and replayed.
 * All ranks must make the same sequence of calls. A peer that never shows up makes the wait run
 * out after wait_limit_us (0 = about 0.4 s): bit 1 of *status is set and everything the call
 * produces (scratch prefixes, remote_out, inclusive_out) is filled with NaN, so that the outputs of
 * the passes built on it are NaN as well. The wait can also run out when ranks reach the call more
 * than the limit apart (a slow data loader, a first-call module load): read *status at the next
 * synchronisation point, or raise the limit. Shapes with more than 592 batch*heads are refused
 * (FLA_ERR_UNSUPPORTED): every block waits for its twin on the other GPUs, so all blocks must be
 * resident at once. */
#define FLA_MAX_RANKS 8
typedef struct FlaExchange {
  int32_t rank, world;
  int32_t reverse; /* 0: add the states of the ranks before this one; 1: of the ranks after it */
  uint32_t epoch;
  float* inbox[FLA_MAX_RANKS];
  uint32_t* flags[FLA_MAX_RANKS];
  float* remote_out;    /* optional, fp32 [batch*heads, dk, dv] */
  float* inclusive_out; /* optional, fp32 [batch*heads, dk, dv] */
  uint32_t* epoch_counter; /* optional device word, see above */
  uint32_t wait_limit_us;  /* how long a block waits for a peer's flag; 0 = 400000 (0.4 s) */
} FlaExchange;
/* Bytes of one rank's inbox (*inbox_bytes) and flag array (*flag_bytes) for these shapes. */
int fla_sm100_exchange_bytes(const FlaArgs* args, int world, size_t* inbox_bytes, size_t* flag_bytes);
/* Scratch needed in args->workspace by fla_sm100_state_exchange (never 0). */
size_t fla_sm100_exchange_workspace_bytes(const FlaArgs* args);
int fla_sm100_state_exchange(const FlaArgs* args, int which, const FlaExchange* exchange);
/* Set-up helpers for the exchange buffers (the only calls of this library that allocate).
 * alloc: cudaMalloc + zero fill on the current device and the 64-byte CUDA IPC handle of the
 * allocation, to be sent to the other ranks of the node. open: maps a peer's allocation into this
 * process WITH THE CALLER'S DEVICE CURRENT, so that this device's kernels can store into it; the
 * mapping is verified with a runtime copy before it is returned. close / free undo them. */
int fla_sm100_exchange_alloc(size_t bytes, void** ptr, unsigned char* handle64);
int fla_sm100_exchange_open(const unsigned char* handle64, void** ptr);
int fla_sm100_exchange_close(void* ptr);
int fla_sm100_exchange_free(void* ptr);
/* Lets kernels on the current device store into memory of `peer_device` (cudaDeviceEnablePeerAccess;
 * already-enabled is not an error). Needed for peer memory that was NOT mapped by
 * fla_sm100_exchange_open (which enables access itself, cudaIpcMemLazyEnablePeerAccess), e.g.
 * buffers of another device of the same process. */
int fla_sm100_enable_peer_access(int peer_device);

/* The building block of both passes: o_i = sum_{j<=i} (q_i . k_j) v_j, or with anticausal != 0 the
 * sum over j >= i (tokens walked from the last to the first; s_init / s_final then refer to the
 * tokens after / up to this call's tokens). fla_sm100_fwd is this product of (q, k, v); the
 * gradients of flashlinear/kernels/linear_attn_kernels.py:179-197 and :291-299 are
 * dQ = product(dO, v, k), dV = anticausal product(k, q, dO), dK = anticausal product(v, dO, q).
 * The Python layer uses it to assemble head dims above 384 from slices. Workspace: as for pass 0. */
int fla_sm100_product(const FlaArgs* args, int anticausal);

/* Head dims above 128 (the SmallVHD shapes of flashlinear/kernels/linear_attn_kernels_smallv_hd.py:
 * q, k wide, v narrow; LinearAttention with head dims up to 256, linear_attn_kernels.py:316-322):
 * fla_sm100_fwd, fla_sm100_bwd and fla_sm100_product accept every dk, dv up to 384 (bf16):
 *   dk in (128, 384]                  q/k tiles streamed in 128-column pieces by a dedicated kernel, one
 *                                     CTA per 64-column slice of v / o (one slice when dv <= 64),
 *   dk <= 128 with dv in (128, 384]   output columns computed in 128-wide slices of one grid,
 * (for the backward the same rules apply to each of the three gradient products with its own
 * operand widths), without running-state arguments, segments or workspace. Row strides must still be multiples of
 * 16 bytes; a contiguous tensor with an odd head dim (273) is first copied to padded rows: */
/* dst[r][0..dpad) = src[r][0..d) followed by zeros; src and dst contiguous bf16, dpad a multiple of 8.
 * The reference pads in registers instead (boundary_check / padding_option="zero",
 * linear_attn_kernels_smallv_hd.py:60-75). */
int fla_sm100_pad_rows(const void* src, void* dst, long long rows, int d, int dpad, void* stream);
/* dst[r][0..d) = src[r][0..d) for src rows of dpad elements: the inverse copy, for gradients that
 * must come back in the contiguous layout of torch.empty_like (linear_attn_kernels_smallv_hd.py:384). */
int fla_sm100_unpad_rows(const void* src, void* dst, long long rows, int d, int dpad, void* stream);

/* ---- normalised attention: the denominator of README.md:27-30 as kernels ----
 * The reference returns the unnormalised product and leaves
 *     denom = (q * k.cumsum(-2)).sum(-1, keepdim=True) + eps;  out = num / denom
 * to PyTorch (several full-tensor passes, the cumulative sum in bf16). These three calls do it in
 * one sweep per tensor with an fp32 running sum; they are opt-in (LinearAttentionNormalized in the
 * Python layer) and change nothing about fla_sm100_fwd / fla_sm100_bwd.
 *
 * normalize_fwd: args->q, k (dk) and args->o (dv) holding the unnormalised product; on return
 *   args->o holds o / den (in place) and den[b*heads + h][i] = q_i . sum_{j<=i} k_j + eps (fp32).
 * normalize_bwd_prepare: args->d_o = gradient g of the normalised output, args->o = the normalised
 *   output; writes args->d_v = g / den (the upstream gradient of the product, feed it to
 *   fla_sm100_bwd as d_o) and dden[..][i] = -(g_i . o_i) / den_i.
 * normalize_bwd_sweep: adds the denominator's part to the gradients fla_sm100_bwd produced, in
 *   place: d_q[i] += dden_i * sum_{j<=i} k_j,  d_k[j] += sum_{i>=j} dden_i q_i  (reads q, k).
 * Long sequences are cut into segments that run as separate CTAs; a column-sum kernel first gives
 * every segment its starting sums. normalize_fwd and normalize_bwd_sweep therefore take scratch
 * in args->workspace (fla_sm100_normalize_workspace_bytes(), pure scratch: nothing is kept in it
 * between calls). Head dims up to 512. */
size_t fla_sm100_normalize_workspace_bytes(const FlaArgs* args);
int fla_sm100_normalize_fwd(const FlaArgs* args, float eps, float* den);
int fla_sm100_normalize_bwd_prepare(const FlaArgs* args, const float* den, float* dden);
int fla_sm100_normalize_bwd_sweep(const FlaArgs* args, const float* dden);

/* ---- second-order Taylor feature map (benchmark configuration 4) ----
 * phi(x) = [1, x / d^(1/4), vec(x x^T) / (sqrt(2) sqrt(d))]: 1 + d + d^2 features, so that
 * phi(q) . phi(k) = 1 + s + s^2 / 2 with s = q . k / sqrt(d). The reference has no such code (its
 * README links the idea only); d = 16 gives the 273 features fed to LinearAttentionSmallVHD.
 * taylor_features writes bf16 rows of `padded` elements (the first `features` valid, the rest zero),
 * i.e. rows the attention kernels address in place (pass stride_n = padded): no pad pass.
 * taylor_features_bwd contracts gradients of such rows back to the d raw dimensions.
 * x, dx: [rows][d] bf16 contiguous; phi, dphi: [rows][padded] bf16. d = 8 or 16. */
int fla_sm100_taylor_dims(int d, int* features, int* padded);
int fla_sm100_taylor_features(const void* x, void* phi, long long rows, int d, void* stream);
int fla_sm100_taylor_features_bwd(const void* dphi, const void* x, void* dx, long long rows, int d,
                                  void* stream);

/* Forward pass for callers that cannot obtain device memory themselves.
 * It has no counterpart in the reference (whose wrappers allocate through torch).
 *
 * Some integrations must not call cudaMalloc or any allocating library routine at the point where
 * the attention runs: for instance a plugin that executes inside another runtime's memory plan, a
 * real-time serving loop that forbids allocation after start-up, or host code that only receives
 * raw input / output pointers. The ordinary fla_sm100_fwd() needs caller-provided scratch as soon as
 * the sequence is split into segments (few heads, long sequences). This variant takes the same
 * FlaArgs (q, k, v, o, optional s_init / s_final, segments, status, stream; workspace fields are
 * ignored) and keeps the per-segment states in a fixed array of FLA_STATIC_SCRATCH_BYTES that is
 * part of the library image on every GPU that loads it. Shapes that fla_sm100_fwd runs without
 * scratch (one segment; q/k wider than 128 with v <= 64) are dispatched exactly as it does.
 *  - It performs no device allocation or free, directly or through a library.
 *  - Shapes whose segment states (batch*heads*segments*dk*dv*4 bytes) exceed the array are refused
 *    with FLA_ERR_SCRATCH_LIMIT before anything is launched; pass a smaller `segments`.
 *  - The first call on each device THAT SPLITS THE SEQUENCE looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current). Make that first call outside any stream
 *    capture.
 *  - All calls on a device share the one array. Calls whose kernels may overlap on the GPU (other
 *    streams, other host threads) race on it; serialise them. Nothing in it needs clearing
 *    between calls: each call writes every entry it later reads. */
int fla_sm100_fwd_static_scratch(const FlaArgs* args);

/* Number of kernels the last fwd / bwd call on this thread launched (for benchmarks). */
int fla_sm100_last_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* FLASHLINEAR_SM100_H_ */
