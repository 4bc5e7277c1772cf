/*
 * cumm_b200 -- C ABI of the B200 (sm_100a) sparse-convolution hot path.
 *
 * Plain pointers and sizes only; every pointer is a CUDA device pointer unless said
 * otherwise.  All entry points are asynchronous on the given stream, keep no reference
 * to caller memory after the launches they enqueue, and are safe to call from several
 * host threads.  They return 0 on success, or a negative CB2_ERR_* code with a message
 * retrievable through cb2_last_error() (thread-local).
 *
 * The two argument structs are the flat kernel-parameter records the reference already
 * passes to its own kernels, extended by the few descriptor fields its dispatcher keys on:
 *   cb2_gemm_args  <->  tv::gemm::GemmNVRTCParams        include/tensorview/gemm/core/nvrtc_params.h:23-36
 *   cb2_conv_args  <->  tv::gemm::SparseConvNVRTCParams  include/tensorview/gemm/core/nvrtc_params.h:38-65
 * dtype codes are tv::DType values (include/tensorview/dtypes.h:39-55): f32 0, i32 1,
 * i8 3, f16 7.
 */
#ifndef CUMM_B200_H_
#define CUMM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CB2_OK 0
#define CB2_ERR_INVALID_ARG (-1) /* maps to std::invalid_argument / ValueError in the reference */
#define CB2_ERR_RUNTIME (-2)     /* maps to std::runtime_error / RuntimeError */
#define CB2_ERR_UNSUPPORTED (-3) /* no kernel for this descriptor ("can't find algo", cumm/gemm/main.py:1323-1333) */
#define CB2_ERR_CUDA (-4)        /* a CUDA call failed (TV_CHECK_CUDA_ERR_V2, include/tensorview/core/common.h:170-175) */

#define CB2_DTYPE_F32 0
#define CB2_DTYPE_I32 1
#define CB2_DTYPE_I8 3
#define CB2_DTYPE_F16 7

/* tv::gemm::ShuffleStrideType, include/tensorview/gemm/core/constants.h:30 */
#define CB2_SHUFFLE_NONE 0
#define CB2_SHUFFLE_AC 1
#define CB2_SHUFFLE_AB 2

/* tv::gemm::ConvOpType, include/tensorview/gemm/core/constants.h:18 */
#define CB2_CONV_FORWARD 0
#define CB2_CONV_BACKWARD_INPUT 1
#define CB2_CONV_BACKWARD_WEIGHT 2

/* tv::gemm::Activation, include/tensorview/gemm/core/constants.h:40-56 */
#define CB2_ACT_NONE 0
#define CB2_ACT_RELU 1
#define CB2_ACT_SIGMOID 2
#define CB2_ACT_LEAKY_RELU 3

/*
 * Gather-GEMM-scatter GEMM.  Replaces the launch made by GemmMainUnitTest::matmul2
 * (cumm/gemm/main.py:1178-1335) after its host prologue (cumm/gemm/nvrtc_code.py:34-146).
 *
 *   ShuffleAC (and NoShuffle, with null index lists):
 *     for i < m:  C[ic(i), :] = act(alpha * A[ia(i), :] * op(B) + beta * D[ic(i), :])
 *     ia = indiceA, ic = indiceBorC; A is [*, k] row-major; B is [n, k] when trans_b
 *     else [k, n].
 *   ShuffleAB (requires trans_a and !trans_b):
 *     C[i, j] = alpha * sum_p A[indiceA[p], i] * B[indiceBorC[p], j] + beta * D[i, j],
 *     p < k.
 * D defaults to C when null.  d_is_vector: D is a length-n vector added to every row
 * (cumm/gemm/nvrtc_code.py:126-128,160-161).  Strides are in elements.
 */
typedef struct cb2_gemm_args {
  int m, n, k;
  const void *ptr_A, *ptr_B, *ptr_D;
  void *ptr_C;
  int64_t stride_A, stride_B, stride_C, stride_D;
  const int32_t *indiceA, *indiceBorC, *indiceD;
  float alpha, beta, act_alpha, act_beta;
  int act_type;
  int split_k_slices; /* accepted for interface parity; the split is chosen internally */
  void *workspace;    /* ShuffleAB only: at least cb2_gemm_workspace_size() bytes */
  size_t workspace_bytes;
  /* descriptor fields (tv::gemm::GemmAlgoDesp, include/tensorview/gemm/core/params.h:24-45) */
  int dtype_a, dtype_b, dtype_c;
  int trans_a, trans_b, trans_c;
  int shuffle_type;
  int d_is_vector;
  int rows_A; /* rows addressable in A (bounds for indiceA); rows_B likewise for ShuffleAB */
  int rows_B;
  /* GemmAlgoDesp::tile_shape[1] and [2] (params.h:24-45): the output columns of one CTA's tile (64 or
   * 128) and the reduction elements per pipeline stage (fp16: 64 or 128); 0 = chosen from the problem.
   * This is what a tuner varies.  ShuffleAB uses tile_n only. */
  int tile_n, tile_k;
  /* Scheduling extensions (no counterpart in the reference; all may be left zero).
   * sched_scratch: 16 bytes of device memory, zero-filled once, owned by THIS argument record: the
   *   tile-ticket counters of the launch (the kernel returns them to zero).  Without it the launch
   *   takes a pair from a per-device pool in round-robin order, which is safe for eager launches
   *   but lets a captured launch (whose pair is fixed at capture) collide with a later eager one
   *   running at the same time on another stream.  Give every captured or replayed call its own;
   *   a caller that launches the SAME record twice in a row alternates between two such blocks
   *   (with programmatic dependent launch the second launch may draw tickets while the first
   *   still runs).
   * max_ctas: upper bound on the CTAs of the launch (0 = one per SM).  The kernels are persistent
   *   and sized to one CTA per SM; calls that are meant to run side by side on different streams
   *   (forward, backward input and backward weight of one layer) each take a share.
   * reuse_plan (ShuffleAB only): the workspace still holds the plan of an earlier, stream-ordered
   *   call on the same workspace with the same reduced masks (contents, not just address), row count,
   *   mask_width, mask_filter, tile_n and max_ctas -- skip the planning kernel.  The plan depends on
   *   the neighbour tables only, so a training loop plans once per scene. */
  void *sched_scratch;
  int max_ctas;
  int reuse_plan;
} cb2_gemm_args;

/*
 * Mask-based implicit-GEMM sparse convolution.  Replaces the launch made by
 * ConvMainUnitTest::implicit_gemm2 (cumm/conv/main.py:485-745) after its host prologue
 * (cumm/conv/nvrtc_code.py:20-260).  ptr_A/B/C follow the reference's role mapping
 * (include/tensorview/gemm/core/utils.h:108-122):
 *   forward          A = input  [*, C],  B = weight [K, kv, C], C = output [N, K]
 *   backward input   A = dout   [*, K],  B = weight [K, kv, C], C = din    [N, C]
 *   backward weight  A = dout   [N, K],  B = input  [*, C],     C = dW     [K, kv, C]
 * N = number of (sorted) rows = second dimension of the neighbour table.
 * indice_ptr [kv, N] int32 in original row order, -1 = no neighbour; mask_ptr: forward /
 * backward input: per-row masks in sorted order [N]; backward weight: reduced masks, one
 * word per mask_width sorted rows (the forward pass's mask_out_ptr).
 * Kernel volumes from 33 to 128 (the reference's dynamic-mask kernels, cumm/gemm/blockmma/mma.py:78-270):
 * W = ceil(kv / 32) words per row, [N, W], word w covering offsets 32w .. 32w+31; mask_out_ptr
 * [ceil(N / 128), W]; reduced masks [chunks, W]; mask_filter applies to every word; with
 * reverse_mask, weight offset p is visited iff the mask bit of offset kv - 1 - p is set.
 * ptr_D: source rows for beta (default C); with d_is_bias a length-(output width) vector.
 * int8 inference (dtype_a == i8, forward only): scale_pointer / bias_pointer fp32 per
 * output channel; ptr_D (if beta != 0) are int8 rows added after scaling
 * (cumm/gemm/output_op/linear.py:279-360).
 */
typedef struct cb2_conv_args {
  const void *ptr_A, *ptr_B, *ptr_D;
  void *ptr_C;
  float alpha, beta, act_alpha, act_beta;
  int act_type;
  int split_k_slices; /* accepted for interface parity; the split is chosen internally */
  void *workspace;    /* backward weight only: at least cb2_conv_workspace_size() bytes */
  size_t workspace_bytes;
  const uint32_t *mask_ptr;
  uint32_t *mask_out_ptr; /* forward only, may be null: [ceil(N / 128)] tile masks */
  const int32_t *indice_ptr;
  const int32_t *mask_argsort_ptr;
  uint32_t mask_filter;
  int reverse_mask;
  int mask_width;
  int ndim, N, C, K;
  int kernel_volume;
  int mode;   /* 1 = cross-correlation (the only mode the reference launches, cumm/conv/nvrtc_code.py:204) */
  int groups; /* 1 */
  int d_is_bias;
  const void *bias_pointer;
  const void *scale_pointer;
  /* descriptor fields (tv::gemm::ConvAlgoDesp, include/tensorview/gemm/core/params.h:166-190) */
  int op_type;
  int dtype_a, dtype_b, dtype_c; /* dtype_c = CB2_DTYPE_F32 is accepted for backward weight */
  int is_int8_inference;
  int rows_A; /* rows addressable in A; rows_B likewise for backward weight */
  int rows_B;
  int mask_words; /* backward weight: number of reduced-mask words available */
  /* ConvAlgoDesp::tile_shape[1] and [2], as in cb2_gemm_args; backward weight uses tile_n only.  Int8
   * kernels exist for tile_k = 128. */
  int tile_n, tile_k;
  /* Scheduling extensions (no counterpart in the reference; all may be left zero).
   * sched_scratch: 16 bytes of device memory, zero-filled once, owned by THIS argument record: the
   *   tile-ticket counters of the launch (the kernel returns them to zero).  Without it the launch
   *   takes a pair from a per-device pool in round-robin order, which is safe for eager launches
   *   but lets a captured launch (whose pair is fixed at capture) collide with a later eager one
   *   running at the same time on another stream.  Give every captured or replayed call its own;
   *   a caller that launches the SAME record twice in a row alternates between two such blocks
   *   (with programmatic dependent launch the second launch may draw tickets while the first
   *   still runs).
   * max_ctas: upper bound on the CTAs of the launch (0 = one per SM).  The kernels are persistent
   *   and sized to one CTA per SM; calls that are meant to run side by side on different streams
   *   (forward, backward input and backward weight of one layer) each take a share.
   * reuse_plan (backward weight only): the workspace still holds the plan of an earlier, stream-ordered
   *   call on the same workspace with the same reduced masks (contents, not just address), row count,
   *   mask_width, mask_filter, tile_n and max_ctas -- skip the planning kernel.  The plan depends on
   *   the neighbour tables only, so a training loop plans once per scene. */
  void *sched_scratch;
  int max_ctas;
  int reuse_plan;
} cb2_conv_args;

/* Launches.  `stream` is a cudaStream_t (the reference passes it as uintptr_t,
 * include/tensorview/gemm/core/params.h:346,420). */
int cb2_gemm_run(const cb2_gemm_args *args, void *stream);
int cb2_conv_run(const cb2_conv_args *args, void *stream);

/*
 * A layer's sequence of ShuffleAC calls in one launch.  (No counterpart in the reference, whose
 * callers launch one GemmParams per filter offset: cumm/gemm/main_real.py:196-232.)
 *
 * `calls[0 .. count)`, count <= 32, are what the caller would pass to cb2_gemm_run one after the
 * other for the filter offsets of one sparse-convolution layer: the same A (ptr_A, stride_A,
 * rows_A), the same C = D (ptr_C, stride_C) with beta = 1 and alpha = 1 (every call accumulates
 * into the output), no activation, and B matrices that are equally spaced slices of one weight
 * tensor (ptr_B of call f = ptr_B of call 0 + f * a constant; same stride_B, trans_b, n, k).
 * Within one call the c_inds are distinct.  The pair lists are scattered into the neighbour
 * table of one convolution (in the workspace: table, masks, sort order) and the layer runs as one
 * mask-convolution launch: out[o] = fp16(out[o] + sum_f A[a_f(o)] B_f), summed in fp32 and
 * rounded once, where the call-by-call sequence rounds to fp16 after every call -- the results
 * agree to a few fp16 ulps, not bit for bit.  `n_out_rows`: rows of C.  `reuse_tables`: the
 * workspace still holds the tables of an earlier call with the same pair lists (they depend on
 * the lists only: build once per scene).  Calls that do not fit these rules are refused with
 * CB2_ERR_UNSUPPORTED and nothing is launched: run them one by one.
 */
typedef struct cb2_gemm_sequence_args {
  const cb2_gemm_args *calls;
  int count;
  int n_out_rows;
  void *workspace; /* at least cb2_gemm_sequence_workspace_size() bytes, 256-byte aligned */
  size_t workspace_bytes;
  int reuse_tables;
} cb2_gemm_sequence_args;

size_t cb2_gemm_sequence_workspace_size(const cb2_gemm_sequence_args *args);
int cb2_gemm_sequence_run(const cb2_gemm_sequence_args *args, void *stream);

/* Bytes of scratch the call needs in args->workspace (0 when none).  Replaces
 * GemmAlgoDesp::query_workspace_size / ConvAlgoDesp::query_conv_workspace_size
 * (include/tensorview/gemm/core/params.h:115-132,286-307); unlike the reference the
 * callee never allocates. */
size_t cb2_gemm_workspace_size(const cb2_gemm_args *args);
size_t cb2_conv_workspace_size(const cb2_conv_args *args);

/*
 * Weight gradient without any allocation.  (No counterpart in the reference: its callee
 * allocates scratch whenever the caller passes none.)
 *
 * For callers that may not allocate device memory where they run: code inside a CUDA
 * stream capture, a real-time or inference-server thread that is forbidden to touch the
 * allocator, a plugin whose host hands it tensors but no allocator.  It computes exactly
 * what cb2_conv_run computes for CB2_CONV_BACKWARD_WEIGHT with the same arguments, except
 * that args->workspace is ignored: the partial sums go to a fixed 16 MiB array that is
 * part of the library image (cb2_static_scratch_bytes()).  Every GPU that loads the library
 * holds that array until the process exits.
 *
 *  - Problems whose scratch does not fit (K * C of 256 * 256 and beyond on a 148-SM part, or
 *    more than about five million rows at K = C = 128: the scratch holds one partial sum per
 *    unit of work and the per-offset lists of row tiles) are refused with CB2_ERR_RUNTIME and a
 *    message naming both sizes; nothing is launched.
 *  - The first call on each device resolves the array's device address.  That one call
 *    should be made before any stream capture begins on that device.
 *  - All calls share the one array and it keeps the previous call's contents; every call
 *    clears the control words it uses and rewrites every partial sum it later reads, so nothing
 *    has to be cleared between calls, but two calls that overlap on the same GPU (different
 *    streams, no ordering) race on it.
 *  - Neither this call nor anything it calls uses cudaMalloc, cudaFree or an allocating
 *    library routine.  Its kernels report through their own status word:
 *    cb2_static_status() is to this entry point what cb2_device_status() is to the others.
 */
int cb2_conv_backward_weight_static(const cb2_conv_args *args, void *stream);
size_t cb2_static_scratch_bytes(void);
int cb2_static_status(int *status);

/*
 * Neighbour tables of a sparse convolution, built on the GPU -- the step before the calls above.
 * (No counterpart inside the reference: its callers build these tables on top of its hash
 * headers, include/tensorview/hash/hash.cu.h:43-263, ops.h:24-150.  The layout produced is the
 * one cb2_conv_args consumes, include/tensorview/gemm/core/nvrtc_params.h:38-65.)
 *
 * Convention: filter offsets in (z, y, x) row-major order; indices [kv, n_out] int32 in original
 * row order, -1 = no neighbour; bit f of a row's mask set iff indices[f, row] >= 0; mask [n_out]
 * holds the masks in ascending order and mask_argsort the rows in that order (stable: equal
 * masks keep their row order); the active outputs of a strided convolution are ordered by their
 * linearised (batch, z, y, x).  The backward arrays are the same for the transposed relation
 * (indices_bwd [kv, n_in], indices_bwd[f, i] = o iff indices[f, o] = i) and may be null.
 * Kernel volumes above 32, up to 128 (the "dynamic mask" kernels): words = ceil(kv / 32) mask words
 * per row, mask [n_out, words], mask_bwd [n_in, words], tile_masks [ceil(n_out / 128), words]; word
 * w holds offsets 32w .. 32w+31, and rows are ordered as one integer whose LAST word is the most
 * significant (stable).
 *
 * Submanifold (subm != 0): outputs are the inputs, n_out = n_in, one call of cb2_pairgen_run.
 * Otherwise call cb2_pairgen_count_outputs first (it finds and sorts the active outputs inside
 * the workspace, synchronises the stream and returns their number), size the output arrays,
 * set n_out and call cb2_pairgen_run with the same workspace.
 * Kernels report through the status word of cb2_device_status(): 3 = a hash table overflowed
 * (cannot happen with a workspace of the stated size), 4 = a coordinate outside the grid or
 * batch.
 */
typedef struct cb2_pairgen_args {
  const int32_t *in_coords; /* [n_in, 4]: batch, z, y, x */
  int n_in;
  int batch_size;           /* coordinates' batch index is in [0, batch_size) */
  int grid[3];              /* input grid extent (z, y, x) */
  int ksize[3], stride[3], pad[3], dil[3];
  int subm;
  int n_out;                /* subm: ignored (= n_in) */
  int32_t *out_coords;      /* [n_out, 4]; not written when subm */
  int32_t *indices;         /* [kv, n_out] */
  uint32_t *mask;           /* [n_out] ([n_out, words] for kernel volumes above 32) */
  int32_t *mask_argsort;    /* [n_out] */
  int32_t *indices_bwd;     /* [kv, n_in] or null */
  uint32_t *mask_bwd;       /* [n_in] ([n_in, words]) or null */
  int32_t *mask_argsort_bwd;/* [n_in] or null */
  void *workspace;          /* at least cb2_pairgen_workspace_size() bytes, 256-byte aligned */
  size_t workspace_bytes;
  uint32_t *tile_masks;     /* [ceil(n_out / 128)] or null: OR of the masks of each 128 sorted rows, i.e. what a
                               forward call with mask_filter = all ones writes to mask_out_ptr and backward
                               weight reads as mask_ptr with mask_width = 128 */
} cb2_pairgen_args;

size_t cb2_pairgen_workspace_size(const cb2_pairgen_args *args);
int cb2_pairgen_count_outputs(const cb2_pairgen_args *args, int *n_out, void *stream);
int cb2_pairgen_run(const cb2_pairgen_args *args, void *stream);

/*
 * Neighbour tables of a DENSE (non-mask) convolution, channels last: with them the dense
 * convolutions of the reference (ConvAlgoDesp::mask_sparse == false; cumm/conv/input_iters.py:2353,
 * harness cumm/conv/main_real.py:41-231) run through cb2_conv_run like a sparse convolution whose
 * voxels fill the grid.  Rows are (batch, z, y, x) row-major; unused leading axes have extent 1.
 * Coordinate rule: in = out * stride - pad + r * dilation per axis (cumm/conv/input_iters.py:2666,2684).
 * indices_fwd [kv, n_out] (forward, backward weight), indices_bwd [kv, n_in] (backward input; may be
 * null), mask_* [rows, ceil(kv / 32)] all-ones masks and identity orders for each direction (may be null).
 */
typedef struct cb2_dense_tables_args {
  int batch;
  int in_dims[3], out_dims[3]; /* (z, y, x) */
  int ksize[3], stride[3], pad[3], dil[3];
  int32_t *indices_fwd;
  int32_t *indices_bwd;
  uint32_t *mask_fwd;
  int32_t *argsort_fwd;
  uint32_t *mask_bwd;
  int32_t *argsort_bwd;
} cb2_dense_tables_args;

int cb2_dense_tables_run(const cb2_dense_tables_args *args, void *stream);

/*
 * Sum of one fp32 array per GPU over NVLink peer memory, for the weight gradient of a
 * convolution whose rows are sharded over the GPUs of a node.  (No counterpart in the
 * reference, which is single-GPU.)  Every GPU makes the same sequence of calls with the same
 * `numel`; each gets the same, bit-identical sum, as fp32 and/or fp16.  The call number that
 * pairs the calls of the GPUs is kept inside the buffers, so a call can be captured in a CUDA
 * graph and replayed.
 * `peer_buffers`: a HOST array of `world` device pointers, the buffer of every GPU as mapped
 * in the calling process (peer_buffers[rank] is the caller's own), each of
 * cb2_peer_allreduce_buffer_size() bytes, zero-filled once before the first call.  The kernel
 * sends shard s of its array to GPU s (plain stores over NVLink), sums the shards it receives
 * in GPU order and sends the sums to every GPU.  Every float travels beside a copy of the call
 * number (8 bytes per float in the buffers), and a reader repeats its load until that number is
 * the current one: no fence or flag round trip separates the GPUs.  Such a wait lasts at most
 * `timeout_ns` (0 = one second); one that runs out sets status word 1 (cb2_device_status) and
 * leaves the outputs untouched.  The kernel's CTAs all have to be resident at the same time;
 * they are small (128 threads), and at most one per SM is launched.
 */
typedef struct cb2_peer_allreduce_args {
  void *const *peer_buffers;
  int rank, world; /* world <= 16 */
  const float *src;
  float *out_f32;  /* may be null */
  void *out_f16;   /* may be null */
  long long numel; /* multiple of 4 */
  unsigned long long timeout_ns;
  int own_sm_smem_bytes; /* 0, or dynamic shared memory to request per CTA (unused by the kernel): a value above
                            what the persistent convolution kernels leave free on an SM (about 11 KB) keeps this
                            kernel's CTAs off the SMs those kernels occupy, so that they run at full speed on the
                            SMs a caller left free (max_ctas of the convolution calls) instead of beside them */
} cb2_peer_allreduce_args;

size_t cb2_peer_allreduce_buffer_size(long long numel, int world);
int cb2_peer_allreduce(const cb2_peer_allreduce_args *args, void *stream);

/*
 * The kernel table: one record per kernel variant a descriptor can select.  Replaces
 * GemmMainUnitTest::get_all_algo_desp (cumm/gemm/main.py:916-965) and
 * ConvMainUnitTest::get_all_conv_algo_desp (cumm/conv/main.py:985-1050); the fields are the
 * ones of tv::gemm::GemmAlgoDesp / ConvAlgoDesp (include/tensorview/gemm/core/params.h:24-45,
 * 166-190) that differ between the variants.  Both calls return the number of variants and
 * fill at most `capacity` records (out may be null to ask for the count); they need no GPU.
 */
typedef struct cb2_kernel_desp {
  int op_type;      /* conv: CB2_CONV_*; gemm: -1 */
  int shuffle_type; /* gemm: CB2_SHUFFLE_*; conv: CB2_SHUFFLE_NONE */
  int dtype_a, dtype_b, dtype_c, dacc, dcomp;
  int trans_a, trans_b, trans_c;
  int tile_shape[3];      /* rows, columns, reduction of one CTA tile */
  int warp_tile_shape[3]; /* = tile_shape: one tcgen05.mma covers the CTA tile */
  int tensorop[3];        /* shape of one tcgen05.mma instruction */
  int num_stage;
  int element_per_access; /* a, b and c alike: 16 bytes */
  int split_k_serial;
  int mask_sparse, increment_k_first, is_int8_inference;
  int min_arch_major, min_arch_minor;
  int dynamic_mask; /* conv: the variant for kernel volumes above 32 (several mask words per row, up to 128
                       offsets; name suffix D, params.h:191-224); it also runs smaller volumes */
} cb2_kernel_desp;

int cb2_enumerate_gemm_desps(cb2_kernel_desp *out, int capacity);
int cb2_enumerate_conv_desps(cb2_kernel_desp *out, int capacity);

/* Rows of one output tile, i.e. the granularity of mask_out_ptr and the mask_width to
 * hand to backward weight (the reference uses the forward kernel's tile_shape[0],
 * cumm/conv/main_real_spconv.py:176-177). */
int cb2_tile_m(void);

/* Message of the last failing call on this host thread. */
const char *cb2_last_error(void);

/* Kernels never spin without bound: a wait that runs out, or a row index outside
 * rows_A / rows_B, sets a per-device status word instead.  This call synchronises the
 * current device, returns the word (0 = ok, 1 = wait timed out, 2 = row index out of
 * range; 3 and 4: see cb2_pairgen_args) in *status and clears it. */
int cb2_device_status(int *status);

/* Registers per thread, threads per CTA and dynamic shared memory of the last convolution / GEMM
 * kernel launched by the calling host thread (what the reference prints for ConvParams::verbose
 * from cudaFuncGetAttributes, cumm/conv/main.py:723-729).  Any pointer may be null. */
int cb2_last_launch_info(int *num_regs, int *num_threads, int *smem_bytes);

/* Number of kernels this library has launched from the calling process (all threads). */
uint64_t cb2_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* CUMM_B200_H_ */
