/*
 * scn_b200.h -- C ABI of the sm_100a submanifold sparse-convolution inference path.
 *
 * This is the drop-in boundary.  The reference (facebookresearch/SparseConvNet) exposes the
 * same operations through a pybind11 module, `sparseconvnet.SCN`
 * (sparseconvnet/SCN/pybind.cpp:201-237, prototypes in sparseconvnet/SCN/sparseconvnet.h);
 * each entry point below names the reference function it replaces.  A binding for the
 * reference only has to turn `at::Tensor` arguments into the plain pointers and sizes used
 * here.
 *
 * Conventions
 *  - every function returns an `int` status (SCN_OK == 0); `scn_last_error()` gives a
 *    thread-local message for the last non-zero status.  Nothing traps or aborts.
 *  - `stream` is a `cudaStream_t` passed as `void*` (NULL = legacy default stream).
 *  - spatial sizes, filter sizes and strides are HOST arrays of `dimension` int64 values,
 *    as in the reference (CPU LongTensors).
 *  - feature matrices are DEVICE pointers to row-major float32 `[rows, planes]`, owned by
 *    the caller.  Rows are the active sites of one spatial scale, numbered as
 *    `scn_md_spatial_locations` reports them.
 *  - a `scn_metadata` owns the device-side site hash tables, the per-filter-offset
 *    rulebooks and their cache, exactly the role of the reference's `Metadata<D>`
 *    (sparseconvnet/SCN/Metadata/Metadata.h:44-167).  It is not thread safe, like the
 *    reference object.
 *  - device memory for tables, rulebooks and per-call scratch comes from a stream-ordered memory
 *    pool that the library creates per device (not the device's default pool); freed blocks stay
 *    in that pool for reuse until scn_trim_memory gives them back to the driver.
 *  - a scn_metadata belongs to the device that was current at its first use; using it with
 *    another device current is SCN_ERR_BAD_ARG.  It may be used on one stream at a time.
 */
#ifndef SCN_B200_H
#define SCN_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define SCN_API __attribute__((visibility("default")))
#else
#define SCN_API
#endif

#define SCN_ABI_VERSION 1
#define SCN_MAX_DIMENSION 6

typedef struct scn_metadata scn_metadata;

enum scn_status {
  SCN_OK = 0,
  SCN_ERR_BAD_ARG = 1,      /* null pointer, bad dimension, bad mode ...                    */
  SCN_ERR_CUDA = 2,         /* a CUDA runtime call failed; message has the CUDA string      */
  SCN_ERR_COORD_RANGE = 3,  /* a coordinate or batch index lies outside its field          */
  SCN_ERR_KEY_BITS = 4,     /* spatial size x batch does not fit a 63-bit site key          */
  SCN_ERR_NO_GRID = 5,      /* no active-site grid exists for that spatial size             */
  SCN_ERR_TABLE_FULL = 6,   /* a bounded hash probe gave up                                 */
  SCN_ERR_UNSUPPORTED = 7,  /* shape outside what the kernels implement                     */
  SCN_ERR_SIZE_MISMATCH = 8 /* row / plane counts disagree with the metadata               */
};

/* arithmetic used inside the convolution kernels */
enum scn_precision {
  SCN_PRECISION_FP32 = 0, /* fp32 FMA, fp32 accumulate (matches the reference's float path)  */
  SCN_PRECISION_TF32 = 1, /* one tf32 product, fp32 accumulate: warp-level mma.sync for 32 / 64 output
                             planes, tcgen05 kind::tf32 with the accumulator in TMEM above          */
  SCN_PRECISION_BF16 = 2, /* one bf16 product, fp32 accumulate: mma.sync for 32 / 64 output planes,
                             tcgen05 kind::f16 with the accumulator in TMEM above                   */
  SCN_PRECISION_TF32X3 = 3 /* fp32-class accuracy on the tensor paths (1e-4 of the reference's fp32
                             results): every operand is split in two bf16 parts, x = h + m, and the
                             three products h h, m h, h m are accumulated in fp32 -- warp-level
                             mma.sync.m16n8k16 for 32 / 64 output planes, tcgen05 kind::f16 in TMEM
                             for wider layers.  (The name is kept from the first form, three tf32
                             products of a tf32 hi / lo split, which SCN_X3_FORM=tf32 still selects.) */
};
/* which convolution kernel the last convolution call of this thread ran (for profiling) */
enum scn_conv_kernel {
  SCN_KERNEL_CONV_SIMT = 0,          /* k_conv_pipe / k_conv_simt / k_conv_thin: fp32 FMA     */
  SCN_KERNEL_CONV_TC = 1,            /* k_conv_tc: tcgen05, one tile per CTA                  */
  SCN_KERNEL_CONV_TC_PERSISTENT = 2, /* k_conv_tma: tcgen05, persistent, double-buffered TMEM */
  SCN_KERNEL_CONV_PIPE_MMA = 3,      /* k_conv_pipe with three tf32 mma.sync passes           */
  SCN_KERNEL_CONV_ROWS = 4,          /* k_conv_rows: row-stationary, warp-level mma.sync      */
  SCN_KERNEL_CONV_WIDE = 5           /* k_conv_wide: tcgen05, persistent, rows split to bf16 parts once per call and copied in by cp.async */
};
/* The tensor-core modes need groups == 1, n_in_planes % 32 == 0, n_out_planes % 16 == 0 and
 * n_out_planes <= 256; other shapes run the fp32 kernel whatever the precision says. */

/* which rulebook of a metadata object an export call refers to */
enum scn_rulebook_kind {
  SCN_RULES_SUBMANIFOLD = 0, /* key (spatial_size, filter_size)          */
  SCN_RULES_STRIDED = 1      /* key (input_size, filter_size, stride)    */
};

SCN_API int scn_abi_version(void);
SCN_API const char *scn_status_string(int status);
SCN_API const char *scn_last_error(void);
/* number of CUDA kernels this library has launched in this process so far (no counterpart in
 * the reference; used to report how many kernels a timed region ran) */
SCN_API long long scn_launch_count(void);
/* number of times this library has made the calling thread wait for the GPU so far (stream or event
 * synchronisations: site counts of the input layer and of strided rulebooks, rule counts asked for
 * before they landed, scn_md_poll_errors).  No counterpart in the reference. */
SCN_API long long scn_host_wait_count(void);
/* number of rulebooks this process has CONSTRUCTED so far (a lookup served from a metadata
 * object's cache does not count).  No counterpart in the reference; lets a profiler credit the
 * bytes of a rulebook build only to the call that built it. */
SCN_API long long scn_rulebook_build_count(void);
/* gives idle blocks of the current device's scratch pool back to the driver, keeping at most
 * `keep_bytes` reserved (0 = everything idle).  No counterpart in the reference. */
SCN_API int scn_trim_memory(uint64_t keep_bytes);
/* bytes the current device's scratch pool holds from the driver, and bytes of them handed out to
 * live allocations (tables, rulebooks, scratch of calls still in flight).  No counterpart in the
 * reference. */
SCN_API int scn_memory_usage(uint64_t *reserved_bytes, uint64_t *used_bytes);

/* ---- Metadata object ------------------------------------------------------------------ */

/* replaces `Metadata_<D>()` (pybind.cpp:12-14, 204-209).  dimension in 1..SCN_MAX_DIMENSION. */
SCN_API int scn_md_create(int dimension, scn_metadata **md);
/* Frees the object's device memory stream-ordered BEHIND THE LAST WORK enqueued with the object
 * (the stream of the most recent call that took it), on the device that owns it whatever device
 * is current: kernels still reading the tables finish first.  If other streams still read the
 * tables (the caller made them wait on that work), use scn_md_destroy_on_stream with a stream
 * that is ordered after all of them. */
SCN_API int scn_md_destroy(scn_metadata *md);
SCN_API int scn_md_destroy_on_stream(scn_metadata *md, void *stream);
/* replaces Metadata<D>::clear (Metadata.cpp:52-66) */
SCN_API int scn_md_clear(scn_metadata *md, void *stream);

/* replaces Metadata<D>::inputLayer + inputLayerRules
 * (Metadata.cpp:413-425, Metadata/IOLayersRules.h:18-121).
 * coords: int64 [n_rows, n_cols], n_cols == dimension (one sample) or dimension+1 (last
 * column = batch index); `coords_on_device` says where the pointer lives (host arrays are
 * copied with one cudaMemcpyAsync).  mode 0..4 as in the reference (0 unique, 1 first,
 * 2 last, 3 sum, 4 mean).  Builds the site hash of `spatial_size` on the GPU, numbers the
 * output rows in order of first occurrence in the input, and returns the active-site count.
 * Coordinates must lie in [0, spatial_size): the reference does not check this, this
 * library reports SCN_ERR_COORD_RANGE. */
SCN_API int scn_md_input_layer(scn_metadata *md, const int64_t *spatial_size, const int64_t *coords,
                       int coords_on_device, int64_t n_rows, int n_cols, int64_t batch_size,
                       int mode, void *stream, int64_t *n_active);

/* replaces Metadata<D>::blLayer + blRules (Metadata.cpp:427-436, Metadata/IOLayersRules.h:134-288),
 * the metadata half of BLInputLayer (CPU/IOLayers.cpp:139-163).
 * coords: int64 [batch_size, length, dimension]; the sample index is the first array index, a point
 * whose first coordinate is negative is an empty slot.  mode as in the reference's BL layers: 0 all
 * present and unique (rows = the batch_size*length points), 1 LAST point of a site, 2 FIRST point,
 * 3 sum, 4 mean.  Sites are numbered sample by sample in order of first occurrence.  The features
 * then go through scn_input_layer_forward (in [batch_size*length, n_planes]) and back through
 * scn_output_layer_forward. */
SCN_API int scn_md_bl_input_layer(scn_metadata *md, const int64_t *spatial_size, const int64_t *coords,
                          int coords_on_device, int64_t batch_size, int64_t length, int mode, void *stream,
                          int64_t *n_active);

/* replaces cpu/cuda_InputLayer_updateOutput's feature pass
 * (CPU/IOLayers.cpp:11-29,49-72; CUDA/IOLayers.cu:14-41) using the rules stored by the last
 * scn_md_input_layer call.  in [n_in, n_planes] -> out [n_active, n_planes]. */
SCN_API int scn_input_layer_forward(scn_metadata *md, const float *in_features, int64_t n_in,
                            float *out_features, int64_t n_out, int n_planes, void *stream);

/* Kernels never trap: they raise a flag in device memory (a rulebook entry outside the feature
 * matrix, an expired bounded wait ...).  This waits for `stream`, reads and clears the flags
 * and returns the matching status.  No counterpart in the reference (which checks nothing). */
SCN_API int scn_md_poll_errors(scn_metadata *md, void *stream);

/* replaces cpu/cuda_OutputLayer_updateOutput and cpu/cuda_BLOutputLayer_updateOutput
 * (CPU/IOLayers.cpp:95-114,197-215; CUDA/IOLayers.cu): in [n_active, n_planes] -> out [n_points,
 * n_planes], n_points = rows read by the last (BL)InputLayer call (batch_size*length for BL).  Each
 * site's row is copied to the points its rule names (mode 0: all rows; first / last point of the
 * site as the input mode kept it; all points for sum / mean -- unscaled, as the reference); every
 * other point gets zeros. */
SCN_API int scn_output_layer_forward(scn_metadata *md, const float *in_features, int64_t n_in,
                             float *out_features, int64_t n_out, int n_planes, void *stream);

/* replaces Metadata<D>::getNActive / getBatchSize (Metadata.cpp:67-70,171-176) */
SCN_API int scn_md_n_active(scn_metadata *md, const int64_t *spatial_size, int64_t *n_active);
SCN_API int scn_md_batch_size(scn_metadata *md, const int64_t *spatial_size, int64_t *batch_size);

/* replaces Metadata<D>::getSpatialLocations (Metadata.cpp:149-170):
 * out_dev int64 [n_active, dimension+1] on the device, row r = coordinates then batch index. */
SCN_API int scn_md_spatial_locations(scn_metadata *md, const int64_t *spatial_size, int64_t *out_dev,
                             void *stream);

/* replaces Metadata<D>::getSubmanifoldRuleBook (Metadata.cpp:437-451,
 * Metadata/SubmanifoldConvolutionRules.h:26-87).  Builds (or finds in the cache) the
 * rulebook on the GPU.  n_rules (may be NULL) receives the total rule count over all filter
 * offsets; asking for it waits for the build. */
SCN_API int scn_md_submanifold_rulebook(scn_metadata *md, const int64_t *spatial_size,
                                const int64_t *filter_size, void *stream, int64_t *n_rules);

/* replaces Metadata<D>::getRuleBook (Metadata.cpp:492-518, Metadata/ConvolutionRules.h:11-105).
 * Creates the output grid (site hash and row numbering of `output_size`) if this is the
 * first use, builds the rulebook, and returns the output active-site count, which the
 * caller needs to size the output of Convolution / MaxPooling. */
SCN_API int scn_md_strided_rulebook(scn_metadata *md, const int64_t *input_size,
                            const int64_t *output_size, const int64_t *filter_size,
                            const int64_t *filter_stride, void *stream, int64_t *n_active_out,
                            int64_t *n_rules);

/* Builds, in one enqueued chain, the grids and rulebooks of up to `levels` consecutive levels of the same
 * downsampling (the same filter_size and filter_stride, each level's output size (in - f) / s + 1 being the
 * next level's input size) below the grid of `input_size`: what an encoder's Convolutions
 * would otherwise request one at a time through scn_md_strided_rulebook (Metadata<D>::getRuleBook,
 * Metadata.cpp:492-518), each request ending in a wait for that level's site count.  The chain waits for
 * `stream` once, for all counts together; the per-level calls that follow find their rulebooks built.
 * Grids, row numbering and rulebooks are the ones the per-level calls would have made.  Where the chain
 * does not apply (fewer than two levels left to build, sizes that do not divide, no grid of `input_size`) nothing
 * is built and the result is SCN_OK.  n_built (may be NULL) receives the number of levels built.  The
 * reference has no such call; it is a hint for callers that know the shape of their network. */
SCN_API int scn_md_strided_chain(scn_metadata *md, const int64_t *input_size, const int64_t *filter_size,
                                 const int64_t *filter_stride, int levels, void *stream, int *n_built);

/* scn_md_strided_chain without the wait: the chain's kernels go to a side stream of the device, ordered behind
 * what `stream` holds at the time of the call (the grid of `input_size` must exist), and run beside whatever the
 * caller enqueues on `stream` afterwards -- for a U-Net, the convolutions of its finest level.  The call returns
 * at once.  The first call that needs one of those levels (scn_md_strided_rulebook, scn_md_strided_chain, a
 * convolution or a query on a level's grid) waits for the chain's event, which has usually long passed, and takes
 * the levels over; until then they do not exist for scn_md_n_active and friends in any other sense.  Nothing is
 * started when a chain is under way already or does not apply.  scn_md_clear / scn_md_input_layer /
 * scn_md_destroy drop a started chain.  The reference has no such call. */
SCN_API int scn_md_strided_chain_start(scn_metadata *md, const int64_t *input_size, const int64_t *filter_size,
                                       const int64_t *filter_stride, int levels, void *stream);

/* Rulebook read-back in the reference's format (RuleBook = one flat list of
 * (input_row, output_row) int32 pairs per filter offset, Metadata.h:35).  The reference does
 * not bind this; it exists so parity tests can compare rulebooks bit for bit.
 * sizes_a / sizes_b / sizes_c: SUBMANIFOLD: (spatial_size, filter_size, NULL);
 * STRIDED: (input_size, filter_size, filter_stride).  The rulebook must have been built.
 * counts_host: int64 [n_offsets] rule count per offset.  pairs_dev (may be NULL): int32
 * [2 * sum(counts)], offsets concatenated in order, rules of one offset ordered by output
 * row. */
SCN_API int scn_md_rulebook_export(scn_metadata *md, int kind, const int64_t *sizes_a,
                           const int64_t *sizes_b, const int64_t *sizes_c, int64_t *n_offsets,
                           int64_t *counts_host, int32_t *pairs_dev, void *stream);

/* ---- Feature operators ----------------------------------------------------------------- */

/* -1 before the first convolution, else an scn_conv_kernel value.  No counterpart in the
 * reference; lets a profiler attribute a call's time to the kernel that ran it. */
SCN_API int scn_last_conv_kernel(void);

/* Self-calibration of the tensor path.  No counterpart in the reference.  Issues `n_mma`
 * tcgen05.mma instructions of shape M x N (x 8 tf32 / 16 bf16 along K) back to back from one
 * thread of each of `n_ctas` CTAs onto disjoint accumulator ranges of TMEM, one commit at the end,
 * and reports SM cycles per instruction (until the last one was issued / until all completed,
 * clock64, averaged over the CTAs) and the CUDA-event duration of the whole launch.
 * a_in_tmem != 0 reads the A operand from TMEM instead of shared memory (M = 128 only).
 * Allocates a few KB for the duration of the call and waits for the stream. */
SCN_API int scn_tc_probe_mma(int m, int n, int kind_bf16, int a_in_tmem, int n_mma, int n_ctas,
                             void *stream, double *cycles_issue, double *cycles_total,
                             double *event_ms);

/* Prepared weight images.  The tensor-path kernels read the weights in operand layouts of their own,
 * made by a small kernel before the convolution (per call: scratch).  A caller whose weights do not
 * change between calls sets a non-zero token for the calling thread before a convolution call: the
 * images made during calls under that token are kept (per device, layout and shape) and found again
 * by later calls under the same token, which then skip the preparation.  The caller chooses tokens so
 * that one token never stands for two different weight contents (e.g. a counter bumped whenever a
 * weight tensor is written), sets 0 again for calls that must not use the cache, and releases a token
 * when its weights change or die (stream-ordered free on `stream`).  An image is built on the stream
 * of the call that first needed it; calls on other streams must be ordered after that one.
 * No counterpart in the reference. */
SCN_API int scn_set_weight_token(uint64_t token);
SCN_API int scn_release_weight_token(uint64_t token, void *stream);

/* The convolution operators return the reference's multiply-add count (rules x planes in x planes
 * out, CPU/Convolution.cpp:141) through `macs`.  The reference knows the rule totals on the host;
 * here they are counted on the device, and fetching them where the operator is called makes the
 * host wait for the stream once per rulebook, with the GPU idle until the next launch.
 * scn_set_deferred_counts(1) lifts that wait for callers that can take the number later: while a
 * rulebook's totals are still on their way the operator stores -(planes in x planes out x groups)
 * in *macs, and scn_md_take_count_ticket hands out a ticket (or NULL) for the total of the last
 * such answer on that metadata object.  scn_count_ticket_total waits for that one copy only (not
 * for the stream) and returns the number of rules; the ticket stays valid after the metadata
 * object is gone and is given back with scn_count_ticket_release.  Off by default: *macs is then
 * always the count.  The switch is process-wide: every client of the library in the process sees the
 * deferred answers once one of them turns it on (the Python mirror does at import).  No counterpart
 * in the reference. */
SCN_API int scn_set_deferred_counts(int on);

/* Arithmetic (an scn_precision value) of the input-gradient pass of the three convolution backward
 * entry points, which runs the forward kernels on the opposite rulebook table with transposed
 * weights.  Default SCN_PRECISION_FP32; SCN_PRECISION_TF32X3 keeps fp32-class gradients on the tensor
 * paths.  The weight and bias gradients are always reduced in fp32, in a fixed order.  No
 * counterpart in the reference. */
SCN_API int scn_set_backward_precision(int precision);
SCN_API int scn_md_take_count_ticket(scn_metadata *md, void **ticket);
SCN_API int scn_count_ticket_total(void *ticket, int64_t *total);
SCN_API int scn_count_ticket_release(void *ticket);

/* replaces SubmanifoldConvolution_updateOutput (sparseconvnet.h:101-104;
 * CPU/Convolution.cpp:117-150; CUDA/Convolution.cu:57-233,444-521,618-642).
 * weight [filter_volume, groups, n_in/groups, n_out/groups], bias [n_out] or NULL.
 * in [n_active, n_in] -> out [n_active, n_out].  macs (may be NULL) receives the
 * reference's return value (rules x n_in/groups x n_out/groups x groups). */
SCN_API int scn_submanifold_convolution_forward(scn_metadata *md, const int64_t *spatial_size,
                                        const int64_t *filter_size, const float *in_features,
                                        float *out_features, const float *weight,
                                        const float *bias, int n_in_planes, int n_out_planes,
                                        int groups, int precision, void *stream, double *macs);

/* Test hook for the failure path of the tensor-core kernels.  Every wait inside them (on an
 * mbarrier another role arrives on) is bounded: when it runs out the kernel raises a status bit,
 * all its roles leave their loops, tensor memory is freed and the kernel returns; the host reads the
 * status through scn_md_poll_errors as SCN_ERR_CUDA with a message naming the wait.  After this call
 * the NEXT per-tile tensor-core convolution of the calling thread (k_conv_tc: a level with at most
 * 148 tiles of 256 rows, precision tf32 / bf16 / tf32x3) leaves out one barrier arrival in one of
 * its CTAs -- a flag that nothing sets -- so that exactly this path runs: the call itself returns
 * SCN_OK (the kernel is asynchronous), its output is incomplete, scn_md_poll_errors reports the
 * expired wait, and the next convolution works again.  Nothing traps, faults or waits without a
 * bound.  No counterpart in the reference. */
SCN_API int scn_test_drop_barrier_arrival(void);

/* Allocation-free SubmanifoldConvolution.  No counterpart in the reference.
 *
 * scn_submanifold_convolution_forward takes a temporary buffer for the prepared weight image
 * from the CUDA allocator on every call.  A caller that must not allocate where it runs the
 * layer -- a fixed launch sequence that is replayed, a latency-critical loop that may not enter
 * the driver's allocator, a process with a pre-assigned memory budget -- uses this entry point
 * instead: the same tensor-core kernels with the image kept in an 8 MiB array that is part of
 * the library (every GPU that loads the library holds those 8 MiB until the process exits).
 * It makes no device allocation: no cudaMalloc / cudaFree, no memory-pool call, no allocating
 * library routine on the device side (the host side uses a few hundred bytes of ordinary heap
 * for the rulebook lookup key).
 *
 *  - precision must be SCN_PRECISION_TF32, _BF16 or _TF32X3, groups == 1, and the shape one the
 *    tensor-core path takes (see scn_precision); anything else is SCN_ERR_UNSUPPORTED.
 *  - limit: filter_volume * n_in_planes * n_out_planes * (4 for tf32, 2 for bf16, 4 for tf32x3 in
 *    its default form of two bf16 parts, 8 in the form of two tf32 parts that SCN_X3_FORM=tf32
 *    selects) bytes <= 8 MiB, otherwise SCN_ERR_UNSUPPORTED with the sizes in scn_last_error().
 *  - the rulebook of (spatial_size, filter_size) must already exist
 *    (scn_md_submanifold_rulebook, which does allocate); otherwise SCN_ERR_NO_GRID.
 *  - the first call on each device looks up the array's device address; make that call with
 *    the device current and before starting any stream capture.
 *  - all calls share the one array and it keeps the last call's image: nothing in it needs
 *    clearing (each call rewrites what it reads), but two calls that overlap on the GPU (other
 *    streams, other threads) race on it -- serialise them.
 *  in [n_active, n_in_planes] -> out [n_active, n_out_planes]; bias [n_out_planes] or NULL. */
SCN_API int scn_submanifold_convolution_forward_static(scn_metadata *md, const int64_t *spatial_size,
                                                       const int64_t *filter_size,
                                                       const float *in_features, float *out_features,
                                                       const float *weight, const float *bias,
                                                       int n_in_planes, int n_out_planes,
                                                       int precision, void *stream);

/* The three convolutions with the eval-mode BatchNormalization (+ leaky ReLU) that FOLLOWS them
 * applied in the kernel's store: out = act((conv + bias) * bn_scale + bn_shift), act(y) = y > 0 ? y :
 * y * leakiness -- BatchNormalization_updateOutput's eval branch (sparseconvnet.h:22-26;
 * CPU/BatchNormalization.cpp:41-61) without a second pass over the activation.  bn_scale / bn_shift
 * [n_out_planes] come from scn_batchnorm_fold (scale = gamma / sqrt(running_var + eps), shift = beta -
 * running_mean * scale, rounded like the stand-alone operator, so the fused result has the same bits
 * as the two calls).  Kernels without a fused store apply the same arithmetic in place afterwards.
 * The reference has no fused form; its Python runs the two operators one after the other. */
SCN_API int scn_batchnorm_fold(const float *running_mean, const float *running_var, const float *weight,
                               const float *bias, double eps, int n_planes, float *scale, float *shift,
                               void *stream);
/* Eval-mode BatchNormalization (+ leaky ReLU) of the column-wise concatenation [in_a | in_b] of two dense
 * matrices with n_rows rows -- a JoinTable (sparseconvnet/tables.py:37-49) followed by
 * BatchNormalization_updateOutput's eval branch -- in one pass, without the joined matrix being written
 * first.  Statistics and affine terms have planes_a + planes_b entries.  Plane counts must be multiples
 * of four. */
SCN_API int scn_batchnorm_join_forward(const float *in_a, int planes_a, const float *in_b, int planes_b,
                                       float *out_features, int64_t n_rows, const float *running_mean,
                                       const float *running_var, const float *weight, const float *bias,
                                       double eps, double leakiness, void *stream);
/* out_features[r, :] = bias + in_features[r, :] * weight for a small weight matrix [n_in_planes]
 * [n_out_planes] (row-major, n_out_planes <= 32, n_in_planes a multiple of four up to 256): the shape of
 * NetworkInNetwork_updateOutput (sparseconvnet/SCN/sparseconvnet.h:51-53, CPU/NetworkInNetwork.cpp:7-23)
 * with few output planes and of the per-voxel class head that follows a segmentation network.  bias may
 * be null.  One read of the rows, one write of the result; wider products return SCN_ERR_UNSUPPORTED and
 * belong to the dense matrix library, as in the reference. */
SCN_API int scn_rows_affine_forward(const float *in_features, float *out_features, int64_t n_rows,
                                    int n_in_planes, int n_out_planes, const float *weight, const float *bias,
                                    void *stream);
SCN_API int scn_submanifold_convolution_bn_forward(scn_metadata *md, const int64_t *spatial_size,
                                                   const int64_t *filter_size, const float *in_features,
                                                   float *out_features, const float *weight, const float *bias,
                                                   const float *bn_scale, const float *bn_shift, double leakiness,
                                                   int n_in_planes, int n_out_planes, int groups, int precision,
                                                   void *stream, double *macs);
SCN_API int scn_convolution_bn_forward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                                       const int64_t *filter_size, const int64_t *filter_stride,
                                       const float *in_features, float *out_features, const float *weight,
                                       const float *bias, const float *bn_scale, const float *bn_shift,
                                       double leakiness, int n_in_planes, int n_out_planes, int groups,
                                       int precision, void *stream, double *macs);
/* SubmanifoldConvolution of the column-wise concatenation [in_a (planes_a) | in_b (planes_b)] of two matrices over
 * the same sites -- a JoinTable (sparseconvnet/tables.py:37-49) in front of the layer, as after the skip connection
 * of a U-Net -- optionally through an eval-mode BatchNormalization (+ leaky ReLU) between the two (pre_scale /
 * pre_shift [planes_a + planes_b] from scn_batchnorm_fold, may be NULL) and with the one behind the layer in its
 * store (bn_scale / bn_shift, may be NULL).  groups = 1; planes_a a multiple of eight, planes_b of four.  The
 * tcgen05 kernels read the two matrices where they lie, in the pass that splits their input rows; for the other
 * kernels the library writes the (normalised) concatenation to a scratch matrix first.  Same bits as JoinTable,
 * BatchNormalization, SubmanifoldConvolution, BatchNormalization one after the other.  Not in the reference. */
SCN_API int scn_submanifold_convolution_joined_forward(scn_metadata *md, const int64_t *spatial_size,
                                                       const int64_t *filter_size, const float *in_a, int planes_a,
                                                       const float *in_b, int planes_b, float *out_features,
                                                       const float *weight, const float *bias, const float *pre_scale,
                                                       const float *pre_shift, double pre_leakiness,
                                                       const float *bn_scale, const float *bn_shift, double leakiness,
                                                       int n_out_planes, int precision, void *stream, double *macs);
/* scn_convolution_bn_forward with a second eval-mode BatchNormalization (+ leaky ReLU), in FRONT of the
 * convolution: the layer sees act(in * pre_scale[plane] + pre_shift[plane]) (scale / shift [n_in_planes] from
 * scn_batchnorm_fold, same roundings as the stand-alone operator, so the result has the bits of the separate calls).
 * bn_scale / bn_shift (the BatchNorm behind) may be NULL.  The tcgen05 kernels apply the one in front in the pass
 * that splits their input rows; for the other kernels the library normalises into a scratch copy first.  The
 * reference has no fused form: a BatchNormalization module followed by a Convolution module
 * (sparseconvnet/networkArchitectures.py:231-238, the way down of a U-Net). */
SCN_API int scn_convolution_bn_bn_forward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                                          const int64_t *filter_size, const int64_t *filter_stride,
                                          const float *in_features, float *out_features, const float *weight,
                                          const float *bias, const float *pre_scale, const float *pre_shift,
                                          double pre_leakiness, const float *bn_scale, const float *bn_shift,
                                          double leakiness, int n_in_planes, int n_out_planes, int groups,
                                          int precision, void *stream, double *macs);
SCN_API int scn_deconvolution_bn_forward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                                         const int64_t *filter_size, const int64_t *filter_stride,
                                         const float *in_features, float *out_features, const float *weight,
                                         const float *bias, const float *bn_scale, const float *bn_shift,
                                         double leakiness, int n_in_planes, int n_out_planes, int groups,
                                         int precision, void *stream, double *macs);

/* replaces Convolution_updateOutput (sparseconvnet.h:87-92; CPU/Convolution.cpp:45-79).
 * out must have the n_active_out rows reported by scn_md_strided_rulebook. */
SCN_API int scn_convolution_forward(scn_metadata *md, const int64_t *input_size,
                            const int64_t *output_size, const int64_t *filter_size,
                            const int64_t *filter_stride, const float *in_features,
                            float *out_features, const float *weight, const float *bias,
                            int n_in_planes, int n_out_planes, int groups, int precision,
                            void *stream, double *macs);

/* replaces Deconvolution_updateOutput (sparseconvnet.h:149-154; CPU/Deconvolution.cpp:7-41):
 * uses the rulebook of the matching Convolution (output_size -> input_size) with the two
 * rule columns swapped.  in [n_active(input_size), n_in] -> out [n_active(output_size), n_out]. */
SCN_API int scn_deconvolution_forward(scn_metadata *md, const int64_t *input_size,
                              const int64_t *output_size, const int64_t *filter_size,
                              const int64_t *filter_stride, const float *in_features,
                              float *out_features, const float *weight, const float *bias,
                              int n_in_planes, int n_out_planes, int groups, int precision,
                              void *stream, double *macs);

/* ---- Backward passes (training) ---------------------------------------------------------------
 * fp32.  Every gradient buffer is overwritten (not accumulated into); d_bias and d_in_features may
 * be NULL when not wanted.  Sums are formed in a fixed order: results are bit-reproducible. */

/* replaces SubmanifoldConvolution_backward (sparseconvnet.h:106-114; CPU/Convolution.cpp:152-190;
 * CUDA/Convolution.cu dConvolution_KMxKN_backward_dW*).  in [n_active, n_in], d_out [n_active, n_out]
 * -> d_in [n_active, n_in], d_weight like weight, d_bias [n_out]. */
SCN_API int scn_submanifold_convolution_backward(scn_metadata *md, const int64_t *spatial_size,
                                         const int64_t *filter_size, const float *in_features,
                                         float *d_in_features, const float *d_out_features,
                                         const float *weight, float *d_weight, float *d_bias,
                                         int n_in_planes, int n_out_planes, int groups, void *stream);

/* replaces Convolution_backward (sparseconvnet.h:94-104; CPU/Convolution.cpp:80-115). */
SCN_API int scn_convolution_backward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                             const int64_t *filter_size, const int64_t *filter_stride,
                             const float *in_features, float *d_in_features, const float *d_out_features,
                             const float *weight, float *d_weight, float *d_bias, int n_in_planes,
                             int n_out_planes, int groups, void *stream);

/* replaces Deconvolution_backward (sparseconvnet.h:156-166; CPU/Deconvolution.cpp). */
SCN_API int scn_deconvolution_backward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                               const int64_t *filter_size, const int64_t *filter_stride,
                               const float *in_features, float *d_in_features, const float *d_out_features,
                               const float *weight, float *d_weight, float *d_bias, int n_in_planes,
                               int n_out_planes, int groups, void *stream);

/* replaces BatchNormalization_updateOutput (sparseconvnet.h:22-26;
 * CPU/BatchNormalization.cpp:12-62; CUDA/BatchNormalization.cu:14-122), which fuses the
 * leaky-ReLU: y = x*w + b, y *= (y > 0 ? 1 : leakiness).  weight / bias may be NULL.
 * train != 0 computes batch statistics and updates running_mean / running_var in place
 * (momentum = weight of the old value).  save_mean / save_invstd: [n_planes] outputs. */
SCN_API int scn_batchnorm_forward(const float *in_features, float *out_features, int64_t n_rows,
                          int n_planes, int64_t in_stride, int64_t out_stride, float *save_mean,
                          float *save_invstd, float *running_mean, float *running_var,
                          const float *weight, const float *bias, double eps, double momentum,
                          int train, double leakiness, void *stream);

/* replaces BatchNormalization_backward (sparseconvnet.h:28-38; CPU/BatchNormalization.cpp:64-107,
 * CUDA/BatchNormalization.cu).  in / d_in share in_stride, out / d_out share out_stride; save_mean and
 * save_invstd are what the forward call left there.  d_weight / d_bias [n_planes] may be NULL; weight
 * may be NULL (no affine).  d_out is not modified (the reference scales it in place). */
SCN_API int scn_batchnorm_backward(const float *in_features, float *d_in_features, const float *out_features,
                           const float *d_out_features, int64_t n_rows, int n_planes, int64_t in_stride,
                           int64_t out_stride, const float *save_mean, const float *save_invstd,
                           const float *weight, float *d_weight, float *d_bias, double leakiness,
                           void *stream);

/* Training-mode BatchNorm over rows that live on several GPUs (data-parallel training), in two phases per
 * direction with the caller's sum over the devices in between.  Not in the reference, which is single-device: its
 * BatchNormalization_updateOutput / _backward (CPU/BatchNormalization.cpp:12-62, 64-107) take the statistics over
 * the one matrix they are given; with one device (sums passed on unchanged, n_rows_total = n_rows) the two phases
 * give what scn_batchnorm_forward / scn_batchnorm_backward give.
 *
 * scn_batchnorm_moments: sums[0..C) = sum of x, sums[C..2C) = sum of x^2 over this device's rows (device doubles,
 * overwritten; n_rows may be 0).  The caller adds the arrays of all devices and the row counts.
 * scn_batchnorm_forward_moments: mean / biased variance from the summed array and n_rows_total, running statistics
 * updated as in training mode (every device computes the same values), this device's rows normalised.
 * n_rows_total = -1 (here and in scn_batchnorm_backward_sums_apply): the total row count is the device double
 * behind the array, sums[2C] / total_sums[2C], which the caller summed over the devices along with it; the host
 * then never waits for the count. */
SCN_API int scn_batchnorm_moments(const float *in_features, int64_t n_rows, int n_planes, int64_t in_stride,
                                  double *sums, void *stream);
SCN_API int scn_batchnorm_forward_moments(const float *in_features, float *out_features, int64_t n_rows,
                                          int64_t n_rows_total, int n_planes, int64_t in_stride,
                                          int64_t out_stride, const double *sums, float *save_mean,
                                          float *save_invstd, float *running_mean, float *running_var,
                                          const float *weight, const float *bias, double eps, double momentum,
                                          double leakiness, void *stream);
/* scn_batchnorm_backward_sums: sums[0..C) = sum of d, sums[C..2C) = sum of (x - mean) d over this device's rows,
 * d = d_out scaled by the leaky ReLU's slope (device doubles, overwritten).
 * scn_batchnorm_backward_sums_apply: d_in of this device's rows from the sums over all devices (total_sums,
 * n_rows_total); d_weight / d_bias (may be NULL) from this device's own sums (local_sums), so that adding the
 * parameter gradients of all devices, as for every other parameter, gives the gradient of the whole batch. */
SCN_API int scn_batchnorm_backward_sums(const float *in_features, const float *out_features,
                                        const float *d_out_features, int64_t n_rows, int n_planes,
                                        int64_t in_stride, int64_t out_stride, const float *save_mean,
                                        double leakiness, double *sums, void *stream);
SCN_API int scn_batchnorm_backward_sums_apply(const float *in_features, float *d_in_features,
                                              const float *out_features, const float *d_out_features,
                                              int64_t n_rows, int64_t n_rows_total, int n_planes,
                                              int64_t in_stride, int64_t out_stride, const float *save_mean,
                                              const float *save_invstd, const float *weight,
                                              const double *local_sums, const double *total_sums,
                                              float *d_weight, float *d_bias, double leakiness, void *stream);

/* replaces MaxPooling_updateOutput (sparseconvnet.h:198-201; CPU/MaxPooling.cpp:7-60):
 * out[o] = max(0, max over rules of in[i]) on planes n_features_to_drop .. n_planes_in-1.
 * out [n_active_out, n_planes_in - n_features_to_drop]. */
SCN_API int scn_max_pooling_forward(scn_metadata *md, const int64_t *input_size,
                            const int64_t *output_size, const int64_t *pool_size,
                            const int64_t *pool_stride, const float *in_features,
                            float *out_features, int n_planes_in, int n_features_to_drop,
                            void *stream);

/* replaces cpu/cuda_AveragePooling_updateOutput (CPU/AveragePooling.cpp:38-61, CUDA/AveragePooling.cu):
 * same arguments as scn_max_pooling_forward; out[o] = sum over the rules of o of in[i] / filter volume
 * (the divisor is the pool volume whatever the number of rules, as in the reference). */
SCN_API int scn_average_pooling_forward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                                const int64_t *pool_size, const int64_t *pool_stride,
                                const float *in_features, float *out_features, int n_planes_in,
                                int n_features_to_drop, void *stream);

/* replaces cpu/cuda_UnPooling_updateOutput (CPU/UnPooling.cpp:35-59, CUDA/UnPooling.cu).  input_size is
 * the coarse scale, output_size = (input_size - 1) * pool_stride + pool_size the fine one, whose grid must
 * already exist in the metadata (SCN_ERR_NO_GRID otherwise; the reference would produce zero rows).
 * in [n_active(input_size), n_planes_in] -> out [n_active(output_size), n_planes_in - n_features_to_drop]:
 * every fine site gets the sum of the coarse sites whose pooling window holds it. */
SCN_API int scn_unpooling_forward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                          const int64_t *pool_size, const int64_t *pool_stride, const float *in_features,
                          float *out_features, int n_planes_in, int n_features_to_drop, void *stream);

/* replaces SparseToDense_updateOutput (sparseconvnet.h:220-222; CPU/SparseToDense.cpp:7-64):
 * out [batch_size, n_planes, *spatial_size] float32, written completely (zeros where
 * inactive). */
SCN_API int scn_sparse_to_dense_forward(scn_metadata *md, const int64_t *spatial_size,
                                const float *in_features, float *out_dense, int n_planes,
                                void *stream);

/* replaces InputLayer_updateGradInput / BLInputLayer_updateGradInput (CPU/IOLayers.cpp:74-93,165-186):
 * d_out [n_active, n_planes] -> d_in [n_points, n_planes]; the points a rule names get the site's
 * gradient (1/count of it in mode 4), the others zero. */
SCN_API int scn_input_layer_backward(scn_metadata *md, float *d_in_features, int64_t n_points,
                             const float *d_out_features, int64_t n_sites, int n_planes, void *stream);

/* replaces OutputLayer_updateGradInput / BLOutputLayer_updateGradInput (CPU/IOLayers.cpp:116-136,217-237):
 * d_out [n_points, n_planes] -> d_in [n_active, n_planes], every site the unscaled sum over its points. */
SCN_API int scn_output_layer_backward(scn_metadata *md, float *d_in_features, int64_t n_sites,
                              const float *d_out_features, int64_t n_points, int n_planes, void *stream);

/* replaces MaxPooling_updateGradInput (sparseconvnet.h:203-212; CPU/MaxPooling.cpp:22-35,61-84): d_out flows
 * to every input that equals the pooled maximum.  d_in [n_active(input_size), n_planes_in] (the dropped
 * planes get zeros), out / d_out [n_active(output_size), n_planes_in - n_features_to_drop]. */
SCN_API int scn_max_pooling_backward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                             const int64_t *pool_size, const int64_t *pool_stride, const float *in_features,
                             float *d_in_features, const float *out_features, const float *d_out_features,
                             int n_planes_in, int n_features_to_drop, void *stream);

/* replaces AveragePooling_updateGradInput (sparseconvnet.h:81-92; CPU/AveragePooling.cpp:21-35,62-85). */
SCN_API int scn_average_pooling_backward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                                 const int64_t *pool_size, const int64_t *pool_stride, float *d_in_features,
                                 const float *d_out_features, int n_planes_in, int n_features_to_drop,
                                 void *stream);

/* replaces UnPooling_updateGradInput (sparseconvnet.h:235-242; CPU/UnPooling.cpp:20-32,60-80): input_size is
 * the coarse scale as in scn_unpooling_forward; d_in [n_active(input_size), n_planes_in]. */
SCN_API int scn_unpooling_backward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                           const int64_t *pool_size, const int64_t *pool_stride, float *d_in_features,
                           const float *d_out_features, int n_planes_in, int n_features_to_drop, void *stream);

/* replaces SparseToDense_updateGradInput (sparseconvnet.h:224-228; CPU/SparseToDense.cpp:20-33,66-85):
 * d_out_dense [batch, n_planes, *spatial_size] -> d_in [n_active, n_planes]. */
SCN_API int scn_sparse_to_dense_backward(scn_metadata *md, const int64_t *spatial_size, float *d_in_features,
                                 const float *d_out_dense, int n_planes, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SCN_B200_H */
