/*
 * nnf_b200 - C ABI of the B200 (sm_100a) kernels that replace nnForge's CUDA batch-norm /
 * activation / add / softmax / max-subsampling layer kernels.
 *
 * Conventions
 *  - Every pointer is a DEVICE pointer to planar fp32 data, offset = ((n*C + c)*H + y)*W + x
 *    (the layout nnforge/cuda/cudnn_util.cpp:27-55 describes to cuDNN), unless stated otherwise.
 *  - Every call only ENQUEUES work on `stream` (a cudaStream_t); nothing synchronises the device,
 *    allocates device memory or touches another device. This is the contract of
 *    layer_tester_cuda::enqueue_forward_propagation (nnforge/cuda/layer_tester_cuda.h:47-57) and of
 *    the layer_updater_cuda::enqueue_* members (nnforge/cuda/layer_updater_cuda.h:50-112).
 *  - Return value: NNF_OK (0) or a negative nnf_status; the text of the last failure of the calling
 *    thread is available from nnf_last_error_string(). Nothing throws. The C++ adapter classes turn
 *    a non-zero status into the neural_network_exception the reference's callers expect.
 *  - `hw` is H*W (1 for a fully-connected shaped tensor). Element counts may exceed 2^32; the
 *    library splits launches internally, the reference's 32-bit indexing limit does not apply.
 *  - Output buffers may alias the first input where the reference layer answers
 *    get_input_index_layer_can_write() == 0; this is stated per function.
 *  - Arithmetic is fp32 with separately rounded multiplies and adds (no FMA contraction), expf and
 *    division at full precision, so results follow nnForge's plain (CPU) backend: bit-exact for
 *    batch-norm-inference, ReLU, PReLU, add and max-subsampling (values and argmax), within
 *    1e-5 relative / 1e-6 absolute elsewhere.
 */
#ifndef NNF_B200_H
#define NNF_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define NNF_API __attribute__((visibility("default")))
#else
#define NNF_API
#endif

typedef void * nnf_stream_t; /* cudaStream_t */

typedef enum nnf_status
{
	NNF_OK = 0,
	NNF_ERR_INVALID_ARGUMENT = -1, /* null pointer, zero/negative extent, misaligned buffer, unknown enum */
	NNF_ERR_UNSUPPORTED = -2,      /* valid nnForge configuration this library does not implement */
	NNF_ERR_WORKSPACE = -3,        /* workspace missing or smaller than nnf_*_workspace_bytes() */
	NNF_ERR_CUDA = -4              /* a CUDA runtime call or launch failed; text has cudaGetErrorString */
} nnf_status;

/* Activation kinds, by nnForge layer type name. */
typedef enum nnf_act_kind
{
	NNF_ACT_NONE = 0,
	NNF_ACT_RELU = 1,    /* "ReLU"    nnforge/rectified_linear_layer.h: p0 = negative_slope */
	NNF_ACT_PRELU = 2,   /* "PReLU"   nnforge/parametric_rectified_linear_layer.h: slope = device float[C] */
	NNF_ACT_ELU = 3,     /* "ELU"     nnforge/exponential_linear_layer.h: alpha fixed at 1 */
	NNF_ACT_TANH = 4,    /* "TanH"    nnforge/hyperbolic_tangent_layer.h: p0 = scale, p1 = steepness */
	NNF_ACT_SIGMOID = 5  /* "Sigmoid" nnforge/sigmoid_layer.h */
} nnf_act_kind;

typedef struct nnf_act
{
	int32_t kind;        /* nnf_act_kind */
	float p0;
	float p1;
	const float * slope; /* PReLU only */
} nnf_act;

#define NNF_MAX_ACTS 2   /* a fused chain applies at most this many activations in sequence */
#define NNF_MAX_ADD_INPUTS 8

NNF_API const char * nnf_last_error_string(void);
NNF_API int nnf_version(void);

/* What the current device offers, by the field names of nnForge's cuda_running_configuration
 * (nnforge/cuda/cuda_running_configuration.h:126-153: device_id, compute_capability_major/minor,
 * multiprocessor_count, ...), filled from cudaDeviceGetAttribute once per device. The launch plans of
 * this library size their grids and shared-memory tiles from it; the host-side layer objects hand it to
 * their factory the way layer_testing_schema::create_tester receives the cuda_running_configuration
 * (nnforge/cuda/layer_testing_schema.cpp:25-51). */
typedef struct nnf_running_configuration
{
	int32_t device_id;
	int32_t compute_capability_major, compute_capability_minor;
	int32_t multiprocessor_count;
	int32_t max_threads_per_multiprocessor;
	int32_t max_shared_memory_per_block_optin;
	int32_t max_shared_memory_per_multiprocessor;
	int32_t l2_cache_size;
	int32_t max_registers_per_multiprocessor;
} nnf_running_configuration;
NNF_API int nnf_get_running_configuration(nnf_running_configuration * out);

/* Knobs of the launch plans (process-wide; nothing in the library reads the environment). No counterpart in
 * the reference. name: "elementwise_waves", "elementwise_group_waves", "pool_waves", "pool_group_floats",
 * "channel_waves", "group_waves", "chain_s_kb", "chain_a_kb", "chain_dist" (-1: built-in), "chain_chunk_mb",
 * "chain_lag" (lag + 1), "no_grouped", "apply_flat", "peer_wait_ns" (how long a batch-sharded launch waits for
 * another rank's statistics before it gives up; default 10 s), or "reset" (all back to the built-in choices).
 * A value <= 0 selects the built-in choice. Meant for tests that walk the geometries and for tuning. */
NNF_API int nnf_set_tuning(const char * name, long long value);

/* ---------------------------------------------------------------------------------------------
 * Inference batch norm (+ residual add) (+ activation chain), one HBM pass.
 *   t = x*mult + add,  mult = gamma*invsigma,  add = beta - mult*mean        (gamma != NULL)
 *   t = x                                                                     (gamma == NULL)
 *   t = ((0 + t) + residual) * add_alpha                                      (residual != NULL)
 *   y = act[n_acts-1](...act[0](t))
 * Replaces batch_norm_layer_tester_cuda::enqueue_forward_propagation
 * (nnforge/cuda/batch_norm_layer_tester_cuda.cu:62-90; weights = gamma, beta, mean, inverse sigma:
 * nnforge/batch_norm_layer.h:26) followed by add_layer_tester_cuda (nnforge/cuda/add_layer_tester_cuda.cu:47-83)
 * and the activation testers (nnforge/cuda/rectified_linear_layer_tester_cuda.cu:52-73,
 * parametric_rectified_linear_layer_tester_cuda.cu:50-74, exponential_linear_layer_tester_cuda.cu:50-70,
 * hyperbolic_tangent_layer_tester_cuda.cu:58-80, sigmoid via activation_layer_cudnn_tester_cuda.cpp:42-72).
 * Arithmetic follows nnforge/plain/batch_norm_layer_tester_plain.cpp:60-72 and
 * nnforge/plain/add_layer_tester_plain.cpp:53-61. y may alias x. */
NNF_API int nnf_bn_infer_act(nnf_stream_t stream, float * y, const float * x,
	const float * gamma, const float * beta, const float * mean, const float * invsigma,
	const float * residual, float add_alpha,
	const nnf_act * acts, int n_acts,
	int64_t n, int64_t c, int64_t hw);

/* The same with the bias of the convolution in front folded into the load: t = x + bias[channel] (its own rounded
 * step, as the reference adds the bias with cudnnAddTensor after the convolution,
 * nnforge/cuda/convolution_layer_tester_cuda.cpp:115), then everything nnf_bn_infer_act does. The convolution is then
 * run WITHOUT its bias and writes x; one pass over HBM is saved. bias may be NULL. */
NNF_API int nnf_bias_bn_infer_act(nnf_stream_t stream, float * y, const float * x, const float * bias,
	const float * gamma, const float * beta, const float * mean, const float * invsigma,
	const float * residual, float add_alpha, const nnf_act * acts, int n_acts,
	int64_t n, int64_t c, int64_t hw);

/* Stand-alone activation forward: y = act(x); the updater-side forward of the same layers
 * (nnforge/cuda/*_layer_updater_cuda.cu enqueue_forward_propagation). y may alias x. */
NNF_API int nnf_act_fwd(nnf_stream_t stream, float * y, const float * x, const nnf_act * act, int64_t n, int64_t c, int64_t hw);

/* Activation backward: dx (+)= dy * act'(.), replacing enqueue_backward_data_propagation of
 * rectified_linear (nnforge/cuda/rectified_linear_layer_updater_cuda.cu:135-167), parametric_rectified_linear
 * (parametric_rectified_linear_layer_updater_cuda.cu:158-199), exponential_linear (exponential_linear_layer_updater_cuda.cu:117-145),
 * hyperbolic_tangent (hyperbolic_tangent_layer_updater_cuda.cu:132-162) and the cuDNN sigmoid
 * (nnforge/cuda/activation_layer_cudnn_updater_cuda.cpp:77-117).
 * `neurons` is the layer INPUT for ReLU and PReLU and the layer OUTPUT for ELU, TanH and Sigmoid, the
 * dependency the plain backend declares (nnforge/plain/rectified_linear_layer_updater_plain.cpp:62-107,
 * exponential_linear_layer_updater_plain.cpp:59-103, ...). dx may alias dy. */
NNF_API int nnf_act_bwd(nnf_stream_t stream, float * dx, const float * dy, const float * neurons, const nnf_act * act,
	int64_t n, int64_t c, int64_t hw, int add_to_destination);

/* PReLU slope gradient: dslope[c] += sum_{n,hw} dy * (x >= 0 ? 0 : x), replacing
 * enqueue_backward_weights_propagation (nnforge/cuda/parametric_rectified_linear_layer_updater_cuda.cu:201-234;
 * plain: parametric_rectified_linear_layer_updater_plain.cpp:137-190). Deterministic (fixed reduction
 * tree, no atomics). workspace: nnf_prelu_bwd_weights_workspace_bytes(n, c, hw) bytes. */
NNF_API size_t nnf_prelu_bwd_weights_workspace_bytes(int64_t n, int64_t c, int64_t hw);
NNF_API int nnf_prelu_bwd_weights(nnf_stream_t stream, float * dslope, const float * dy, const float * x,
	int64_t n, int64_t c, int64_t hw, void * workspace, size_t workspace_bytes);

/* Add layer: y = ((0 + in[0]) + in[1] + ...) * alpha in one pass for any input count <= NNF_MAX_ADD_INPUTS
 * (the reference launches one kernel per extra input: nnforge/cuda/add_layer_tester_cuda.cu:59-82;
 * arithmetic: nnforge/plain/add_layer_tester_plain.cpp:53-61). `inputs` is a HOST array of device pointers.
 * y may alias inputs[0]. */
NNF_API int nnf_add_fwd(nnf_stream_t stream, float * y, const float * const * inputs, int input_count, float alpha, int64_t count);

/* Add layer backward: dx (+)= dy*alpha (nnforge/cuda/add_layer_updater_cuda.cu:88-116); a no-op when
 * dx == dy, alpha == 1 and not accumulating, as in the reference. */
NNF_API int nnf_add_bwd(nnf_stream_t stream, float * dx, const float * dy, float alpha, int64_t count, int add_to_destination);

/* ---------------------------------------------------------------------------------------------
 * Channel softmax over C at every (n, pixel), replacing the cuDNN calls of
 * softmax_layer_tester_cuda (nnforge/cuda/softmax_layer_tester_cuda.cpp:37-68) and softmax_layer_updater_cuda
 * (nnforge/cuda/softmax_layer_updater_cuda.cpp:38-71, 73-112); arithmetic of
 * nnforge/plain/softmax_layer_tester_plain.cpp:65-88 and softmax_layer_updater_plain.cpp:100-166.
 * y may alias x; dx may alias dy. */
NNF_API int nnf_softmax_fwd(nnf_stream_t stream, float * y, const float * x, int64_t n, int64_t c, int64_t hw);
NNF_API int nnf_softmax_bwd(nnf_stream_t stream, float * dx, const float * dy, const float * y, int64_t n, int64_t c, int64_t hw,
	int add_to_destination);

/* ---------------------------------------------------------------------------------------------
 * 2-D max subsampling (H = 1 gives 1-D). Extents and flags are in the reference's dimension order
 * (x = width first). Output extent per dimension: (in + stride - win + (round_up ? win-1 : 0)) / stride
 * (nnforge/max_subsampling_layer.cpp:125-133). */
typedef struct nnf_pool
{
	int32_t win_w, win_h;
	int32_t stride_w, stride_h;
	int32_t round_up_w, round_up_h; /* clip the last window to the input instead of dropping it */
	int32_t is_min;
} nnf_pool;

NNF_API int64_t nnf_pool_out_size(int64_t in_size, int32_t window, int32_t stride, int32_t round_up);

/* Forward, replacing max_subsampling_layer_tester_cuda / max_subsampling_layer_updater_cuda forward
 * (nnforge/cuda/max_subsampling_layer_tester_cuda.cuh:194-217, max_subsampling_layer_updater_cuda.cuh:539-818).
 * Tie-break and argmax format are the PLAIN backend's (nnforge/plain/max_subsampling_layer_updater_plain.cpp:139-159):
 * window scanned x-fastest, first strict maximum wins, argmax = absolute input element offset as
 * uint32 (so n*c*h*w must be < 2^32 when argmax is requested). argmax may be NULL. */
NNF_API int nnf_maxpool_fwd(nnf_stream_t stream, float * y, uint32_t * argmax, const float * x,
	int64_t n, int64_t c, int64_t h, int64_t w, const nnf_pool * pool);

/* Backward as a deterministic gather: every input element sums dy of the (few) windows whose stored
 * argmax points at it, in ascending output index, which equals the plain backend's scatter
 * (nnforge/plain/max_subsampling_layer_updater_plain.cpp:173-231) run serially with accumulation onto a
 * zeroed buffer. No zero-fill pass, no atomics (reference: nnforge/cuda/max_subsampling_layer_updater_cuda.cuh:820-977). */
NNF_API int nnf_maxpool_bwd(nnf_stream_t stream, float * dx, const float * dy, const uint32_t * argmax,
	int64_t n, int64_t c, int64_t h, int64_t w, const nnf_pool * pool, int add_to_destination);

/* ResNet block tail in one pass: z = relu(((0 + bn(x)) + residual) * 1, slope), pooled = maxpool(z).
 * z is written because later layers and the backward pass need it. gamma == NULL skips the batch norm. */
NNF_API int nnf_bn_add_relu_maxpool_fwd(nnf_stream_t stream, float * z, float * pooled, uint32_t * argmax,
	const float * x, const float * residual,
	const float * gamma, const float * beta, const float * mean, const float * invsigma,
	float relu_slope, int64_t n, int64_t c, int64_t h, int64_t w, const nnf_pool * pool);

/* Backward of the same chain with frozen batch-norm statistics:
 *   dz = maxpool_bwd(dpooled), ds = (z sign bit clear) ? dz : dz*slope, dresidual = ds,
 *   dx = ds * (gamma*invsigma).   Requires relu_slope >= 0 (the gate is read from the sign of z).
 * dresidual and/or dx may be NULL. */
NNF_API int nnf_bn_add_relu_maxpool_bwd(nnf_stream_t stream, float * dx, float * dresidual,
	const float * dpooled, const uint32_t * argmax, const float * z,
	const float * gamma, const float * invsigma,
	float relu_slope, int64_t n, int64_t c, int64_t h, int64_t w, const nnf_pool * pool);

/* ---------------------------------------------------------------------------------------------
 * Training-mode batch norm fused with the following activation chain, replacing the cuDNN calls
 * cudnnBatchNormalizationForwardTraining / cudnnBatchNormalizationBackward of batch_norm_layer_updater_cuda
 * (nnforge/cuda/batch_norm_layer_updater_cuda.cu:60-107, 109-183) plus the activation updaters that follow.
 * The work is split so that a batch-sharded multi-GPU caller can all-reduce 2*C floats between the steps:
 *
 *   forward : nnf_bn_train_stats      -> sums[2C] = {sum x, sum x^2} of THIS shard
 *             (all-reduce sums over shards; skip with one GPU)
 *             nnf_bn_train_apply_act  -> saved[2C] = {mean, invstd}, y = acts(x*mult + add)
 *   backward: nnf_bn_train_bwd_stats  -> bsums[3C] = {sum du, sum du*xhat, sum dv*(u>=0?0:u)} of this shard,
 *                                        and, when gsums != NULL, a copy of its first 2C floats in gsums[2C]
 *             (all-reduce gsums in place over shards; with one GPU pass bsums itself as gsums below)
 *             nnf_bn_train_bwd_apply  -> dx, and the per-channel gradients accumulated from bsums
 *
 * u = bn output, v = act[0](u), du/dv = gradient reaching u/v through the chain, xhat = (x-mean)*invstd.
 * count_total = number of elements per channel over ALL shards (N_global * hw).
 * saved has the layout of the reference's temporary_fixed_buffer (mean then inverse std-dev,
 * nnforge/cuda/batch_norm_layer_updater_cuda.cu:105-106, 209-212).
 * workspace: nnf_bn_train_workspace_bytes(n, c, hw) bytes, used by the two *_stats calls. */
NNF_API size_t nnf_bn_train_workspace_bytes(int64_t n, int64_t c, int64_t hw);

NNF_API int nnf_bn_train_stats(nnf_stream_t stream, float * sums, const float * x, int64_t n, int64_t c, int64_t hw,
	void * workspace, size_t workspace_bytes);

/* Same result as nnf_bn_train_stats, for callers that cannot supply a workspace. It has no counterpart
 * in the reference. An nnForge layer object may only use the buffers its scheduler planned from the
 * layer's size answers, and must not allocate while enqueueing (an allocation can fail once the
 * scheduler has filled the memory it measured as free, and it stalls every stream of the device); the
 * stock batch-norm updater plans no working buffer at all. This variant therefore keeps its per-CTA
 * partial sums in a 1.5 MiB array built into the library (held by every GPU that loads it until the
 * process ends) and calls no allocating routine.
 *  - Limit: c <= 1024 channels; more returns NNF_ERR_UNSUPPORTED with a message naming the limit.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *    that device current). Make that first call before starting any stream capture on the device.
 *  - All calls on a device share the array. Calls that overlap on the GPU (issued on different
 *    streams without ordering between them) race on it; calls on one stream are safe. Nothing in the
 *    array needs clearing between calls: each call writes every slot it later reads. */
NNF_API int nnf_bn_train_stats_static(nnf_stream_t stream, float * sums, const float * x, int64_t n, int64_t c, int64_t hw);

NNF_API int nnf_bn_train_apply_act(nnf_stream_t stream, float * y, float * saved, const float * x,
	const float * gamma, const float * beta, const float * sums, double count_total, float eps,
	const nnf_act * acts, int n_acts, int64_t n, int64_t c, int64_t hw);

/* Single-GPU forward in one call and, for 16-byte aligned tensors whose planes are whole float4s or fill
 * channel groups, one launch: statistics items and apply items share it and the second read of x comes
 * from L2 (8 bytes/element through HBM). Other shapes run nnf_bn_train_stats + nnf_bn_train_apply_act,
 * for which `sums` (2C floats) is required. The workspace (nnf_bn_train_workspace_bytes, 16-byte aligned)
 * is always required: NNF_ERR_WORKSPACE without it. saved receives {mean, invstd}; sums (may be NULL for
 * single-launch shapes) receives {sum x, sum x^2}. Replaces
 * batch_norm_layer_updater_cuda::enqueue_forward_propagation
 * (nnforge/cuda/batch_norm_layer_updater_cuda.cu:60-107) plus the activation layers behind it. */
NNF_API int nnf_bn_train_fwd(nnf_stream_t stream, float * y, float * saved, float * sums, const float * x,
	const float * gamma, const float * beta, float eps,
	const nnf_act * acts, int n_acts, int64_t n, int64_t c, int64_t hw,
	void * workspace, size_t workspace_bytes);

/* Single-GPU backward in one call: dx, bsums[3C] = {sum du, sum du*xhat, sum dslope} and the accumulated
 * per-channel gradients (see nnf_bn_train_bwd_apply). The shapes of nnf_bn_train_fwd's single launch take
 * one launch here too (x and dy read from HBM once, a second time from L2, dx written once: 12
 * bytes/element); other shapes, and add_to_destination, run nnf_bn_train_bwd_stats +
 * nnf_bn_train_bwd_apply. dx may be dy or x. Replaces enqueue_backward_data_and_weights_propagation
 * (nnforge/cuda/batch_norm_layer_updater_cuda.cu:109-183) plus the activation layers' backward actions. */
NNF_API int nnf_bn_train_bwd(nnf_stream_t stream, float * dx, float * bsums, const float * dy, const float * x,
	const float * gamma, const float * beta, const float * saved,
	const nnf_act * acts, int n_acts,
	float * grad_gamma, float * grad_beta, float * grad_mean, float * grad_invsigma, float * grad_slope,
	const float * mean, const float * invsigma, float entry_count,
	int64_t n, int64_t c, int64_t hw, int add_to_destination,
	void * workspace, size_t workspace_bytes);

/* What a single-launch training batch-norm call (nnf_bn_train_fwd / _bwd and their _sharded forms) reports:
 * every such launch starts by clearing this block at the head of its workspace and leaves in it
 *   status        0, or the code of a bounded wait that ran out: 2 = another rank's statistics did not
 *                 arrive within the limit ("peer_wait_ns"), 4 = this GPU's own items did not finish;
 *                 the launch then completed with what it had and its outputs are not to be used
 *   wait_ns_*     how long its waiting items waited, summed and the longest
 * nnf_bn_train_read_report enqueues the copy of the block into host memory (pinned, for an asynchronous
 * copy) on `stream`, after the launches already enqueued there; the caller looks at it once the stream
 * has passed that point - e.g. before the next step - and repeats the step another way (the split entry
 * points with an NCCL all-reduce) when status is not 0. A failed launch does not affect later ones. No
 * counterpart in the reference, whose layers cannot fail on the device. */
typedef struct nnf_launch_report
{
	uint64_t wait_ns_total;
	uint64_t wait_ns_max;
	uint32_t reserved;
	int32_t status;
} nnf_launch_report;
NNF_API int nnf_bn_train_read_report(nnf_stream_t stream, nnf_launch_report * host_report, const void * workspace);

/* Returns the library's process-wide error word (and clears it): the code of the last bounded wait that
 * ran out anywhere since the last check (2 = a peer exchange, 4 = a single-launch kernel's own items), 0
 * otherwise, -1 if the word cannot be read. Kernels only ever raise it. Synchronises the device: for
 * tests and diagnosis; nnf_bn_train_read_report is the per-launch, asynchronous way. */
NNF_API int nnf_fused_error_check(void);

/* Where the launches raise the process-wide error word. By default a device variable inside the library, which the host
 * can only read with a synchronising copy (nnf_fused_error_check). A host that wants to look at it after every step hands
 * over ONE 32-bit word of pinned host memory here (cudaHostAlloc / cudaHostRegister; under unified addressing the device
 * reaches it at the same address): a kernel whose bounded wait runs out then stores its code (2 or 4, as in
 * nnf_launch_report.status) straight into that word, and the host reads it as ordinary memory once the stream has passed
 * the launch - no copy, no event, nothing added to the stream. The host clears it (or calls nnf_fused_error_check) after it has
 * dealt with the failure, e.g. by reading the launch reports to find the launch. NULL restores the default. The word must
 * outlive every launch enqueued while it is set. No counterpart in the reference. */
NNF_API int nnf_set_error_sink(int32_t * host_visible_word);

NNF_API int nnf_bn_train_bwd_stats(nnf_stream_t stream, float * bsums, float * gsums, const float * dy, const float * x,
	const float * gamma, const float * beta, const float * saved,
	const nnf_act * acts, int n_acts, int64_t n, int64_t c, int64_t hw,
	void * workspace, size_t workspace_bytes);

/* dx (+)= gamma*invstd/m * (m*du - gsums[c] - xhat*gsums[C+c]).
 * Per-channel gradients (each may be NULL) are ACCUMULATED from the LOCAL sums, as the reference
 * accumulates (beta_weights = 1, nnforge/cuda/batch_norm_layer_updater_cuda.cu:138-139) and leaves the
 * cross-device sum to the weight all-reduce: grad_gamma += bsums[C+c], grad_beta += bsums[c],
 * grad_slope += bsums[2C+c], and the running-statistics pseudo-gradients
 * grad_mean += entry_count*(saved_mean - mean), grad_invsigma += entry_count*(saved_invstd - invsigma)
 * (nnforge/cuda/batch_norm_layer_updater_cuda.cu:28-44, 167-182). dx may alias dy. */
NNF_API int nnf_bn_train_bwd_apply(nnf_stream_t stream, float * dx, const float * dy, const float * x,
	const float * gamma, const float * beta, const float * saved,
	const float * gsums, const float * bsums, double count_total,
	const nnf_act * acts, int n_acts,
	float * grad_gamma, float * grad_beta, float * grad_mean, float * grad_invsigma, float * grad_slope,
	const float * mean, const float * invsigma, float entry_count,
	int64_t n, int64_t c, int64_t hw, int add_to_destination);

/* ---------------------------------------------------------------------------------------------
 * Sum of a small message (the 2*C floats of batch-norm statistics) over the GPUs of one machine through
 * peer memory, in place of the reference's per-part all-reduce (nnforge/cuda/nccl_cuda_communicator.cpp:72-94,
 * host_staged_cuda_communicator.cpp:39-152). Every rank owns one zero-initialised buffer of
 * nnf_peer_exchange_bytes(kmax) bytes that all ranks can address; peer_bufs[r] is rank r's buffer as seen
 * from this GPU. seq is the number of this exchange (1, 2, 3, ... identical on all ranks).
 * publish stores `local[k]` into every rank's buffer and raises this rank's flag there; gather_sum waits
 * (bounded; expiry raises the word read by nnf_fused_error_check, value 2) for all ranks' flags in its own
 * buffer and writes the sum in rank order to `out` (may alias local). exchange_sum = publish + gather_sum. */
NNF_API size_t nnf_peer_exchange_bytes(int kmax);
NNF_API int nnf_peer_publish(nnf_stream_t stream, const float * local, void * const * peer_bufs, int rank, int world, int k, int kmax, uint32_t seq);
NNF_API int nnf_peer_gather_sum(nnf_stream_t stream, float * out, const void * my_buf, int world, int k, int kmax, uint32_t seq);
NNF_API int nnf_peer_exchange_sum(nnf_stream_t stream, float * out, const float * local, void * const * peer_bufs, int rank, int world, int k, int kmax, uint32_t seq);

/* The same exchange folded into the batch-norm kernels, so that it costs no launch of its own: the
 * *_publish variants store this shard's sums into every rank's peer buffer from the kernel that finishes
 * the reduction (first 2*C floats, kmax >= 2*C); the *_peer variants take the sums of all ranks from the
 * rank's own peer buffer in their prologue (bounded wait) instead of from a sums / gsums array. Use the two
 * of a pass with the same seq. When H*W is not a multiple of 4 (or a buffer is not 16-byte aligned) the
 * forward _peer variant returns NNF_ERR_UNSUPPORTED: use nnf_peer_exchange_sum and the plain entry points. */
NNF_API int nnf_bn_train_stats_publish(nnf_stream_t stream, float * sums, const float * x, int64_t n, int64_t c, int64_t hw,
	void * workspace, size_t workspace_bytes, void * const * peer_bufs, int rank, int world, int kmax, uint32_t seq);
NNF_API int nnf_bn_train_apply_act_peer(nnf_stream_t stream, float * y, float * saved, const float * x,
	const float * gamma, const float * beta, const void * my_buf, int world, int kmax, uint32_t seq, double count_total, float eps,
	const nnf_act * acts, int n_acts, int64_t n, int64_t c, int64_t hw);
NNF_API int nnf_bn_train_bwd_stats_publish(nnf_stream_t stream, float * bsums, const float * dy, const float * x,
	const float * gamma, const float * beta, const float * saved,
	const nnf_act * acts, int n_acts, int64_t n, int64_t c, int64_t hw,
	void * workspace, size_t workspace_bytes, void * const * peer_bufs, int rank, int world, int kmax, uint32_t seq);
NNF_API int nnf_bn_train_bwd_apply_peer(nnf_stream_t stream, float * dx, const float * dy, const float * x,
	const float * gamma, const float * beta, const float * saved,
	const void * my_buf, int world, int kmax, uint32_t seq, const float * bsums, double count_total,
	const nnf_act * acts, int n_acts,
	float * grad_gamma, float * grad_beta, float * grad_mean, float * grad_invsigma, float * grad_slope,
	const float * mean, const float * invsigma, float entry_count,
	int64_t n, int64_t c, int64_t hw, int add_to_destination);

/* ---------------------------------------------------------------------------------------------
 * average_subsampling_layer over the two spatial dimensions (replaces average_subsampling_layer_tester_cuda /
 * _updater_cuda; semantics of nnforge/plain/average_subsampling_layer_tester_plain.cpp:120-135 and
 * average_subsampling_layer_updater_plain.cpp:270-285): windows win_w x win_h that do not overlap (stride = window; they
 * must divide the plane), global average pooling being win = (w, h).
 *   forward : y[n][c][h/win_h][w/win_w] = (sum of the window, x fastest then y, from +0) * mult
 *   backward: dx = dy[window of the element] * mult (accumulated with add_to_destination)
 * mult is the layer's effective alpha. NOTE: the plain backend's default is 1 / (feature-map x entry subsampling), i.e. 1
 * for spatial windows - it passes feature-map counts where get_effective_alpha expects layer configurations
 * (average_subsampling_layer_tester_plain.cpp:82) - so it sums; pass 1.0f / (win_w*win_h) for a true average.
 * The fused forms run batch norm (running statistics) -> residual add (alpha 1) -> ReLU -> average pooling in one pass and
 * its backward, like nnf_bn_add_relu_maxpool_fwd/bwd: z = relu(bn(x) + residual) is written for the backward pass;
 * dresidual = gate(z) * dpooled-window * mult, dx = dresidual * gamma * invsigma. gamma == NULL: no batch norm;
 * residual == NULL: no add; dx or dresidual may be NULL. */
NNF_API int nnf_avgpool_fwd(nnf_stream_t stream, float * y, const float * x, int64_t n, int64_t c, int64_t h, int64_t w,
	int win_w, int win_h, float mult);
NNF_API int nnf_avgpool_bwd(nnf_stream_t stream, float * dx, const float * dy, int64_t n, int64_t c, int64_t h, int64_t w,
	int win_w, int win_h, float mult, int add_to_destination);
NNF_API int nnf_bn_add_relu_avgpool_fwd(nnf_stream_t stream, float * z, float * pooled, const float * x, const float * residual,
	const float * gamma, const float * beta, const float * mean, const float * invsigma,
	float relu_slope, int64_t n, int64_t c, int64_t h, int64_t w, int win_w, int win_h, float mult);
NNF_API int nnf_bn_add_relu_avgpool_bwd(nnf_stream_t stream, float * dx, float * dresidual, const float * dpooled, const float * z,
	const float * gamma, const float * invsigma, float relu_slope,
	int64_t n, int64_t c, int64_t h, int64_t w, int win_w, int win_h, float mult);

/* ---------------------------------------------------------------------------------------------
 * The loss behind softmax: negative_log_likelihood_layer, stand-alone (replaces
 * negative_log_likelihood_layer_tester_cuda / _updater_cuda, nnforge/cuda/negative_log_likelihood_layer_*_cuda.cu;
 * semantics of nnforge/plain/negative_log_likelihood_layer_updater_plain.cpp:60-92, 131-157) and fused with the
 * softmax layer in front of it (softmax_layer_*_cuda + the loss in one pass over HBM).
 *   predicted / probs / logits / targets / dlogits / dpredicted: [n][c][hw];  err, mask: [n][hw] (mask may be NULL)
 *   forward : err = scale*mask * ( - sum over channels with target > 0 of target * logf(max(p, 1e-20)) )
 *   backward: dpredicted = (target > 0 ? target / max(p, 1e-20) : 0) * scale*mask   (the layer is a loss: no output errors)
 *   fused forward : probs = softmax(logits) over channels, err as above from probs
 *   fused backward: dlogits = probs * (g - sum_f g_f*probs_f), g = the gradient above (softmax_layer_updater_plain.cpp:100-166)
 * add_to_destination accumulates into dpredicted / dlogits. */
NNF_API int nnf_nll_fwd(nnf_stream_t stream, float * err, const float * predicted, const float * targets, const float * mask,
	float scale, int64_t n, int64_t c, int64_t hw);
NNF_API int nnf_nll_bwd(nnf_stream_t stream, float * dpredicted, const float * predicted, const float * targets, const float * mask,
	float scale, int64_t n, int64_t c, int64_t hw, int add_to_destination);
NNF_API int nnf_softmax_nll_fwd(nnf_stream_t stream, float * probs, float * err, const float * logits, const float * targets, const float * mask,
	float scale, int64_t n, int64_t c, int64_t hw);
NNF_API int nnf_softmax_nll_bwd(nnf_stream_t stream, float * dlogits, const float * probs, const float * targets, const float * mask,
	float scale, int64_t n, int64_t c, int64_t hw, int add_to_destination);

/* cross_entropy_layer, the loss behind sigmoid outputs (replaces cross_entropy_layer_tester_cuda / _updater_cuda,
 * nnforge/cuda/cross_entropy_layer_*_cuda.cu; semantics of nnforge/plain/cross_entropy_layer_updater_plain.cpp:60-101, 131-173):
 *   forward : err = scale*mask * sum over channels of ( t > 0 ? -t*logf(max(p, 1e-20)) : 0 ) + ( t < 1 ? -(1-t)*logf(max(1-p, 1e-20)) : 0 )
 *   backward: dpredicted = ( (t > 0 ? t/max(p, 1e-20) : 0) - (t < 1 ? (1-t)/max(1-p, 1e-20) : 0) ) * scale*mask
 * Layouts as for the negative log likelihood. Two remarks on the reference: its plain TESTER takes the mask INSTEAD of the scale
 * when a mask is given (cross_entropy_layer_tester_plain.cpp:72-74) - a tester adapter passes scale = 1 then; and its plain
 * updater computes this gradient into a variable that shadows the stored one and so writes zeros (:150-168) - the value here is
 * the one the expression in that file and the CUDA backend (cross_entropy_layer_updater_cuda.cu:115-183) define. */
NNF_API int nnf_cross_entropy_fwd(nnf_stream_t stream, float * err, const float * predicted, const float * targets, const float * mask,
	float scale, int64_t n, int64_t c, int64_t hw);
NNF_API int nnf_cross_entropy_bwd(nnf_stream_t stream, float * dpredicted, const float * predicted, const float * targets, const float * mask,
	float scale, int64_t n, int64_t c, int64_t hw, int add_to_destination);

/* accuracy_layer (replaces accuracy_layer_tester_cuda / _updater_cuda, nnforge/cuda/accuracy_layer_tester_cuda.cu; semantics of
 * nnforge/plain/accuracy_layer_tester_plain.cpp:64-110): per (entry, pixel) the actual class is the first channel with the
 * largest target; rank = number of channels whose prediction is larger than that class's, or equal with a smaller index.
 * out[n][top_n + 1][hw]: out[k] = (rank <= k ? mask : 0) for k < top_n, out[top_n] = mask (1 without a mask). */
NNF_API int nnf_accuracy_fwd(nnf_stream_t stream, float * out, const float * predicted, const float * targets, const float * mask,
	int top_n, int64_t n, int64_t c, int64_t hw);

/* Batch-sharded training batch norm in ONE launch per direction and GPU (the sharded form of
 * nnf_bn_train_fwd / nnf_bn_train_bwd): statistics and apply work items share the launch, the second read
 * of x (and dy) comes from L2, and the per-channel sums cross the GPUs inside the launch - the item that
 * finishes a channel's statistics stores this rank's two sums into every rank's mailbox, an apply item
 * waits (bounded by "peer_wait_ns"; expiry sets status 2 in the launch's report, see nnf_bn_train_read_report) until
 * its own mailbox holds the sums of all ranks for its channel and adds them in rank order. Replaces the
 * sequence statistics kernel -> all-reduce (nnforge/cuda/nccl_cuda_communicator.cpp:72-94) -> apply kernel.
 * Every rank owns one zero-initialised mailbox of nnf_bn_train_mailbox_bytes(c) bytes that all ranks can
 * address; mailboxes[r] is rank r's mailbox as seen from this GPU. seq numbers the exchanges (1, 2, 3, ...,
 * the same on all ranks, one per call). Every rank must make the same call with its own shard; count_total
 * = elements per channel over all shards. sums / bsums receive THIS shard's sums; the per-channel gradients
 * accumulate this shard's sums. Needs 16-byte aligned tensors and a shape for which
 * nnf_bn_train_sharded_supported(n, c, hw) answers 1: planes of whole float4s, or planes whose channel groups fill a
 * CTA (7x7, 13x13, ...: channels a multiple of 4 / gcd(H*W, 4)); NNF_ERR_UNSUPPORTED otherwise: use the split entry
 * points. Workspace as for nnf_bn_train_stats. No add_to_destination. */
NNF_API int nnf_bn_train_sharded_supported(int64_t n, int64_t c, int64_t hw);
NNF_API size_t nnf_bn_train_mailbox_bytes(int64_t c);
NNF_API int nnf_bn_train_fwd_sharded(nnf_stream_t stream, float * y, float * saved, float * sums, const float * x,
	const float * gamma, const float * beta, float eps, const nnf_act * acts, int n_acts,
	int64_t n, int64_t c, int64_t hw, double count_total, void * workspace, size_t workspace_bytes,
	void * const * mailboxes, int rank, int world, uint32_t seq);
NNF_API int nnf_bn_train_bwd_sharded(nnf_stream_t stream, float * dx, float * bsums, const float * dy, const float * x,
	const float * gamma, const float * beta, const float * saved, const nnf_act * acts, int n_acts,
	float * grad_gamma, float * grad_beta, float * grad_mean, float * grad_invsigma, float * grad_slope,
	const float * mean, const float * invsigma, float entry_count,
	int64_t n, int64_t c, int64_t hw, double count_total, void * workspace, size_t workspace_bytes,
	void * const * mailboxes, int rank, int world, uint32_t seq);

/* ---------------------------------------------------------------------------------------------
 * Optimiser step for many weight chunks in one launch (replaces cuda_util::apply_gradient,
 * apply_gradient_with_vanilla_momentum, _nesterov_momentum and _adam_momentum, nnforge/cuda/util_cuda.cu:337-596,
 * which backward_propagation_cuda::enqueue_apply_gradient calls once per chunk, nnforge/cuda/backward_propagation_cuda.cpp:2008-2096;
 * arithmetic order of nnforge/plain/backward_propagation_plain.cpp:826-985). Per weight, with g = gradient*normalizer - w*weight_decay:
 *   NONE      upd = lr*g
 *   VANILLA   upd = prev*momentum + lr*g;                         prev_upd = upd
 *   NESTEROV  fresh = prev*momentum + lr*g; upd = (momentum+1)*fresh - momentum*prev;   prev_upd = fresh
 *   ADAM      m1 = beta1*prev + (1-beta1)*g; m2 = beta2*prev2 + (1-beta2)*g*g;  (momentum = beta1, momentum2 = beta2)
 *             upd = lr*(m1/(1-beta1^t)) / (sqrt(m2/(1-beta2^t)) + 1e-8), t = iteration_id >= 1;   prev_upd = m1, prev_upd2 = m2
 *   w += upd; gradient = 0; *update_accum += sum |upd| (double; skipped when update_accum is NULL).
 * `parts` is a HOST array; the chunk table travels in the kernel parameters (48 chunks per launch), so a batch-norm
 * layer's four chunks, or all per-channel chunks of a network, cost one launch. weight_decay is the value that applies
 * to the chunk (0 for chunks outside layer::get_weight_decay_part_id_set()). Results are bit-identical to the plain
 * backend's expressions compiled without FMA contraction; a chunk of up to 1024 weights sums |upd| in a fixed order. */
typedef enum nnf_momentum_type
{
	NNF_MOMENTUM_NONE = 0,      /* training_momentum::no_momentum (nnforge/training_momentum.h) */
	NNF_MOMENTUM_VANILLA = 1,
	NNF_MOMENTUM_NESTEROV = 2,
	NNF_MOMENTUM_ADAM = 3
} nnf_momentum_type;

typedef struct nnf_opt_part
{
	float * data;            /* weights, updated in place */
	float * gradient;        /* accumulated gradient, zeroed */
	float * prev_upd;        /* previous update / first moment (not NONE) */
	float * prev_upd2;       /* second moment (ADAM) */
	double * update_accum;   /* one double, or NULL */
	float learning_rate;
	float weight_decay;
	int64_t elem_count;
} nnf_opt_part;

NNF_API int nnf_apply_gradient(nnf_stream_t stream, const nnf_opt_part * parts, int n_parts, int momentum_type, float momentum,
	float momentum2, float normalizer, unsigned int iteration_id);

/* Recalibration of a batch-norm layer's running statistics on a data set (the GPU form of toolset::update_bn_weights,
 * nnforge/toolset.cpp:1562-1630, which runs the network with gamma = 1 and beta = 0 up to the layer, collects per-feature-map
 * statistics of its output on the host with stat_data_bunch_writer, nnforge/stat_data_bunch_writer.cpp:44-111, and rewrites
 * mean and inverse sigma). nnf_bn_calibrate_accumulate reads the layer's INPUT x once, forms y = x*invsigma + (0 - invsigma*mean)
 * exactly as the inference kernel does and merges count, mean, M2 (double) and min, max of y per feature map into the
 * accumulator (nnf_bn_calibrate_accumulator_bytes(c) bytes, zeroed before the first batch; batches may have any size).
 * nnf_bn_calibrate_finish writes stats[4][c] = {min, max, average, std_dev} (may be NULL) and, when mean / invsigma are given,
 * invsigma' = invsigma / std_dev, mean' = mean + average / invsigma. The reference accumulates value by value (Welford) in
 * double; sums of y and y*y in double followed by a pairwise merge agree with it to double rounding, i.e. to the last
 * bit or two of the fp32 results. */
NNF_API size_t nnf_bn_calibrate_workspace_bytes(int64_t c);
NNF_API size_t nnf_bn_calibrate_accumulator_bytes(int64_t c);
NNF_API int nnf_bn_calibrate_accumulate(nnf_stream_t stream, void * accumulator, const float * x, const float * mean, const float * invsigma,
	int64_t n, int64_t c, int64_t hw, void * workspace, size_t workspace_bytes);
NNF_API int nnf_bn_calibrate_finish(nnf_stream_t stream, float * mean, float * invsigma, float * stats, const void * accumulator, int64_t c);

#ifdef __cplusplus
}
#endif

#endif /* NNF_B200_H */
