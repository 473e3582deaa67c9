/* dk_b200.h -- C ABI of the B200 (sm_100a) deformable-kernel operator library.
 *
 * This is the drop-in boundary: one entry point per function the reference binds
 * through pybind11 (9 in csrc/filter_sample_depthwise_cuda.cpp:540-569, 3 in
 * csrc/nd_linear_sample_cuda.cpp:67-74; paths relative to
 * deformable_kernels/ops/deform_kernel/ of the reference project), plus fused
 * variants that the autograd functions of this package prefer.
 *
 * Conventions, same for every entry point
 *   - all tensor pointers are DEVICE pointers to dense NCHW (row-major) arrays; all
 *     tensors of one call share one element type, given by `dtype`;
 *   - the caller owns and allocates every buffer, outputs and workspaces included;
 *     nothing is allocated, freed or kept by the library between calls;
 *   - outputs are fully written: no output needs to be zeroed by the caller (the
 *     reference needs zeroed grad buffers, functions/filter_sample_depthwise.py:64-80);
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = the
 *     legacy default stream) of the CURRENT device and the call returns without
 *     synchronising;
 *   - the return value is a dk_status; nothing is printed and the process is never
 *     terminated (the reference prints launch errors and returns 1 regardless,
 *     csrc/filter_sample_depthwise_cuda_kernel.cu:427-430);
 *   - half inputs are read as fp16 and every sum is accumulated in fp32, results are
 *     rounded once on store (what the tensor-core path of fp16 calls rounds on the way
 *     is stated under "numeric limits" below); DK_F64 computes in fp64.
 *   - entry points are thread-safe; the only global state is a per-device attribute
 *     cache behind a mutex.
 */
#ifndef DK_B200_H
#define DK_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum dk_status {
  DK_OK = 0,
  DK_ERR_BAD_ARGUMENT = 1,    /* null pointer, non-positive size, channels % groups != 0, ... */
  DK_ERR_UNSUPPORTED = 2,     /* valid request outside what the kernels cover (e.g. > 8 sample dims) */
  DK_ERR_WORKSPACE = 3,       /* workspace missing or smaller than the matching *_workspace_bytes() */
  DK_ERR_CUDA = 4             /* a CUDA runtime call or launch failed; see dk_last_cuda_error() */
} dk_status;

typedef enum dk_dtype { DK_F32 = 0, DK_F16 = 1, DK_F64 = 2 } dk_dtype;

/* Devices and numeric limits.  Every pointer of a call must belong to the CURRENT device (cudaGetDevice()): the library
 * launches there, on the given stream, and never checks ownership.  fp16 calls on the tensor-core path (3x3, pad 1,
 * stride 1 or 2, at most 16 bank cells, channels a multiple of 16): forward and grad-input take the resampled kernel
 * value of a (pixel, tap, channel) from the tensor cores rounded to fp16 (relative 2^-11, the precision of the tensors
 * themselves), multiply it exactly with the fp16 input and sum in fp32;
 * grad-offsets and grad-bank feed the products grad_output * input to the tensor cores as fp16, so
 * |grad_output * input| must stay below 65504 (an overflow gives Inf / NaN gradients, which a loss scaler's
 * overflow check catches and answers by lowering its scale); all sums are fp32. */

/* Geometry of one depthwise call.  Same fields as the reference's
 * SampleDepthwiseArgs (csrc/filter_sample_depthwise_cuda.h:1-28) minus the output
 * extent, which is derived as in csrc/filter_sample_depthwise_cuda.cpp:42-43:
 *   out = (in + 2*pad - (dil*(kernel-1)+1)) / stride + 1   (integer division).
 * Tensor shapes: input [batch, channels, in_h, in_w]; filter (the weight bank)
 * [channels, 1, scope_h, scope_w]; rotation (kernel-space offsets)
 * [batch, rotation_groups*kernel_h*kernel_w*2, out_h, out_w] with channel index
 * ((g*kernel_h*kernel_w + tap)*2 + dir), dir 0 = h, 1 = w, and channel c using group
 * c % rotation_groups; offset (image-space offsets)
 * [batch, kernel_h*kernel_w*2, out_h, out_w]; output [batch, channels, out_h, out_w]. */
typedef struct dk_geom {
  int batch, channels, in_h, in_w;
  int kernel_h, kernel_w;
  int stride_h, stride_w;
  int pad_h, pad_w;
  int dil_h, dil_w;
  int scope_h, scope_w;
  int rotation_groups;
} dk_geom;

const char *dk_status_string(int status);
/* cudaError_t of the most recent DK_ERR_CUDA on the calling thread (0 if none). */
int dk_last_cuda_error(void);
const char *dk_version(void);

/* Block shape the fp16 tensor-core kernels of the local deformable kernel would launch for this geometry (no counterpart
 * in the reference; for tuning tools and tests, touches no GPU: without a device it plans for 227 KB of shared memory and
 * 148 SMs).  Band kernels, pass: 0 forward, 1 grad-input, 2 grad-offsets, 3 grad-bank; out8 = {band height, channels per
 * block, channel groups, warps per block, bands, dynamic shared memory in bytes, blocks in the grid, workspace bytes}.
 * Row-ring kernels, pass: 4 forward, 5 grad-input, 6 grad-offsets + grad-bank, 7 the one-pass backward; out8 = {slots of
 * the source-row ring, slots of the per-output-row rings, warps per block, producer warps among them, channels per block,
 * channel groups, dynamic shared memory in bytes, blocks in the grid}.  DK_ERR_UNSUPPORTED when the geometry or dtype
 * does not take that family of kernels. */
int dk_local_plan_query(const dk_geom *g, int dtype, int pass, long long *out8);
/* The producer / consumer kernels of the fp16 path bound every wait on a shared-memory barrier; a wait that
 * runs out records a non-zero code on the device and the kernel returns early instead of hanging.  This reads
 * that code for the current device (0 = no wait ever ran out, -1 = the query itself failed).  It synchronises with
 * the device, so it is for tests and diagnosis, not for the hot path.  No counterpart in the reference. */
int dk_ring_error_status(void);
/* Output extent for a geometry; returns DK_ERR_BAD_ARGUMENT if it is not positive. */
int dk_output_size(const dk_geom *g, int *out_h, int *out_w);

/* ---------------------------------------------------------------- local DK
 * y[n,c,oh,ow] = sum over taps of x[n,c,oh*s-p+fh*d, ow*s-p+fw*d] * B(W[c]; u, v),
 * u = fh + rot_h + (scope_h-kernel_h)/2, v alike; B = zero-extended bilinear read. */

/* replaces sample_depthwise_forward_cuda, csrc/filter_sample_depthwise_cuda.cpp:8-62 */
int dk_sample_depthwise_forward(const void *input, const void *rotation, const void *filter, void *output,
                                const dk_geom *g, int dtype, void *stream);

/* replaces sample_depthwise_backward_data_cuda, csrc/filter_sample_depthwise_cuda.cpp:64-119
 * (the reference also takes `input`, for its shape only) */
int dk_sample_depthwise_backward_data(const void *grad_output, const void *rotation, const void *filter,
                                      void *grad_input, const dk_geom *g, int dtype, void *stream);

/* replaces sample_depthwise_backward_filter_cuda, csrc/filter_sample_depthwise_cuda.cpp:121-176.
 * Needs a workspace of dk_sample_depthwise_backward_filter_workspace_bytes() bytes:
 * per-block fp32 partial sums, reduced in a fixed order (no atomics, deterministic). */
size_t dk_sample_depthwise_backward_filter_workspace_bytes(const dk_geom *g, int dtype);
int dk_sample_depthwise_backward_filter(const void *grad_output, const void *input, const void *rotation,
                                        void *grad_filter, const dk_geom *g, int dtype, void *workspace,
                                        size_t workspace_bytes, void *stream);

/* No counterpart in the reference (which runs three launches, functions/filter_sample_depthwise.py:53-87): all three
 * gradients in ONE pass in which every row of grad_output, of the offsets and of input crosses HBM once (fp16, 3x3, pad 1,
 * stride 1 or 2, rows of 112 or 56 elements, at most 144 channels; DK_ERR_UNSUPPORTED otherwise).  It moves the least
 * memory but is not the fastest way on most shapes, so dk_sample_depthwise_backward picks it only where it is.
 * Workspace: dk_sample_depthwise_backward_workspace_bytes(). */
int dk_sample_depthwise_backward_one_pass(const void *grad_output, const void *input, const void *rotation, const void *filter,
                                          void *grad_input, void *grad_rotation, void *grad_filter, const dk_geom *g, int dtype,
                                          void *workspace, size_t workspace_bytes, void *stream);

/* No counterpart in the reference.  Same result as dk_sample_depthwise_backward_filter, for callers
 * that cannot supply a workspace because they may not allocate device memory at call time (plugins
 * inside a memory-planned runtime, fixed-memory control loops, FFI hosts without a CUDA allocator):
 * the partial sums go to a fixed array built into the library, of
 * dk_sample_depthwise_backward_filter_noalloc_max_bytes() bytes (8 MiB, held by every GPU that loads the
 * library until the process exits).  Nothing is allocated or freed on this path.  The call sizes itself for the
 * kernel it launches: the fp16 tensor-core kernel when its partial sums fit, otherwise the general kernel with as
 * many pixel blocks as fit (slower, same result up to summation order); DK_ERR_WORKSPACE only when one block's
 * partial sums (channels x bank cells x 4 bytes; x 8 for fp64) exceed the array.
 * dk_sample_depthwise_backward_filter_noalloc_bytes() returns, without touching a GPU, the bytes of the array a
 * call would use (0 = refused).  All calls on one device share that array, so calls that overlap on the GPU race:
 * serialise them.  The first call on a device queries the array's address; make it before any stream capture
 * begins.  The tensors must live on the current device. */
size_t dk_sample_depthwise_backward_filter_noalloc_max_bytes(void);
size_t dk_sample_depthwise_backward_filter_noalloc_bytes(const dk_geom *g, int dtype);
int dk_sample_depthwise_backward_filter_noalloc(const void *grad_output, const void *input, const void *rotation,
                                                void *grad_filter, const dk_geom *g, int dtype, void *stream);

/* replaces sample_depthwise_backward_rotation_cuda, csrc/filter_sample_depthwise_cuda.cpp:178-235.
 * The workspace (fp32 partial sums over channel groups, used for fp16 tensors on small planes)
 * may be 0 bytes; ask dk_sample_depthwise_backward_rotation_workspace_bytes(). */
size_t dk_sample_depthwise_backward_rotation_workspace_bytes(const dk_geom *g, int dtype);
int dk_sample_depthwise_backward_rotation(const void *grad_output, const void *input, const void *rotation,
                                          const void *filter, void *grad_rotation, const dk_geom *g, int dtype,
                                          void *workspace, size_t workspace_bytes, void *stream);

/* All gradients of the local operator in one call (what
 * SampleDepthwiseFunction.backward, functions/filter_sample_depthwise.py:53-87, does
 * with three).  Any of the three outputs may be NULL to skip it.  Workspace:
 * dk_sample_depthwise_backward_workspace_bytes() (shared by the passes). */
size_t dk_sample_depthwise_backward_workspace_bytes(const dk_geom *g, int dtype);
int dk_sample_depthwise_backward(const void *grad_output, const void *input, const void *rotation,
                                 const void *filter, void *grad_input, void *grad_rotation, void *grad_filter,
                                 const dk_geom *g, int dtype, void *workspace, size_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------- DK + DCN
 * as above, with x read by zero-extended bilinear sampling at
 * (oh*s-p+fh*d + off_h, ow*s-p+fw*d + off_w); a tap is used only if -1 < pos < size. */

/* replaces deformable_sample_depthwise_forward_cuda, csrc/filter_sample_depthwise_cuda.cpp:237-294.
 * `rotation` may be NULL here and in dk_deform_sample_depthwise_backward, meaning zero kernel-space offsets (what
 * DeformKernelConv2d / DeformConv2d pass, modules/deform_kernel.py:276): the sampled kernel is then the same for every
 * pixel and is built once.  Only the fp16 tensor-core path takes NULL; otherwise DK_ERR_UNSUPPORTED is returned and
 * the caller passes a tensor of zeros, as the reference does. */
int dk_deform_sample_depthwise_forward(const void *input, const void *offset, const void *rotation,
                                       const void *filter, void *output, const dk_geom *g, int dtype, void *stream);

/* replaces deformable_sample_depthwise_backward_data_cuda, csrc/filter_sample_depthwise_cuda.cpp:296-354.
 * For DK_F16 the scatter accumulates in an fp32 workspace of
 * dk_deform_sample_depthwise_backward_data_workspace_bytes() bytes (0 for F32/F64). */
size_t dk_deform_sample_depthwise_backward_data_workspace_bytes(const dk_geom *g, int dtype);
int dk_deform_sample_depthwise_backward_data(const void *grad_output, const void *offset, const void *rotation,
                                             const void *filter, void *grad_input, const dk_geom *g, int dtype,
                                             void *workspace, size_t workspace_bytes, void *stream);

/* replaces deformable_sample_depthwise_backward_filter_cuda, csrc/filter_sample_depthwise_cuda.cpp:356-414 */
size_t dk_deform_sample_depthwise_backward_filter_workspace_bytes(const dk_geom *g, int dtype);
int dk_deform_sample_depthwise_backward_filter(const void *grad_output, const void *input, const void *offset,
                                               const void *rotation, void *grad_filter, const dk_geom *g, int dtype,
                                               void *workspace, size_t workspace_bytes, void *stream);

/* replaces deformable_sample_depthwise_backward_offset_cuda, csrc/filter_sample_depthwise_cuda.cpp:416-476 */
int dk_deform_sample_depthwise_backward_offset(const void *grad_output, const void *input, const void *offset,
                                               const void *rotation, const void *filter, void *grad_offset,
                                               const dk_geom *g, int dtype, void *stream);

/* replaces deformable_sample_depthwise_backward_rotation_cuda, csrc/filter_sample_depthwise_cuda.cpp:478-538 */
int dk_deform_sample_depthwise_backward_rotation(const void *grad_output, const void *input, const void *offset,
                                                 const void *rotation, const void *filter, void *grad_rotation,
                                                 const dk_geom *g, int dtype, void *stream);

/* All gradients of DK+DCN in one call (DeformableSampleDepthwiseFunction.backward,
 * functions/filter_sample_depthwise.py:142-191, uses four).  Outputs may be NULL.
 * Workspace: dk_deform_sample_depthwise_backward_workspace_bytes(). */
size_t dk_deform_sample_depthwise_backward_workspace_bytes(const dk_geom *g, int dtype);
int dk_deform_sample_depthwise_backward(const void *grad_output, const void *input, const void *offset,
                                        const void *rotation, const void *filter, void *grad_input,
                                        void *grad_offset, void *grad_rotation, void *grad_filter, const dk_geom *g,
                                        int dtype, void *workspace, size_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------- N-d linear sample
 * data [channels, shape[0..dims-1]], coord [batch, dims], output [batch, channels];
 * `shape` is a HOST array of `dims` ints (the reference passes a floating device
 * tensor and casts it per use, csrc/nd_linear_sample_cuda_kernel.cu:49).  dims <= 8. */

/* replaces nd_linear_sample_forward_cuda, csrc/nd_linear_sample_cuda.cpp:10-26 */
int dk_nd_linear_sample_forward(const void *data, const void *coord, void *output, int batch, int channels,
                                int dims, const int *shape, int dtype, void *stream);

/* replaces nd_linear_sample_backward_data_cuda, csrc/nd_linear_sample_cuda.cpp:29-45
 * (gather form: no atomics, grad_data needs no zeroing) */
int dk_nd_linear_sample_backward_data(const void *grad_output, const void *coord, void *grad_data, int batch,
                                      int channels, int dims, const int *shape, int dtype, void *stream);

/* replaces nd_linear_sample_backward_coord_cuda, csrc/nd_linear_sample_cuda.cpp:47-64:
 * per-channel coordinate gradient [batch, dims, channels] */
int dk_nd_linear_sample_backward_coord(const void *grad_output, const void *data, const void *coord,
                                       void *grad_coord_per_channel, int batch, int channels, int dims,
                                       const int *shape, int dtype, void *stream);

/* The same summed over channels inside the kernel: grad_coord [batch, dims] (the
 * reference sums in Python, functions/nd_linear_sample.py:55). */
int dk_nd_linear_sample_backward_coord_sum(const void *grad_output, const void *data, const void *coord,
                                           void *grad_coord, int batch, int channels, int dims, const int *shape,
                                           int dtype, void *stream);

/* ---------------------------------------------------------------- global DK with a 1x1 depthwise kernel
 * The reference evaluates it as F.conv2d(x.view(1, N*C, H, W), weight[N*C,1,1,1], groups=N*C)
 * (modules/deform_kernel.py:105-118): y[plane, :] = x[plane, :] * scale[plane], plane = n*C + c.
 * Backward gives grad_input = grad_output * scale and grad_scale[plane] = sum(grad_output * input);
 * either output may be NULL. */
int dk_plane_scale_forward(const void *input, const void *scale, void *output, long long planes, int plane_size,
                           int dtype, void *stream);
int dk_plane_scale_backward(const void *grad_output, const void *input, const void *scale, void *grad_input,
                            void *grad_scale, long long planes, int plane_size, int dtype, void *stream);

/* ---------------------------------------------------------------- fused global DK with a 1x1 depthwise kernel
 * GlobalDeformKernel2d.forward for kernel_size 1, groups == channels (modules/deform_kernel.py:76-118) as one call:
 * global average pool -> linear coordinate head (+ tap_bias) -> clamp to [0, shape[0]-1] -> N-d linear sample of
 * the bank [channels, shape...] -> y = x * scale.  The head runs in fp32: bank, fc_weight [dims, channels], fc_bias,
 * tap_bias [dims] and the four saved tensors pooled [batch, channels], raw_coord, coord [batch, dims], scale
 * [batch, channels] are float whatever `dtype` (that of input/output) is.  The backward call takes the saved
 * tensors back; any of its four outputs may be NULL. */
int dk_global_dk_forward(const void *input, const void *bank, const void *fc_weight, const void *fc_bias,
                         const void *tap_bias, void *output, void *pooled, void *raw_coord, void *coord, void *scale,
                         int batch, int channels, int plane_size, int dims, const int *shape, int dtype, void *stream);
size_t dk_global_dk_backward_workspace_bytes(int batch, int channels, int dims);
int dk_global_dk_backward(const void *grad_output, const void *input, const void *bank, const void *fc_weight,
                          const void *pooled, const void *raw_coord, const void *coord, const void *scale,
                          void *grad_input, void *grad_bank, void *grad_fc_weight, void *grad_fc_bias, int batch,
                          int channels, int plane_size, int dims, const int *shape, int dtype, void *workspace,
                          size_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------- offset clipping
 * What LocalDeformKernel2d._clip_rotation, `rotation * weight_dilate` and DeformKernelConv2d's offset clamp / `* dilation`
 * (modules/deform_kernel.py:185-218, 165-170, 273-276) do in up to five elementwise passes, as one:
 *   v = offsets * dilate + bias[channel];   output = (clamp(v, lo, hi) - bias[channel]) / dilate * post_scale
 * offsets [batch, channels, plane_size]; bias [channels] float or NULL (zero).  The backward passes
 * grad_output * post_scale where lo <= v <= hi.  No counterpart among the reference's compiled functions. */
int dk_offset_clip_forward(const void *offsets, const void *bias, void *output, int batch, int channels, int plane_size,
                           double lo, double hi, double dilate, double post_scale, int dtype, void *stream);
int dk_offset_clip_backward(const void *grad_output, const void *offsets, const void *bias, void *grad_offsets, int batch,
                            int channels, int plane_size, double lo, double hi, double dilate, double post_scale, int dtype,
                            void *stream);

#ifdef __cplusplus
}
#endif
#endif /* DK_B200_H */
