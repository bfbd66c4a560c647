/*
 * eddl_b200 -- C ABI of the B200 (sm_100a) backend for EDDL's convnet training step.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, and returns an
 * int status: 0 = ok, >0 = a cudaError_t, <0 = one of the EDDLB200_E* codes below
 * (eddlb200_last_error() gives the text).  `dev` is a CUDA device ordinal; every call
 * makes that device current and enqueues its work on that device's single compute
 * stream (eddlb200_stream).  Calls are stream-ordered and asynchronous unless the
 * comment says "blocking".  Device pointers are float* (fp32) in NCHW / row-major
 * layout, exactly what EDDL's Tensor::ptr holds.  There is no CPU fallback: a call
 * made without a usable GPU fails with a CUDA error.
 *
 * Each declaration cites the EDDL v1.1 function it replaces (path inside the EDDL
 * source tree : line) -- the `gpu_*` function the reference's Tensor / tensorNN
 * dispatch calls, and the `cpu_*` twin that defines the arithmetic.
 */
#ifndef EDDL_B200_H
#define EDDL_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EDDLB200_EINVAL   (-1)  /* bad argument (null pointer, negative size, unsupported shape) */
#define EDDLB200_ENOINIT  (-2)  /* device context not initialised / device ordinal out of range */
#define EDDLB200_ENCCL    (-3)  /* NCCL reported an error */
#define EDDLB200_ETIMEOUT (-4)  /* a bounded device-side wait gave up */
#define EDDLB200_ELIMIT   (-5)  /* size beyond a documented maximum */

const char *eddlb200_last_error(void);
int eddlb200_version(void);

/* ---- lifecycle, memory, copies ------------------------------------------------
 * gpu_devices / gpu_init / gpu_create_tensor / gpu_delete_tensor
 *   (src/hardware/gpu/gpu_tensor.cu:133-233);  gpu_copy_to_gpu / gpu_copy_from_gpu /
 *   gpu_copy_gpu (src/hardware/gpu/gpu_core.cu:49-78). */
int eddlb200_device_count(int *n);
int eddlb200_init(int dev);                                  /* idempotent, thread-safe */
int eddlb200_alloc(int dev, size_t bytes, void **out);       /* caching allocator, 256-byte aligned */
int eddlb200_free(int dev, void *p);
int eddlb200_memcpy_h2d(int dev, void *dst, const void *src, size_t bytes);  /* blocking */
int eddlb200_memcpy_d2h(int dev, void *dst, const void *src, size_t bytes);  /* blocking */
int eddlb200_memcpy_d2d(int dev, void *dst, const void *src, size_t bytes);
/* Copy between two devices of this process (gpu_copy_gpu with tensors on different devices: the single-process
 * multi-GPU path of Net::sync_weights / Net::load, src/net/net_func.cpp:111-127).  A direct peer copy over NVLink,
 * ordered after the work already enqueued on both devices' streams and before what is enqueued on either afterwards. */
int eddlb200_memcpy_peer(int dst_dev, void *dst, int src_dev, const void *src, size_t bytes);
/* For device code OUTSIDE this library that writes memory this library also works on: call it before enqueueing the write on
 * the library's stream (eddlb200_stream).  Zeros, copies and averages the library still owes the range are written first, and
 * what it caches about the range's contents (packed weight images of the convolutions, the loss / metric pair) is dropped.
 * The reference's host code never needs it: all its device writes are calls of this library. */
int eddlb200_notify_write(int dev, void *p, size_t bytes);
/* Pinned-host staged copies for a caller that overlaps transfers itself
 * (Net::train_batch does blocking copies: src/net/net_api.cpp:1269-1285). */
int eddlb200_host_alloc(size_t bytes, void **out);
int eddlb200_host_free(void *p);
int eddlb200_memcpy_h2d_async(int dev, void *dst, const void *src, size_t bytes);
/* Host->device copy from ordinary (pageable) host memory that does not wait for the GPU: the bytes are copied into a
 * pinned staging buffer of the library (the call returns as soon as `src` may be reused), travel to a device staging
 * buffer on a separate copy stream while the compute stream keeps working, and a device-side copy ordered on the compute
 * stream delivers them to `dst`.  A ring of four staging pairs, grown to the largest copy seen; a call waits only when
 * the pair it is about to reuse has not been delivered yet.  This is how the drop-in's gpu_copy_to_gpu feeds
 * Net::train_batch's per-step input and target copies (src/net/net_api.cpp:1273-1283). */
int eddlb200_memcpy_h2d_staged(int dev, void *dst, const void *src, size_t bytes);
int eddlb200_stream(int dev, void **cuda_stream);
int eddlb200_sync(int dev);                                  /* blocking */
int eddlb200_mem_info(int dev, size_t *in_use, size_t *cached);
/* Device timers on the compute stream (CUDA events); slot in [0,16). */
int eddlb200_timer_start(int dev, int slot);
int eddlb200_timer_stop(int dev, int slot);
int eddlb200_timer_elapsed_ms(int dev, int slot, float *ms);  /* blocking */
/* Per-family device timing, off by default: when enabled every call of a family is bracketed by
 * CUDA events on the compute stream.  kind: 0 conv fwd, 1 conv bwd-data, 2 conv bwd-weight, 3 BN fwd,
 * 4 BN bwd, 5 elementwise, 6 pooling, 7 dense, 8 optimizer, 9 collectives.  total_work is the sum of
 * the calls' algorithmic work (FLOPs for 0-2 and 7, bytes otherwise).  read is blocking. */
int eddlb200_profile_enable(int dev, int on);
int eddlb200_profile_read(int dev, int kind, unsigned long long *calls, double *total_ms, double *total_work);
/* Individual records of one family, in call order: duration (ms) and work of up to `capacity` calls; *count = calls recorded. */
int eddlb200_profile_records(int dev, int kind, double *ms, double *work, int capacity, int *count);
int eddlb200_profile_reset(int dev);
/* Number of kernels this library has launched on `dev` since init. */
int eddlb200_launch_count(int dev, unsigned long long *n);

/* ---- elementwise (src/hardware/gpu/gpu_math.cu:108-116,148-156,275-284,390-410,
 *      446-455,493-503; gpu_core.cu:139-147; cpu twins in src/hardware/cpu/cpu_math.cpp) */
int eddlb200_fill(int dev, float *a, size_t n, float v);                      /* gpu_fill_ */
/* ntensors fills in ONE launch (Net::do_reset / do_reset_grads issue one gpu_fill_ per delta and per gradient tensor:
 * src/layers/layer.cpp:190-205). */
int eddlb200_fill_multi(int dev, float *const *ptrs, const size_t *sizes, const float *values, int ntensors);
/* gpu_add(scA,A,scB,B,C,incC): C = (incC ? C : 0) + scA*A + scB*B */
int eddlb200_axpby(int dev, float sca, const float *a, float scb, const float *b, float *c, int inc_c, size_t n);
int eddlb200_inc(int dev, const float *a, float *b, size_t n);                /* gpu_inc: B += A */
int eddlb200_scale(int dev, const float *a, float *b, float v, size_t n);     /* gpu_mult: B = A*v */
int eddlb200_addc(int dev, const float *a, float *b, float v, size_t n);      /* gpu_add(A,B,v): B = A+v */
int eddlb200_sqr(int dev, const float *a, float *b, size_t n);                /* gpu_sqr */
int eddlb200_sqrt(int dev, const float *a, float *b, size_t n);               /* gpu_sqrt */
int eddlb200_clamp(int dev, const float *a, float *b, float lo, float hi, size_t n);   /* gpu_clamp */
int eddlb200_el_div(int dev, const float *a, const float *b, float *c, int inc_c, size_t n);  /* gpu_el_div */
int eddlb200_el_mult(int dev, const float *a, const float *b, float *c, int inc_c, size_t n); /* gpu_el_mult */

/* ---- activations (src/hardware/gpu/nn/gpu_activations.cu:25-45,294-385;
 *      src/hardware/cpu/nn/cpu_activations.cpp:20-45,329-436) */
int eddlb200_relu_fwd(int dev, const float *a, float *b, size_t n);
/* pd += (i > 0) ? d : 0   (tests the layer INPUT i, accumulates) */
int eddlb200_relu_bwd(int dev, const float *d, const float *i, float *pd, size_t n);
/* Row softmax over the last axis of a [rows, cols] view; the denominator starts at
 * 1.19209e-07 like the reference. */
int eddlb200_softmax_fwd(int dev, const float *a, float *b, int rows, int cols);
/* pd[r,i] += sum_j d[r,j] * (s[r,i]*[i==j] - s[r,j]*s[r,i]) ; s = softmax OUTPUT */
int eddlb200_softmax_bwd(int dev, const float *d, const float *s, float *pd, int rows, int cols);
/* Same over the middle axis of an [outer, cols, inner] view (gpu_full_softmax's `axis`). */
int eddlb200_softmax_fwd_nd(int dev, const float *a, float *b, int outer, int cols, int inner);
int eddlb200_softmax_bwd_nd(int dev, const float *d, const float *s, float *pd, int outer, int cols, int inner);

/* ---- losses / metrics (src/hardware/gpu/nn/gpu_losses.cu:49-92, gpu_metrics.cu:26-49;
 *      src/hardware/cpu/nn/cpu_losses.cpp:29-57, cpu_metrics.cpp:17-29) */
/* value = -sum_rows sum_cols y*logf(p + 1e-7)   (a SUM over the batch).
 * Net::train_batch asks for the loss and the metric of the same (target, prediction) pair twice per step
 * (src/net/net_func.cpp:78-90, called from net_api.cpp:46 and :1300): the first of these calls computes BOTH scalars and
 * reads them back with one blocking copy; eddlb200_cce_value / eddlb200_accuracy calls that follow with the same pointers
 * and shape return the remembered values without touching the GPU, until an entry point of this library writes either
 * tensor.  Values are those a fresh evaluation would give. */
int eddlb200_cce_value(int dev, const float *y_true, const float *y_pred, int rows, int cols, float *host_out);
int eddlb200_cce_delta(int dev, const float *y_true, const float *y_pred, float *delta, size_t n);
/* rows whose argmax(y_true) == argmax(y_pred), first maximum wins.  Blocking unless remembered (see above). */
int eddlb200_accuracy(int dev, const float *y_true, const float *y_pred, int rows, int cols, int *host_out);

/* ---- batch normalisation (src/hardware/gpu/nn/gpu_bn.cu:65-117;
 *      src/hardware/cpu/nn/cpu_bn.cpp:118-249).  x is [b, z, rc].  Argument order and
 *      meaning are those of gpu_batchnorm_forward / gpu_batchnorm_backward:
 *      train: mean = sum/N, var = sumsq/N - mean^2, running stats updated when
 *      momentum != 0, then `variance` receives sqrt(var + eps); opa = (x-mean)/variance;
 *      y = opa*g + b.  `relu_out`, when not null, additionally receives max(y, 0)
 *      (what a following ReLU layer would compute), so a BN+ReLU pair costs one pass. */
int eddlb200_bn_fwd(int dev, int b, int z, int rc,
                    const float *input, float *output, float *opa,
                    float *global_mean, float *global_variance,
                    const float *affine_g, const float *affine_b,
                    float *mean, float *variance,
                    int trmode, float epsilon, float momentum, float *relu_out);
/* Same operation as eddlb200_bn_fwd for callers that must not allocate device memory.  It has no
 * counterpart in EDDL.  It performs no cudaMalloc / cudaFree (neither directly nor through the library's
 * device context, which it does not create): the per-channel partial sums live in a fixed 2 MiB array
 * inside the library image, and the work is enqueued on the caller's `cuda_stream` (a cudaStream_t; null is
 * the default stream).  Intended for hosts whose device memory is wholly owned by another allocator, or
 * that cannot accept the device-wide synchronisation cudaMalloc / cudaFree imply.  Limits and rules:
 *   - in training mode channels x slices must not exceed 262144, else EDDLB200_ELIMIT.  The slice count (1..256 per
 *     channel) follows from the shape and from the "bn_waves" / "bn_min_items" options in force at the call: channels x
 *     slices stays below 1184 x bn_waves + z, so with the defaults every z up to 243200 fits.  Inference mode
 *     (trmode = 0) uses no partial sums and has no such limit;
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress): make
 *     that call before any stream capture starts;
 *   - all calls on a device share the array; calls that overlap on the GPU race on it, so order them;
 *   - if the library's device context exists (eddlb200_init or any other entry point was used on `dev`), work that it
 *     still owes -- deferred zero fills, a recorded first term of a sum -- is settled on the LIBRARY's compute stream
 *     first, and a different `cuda_stream` is then made to wait for that stream, so these kernels see every buffer as
 *     the earlier library calls left it.  Ordering work that follows on other streams after this call is the caller's job.
 * Results are identical to eddlb200_bn_fwd called with the same options (same kernels, same slicing). */
int eddlb200_bn_fwd_noalloc(int dev, int b, int z, int rc,
                            const float *input, float *output, float *opa,
                            float *global_mean, float *global_variance,
                            const float *affine_g, const float *affine_b,
                            float *mean, float *variance,
                            int trmode, float epsilon, float momentum, float *relu_out, void *cuda_stream);
/* gbn_g += mean(delta*opa); gbn_b += mean(delta)  (means, not sums);
 * delta *= bn_g in place; pdelta += (delta - (opa*m1 + m2)) / variance. */
int eddlb200_bn_bwd(int dev, int b, int z, int rc,
                    float *delta, const float *opa, float *pdelta,
                    float *gbn_g, float *gbn_b, const float *bn_g,
                    const float *variance, float *mean1, float *mean2);

/* ---- pooling (src/hardware/gpu/nn/gpu_pool.cu:26-60,101-135;
 *      src/hardware/cpu/nn/cpu_pool.cpp:74-145,226-304).  Input [n,c,ih,iw], output
 *      [n,c,oh,ow]; ind_x/ind_y are float tensors shaped like the output that hold the
 *      absolute input column/row of the maximum (first in row-major window order). */
int eddlb200_maxpool2d_fwd(int dev, const float *in, float *out, float *ind_x, float *ind_y,
                           int n, int c, int ih, int iw, int oh, int ow,
                           int kr, int kc, int sr, int sc, int pad_top, int pad_left);
int eddlb200_maxpool2d_bwd(int dev, const float *d, const float *ind_x, const float *ind_y, float *id,
                           int n, int c, int ih, int iw, int oh, int ow,
                           int kr, int kc, int sr, int sc, int pad_top, int pad_left);
int eddlb200_avgpool2d_fwd(int dev, const float *in, float *out,
                           int n, int c, int ih, int iw, int oh, int ow,
                           int kr, int kc, int sr, int sc, int pad_top, int pad_left);
int eddlb200_avgpool2d_bwd(int dev, const float *d, float *id,
                           int n, int c, int ih, int iw, int oh, int ow,
                           int kr, int kc, int sr, int sc, int pad_top, int pad_left);

/* ---- padding (src/hardware/gpu/gpu_da.cu:144-168; spec src/hardware/cpu/cpu_da.cpp:502-534)
 *      a [n,c,h,w] -> b [n,c,h+top+bottom,w+left+right]; only the interior of b is written. */
int eddlb200_pad(int dev, const float *a, float *b, int n, int c, int h, int w,
                 int top, int bottom, int left, int right);
int eddlb200_pad_bwd(int dev, float *a_delta, const float *b_delta, int n, int c, int h, int w,
                     int top, int bottom, int left, int right);   /* a_delta += crop(b_delta) */

/* ---- layers beside the benchmark nets that EDDL's own convnet examples use (examples/nn/2_cifar10): Concat, UpSampling,
 *      Dropout, RandomFlip, RandomCropScale.  gpu_concat (src/hardware/gpu/gpu_core.cu:384-409; cpu_concat,
 *      src/hardware/cpu/cpu_core.cpp:368-396); gpu_repeat_nn / gpu_d_repeat_nn (src/hardware/cpu/nn/cpu_tensor_nn.cpp:13-50);
 *      gpu_rand_binary; gpu_flip_random / gpu_crop_scale_random (src/hardware/gpu/gpu_da.cu:250-302; cpu_single_flip and
 *      cpu_single_crop_scale, src/hardware/cpu/cpu_da.cpp:315-336, 363-384). */
/* Concatenation along one axis of `a`: part i holds part_sizes[i] floats in runs of part_strides[i] (= stride[axis] *
 * shape[axis] of that tensor); `steps` is the same product for `a`.  derivative != 0 runs it backwards: part += slice of a. */
int eddlb200_concat(int dev, float *a, float *const *parts, const size_t *part_sizes, const size_t *part_strides, int nparts,
                    size_t steps, int derivative);
/* UpSampling by whole factors: b[row*size_r + i][col*size_c + j] = a[row][col] over rows_a = batch*channels*height rows;
 * backward adds every block of d into a, one value at a time in row-major order of the block. */
int eddlb200_repeat_nn(int dev, const float *a, float *b, size_t rows_a, int cols_a, int size_r, int size_c);
int eddlb200_repeat_nn_bwd(int dev, const float *d, float *a, size_t rows_a, int cols_a, int size_r, int size_c);
/* Nearest-neighbour resize of a [n,c,ah,aw] to b [n,c,bh,bw] thought of as a (new_h, new_w) image cropped at its centre
 * (gpu_scale / gpu_scale_back, src/hardware/gpu/gpu_da.cu:61-88; cpu_single_scale(_back), src/hardware/cpu/cpu_da.cpp:88-190):
 * eddl::UpSampling2D is this with new shape = b's shape.  mode: 0 half-pixel, 2 align-corners, 3 asymmetric (the source index
 * uses the reference's float arithmetic and truncation).  wrap: where a source index leaves a, 0 writes cval and 5
 * ("original", forward only) copies a at b's own position; other wrapping modes are accepted only when no index leaves a.
 * The backward pass adds every b_delta value into its source position of a_delta, in row-major order of b. */
int eddlb200_resize(int dev, const float *a, float *b, int n, int c, int ah, int aw, int bh, int bw, int new_h, int new_w,
                   int wrap, float cval, int mode);
int eddlb200_resize_bwd(int dev, float *a_delta, const float *b_delta, int n, int c, int ah, int aw, int bh, int bw,
                       int new_h, int new_w, int wrap, float cval, int mode);
/* Image i of the batch is mirrored along axis (0 = rows, 1 = columns) when apply_host[i] != 0, copied otherwise.
 * apply_host is a HOST array of n bytes: the caller draws the decisions (uniform >= 0.5 in the reference). */
int eddlb200_flip_batch(int dev, const float *a, float *b, int n, int c, int h, int w, int axis, const unsigned char *apply_host);
/* Image i of b [n,c,bh,bw] is the box (y0, x0) .. (y1, x1) of image i of a [n,c,ah,aw], resized by nearest neighbour with
 * the reference's integer arithmetic Ai = Bi*(y1-y0+1)/bh + y0.  boxes_host is a HOST array of 4n ints (y0, x0, y1, x1). */
int eddlb200_crop_scale_batch(int dev, const float *a, float *b, int n, int c, int ah, int aw, int bh, int bw, const int *boxes_host);
/* a[i] = 1 with probability p, else 0: value i of the stream (seed, offset) of a counter-based generator, so equal
 * arguments give equal masks whatever the launch geometry (the reference draws from cuRAND; no stream is shared with it). */
int eddlb200_rand_binary(int dev, float *a, size_t n, float p, size_t seed, size_t offset);

/* ---- dense algebra (src/hardware/gpu/gpu_math.cu:457-528; gpu_reduction.cu:232-244;
 *      src/hardware/cpu/cpu_math.cpp:302-325,369-401) */
/* gpu_mult2D: C[m,n] = (inc_c ? C : 0) + op(A) * op(B), row-major; A is [m,k] (or [k,m]
 * when ta), B is [k,n] (or [n,k] when tb).  Large products (k >= 32, m n k >= 2^26) run on the
 * tensor-core kernel of the convolutions in its fp32-equivalent 3xTF32 mode (about 1e-6 relative); smaller ones, and all of
 * them under "conv_path" 1, on an exact-fp32 FMA kernel. */
int eddlb200_mult2d(int dev, const float *a, int ta, const float *b, int tb, float *c, int inc_c,
                    int m, int n, int k);
int eddlb200_sum2d_rowwise(int dev, const float *a, const float *b, float *c, int rows, int cols); /* C = A + b[col] */
/* gpu_reduce_sum2D: axis 0 -> B[cols] (+)= sum over rows; axis 1 -> B[rows] (+)= sum over cols */
int eddlb200_reduce_sum2d(int dev, const float *a, float *b, int rows, int cols, int axis, int inc_b);

/* ---- Conv2D (src/hardware/gpu/nn/gpu_conv.cu:159-372;
 *      src/hardware/cpu/nn/cpu_conv.cpp:114-280,316-527).  Cross-correlation, zero padding,
 *      x [n,c,ih,iw], w [k,c,kr,kc], y [n,k,oh,ow].  precision: 0 = fp32-equivalent
 *      (3xTF32 split on the tensor cores or fp32 FMA), 1 = plain TF32, 2 = TF32 main product plus
 *      bf16 cross terms of the split (forward and backward-data; about four times the rounding error
 *      of 0, still below 1e-5 relative; backward-weight runs as 0).  Any other value is EINVAL. */
/* Options: "conv_path" 0 = tensor-core kernel where it applies (default), 1 = fp32 FMA kernel only.
 *          "lazy_zero" 1 = eddlb200_fill / eddlb200_fill_multi of 256 KB or more with 0.0f only record the range; the
 *          zeros are written when an entry point of this library reads the range, dropped when one overwrites all of
 *          it, and an accumulating kernel (conv2d_bwd_data, bn_bwd, relu_bwd, inc, axpby with inc_c, pool backward)
 *          that owns the whole range stores its result instead of adding to it (same bits); the in-place form
 *          eddlb200_axpby(s, a, t, c, c, 0) into such a c is recorded and runs with the next call (fused with it when
 *          that is the second in-place add into c; the sum then stays on record for one more call and is fused
 *          with an eddlb200_relu_fwd of c).  Off by default: device
 *          code outside this library does not see a deferred fill.  0 writes everything still deferred and returns
 *          to immediate fills.
 *          "conv_prefetch" 1 (default) = in 1x1 unpadded layers a spare warp of the tensor-core kernel prefetches the
 *          activation operand into L2 ahead of the gather (results unchanged); 0 = off.
 *          "conv_tma" 2 (default) = forward and backward-data of 1x1 stride-1 unpadded layers (planes of a multiple of 4
          pixels, at least 32 channels on both sides) are fed by TMA tensor copies of the activations and drained by TMA
          stores, or TMA fp32 adds where the output accumulates; 1 = only where the output is stored; 0 = the gather
          kernel everywhere.  Results are the same bits at every level.
 *          "conv_tma_3x3" 1 (default) = forward and backward-data of 3x3 stride-1 pad-1 layers (planes of a multiple of 4
 *          pixels and at least 64, rows of at most 125 pixels, at least 32 channels on both sides) read raw slabs of the
 *          activations delivered by TMA, one per tile and 32-channel group for all nine taps; the reduction is then
 *          ordered (channel group, tap, channel), so results agree with the gather kernel to rounding (3e-6), not to
 *          the bit; 0 = the gather kernel.  Needs "conv_tma" >= 1.
 *          "conv_tma_wgrad" 2 (default) = backward-weight of 1x1 stride-1 unpadded layers: both operands are copied by TMA
 *          straight into the operand ring and the landed fp32 values serve as the hi planes as they are (the tensor core
 *          reads only their upper 19 bits: same bits as 1); 1 = the hi planes are rewritten with the low bits cleared;
 *          0 = the gather kernel.
 *          "conv_tma_wgrad_3x3" 1 (default) = backward-weight of 3x3 stride-1 pad-1 layers (rows of at most 60 pixels, planes of a
 *          multiple of 4 pixels, at least 14 channels and 32 filters): dy is copied by TMA into the operand ring and the
 *          tap-shifted x operand is built in shared memory from raw slabs that TMA delivers, one per K-block for the nine
 *          taps of 14 channels; 0 = the gather kernel.  Agreement to rounding (K-blocks end at image boundaries).
 *          "conv_dense_1x1" 1 (default) = 1x1 unpadded layers that skip pixels (stride > 1) or whose planes are not a
 *          multiple of 4 pixels run as dense 1x1 stride-1 layers over gathered copies of their operands (library-owned
 *          device buffers that only grow); 0 = the strided gather kernels.  Agreement to rounding.
 *          "conv_pack_cache" 1 (default) = the packed weight images of forward / backward-data are kept per weight tensor
 *          and re-packed only after a call of this library has written the tensor; 0 = packed at every call.  Device
 *          code outside this library that writes weights must go through eddlb200_notify_write or switch this off.
          "bn_waves" (1..64, default 16) and "bn_min_items" (>= 1024, default 8192): grid sizing of the BatchNorm
 *          kernels -- every channel is cut into slices so that a launch has about bn_waves x (8 blocks per SM) blocks
 *          of at least bn_min_items elements each.  Results depend on the slicing only through the fp32 order of the
 *          partial sums (about 1e-7 relative on the statistics). */
int eddlb200_set_option(const char *name, int value);
/* Conv2D calls (forward, backward-data, backward-weight alike) that `dev` has served on the tensor-core kernels and on the fp32
 * FMA kernels since the library was loaded.  The FMA path is taken for shapes the tensor-core kernel refuses (a plane side of
 * 16000 pixels or more) and when "conv_path" forces it; it is about 100 times slower, so a non-zero fma count in a training
 * run is worth knowing.  Either pointer may be null. */
int eddlb200_conv_path_counts(int dev, unsigned long long *tensor_core_calls, unsigned long long *fma_calls);
int eddlb200_conv2d_fwd(int dev, const float *x, const float *w, const float *bias /* may be null */, float *y,
                        int n, int c, int ih, int iw, int k, int kr, int kc, int oh, int ow,
                        int sr, int sc, int pad_top, int pad_left, int precision);
/* gw += sum_{n,p,q} dy * x ; gbias += sum dy when gbias != null  (accumulates) */
int eddlb200_conv2d_bwd_weight(int dev, const float *x, const float *dy, float *gw, float *gbias,
                               int n, int c, int ih, int iw, int k, int kr, int kc, int oh, int ow,
                               int sr, int sc, int pad_top, int pad_left, int precision);
/* dx += sum_{k,r,s} dy * w  (accumulates into the parent delta) */
int eddlb200_conv2d_bwd_data(int dev, const float *dy, const float *w, float *dx,
                             int n, int c, int ih, int iw, int k, int kr, int kc, int oh, int ow,
                             int sr, int sc, int pad_top, int pad_left, int precision);

/* ---- optimizers (src/optimizers/optim_sgd.cpp:68-89; optim_adam.cpp:85-120) */
/* m = lr*g + mu*m ; p = p - m   (no weight decay, no nesterov: the reference ignores both) */
int eddlb200_sgd_momentum(int dev, float *p, const float *g, float *m, float lr, float mu, size_t n);
/* Multi-tensor form: ntensors triples (p[i], g[i], m[i]) of sizes[i] floats, one launch. */
int eddlb200_sgd_momentum_multi(int dev, float *const *p, const float *const *g, float *const *m,
                                const size_t *sizes, int ntensors, float lr, float mu);
/* m = b1*m + (1-b1)*g ; g = g*g (in place, like the reference) ; v = b2*v + (1-b2)*g ;
 * p -= lr * (m/(1-b1^t)) / sqrt(v/(1-b2^t) + eps)      (eps inside the sqrt) */
int eddlb200_adam(int dev, float *p, float *g, float *m, float *v,
                  float lr, float beta1, float beta2, float eps, int t, size_t n);
/* Multi-tensor form of the same step (Adam::applygrads walks every trainable tensor with ten launches each:
 * src/optimizers/optim_adam.cpp:85-120): ntensors quadruples (p[i], g[i], m[i], v[i]) of sizes[i] floats, one launch,
 * every tensor bit-identical to eddlb200_adam. */
int eddlb200_adam_multi(int dev, float *const *p, float *const *g, float *const *m, float *const *v,
                        const size_t *sizes, int ntensors, float lr, float beta1, float beta2, float eps, int t);

/* ---- cross-replica averaging (replaces Net::sync_weights, src/net/net_func.cpp:111-127:
 *      acc = sum over replicas in fp32, acc *= 1.0f/N, every replica receives acc).
 *      One process per GPU; the 128-byte id is made on rank 0 and given to every rank. */
int eddlb200_comm_unique_id(void *id128);
int eddlb200_comm_init_rank(int dev, int nranks, int rank, const void *id128);
int eddlb200_comm_destroy(int dev);
int eddlb200_comm_info(int dev, int *nranks, int *rank);
int eddlb200_allreduce_avg(int dev, float *buf, size_t n);            /* in place */
int eddlb200_allreduce_avg_multi(int dev, float *const *bufs, const size_t *sizes, int ntensors);
/* The same averaging, overlapped with whatever the compute stream does next: the tensors are cut, in the order given, into
 * buckets (a first one of about 2 MB, then `bucket_bytes` each; 0 = 32 MB); each bucket is all-reduced on a separate
 * communication stream -- tensors of 1 MB or more where they lie, the small ones packed into one message -- and scaled by
 * 1.0f/N there.  The call returns at once.  Any later entry point of this library that reads or writes one of the tensors
 * first makes the compute stream wait for THAT tensor's bucket, so with the parameters given in forward order the next
 * step's first layers start while the last layers are still being averaged.  Code outside the library must call
 * eddlb200_sync before it touches the tensors. */
int eddlb200_allreduce_avg_multi_async(int dev, float *const *bufs, const size_t *sizes, int ntensors, size_t bucket_bytes);
/* Health of the communicator (ncclCommGetAsyncError) and progress of the collectives enqueued so far: 0 = all done;
 * EDDLB200_ETIMEOUT = still running after wait_ms milliseconds (wait_ms < 0 waits without limit); EDDLB200_ENCCL = NCCL
 * reported an asynchronous error, in which case the communicator has been aborted and this rank is back to N = 1.  The
 * wait is a host-side poll: nothing is left waiting on the GPU by this call. */
int eddlb200_comm_check(int dev, int wait_ms);
int eddlb200_broadcast(int dev, float *buf, size_t n, int root);
/* Gradient averaging fused with the SGD-momentum step of an equal-size parameter
 * buffer: g <- allreduce(g)/N ; m = lr*g + mu*m ; p -= m. */
int eddlb200_avg_grad_sgd(int dev, float *p, float *g, float *m, float lr, float mu, size_t n);

#ifdef __cplusplus
}
#endif
#endif
