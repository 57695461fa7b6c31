/*
 * snntc_b200 -- C ABI of the B200 (sm_100a) implementation of the four SNN-TC operators.
 *
 * One shared library (libsnntc_b200.so), plain pointers and sizes, no framework types. Every data
 * pointer is a DEVICE pointer except the `params*_host` vectors, which are read on the host (the
 * reference pins `params` to host memory as well: snntc/snnfc_kernels.cc:224). The library allocates
 * nothing: outputs and the scratch `workspace` belong to the caller, who sizes the workspace with the
 * matching *_workspace_bytes() call and aligns it to 256 bytes (what cudaMalloc and every framework allocator
 * give). All work is queued on `stream` (a cudaStream_t passed as void*)
 * and the call returns without waiting for it; the reference blocks the host after every launch
 * (snntc/snnfc_kernels.cu.cc:187), callers that relied on that must synchronise the stream.
 *
 * Every entry point returns 0 on success or a negative SNNTC_E_* code (see snntc_status_string);
 * nothing is printed and nothing aborts.
 */
#ifndef SNNTC_B200_H_
#define SNNTC_B200_H_

#include <stddef.h>

#if defined(__GNUC__)
#define SNNTC_API __attribute__((visibility("default")))
#else
#define SNNTC_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum {
  SNNTC_OK = 0,
  SNNTC_E_NULL = -1,       /* a required pointer is null */
  SNNTC_E_SHAPE = -2,      /* a dimension is <= 0 or inconsistent (e.g. grad rows != 2*B) */
  SNNTC_E_WEIGHT_ROWS = -3,/* weight rows != fan-in (+1 when params say bias is on) */
  SNNTC_E_TOO_LARGE = -4,  /* a tensor has more than 2^31-1 elements */
  SNNTC_E_WORKSPACE = -5,  /* workspace pointer null, not 256-byte aligned, or smaller than *_workspace_bytes() */
  SNNTC_E_UNSUPPORTED = -6,/* configuration the kernels cannot run (e.g. fan-in too large for shared memory) */
  SNNTC_E_CUDA = -7,       /* a CUDA runtime call failed; see snntc_last_cuda_error() */
  SNNTC_E_PARAMS = -8      /* params vector holds an invalid kernel size / stride / sentinel */
};

SNNTC_API const char* snntc_status_string(int status);
/* Text of the last CUDA runtime error seen by this thread inside the library ("" if none). */
SNNTC_API const char* snntc_last_cuda_error(void);
/* Library version, e.g. "snntc_b200 0.1 sm_100a". */
SNNTC_API const char* snntc_version(void);

/* ------------------------------------------------------------------------------------------------
 * SnnFc -- dense forward.  Replaces the op registered at snntc/snnfc_ops.cc:6-30 with the kernel
 * dispatch of snntc/snnfc_kernels.cc:155-208 and the GPU functor snntc/snnfc_kernels.cu.cc:93-194.
 *   x[B,I] row-major inputs (spike values z=exp(t)); w[w_rows,J] with w_rows = I (+1 bias row, LAST)
 *   params6_host = [MAX_SPIKE_TIME, Epsilon, Spike_Threshold, Thread_per_Block, Blocks, biasvolt]
 *                  (SNN_TC_Modules.py:48-49; entries 1,3,4 are accepted and ignored)
 *   out[2B,J]: rows [0,B) spike value or MAX; rows [B,2B) 1/(sum w - threshold) or 0.
 */
SNNTC_API size_t snntc_fc_forward_workspace_bytes(int B, int I, int J);
SNNTC_API int snntc_fc_forward(const float* x, const float* w, const float* params6_host, float* out_2BJ,
                     int B, int I, int w_rows, int J,
                     void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * SnnFcGrad -- dense backward.  Replaces snntc/snnfcgrad_ops.cc:6-23, snntc/snnfcgrad_kernels.cc:88-132
 * and the GPU functor snntc/snnfcgrad_kernels.cu.cc:137-225.
 *   grad[2B,J] (only rows [0,B) are read), out[2B,J] = the forward's output.
 *   dx[B,I] may be null (first layer of a network); dw[w_rows,J]; dparams6 (device, may be null) is
 *   zero-filled -- the reference never writes it on the GPU.
 */
SNNTC_API size_t snntc_fc_backward_workspace_bytes(int B, int I, int w_rows, int J);
SNNTC_API int snntc_fc_backward(const float* grad_2BJ, const float* x, const float* w, const float* params6_host,
                      const float* out_2BJ, float* dx, float* dw, float* dparams6,
                      int B, int I, int w_rows, int J,
                      void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * SnnCv -- convolution forward.  Replaces snntc/snncv_ops.cc:6-35, snntc/snncv_kernels.cc:186-243 and
 * the GPU functor snntc/snncv_kernels.cu.cc:95-210 (im2col + segmented sort + walk, here fused).
 *   x[B,H,W,C] NHWC, UNPADDED. The reference op receives a tensor already padded with MAX by
 *   SNN_conv.call (SNN_TC_Modules.py:147-161); here pad_top/pad_left say where the image sits in that
 *   virtual padded frame and taps outside [0,H)x[0,W) read as MAX. pad_top = pad_left = 0 with
 *   Nh=(H-Kh)/Sh+1 reproduces the reference op on a pre-padded tensor exactly.
 *   w[w_rows,Kc], row (kh*Kw+kw)*C+c, bias row last.
 *   params12_host = [MAX, Thread_per_Block, Blocks, Epsilon, Threshold, cudaflag, Kh, Kw, Sh, Sw,
 *                    SAME?1:0, biasvolt] (SNN_TC_Modules.py:121-123)
 *   out[2B,Nh,Nw,Kc] packed like SnnFc.
 */
SNNTC_API size_t snntc_cv_forward_workspace_bytes(int B, int H, int W, int C, int Kc, int Kh, int Kw, int Nh, int Nw);
SNNTC_API int snntc_cv_forward(const float* x_nhwc, const float* w, const float* params12_host, float* out,
                     int B, int H, int W, int C, int w_rows, int Kc,
                     int pad_top, int pad_left, int Nh, int Nw,
                     void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * SnnCvGrad -- convolution backward.  Replaces snntc/snncvgrad_ops.cc:6-23,
 * snntc/snncvgrad_kernels.cc:126-184 and the GPU functor snntc/snncvgrad_kernels.cu.cc:164-263.
 *   dx[B,H,W,C] is the gradient of the UNPADDED input (what tf.pad's gradient leaves of the
 *   reference's padded-shape result); it is written, not accumulated, and may be null.
 */
SNNTC_API size_t snntc_cv_backward_workspace_bytes(int B, int H, int W, int C, int w_rows, int Kc, int Nh, int Nw);
SNNTC_API int snntc_cv_backward(const float* grad, const float* x_nhwc, const float* w, const float* params12_host,
                      const float* out, float* dx, float* dw, float* dparams12,
                      int B, int H, int W, int C, int w_rows, int Kc,
                      int pad_top, int pad_left, int Nh, int Nw,
                      void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Earliest-spike pooling between conv layers. The reference has no native code for it: SNN_maxpool2d
 * pads with 1e5 and calls -MaxPool2D(-x) in TensorFlow (SNN_TC_Modules.py:216-246). Here: window
 * minimum over the UNPADDED NHWC input with out-of-image taps reading `padvalue`; arg[B,Nh,Nw,C]
 * receives the flat input index of each winner (first minimum in (kh,kw) order, -1 for padding) and
 * drives the backward: every input element sums gy over the windows it won, in window order (a gather --
 * no atomics, so overlapping windows give the same bits every run); dx[B,H,W,C] is written in full.
 */
SNNTC_API int snntc_minpool_forward(const float* x_nhwc, float* y, int* arg, int B, int H, int W, int C,
                                    int Kh, int Kw, int Sh, int Sw, int pad_top, int pad_left, int Nh, int Nw,
                                    float padvalue, void* stream);
SNNTC_API int snntc_minpool_backward(const float* gy, const int* arg, float* dx, int B, int H, int W, int C,
                                     int Kh, int Kw, int Sh, int Sw, int pad_top, int pad_left, int Nh, int Nw,
                                     void* stream);

/* ------------------------------------------------------------------------------------------------
 * Inference-only forward: SnnFc / SnnCv writing only the spike values, out[B,J] / out[B,Nh,Nw,Kc], without
 * the 1/(sum w - theta) half that only the gradient operators read. Same arguments, workspace
 * (snntc_fc_forward_workspace_bytes / snntc_cv_forward_workspace_bytes) and values as snntc_fc_forward /
 * snntc_cv_forward. The reference has one operator for training and evaluation (snntc-mnist.py:88-94 calls
 * the training forward with training=False); this is its serving-side half.
 *   khist (device, may be null): fan_in + 2 counters, fan_in without the bias row (Kh*Kw*C for the convolution).
 *   khist[k] is incremented for every output that fired after consuming k inputs (its causal-set size; the bias
 *   input is not counted), khist[fan_in + 1] for every output that did not fire. The caller zeroes it. The
 *   reference has no such output: its kernel only breaks out of the walk (snntc/snnfc_kernels.cu.cc:45-48); the
 *   histogram says how early the outputs of a layer fire, i.e. what stopping early can save.
 */
SNNTC_API int snntc_fc_infer(const float* x, const float* w, const float* params6_host, float* out_BJ, int* khist,
                             int B, int I, int w_rows, int J,
                             void* workspace, size_t workspace_bytes, void* stream);
SNNTC_API int snntc_cv_infer(const float* x_nhwc, const float* w, const float* params12_host, float* out, int* khist,
                             int B, int H, int W, int C, int w_rows, int Kc,
                             int pad_top, int pad_left, int Nh, int Nw,
                             void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * The rest of a training step of the reference's example trainers, which the reference runs as TensorFlow
 * graph ops: each is one or two kernels over flat fp32 device buffers, queued on `stream`.
 *
 * snntc_encode       x[e] = exp(scale * (one_minus ? 1 - p[e] : p[e]))   (snntc-mnist.py:75: exp(1.0*(1-images)))
 * snntc_loss_ce      SNN_TC_Modules.loss_func (SNN_TC_Modules.py:286-288): softmax cross-entropy on the negated
 *                    spike times y[B,J] against integer labels[B] (int64). sums2[0] += loss_scale * sum_b loss_b,
 *                    sums2[1] += number of samples whose arg-min_j y equals the label (snntc-mnist.py:82); the
 *                    caller zeroes sums2. grad (may be null) receives d(sum_b loss_b)/dy * grad_scale, i.e.
 *                    -(softmax(-y) - onehot) * grad_scale; use loss_scale = grad_scale = 1/B for the mean.
 * snntc_weight_cost  MyModel.constraint_cost for one weight tensor w[rows,J] (snntc-mnist.py:55-59):
 *                    cost[0] += K * mean_j max(0, 1 - sum_i w_ij) + K2 * mean(w^2); gw (may be null) +=
 *                    its gradient. workspace: snntc_weight_cost_workspace_bytes(J) bytes.
 * snntc_adam_step    tf.keras.optimizers.Adam (snntc-mnist.py:70) on n elements: g is multiplied by grad_scale
 *                    first (1/world size for an all-reduced sum). step[0] is a device int holding the number of
 *                    steps taken so far (0 before the first); the call reads it for the bias correction and
 *                    increments it, so a captured CUDA graph can be replayed. eps is added to sqrt(v) (Keras: 1e-7).
 * snntc_sgdm_step    tf.keras.optimizers.SGD(momentum) (snntc-imagenet.py:238): vel = momentum*vel - lr*g; w += vel.
 */
SNNTC_API int snntc_encode(const float* p, float* x, size_t n, float scale, int one_minus, void* stream);
SNNTC_API int snntc_loss_ce(const float* y, const long long* labels, float* grad, float* sums2, int B, int J,
                            float loss_scale, float grad_scale, void* stream);
SNNTC_API size_t snntc_weight_cost_workspace_bytes(int J);
SNNTC_API int snntc_weight_cost(const float* w, float* gw, float* cost, int rows, int J, float K, float K2,
                                void* workspace, size_t workspace_bytes, void* stream);
SNNTC_API int snntc_adam_step(float* w, const float* g, float* m, float* v, size_t n, float lr, float beta1,
                              float beta2, float eps, float grad_scale, int* step, void* stream);
SNNTC_API int snntc_sgdm_step(float* w, const float* g, float* vel, size_t n, float lr, float momentum,
                              float grad_scale, void* stream);

/* ------------------------------------------------------------------------------------------------
 * SnnFcGrad without a caller workspace. This entry point has no counterpart in the reference.
 *
 * For callers that have no way to allocate device memory when the dense backward runs (an operator
 * plugin that is handed only its declared inputs and outputs, a loop with a fixed memory plan, a
 * process whose device memory belongs to another pool): same arguments and results as
 * snntc_fc_backward, minus the workspace. Everything snntc_fc_backward keeps in its workspace -- the
 * per-output factor u[B,J] = grad/(sum w - threshold), the range flag of the weight-gradient kernel and
 * that kernel's partial tiles -- goes to a fixed array of SNNTC_NOALLOC_SCRATCH_BYTES that is part of the
 * library image, so every GPU that loads the library holds that much memory until the process exits.
 * The call allocates and frees nothing, on the device or through the CUDA runtime: it also keeps all its
 * kernels on `stream` (the regular entry point may run two of them side by side on a library-owned
 * auxiliary stream, which is created on first use).
 *   - Problems that need more than the array (snntc_fc_backward_workspace_bytes() >
 *     snntc_noalloc_scratch_bytes()) are refused with SNNTC_E_WORKSPACE; nothing is launched.
 *   - The first call on each device resolves the array's device address and reads two device
 *     attributes; make that first call outside any stream capture, with the device current.
 *   - All calls on a device share the one array. Calls whose kernels can overlap on the GPU (two
 *     streams, two host threads) race on it -- on u and the flag even when the problem is too small to
 *     have partial tiles: run them one after the other on one stream, or order the streams with events.
 *     The array keeps the previous call's contents; the kernels write every element before they read
 *     it, so no clearing is needed between calls.
 */
#define SNNTC_NOALLOC_SCRATCH_BYTES (8u << 20)
SNNTC_API size_t snntc_noalloc_scratch_bytes(void);
SNNTC_API int snntc_fc_backward_noalloc(const float* grad_2BJ, const float* x, const float* w,
                                        const float* params6_host, const float* out_2BJ,
                                        float* dx, float* dw, float* dparams6,
                                        int B, int I, int w_rows, int J, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Library-wide helpers (no counterpart in the reference).
 *   snntc_launch_count   kernels launched by this library since it was loaded
 *   snntc_set_overlap    1 (default): the two independent kernels of a backward call (dX, dW) run side by side,
 *                        dX on a library-owned auxiliary stream that is joined back with events, so the caller
 *                        still sees plain stream order; 0: everything runs on the caller's stream. The setting
 *                        only chooses between two schedules of the same kernels. Entry points may be called
 *                        from several host threads and on several streams at once: the library keeps no state
 *                        between calls apart from per-device caches behind a lock.
 *   snntc_copy_timeouts  Two kernels wait for asynchronous bulk copies, each wait with a time limit of about a second:
 *                        the forward walk of layers whose weights fit in shared memory (64 outputs x all fan-in rows)
 *                        waits for its weight slice and reads the weights from global memory instead when it does
 *                        not arrive (same results); the weight-gradient kernel of stride-1 convolutions waits for
 *                        the tiles of a stage and, when they do not arrive, stops and leaves its part of the
 *                        gradient incomplete. Either way the CTA counts here. Returns the count on the current
 *                        device since the library was loaded (synchronises the device): 0 in a healthy process.
 */
SNNTC_API unsigned long long snntc_launch_count(void);
SNNTC_API void snntc_set_overlap(int on);
SNNTC_API unsigned long long snntc_copy_timeouts(void);

#ifdef SNNTC_MEASURE
/* ------------------------------------------------------------------------------------------------
 * Measurement build only (libsnntc_b200_measure.so, compiled with -DSNNTC_MEASURE; the default library does
 * not export these). The four operators with the kernel choice of THE CALL given explicitly, so that a
 * benchmark can time the kernels of an operator apart and a test can check the variants against each other:
 *   opts8 = { forward_parts   bit 0: build the sorted lists, bit 1: walk them (default 3; without bit 1 the
 *                             output is not written),
 *             walk_layout     0 auto, 1 output pairs, 2 outputs lane+32m, 3 consecutive outputs per lane; +4: list
 *                             entries straight from global memory instead of staged through shared memory,
 *             walk_outputs    0 auto, 1..4: 1, 2, 4, 8 outputs per lane,
 *             list_builder    0 auto, 1 per-row radix sort, 2 per-pixel sort + merges,
 *             backward_parts  bit 0: dX, bit 1: dW (default 3),
 *             dw_kernel       0 auto, 1 dense register tile, 2 row-skipping kernel,
 *             overlap         -1 library setting, 0 one stream, 1 dX beside dW,
 *             dx_kernel       0 auto, 1 dense register tile, 2 list-walking kernel }
 * A null opts8 means the defaults. All variants of a kernel give the same values (the walk variants the same
 * bits). snntc_fp32_probe queues `ctas` CTAs of 256 threads running `iters` rounds of 8 independent FMAs each
 * and reports the flop count: timed by the caller, it gives the FP32 issue ceiling the kernels are judged against.
 */
SNNTC_API int snntc_measure_fc_forward(const float* x, const float* w, const float* params6_host, float* out_2BJ,
                                       int B, int I, int w_rows, int J, void* workspace, size_t workspace_bytes,
                                       const int* opts8, void* stream);
SNNTC_API int snntc_measure_fc_backward(const float* grad_2BJ, const float* x, const float* w,
                                        const float* params6_host, const float* out_2BJ, float* dx, float* dw,
                                        float* dparams6, int B, int I, int w_rows, int J,
                                        void* workspace, size_t workspace_bytes, const int* opts8, void* stream);
SNNTC_API int snntc_measure_cv_forward(const float* x_nhwc, const float* w, const float* params12_host, float* out,
                                       int B, int H, int W, int C, int w_rows, int Kc,
                                       int pad_top, int pad_left, int Nh, int Nw,
                                       void* workspace, size_t workspace_bytes, const int* opts8, void* stream);
SNNTC_API int snntc_measure_cv_backward(const float* grad, const float* x_nhwc, const float* w,
                                        const float* params12_host, const float* out, float* dx, float* dw,
                                        float* dparams12, int B, int H, int W, int C, int w_rows, int Kc,
                                        int pad_top, int pad_left, int Nh, int Nw,
                                        void* workspace, size_t workspace_bytes, const int* opts8, void* stream);
SNNTC_API int snntc_fp32_probe(float* sink, int iters, int ctas, double* flops_out, void* stream);
#endif /* SNNTC_MEASURE */

#ifdef __cplusplus
}
#endif
#endif /* SNNTC_B200_H_ */
