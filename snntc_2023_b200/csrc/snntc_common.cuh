// Shared definitions for the SNN-TC sm_100a kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace snntc {

// How a logical "row" of the operator (a dense sample, or one conv receptive field) maps to memory.
// Dense: row r is x[r*I .. r*I+I). Conv: row r = (b*Nh+nh)*Nw+nw, element i = (kh*Kw+kw)*C+c reads
// x[b, nh*Sh+kh-pad_top, nw*Sw+kw-pad_left, c] of the unpadded NHWC image, MAX outside it
// (patch order as in snntc/snncvgrad_kernels.cu.cc:39-43).
struct Geometry {
  int is_conv;
  int R;   // rows: B (dense) or B*Nh*Nw (conv)
  int I;   // fan-in without bias
  int J;   // fan-out
  int has_bias;
  float maxv, theta, biasvolt;
  // conv only
  int B, H, W, C, Kh, Kw, Sh, Sw, pad_top, pad_left, Nh, Nw;
  // forward only: 1 = inference (the output is [R,J] spike values; 1/(sum w - theta) is not written)
  int infer;
  // inference only, may be null: I+2 counters. khist[k] += 1 for every output that fired after consuming k inputs
  // (the bias input is not counted), khist[I+1] += 1 for every output that did not fire.
  int* khist;
  // forward only, set by launch_forward: wbound_n (<= 32) floats whose sum is an upper bound on sum_i |w_ij| for
  // every output j (the walk derives from it how close to zero its sign test must hand over to the reference's
  // rounded comparisons)
  const float* wbound;
  int wbound_n;
};

struct LaunchInfo {
  int num_sms;
  int max_smem_optin;  // bytes of dynamic shared memory one CTA may opt in to
};

// Per-call choices among kernels that compute the same thing. The default (all zero / all parts) is the
// library's own choice; anything else comes from the measurement entry points of a -DSNNTC_MEASURE build
// and from the tests that check the variants against each other. Nothing here is process-wide state.
struct Options {
  int forward_parts = 3;    // bit 0: build the sorted lists, bit 1: walk them
  int walk_layout = 0;      // 0 auto, 1 output pairs, 2 outputs lane+32m, 3 consecutive outputs per lane;
                            // +4: read list entries straight from global memory instead of through shared memory
                            // +8: output pairs with the weights staged in shared memory (where they fit)
  int walk_outputs = 0;     // 0 auto, 1..4: 1, 2, 4, 8 outputs per lane (pairs layout: 2 only)
  int list_builder = 0;     // 0 auto, 1 per-row radix sort, 2 per-pixel sort + merges (3x3 stride-1 conv only),
                            // 3 per-row sorting network in registers (rows of at most 256 inputs);
                            // + 4*(k+1): the merges are cut into 2^k pieces each (k = 0 .. 5) instead of auto
  int backward_parts = 3;   // bit 0: dX, bit 1: dW
  int dw_kernel = 0;        // 0 auto, 1 dense register tile, 2 row-skipping kernel (conv, C % 4 == 0) with per-thread
                            // copies, 4 the row-skipping kernel fed through tensor maps (where the shape allows)
  int dx_kernel = 0;        // 0 auto (conv layers the list-walking kernel supports: both queued, the device picks by
                            // the share of outputs with a gradient), 1 dense register tile, 2 list-walking kernel
  int overlap = -1;         // -1 library setting (snntc_set_overlap), 0 one stream, 1 dX beside dW
};

// number of kernels this library has launched since it was loaded (read by snntc_launch_count)
void count_launch(int n = 1);
// remembers the text of a CUDA runtime error for snntc_last_cuda_error() (per host thread)
void note_cuda_error(cudaError_t e);

// A few auxiliary streams per device, each with its own fork/join events, created on first use and kept for
// the life of the process. Kernels of one call that do not depend on each other (dX and dW) are forked onto
// one of them and joined back into the caller's stream with events, so the caller still sees ordinary stream
// order. Slots are handed out round robin; an event record and the wait that refers to it are issued under one
// lock, so calls from several host threads (or one thread alternating streams) never wait on each other's
// fork points. aux_acquire returns nullptr when the resources cannot be created or overlap is off: callers then
// run everything on the one stream.
struct AuxSlot {
  cudaStream_t stream;
  cudaEvent_t fork;   // recorded on the caller's stream, waited on by the auxiliary stream
  cudaEvent_t join;   // recorded on the auxiliary stream, waited on by the caller's stream
};
AuxSlot* aux_acquire(int overlap_option);
cudaError_t aux_fork(AuxSlot* a, cudaStream_t caller);   // a->stream waits for everything queued on caller so far
cudaError_t aux_join(AuxSlot* a, cudaStream_t caller);   // caller waits for everything queued on a->stream so far

// status codes mirrored from include/snntc_b200.h
enum { OK = 0, E_WORKSPACE = -5, E_UNSUPPORTED = -6, E_CUDA = -7 };

// Entry of a sorted list handed from the list builders to the walk kernels: x = input value (float bits),
// y = element offset of its weight row (source index * J).
typedef uint2 WalkEntry;

// ---- forward ---------------------------------------------------------------------------------
size_t forward_workspace_bytes(const Geometry& g);
// CTAs of the walk that gave up waiting for their weight copies (current device, since the library was loaded)
unsigned long long walk_copy_timeouts();
int launch_forward(const Geometry& g, const float* x, const float* w, float* out, void* ws, size_t ws_bytes,
                   const LaunchInfo& li, const Options& opt, cudaStream_t s);

// Sorted lists of a 3x3 (any Kh x Kw up to 3x3 here), stride-1 convolution by per-pixel sorting and two levels of
// merging (snntc_lists.cu). merge_lists_supported says whether the geometry qualifies, merge_lists_shape_ok the same
// without looking at the strides (what a workspace query knows); merge_lists_bytes is the scratch it needs beyond
// the lists themselves.
bool merge_lists_shape_ok(const Geometry& g);
bool merge_lists_supported(const Geometry& g);
size_t merge_lists_bytes(const Geometry& g);
// split_log2: pieces per merge as a power of two (0 .. 5), -1 = chosen from the number of merges
int launch_merge_lists(const Geometry& g, const float* x, WalkEntry* lists, int* nvalid, int istride,
                       void* scratch, int split_log2, const LaunchInfo& li, cudaStream_t s);

// Sorted lists of rows of at most 256 inputs by a sorting network in registers, one warp per row (snntc_lists.cu).
bool small_rows_supported(const Geometry& g);
int launch_small_rows(const Geometry& g, const float* x, WalkEntry* lists, int* nvalid, int istride,
                      const LaunchInfo& li, cudaStream_t s);

// ---- backward --------------------------------------------------------------------------------
size_t backward_workspace_bytes(const Geometry& g, const LaunchInfo& li);
int launch_backward(const Geometry& g, const float* grad, const float* x, const float* w, const float* out,
                    float* dx, float* dw, void* ws, size_t ws_bytes, const LaunchInfo& li, const Options& opt,
                    cudaStream_t s);

// dW by a kernel that skips the (row, output) pairs that did not fire (snntc_dw_skip.cu); conv layers whose
// channel count is a multiple of 4.
bool dw_skip_supported(const Geometry& g, const float* x, const float* uv, const float* out);
int dw_skip_splits(const Geometry& g, const LaunchInfo& li, int* rows_per_split);
int launch_dw_skip(const Geometry& g, const float* uv, const float* x, const float* out, float* partial,
                   int splits, int rows_per_split, float scale, const int* exact_flag,
                   const LaunchInfo& li, cudaStream_t s);

// The same kernel with its tiles brought in by tiled bulk copies through tensor maps (snntc_dw_tma.cu): stride-1
// convolutions on a power-of-two number of channels (<= 256). Its slices are counted in stages of 16 fields.
bool dw_tma_shape_ok(const Geometry& g);
bool dw_tma_supported(const Geometry& g, const float* x, const float* uv, const float* out);
int dw_tma_splits(const Geometry& g, const LaunchInfo& li, int* stages_per_split);
int launch_dw_tma(const Geometry& g, const float* uv, const float* x, const float* out, float* partial, int splits,
                  int stages_per_split, float scale, const int* exact_flag, const LaunchInfo& li, cudaStream_t s);
// CTAs of that kernel that gave up waiting for their copies (current device, since the library was loaded)
unsigned long long dw_copy_timeouts();

// Which dX kernel of a conv layer is faster depends on how many outputs carry a gradient, which only the device knows
// (snn_u_kernel counts them into *nz): the library queues BOTH, and each looks at the count first -- the list-walking
// kernels return at once when more than `threshold` outputs carry one, the dense register-tile kernel when at most
// that many do. nz == nullptr: no gate, the kernel runs. Both kernels give the same bits.
struct DxGate {
  const unsigned* nz;
  unsigned threshold;
};

// dX by a kernel that walks, per input pixel, the lists of outputs with a non-zero gradient factor
// (snntc_dx_sparse.cu). dx_sparse_bytes is its scratch (lists, their lengths, transposed weights).
bool dx_sparse_shape_ok(const Geometry& g);
bool dx_sparse_supported(const Geometry& g, const float* x, const float* dx);
size_t dx_sparse_bytes(const Geometry& g);
int launch_dx_sparse(const Geometry& g, const float* uv, const float* x, const float* w, const float* out, float* dx,
                     void* scratch, DxGate gate, const LaunchInfo& li, cudaStream_t s);

// monotone map float bits -> unsigned so that an unsigned compare orders like the float compare
__host__ __device__ __forceinline__ uint32_t float_to_sortable(float f) {
#ifdef __CUDA_ARCH__
  uint32_t b = __float_as_uint(f);
#else
  union { float f; uint32_t u; } cv; cv.f = f; uint32_t b = cv.u;
#endif
  return b ^ ((b >> 31) ? 0xFFFFFFFFu : 0x80000000u);
}
__device__ __forceinline__ float sortable_to_float(uint32_t k) {
  return __uint_as_float(k ^ ((k >> 31) ? 0x80000000u : 0xFFFFFFFFu));
}

}  // namespace snntc
