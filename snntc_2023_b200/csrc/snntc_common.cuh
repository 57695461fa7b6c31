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
};

struct LaunchInfo {
  int num_sms;
  int max_smem_optin;  // bytes of dynamic shared memory one CTA may opt in to
};

// number of kernels this library has launched since it was loaded (read by snntc_launch_count)
void count_launch(int n = 1);
// profiling aid: bit 0 = run the dX kernel, bit 1 = run the dW kernels (default 3)
int backward_parts();
// profiling aid: bit 0 = run the sort kernel, bit 1 = run the walk kernel (default 3)
int forward_parts();

// One auxiliary stream and a few events per device, created on first use and kept for the life of the
// process. Kernels of one call that do not depend on each other (dX and dW) are forked onto it and
// joined back into the caller's stream with events, so the caller still sees ordinary stream order. Returns nullptr when the
// resources cannot be created or overlap is switched off (snntc_set_overlap(0)): callers then run
// everything on the one stream.
struct AuxStream {
  cudaStream_t stream;
  cudaEvent_t fork;       // recorded on the caller's stream, waited on by the auxiliary stream
  cudaEvent_t join[8];    // recorded on the auxiliary stream, waited on by the caller's stream
};
AuxStream* aux_stream();

// status codes mirrored from include/snntc_b200.h
enum { OK = 0, E_UNSUPPORTED = -6, E_CUDA = -7 };

// ---- forward ---------------------------------------------------------------------------------
size_t forward_workspace_bytes(const Geometry& g);
int launch_forward(const Geometry& g, const float* x, const float* w, float* out, void* ws, size_t ws_bytes,
                   const LaunchInfo& li, cudaStream_t s);

// ---- backward --------------------------------------------------------------------------------
size_t backward_workspace_bytes(const Geometry& g, const LaunchInfo& li);
int launch_backward(const Geometry& g, const float* grad, const float* x, const float* w, const float* out,
                    float* dx, float* dw, void* ws, size_t ws_bytes, const LaunchInfo& li, cudaStream_t s);

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
