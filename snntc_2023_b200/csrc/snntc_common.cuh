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
};

struct LaunchInfo {
  int num_sms;
  int max_smem_optin;  // bytes of dynamic shared memory one CTA may opt in to
};

// number of kernels this library has launched since it was loaded (read by snntc_launch_count)
void count_launch(int n = 1);
// profiling aid: bit 0 = run the dX kernel, bit 1 = run the dW kernels (default 3)
int backward_parts();

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
