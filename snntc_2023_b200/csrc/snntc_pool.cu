// Earliest-spike ("min") pooling for NHWC spike maps: pad with padvalue, window minimum, VALID.
// The reference does this with TensorFlow glue, -MaxPool2D(-x) after tf.pad with 1e5
// (SNN_TC_Modules.py:216-246); here it is one kernel that also records the winner for the backward.
#include "../../include/snntc_b200.h"

#include <cuda_runtime.h>
#include <stdint.h>

namespace snntc { void count_launch(int n = 1); }

namespace {

// One thread per V consecutive channels of one output (V = 4 when C % 4 == 0: 16-byte accesses; else 1).
// All indices fit 32 bits (checked by the callers).
template <int V>
__global__ void minpool_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, int* __restrict__ arg,
                                   int B, int H, int W, int C, int Kh, int Kw, int Sh, int Sw, int pt, int pl,
                                   int Nh, int Nw, float padvalue) {
  const unsigned CV = (unsigned)C / V;
  const unsigned n = (unsigned)B * Nh * Nw * CV;
  const unsigned stride = gridDim.x * blockDim.x;
  for (unsigned o = blockIdx.x * blockDim.x + threadIdx.x; o < n; o += stride) {
    const unsigned cv = o % CV;
    unsigned t = o / CV;
    const int nw = (int)(t % (unsigned)Nw); t /= (unsigned)Nw;
    const int nh = (int)(t % (unsigned)Nh);
    const int b = (int)(t / (unsigned)Nh);
    float best[V];
    int bi[V];
#pragma unroll
    for (int k = 0; k < V; ++k) { best[k] = 0.f; bi[k] = -1; }
    bool first = true;
    for (int kh = 0; kh < Kh; ++kh) {
      const int h = nh * Sh + kh - pt;
      for (int kw = 0; kw < Kw; ++kw) {
        const int w = nw * Sw + kw - pl;
        float v[V];
        int idx = -1;
#pragma unroll
        for (int k = 0; k < V; ++k) v[k] = padvalue;
        if (h >= 0 && h < H && w >= 0 && w < W) {
          idx = ((b * H + h) * W + w) * C + (int)cv * V;
          if constexpr (V == 4) {
            const float4 q = __ldg(reinterpret_cast<const float4*>(x + idx));
            v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
          } else {
            v[0] = __ldg(x + idx);
          }
        }
#pragma unroll
        for (int k = 0; k < V; ++k)
          if (first || v[k] < best[k]) { best[k] = v[k]; bi[k] = idx < 0 ? -1 : idx + k; }
        first = false;
      }
    }
    if constexpr (V == 4) {
      reinterpret_cast<float4*>(y)[o] = make_float4(best[0], best[1], best[2], best[3]);
      reinterpret_cast<int4*>(arg)[o] = make_int4(bi[0], bi[1], bi[2], bi[3]);
    } else {
      y[o] = best[0];
      arg[o] = bi[0];
    }
  }
}

// Backward as a gather: every input element adds up, in (nh, nw) order, the gradients of the windows that
// contain it and whose winner it was. No atomics and no zero-fill: the sum of an element that overlapping
// windows (kernel larger than stride) share is formed in a fixed order, so the result is the same bits every run.
template <int V>
__global__ void minpool_bwd_kernel(const float* __restrict__ gy, const int* __restrict__ arg, float* __restrict__ dx,
                                   int B, int H, int W, int C, int Kh, int Kw, int Sh, int Sw, int pt, int pl,
                                   int Nh, int Nw) {
  const unsigned CV = (unsigned)C / V;
  const unsigned n = (unsigned)B * H * W * CV;
  const unsigned stride = gridDim.x * blockDim.x;
  for (unsigned ev = blockIdx.x * blockDim.x + threadIdx.x; ev < n; ev += stride) {
    const unsigned cv = ev % CV;
    unsigned t = ev / CV;
    const int w = (int)(t % (unsigned)W); t /= (unsigned)W;
    const int h = (int)(t % (unsigned)H);
    const int b = (int)(t / (unsigned)H);
    const int e = (int)ev * V;                       // flat index of this thread's first element
    // windows nh with nh*Sh - pt <= h <= nh*Sh - pt + Kh - 1
    int nh0 = h + pt - Kh + 1; nh0 = nh0 <= 0 ? 0 : (nh0 + Sh - 1) / Sh;
    int nh1 = (h + pt) / Sh; if (nh1 > Nh - 1) nh1 = Nh - 1;
    int nw0 = w + pl - Kw + 1; nw0 = nw0 <= 0 ? 0 : (nw0 + Sw - 1) / Sw;
    int nw1 = (w + pl) / Sw; if (nw1 > Nw - 1) nw1 = Nw - 1;
    float s[V];
#pragma unroll
    for (int k = 0; k < V; ++k) s[k] = 0.f;
    for (int nh = nh0; nh <= nh1; ++nh)
      for (int nw = nw0; nw <= nw1; ++nw) {
        const int o = ((b * Nh + nh) * Nw + nw) * C + (int)cv * V;
        if constexpr (V == 4) {
          const int4 a = __ldg(reinterpret_cast<const int4*>(arg + o));
          if (a.x == e || a.y == e + 1 || a.z == e + 2 || a.w == e + 3) {
            const float4 g4 = __ldg(reinterpret_cast<const float4*>(gy + o));
            if (a.x == e) s[0] += g4.x;
            if (a.y == e + 1) s[1] += g4.y;
            if (a.z == e + 2) s[2] += g4.z;
            if (a.w == e + 3) s[3] += g4.w;
          }
        } else {
          if (__ldg(arg + o) == e) s[0] += __ldg(gy + o);
        }
      }
    if constexpr (V == 4) reinterpret_cast<float4*>(dx)[ev] = make_float4(s[0], s[1], s[2], s[3]);
    else dx[ev] = s[0];
  }
}

int grid_for(size_t n) {
  size_t b = (n + 255) / 256;
  if (b > 148 * 16) b = 148 * 16;
  if (b < 1) b = 1;
  return (int)b;
}

}  // namespace

extern "C" {

int snntc_minpool_forward(const float* x, float* y, int* arg, int B, int H, int W, int C, int Kh, int Kw,
                          int Sh, int Sw, int pad_top, int pad_left, int Nh, int Nw, float padvalue, void* stream) {
  if (!x || !y || !arg) return SNNTC_E_NULL;
  if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || Kh <= 0 || Kw <= 0 || Sh <= 0 || Sw <= 0 || Nh <= 0 || Nw <= 0 ||
      pad_top < 0 || pad_left < 0)
    return SNNTC_E_SHAPE;
  if ((long long)B * H * W * C > 0x7fffffffLL || (long long)B * Nh * Nw * C > 0x7fffffffLL) return SNNTC_E_TOO_LARGE;
  const size_t n = (size_t)B * Nh * Nw * C;
  const bool v4 = (C % 4) == 0 && (((uintptr_t)x | (uintptr_t)y | (uintptr_t)arg) & 15) == 0;
  if (v4)
    minpool_fwd_kernel<4><<<grid_for(n / 4), 256, 0, (cudaStream_t)stream>>>(x, y, arg, B, H, W, C, Kh, Kw, Sh, Sw, pad_top,
                                                                           pad_left, Nh, Nw, padvalue);
  else
    minpool_fwd_kernel<1><<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(x, y, arg, B, H, W, C, Kh, Kw, Sh, Sw, pad_top,
                                                                     pad_left, Nh, Nw, padvalue);
  snntc::count_launch();
  return cudaGetLastError() == cudaSuccess ? SNNTC_OK : SNNTC_E_CUDA;
}

int snntc_minpool_backward(const float* gy, const int* arg, float* dx, int B, int H, int W, int C, int Kh, int Kw,
                           int Sh, int Sw, int pad_top, int pad_left, int Nh, int Nw, void* stream) {
  if (!gy || !arg || !dx) return SNNTC_E_NULL;
  if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || Kh <= 0 || Kw <= 0 || Sh <= 0 || Sw <= 0 || Nh <= 0 || Nw <= 0 ||
      pad_top < 0 || pad_left < 0)
    return SNNTC_E_SHAPE;
  if ((long long)B * H * W * C > 0x7fffffffLL || (long long)B * Nh * Nw * C > 0x7fffffffLL) return SNNTC_E_TOO_LARGE;
  const size_t n = (size_t)B * H * W * C;
  const bool v4 = (C % 4) == 0 && (((uintptr_t)gy | (uintptr_t)arg | (uintptr_t)dx) & 15) == 0;
  if (v4)
    minpool_bwd_kernel<4><<<grid_for(n / 4), 256, 0, (cudaStream_t)stream>>>(gy, arg, dx, B, H, W, C, Kh, Kw, Sh, Sw, pad_top,
                                                                           pad_left, Nh, Nw);
  else
    minpool_bwd_kernel<1><<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(gy, arg, dx, B, H, W, C, Kh, Kw, Sh, Sw, pad_top,
                                                                         pad_left, Nh, Nw);
  snntc::count_launch();
  return cudaGetLastError() == cudaSuccess ? SNNTC_OK : SNNTC_E_CUDA;
}

}  // extern "C"
