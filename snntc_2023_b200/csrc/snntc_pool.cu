// Earliest-spike ("min") pooling for NHWC spike maps: pad with padvalue, window minimum, VALID.
// The reference does this with TensorFlow glue, -MaxPool2D(-x) after tf.pad with 1e5
// (SNN_TC_Modules.py:216-246); here it is one kernel that also records the winner for the backward.
#include "../../include/snntc_b200.h"

#include <cuda_runtime.h>

namespace snntc { void count_launch(int n = 1); }

namespace {

__global__ void minpool_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, int* __restrict__ arg,
                                   int B, int H, int W, int C, int Kh, int Kw, int Sh, int Sw, int pt, int pl,
                                   int Nh, int Nw, float padvalue) {
  const size_t n = (size_t)B * Nh * Nw * C;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < n; o += stride) {
    const int c = (int)(o % C);
    size_t t = o / C;
    const int nw = (int)(t % Nw); t /= Nw;
    const int nh = (int)(t % Nh);
    const int b = (int)(t / Nh);
    float best = 0.f;
    int bi = -1;
    bool first = true;
    for (int kh = 0; kh < Kh; ++kh) {
      const int h = nh * Sh + kh - pt;
      for (int kw = 0; kw < Kw; ++kw) {
        const int w = nw * Sw + kw - pl;
        float v = padvalue;
        int idx = -1;
        if (h >= 0 && h < H && w >= 0 && w < W) {
          idx = ((b * H + h) * W + w) * C + c;
          v = __ldg(x + idx);
        }
        if (first || v < best) { best = v; bi = idx; first = false; }
      }
    }
    y[o] = best;
    arg[o] = bi;
  }
}

// Backward as a gather: every input element adds up, in (nh, nw) order, the gradients of the windows that
// contain it and whose winner it was. No atomics and no zero-fill: the sum of an element that overlapping
// windows (kernel larger than stride) share is formed in a fixed order, so the result is the same bits every run.
__global__ void minpool_bwd_kernel(const float* __restrict__ gy, const int* __restrict__ arg, float* __restrict__ dx,
                                   int B, int H, int W, int C, int Kh, int Kw, int Sh, int Sw, int pt, int pl,
                                   int Nh, int Nw) {
  const size_t n = (size_t)B * H * W * C;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
    const int c = (int)(e % C);
    size_t t = e / C;
    const int w = (int)(t % W); t /= W;
    const int h = (int)(t % H);
    const int b = (int)(t / H);
    // windows nh with nh*Sh - pt <= h <= nh*Sh - pt + Kh - 1
    int nh0 = h + pt - Kh + 1; nh0 = nh0 <= 0 ? 0 : (nh0 + Sh - 1) / Sh;
    int nh1 = (h + pt) / Sh; if (nh1 > Nh - 1) nh1 = Nh - 1;
    int nw0 = w + pl - Kw + 1; nw0 = nw0 <= 0 ? 0 : (nw0 + Sw - 1) / Sw;
    int nw1 = (w + pl) / Sw; if (nw1 > Nw - 1) nw1 = Nw - 1;
    float s = 0.f;
    for (int nh = nh0; nh <= nh1; ++nh)
      for (int nw = nw0; nw <= nw1; ++nw) {
        const size_t o = (((size_t)b * Nh + nh) * Nw + nw) * C + c;
        if (__ldg(arg + o) == (int)e) s += __ldg(gy + o);
      }
    dx[e] = s;
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
  minpool_fwd_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(x, y, arg, B, H, W, C, Kh, Kw, Sh, Sw, pad_top,
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
  minpool_bwd_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(gy, arg, dx, B, H, W, C, Kh, Kw, Sh, Sw, pad_top,
                                                                     pad_left, Nh, Nw);
  snntc::count_launch();
  return cudaGetLastError() == cudaSuccess ? SNNTC_OK : SNNTC_E_CUDA;
}

}  // extern "C"
