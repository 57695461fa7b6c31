/*
 * TEST INFRASTRUCTURE ONLY -- plain-C entry points over the reference's own GPU functors
 * (SnnFcFunctor<GPUDevice,float> etc., compiled unmodified for sm_100a against the stand-in header
 * in this folder). All tensor pointers are device pointers, `params` is a host vector, `pool` is
 * device scratch for the functors' temporaries. The functors synchronise the device after every
 * launch, as they do under TensorFlow; that is part of what is being timed.
 */
#include "snnfc.h"
#include "snnfcgrad.h"
#include "snncv.h"
#include "snncvgrad.h"

using namespace tensorflow;
typedef Eigen::GpuDevice GPUDevice;

static Tensor view(std::initializer_list<int64> dims, const void* p) {
  Tensor t;
  for (auto v : dims) t.s.AddDim(v);
  t.dev = (void*)p;
  return t;
}

static int finish(OpKernelContext& c) {
  cudaError_t e = cudaStreamSynchronize(c.gpu.s);
  for (void* p : c.overflow) cudaFree(p);
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

static void init(OpKernelContext& c, void* pool, size_t pool_bytes, void* stream) {
  c.gpu.s = (cudaStream_t)stream;
  c.pool = (char*)pool;
  c.pool_bytes = pool_bytes;
}

extern "C" {

int refgpu_fc_forward(const float* x, const float* w, const float* params6_host, float* out_2BJ, int B, int I,
                      int wrows, int J, void* pool, size_t pool_bytes, void* stream) {
  OpKernelContext c; init(c, pool, pool_bytes, stream);
  Tensor X = view({B, I}, x), W = view({wrows, J}, w), P = view({6}, params6_host), O = view({2 * (int64)B, J}, out_2BJ);
  functor::SnnFcFunctor<GPUDevice, float>()(&c, X, W, P, &O, B, I, J);
  return finish(c);
}

int refgpu_fc_backward(const float* grad_2BJ, const float* x, const float* w, const float* params6_host,
                       const float* oldout_2BJ, float* dx, float* dw, float* dparams, int B, int I, int wrows, int J,
                       void* pool, size_t pool_bytes, void* stream) {
  OpKernelContext c; init(c, pool, pool_bytes, stream);
  Tensor G = view({2 * (int64)B, J}, grad_2BJ), X = view({B, I}, x), W = view({wrows, J}, w), P = view({6}, params6_host),
         Y = view({2 * (int64)B, J}, oldout_2BJ), DX = view({B, I}, dx), DW = view({wrows, J}, dw), DP = view({6}, dparams);
  functor::SnnFcGradFunctor<GPUDevice, float>()(&c, G, X, W, P, Y, &DX, &DW, &DP, B, I, J);
  return finish(c);
}

/* x is the ALREADY padded/cropped NHWC input [B,H,W,C]; Nh = (H-Kh)/Sh+1 as the op computes it. */
int refgpu_cv_forward(const float* x, const float* w, const float* params12_host, float* out, int B, int H, int Wd,
                      int C, int wrows, int Kc, int Nh, int Nw, void* pool, size_t pool_bytes, void* stream) {
  OpKernelContext c; init(c, pool, pool_bytes, stream);
  int dimparams[10] = {B, H, Wd, C, wrows, Kc, Nh, Nw, 0, 0};
  Tensor X = view({B, H, Wd, C}, x), W = view({wrows, Kc}, w), P = view({12}, params12_host),
         O = view({2 * (int64)B, Nh, Nw, Kc}, out);
  functor::SnnCvFunctor<GPUDevice, float>()(&c, X, W, P, dimparams, &O);
  return finish(c);
}

int refgpu_cv_backward(const float* grad, const float* x, const float* w, const float* params12_host,
                       const float* oldout, float* dx, float* dw, float* dparams, int B, int H, int Wd, int C,
                       int wrows, int Kc, int Nh, int Nw, void* pool, size_t pool_bytes, void* stream) {
  OpKernelContext c; init(c, pool, pool_bytes, stream);
  int dimparams[10] = {B, H, Wd, C, wrows, Kc, Nh, Nw, 0, 0};
  Tensor G = view({2 * (int64)B, Nh, Nw, Kc}, grad), X = view({B, H, Wd, C}, x), W = view({wrows, Kc}, w),
         P = view({12}, params12_host), Y = view({2 * (int64)B, Nh, Nw, Kc}, oldout), DX = view({B, H, Wd, C}, dx),
         DW = view({wrows, Kc}, dw), DP = view({12}, dparams);
  functor::SnnCvGradFunctor<GPUDevice, float>()(&c, G, X, W, P, Y, dimparams, &DX, &DW, &DP);
  return finish(c);
}

}  // extern "C"
