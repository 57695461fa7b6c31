/*
 * TEST INFRASTRUCTURE ONLY -- plain-C entry points over the reference's own CPU operators
 * (compiled unmodified against the stand-in op_kernel.h in this folder). Each call builds tensors
 * that view the caller's buffers, runs OpKernel::Compute of the registered float kernel and copies
 * nothing but the outputs. Calls are independent, so several threads may run sub-batches at once.
 *
 * Known limits of the reference CPU code that callers must respect (they are properties of the
 * reference, not of this wrapper): the dense CPU pair is only right without bias
 * (snntc/readme.txt:28-30); the dense forward stores (sum w - theta), not its reciprocal, in rows
 * [B,2B) (snnfc_kernels.cc:136,140); the conv forward leaves rows [B,2B) unwritten
 * (snncv_kernels.cc:109,180); both gradients recompute the denominator from a strict x<y mask.
 */
#include <cstring>
#include <memory>

#include "tensorflow/core/framework/op_kernel.h"

using namespace tensorflow;

static Tensor view(std::initializer_list<int64> dims, const float* p) {
  Tensor t;
  for (auto v : dims) t.s.AddDim(v);
  t.ext = (void*)p;
  return t;
}

static int run(const char* key, OpKernelContext& c) {
  auto it = kernel_table().find(key);
  if (it == kernel_table().end()) return -2;
  std::unique_ptr<OpKernel> k(it->second());
  k->Compute(&c);
  return c.st.ok() ? 0 : -1;
}

extern "C" {

int ref_fc_forward(const float* x, int B, int I, const float* w, int wrows, int J, const float* params6,
                   float* out_2BJ) {
  Tensor X = view({B, I}, x), W = view({wrows, J}, w), P = view({6}, params6);
  OpKernelContext c;
  c.in = {&X, &W, &P};
  c.out_ext[0] = out_2BJ;
  return run("SnnFc/float", c);
}

int ref_fc_backward(const float* grad_2BJ, const float* x, int B, int I, const float* w, int wrows, int J,
                    const float* params6, const float* oldout_2BJ, float* dx, float* dw, float* dparams) {
  Tensor G = view({2 * (int64)B, J}, grad_2BJ), X = view({B, I}, x), W = view({wrows, J}, w),
         P = view({6}, params6), Y = view({2 * (int64)B, J}, oldout_2BJ);
  OpKernelContext c;
  c.in = {&G, &X, &W, &P, &Y};
  c.out_ext[0] = dx; c.out_ext[1] = dw; c.out_ext[2] = dparams;
  return run("SnnFcGrad/float", c);
}

/* x is the ALREADY padded/cropped NHWC input, exactly what the reference op receives. */
int ref_cv_forward(const float* x, int B, int H, int Wd, int C, const float* w, int wrows, int Kc,
                   const float* params12, float* out, int out_capacity_floats, int* nh_nw) {
  Tensor X = view({B, H, Wd, C}, x), W = view({wrows, Kc}, w), P = view({12}, params12);
  OpKernelContext c;
  c.in = {&X, &W, &P};
  int rc = run("SnnCv/float", c);
  if (rc) return rc;
  const Tensor& o = c.out[0];
  if (o.NumElements() > out_capacity_floats) return -3;
  nh_nw[0] = (int)o.s.d[1]; nh_nw[1] = (int)o.s.d[2];
  std::memcpy(out, o.raw(), (size_t)o.NumElements() * 4);
  return 0;
}

int ref_cv_backward(const float* grad, const float* x, int B, int H, int Wd, int C, const float* w, int wrows,
                    int Kc, const float* params12, const float* oldout, int Nh, int Nw,
                    float* dx, float* dw, float* dparams) {
  Tensor G = view({2 * (int64)B, Nh, Nw, Kc}, grad), X = view({B, H, Wd, C}, x), W = view({wrows, Kc}, w),
         P = view({12}, params12), Y = view({2 * (int64)B, Nh, Nw, Kc}, oldout);
  OpKernelContext c;
  c.in = {&G, &X, &W, &P, &Y};
  c.out_ext[0] = dx; c.out_ext[1] = dw; c.out_ext[2] = dparams;
  return run("SnnCvGrad/float", c);
}

}  // extern "C"
