/*
 * TEST INFRASTRUCTURE ONLY -- a stand-in for the small part of TensorFlow's op-kernel API that the
 * reference CPU operators (snntc/snnfc_kernels.cc, snnfcgrad_kernels.cc, snncv_kernels.cc,
 * snncvgrad_kernels.cc) touch, so those four files compile unmodified, from where they lie, without
 * TensorFlow. Tensors are host buffers; REGISTER_KERNEL_BUILDER feeds a name -> factory table that
 * ref_capi.cc drives. Nothing here is part of the product.
 */
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <map>
#include <string>
#include <type_traits>
#include <vector>

namespace Eigen {
struct ThreadPoolDevice {};
struct GpuDevice {};
}  // namespace Eigen

namespace tensorflow {

typedef uint64_t uint64;
typedef int64_t int64;
typedef int32_t int32;
typedef int8_t int8;
static const int32 kint32max = 0x7fffffff;

struct Status {
  bool good = true;
  std::string msg;
  bool ok() const { return good; }
};
namespace errors {
template <class... A>
Status InvalidArgument(const char* m, A...) {
  Status s;
  s.good = false;
  s.msg = m;
  return s;
}
}  // namespace errors

struct TensorShape {
  std::vector<int64> d;
  int64 dim_size(int i) const { return d[i]; }
  void AddDim(int64 v) { d.push_back(v); }
  int dims() const { return (int)d.size(); }
  int64 num_elements() const {
    int64 n = 1;
    for (auto v : d) n *= v;
    return n;
  }
};

template <class T>
struct FlatView {
  T* p;
  T* data() const { return p; }
};

/* A tensor either owns its bytes (outputs) or views caller memory (inputs). */
struct Tensor {
  TensorShape s;
  std::vector<char> own;
  void* ext = nullptr;
  const TensorShape& shape() const { return s; }
  int64 NumElements() const { return s.num_elements(); }
  void* raw() const { return ext ? ext : (void*)own.data(); }
  template <class T>
  FlatView<T> flat() { return FlatView<T>{(T*)raw()}; }
  template <class T>
  FlatView<const T> flat() const { return FlatView<const T>{(const T*)raw()}; }
};

struct OpKernelConstruction {};

struct OpKernelContext {
  std::vector<const Tensor*> in;
  Tensor out[4];          /* fixed slots: an output must not move when a later one is allocated */
  void* out_ext[4] = {nullptr, nullptr, nullptr, nullptr}; /* optional caller-owned output storage */
  Status st;
  const Tensor& input(int i) { return *in[i]; }
  Status allocate_output(int i, const TensorShape& sh, Tensor** t) {
    out[i].s = sh;
    if (out_ext[i]) out[i].ext = out_ext[i];
    else out[i].own.assign((size_t)sh.num_elements() * 4, 0);
    *t = &out[i];
    return Status();
  }
  template <class D>
  const D& eigen_device() {
    static D d;
    return d;
  }
};

struct OpKernel {
  explicit OpKernel(OpKernelConstruction*) {}
  virtual void Compute(OpKernelContext*) = 0;
  virtual ~OpKernel() {}
};

#define OP_REQUIRES(ctx, cond, status) \
  do {                                 \
    if (!(cond)) {                     \
      (ctx)->st = (status);            \
      return;                          \
    }                                  \
  } while (0)
#define OP_REQUIRES_OK(ctx, expr)          \
  do {                                     \
    ::tensorflow::Status _s = (expr);      \
    if (!_s.ok()) {                        \
      (ctx)->st = _s;                      \
      return;                              \
    }                                      \
  } while (0)

static const char* const DEVICE_CPU = "CPU";

struct KernelKey {
  std::string name, dev, ty;
  KernelKey& Device(const char* d) { dev = d; return *this; }
  template <class T>
  KernelKey& TypeConstraint(const char*) {
    ty = std::is_floating_point<T>::value ? "float" : "int";
    return *this;
  }
};
inline KernelKey Name(const char* n) { KernelKey k; k.name = n; return k; }

typedef std::function<OpKernel*()> KernelFactory;
inline std::map<std::string, KernelFactory>& kernel_table() {
  static std::map<std::string, KernelFactory> t;
  return t;
}
struct KernelRegistrar {
  KernelRegistrar(const KernelKey& k, KernelFactory f) { kernel_table()[k.name + "/" + k.ty] = f; }
};
#define SNNTC_SHIM_CAT2(a, b) a##b
#define SNNTC_SHIM_CAT(a, b) SNNTC_SHIM_CAT2(a, b)
/* variadic: the registered class name contains a comma (Op<Device, T>) */
#define REGISTER_KERNEL_BUILDER(key, ...)                                             \
  static ::tensorflow::KernelRegistrar SNNTC_SHIM_CAT(snntc_shim_reg_, __COUNTER__)( \
      key, []() -> ::tensorflow::OpKernel* { return new __VA_ARGS__(nullptr); });

}  // namespace tensorflow
