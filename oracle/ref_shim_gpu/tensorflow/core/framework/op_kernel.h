/*
 * TEST INFRASTRUCTURE ONLY -- a stand-in for the part of the TensorFlow / Eigen GPU surface that the
 * reference GPU operators (snntc/snnfc_kernels.cu.cc, snnfcgrad_kernels.cu.cc, snncv_kernels.cu.cc,
 * snncvgrad_kernels.cu.cc) touch, so that those four files compile unmodified for sm_100a, from
 * where they lie, without TensorFlow. Tensors are views of device memory; the few Eigen tensor
 * expressions the functors assign (`generate`, `constant`, product of two leading-dimension slices,
 * `extract_image_patches(...VALID).reshape`) each become one small elementwise kernel on the
 * context's stream; `allocate_temp` carves from a caller-provided pool (TensorFlow's allocator is a
 * pool too) and only falls back to cudaMalloc when the pool is exhausted. Nothing here is part of
 * the product; it exists to time the reference's own GPU kernels on a B200 and to compare results.
 */
#pragma once
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <initializer_list>
#include <string>
#include <type_traits>
#include <vector>

#define EIGEN_DEVICE_FUNC __host__ __device__
#define EIGEN_STRONG_INLINE __forceinline__

namespace Eigen {
typedef long Index;
template <class T, size_t N>
struct array {
  T v[N];
  EIGEN_DEVICE_FUNC T& operator[](size_t i) { return v[i]; }
  EIGEN_DEVICE_FUNC const T& operator[](size_t i) const { return v[i]; }
};
enum PaddingType { PADDING_VALID = 1, PADDING_SAME = 2 };
struct ThreadPoolDevice {};
struct GpuDevice {
  cudaStream_t s = 0;
  cudaStream_t stream() const { return s; }
};
}  // namespace Eigen

namespace tensorflow {

typedef uint64_t uint64;
typedef int64_t int64;
typedef int32_t int32;
typedef int8_t int8;
enum DataType { DT_FLOAT, DT_INT32, DT_INT8 };

struct Status {
  int c = 0;
  bool ok() const { return c == 0; }
  int code() const { return c; }
};

struct TensorShape {
  std::vector<int64> d;
  TensorShape() {}
  TensorShape(std::initializer_list<int64> l) : d(l) {}
  int64 dim_size(int i) const { return d[i]; }
  void AddDim(int64 v) { d.push_back(v); }
  int64 num_elements() const {
    int64 n = 1;
    for (auto v : d) n *= v;
    return n;
  }
};

namespace shim {
// ---- the elementwise kernels behind the Eigen expressions
template <class F>
__global__ void generate_kernel(int* p, long n, F f) {
  long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
  if (i < n) {
    Eigen::array<int, 1> ix;
    ix[0] = (int)i;
    p[i] = f(ix);
  }
}
template <class T>
__global__ void fill_kernel(T* p, long n, T v) {
  long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
  if (i < n) p[i] = v;
}
template <class T>
__global__ void product_kernel(T* o, const T* a, const T* b, long n) {
  long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
  if (i < n) o[i] = a[i] * b[i];
}
// patches[(b,nh,nw), (kh,kw,c)] = in[b, nh*Sh+kh, nw*Sw+kw, c]  (VALID)
template <class T>
__global__ void patches_kernel(T* o, const T* in, int B, int H, int W, int C, int Nh, int Nw, int Kh, int Kw,
                               int Sh, int Sw) {
  long n = (long)B * Nh * Nw * Kh * Kw * C;
  long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
  if (i >= n) return;
  int c = (int)(i % C);
  long r = i / C;
  int kw = (int)(r % Kw); r /= Kw;
  int kh = (int)(r % Kh); r /= Kh;
  int nw = (int)(r % Nw); r /= Nw;
  int nh = (int)(r % Nh);
  int b = (int)(r / Nh);
  o[i] = in[(((long)b * H + nh * Sh + kh) * W + nw * Sw + kw) * C + c];
}
inline unsigned blocks_for(long n) { return (unsigned)((n + 255) / 256 > 0 ? (n + 255) / 256 : 1); }

template <class F> struct Gen { F f; };
template <class T> struct Const { T v; };
template <class T> struct Slice { const T* p; long n; };
template <class T> struct Product { Slice<T> a, b; };
template <class T>
Product<T> operator*(Slice<T> a, Slice<T> b) { return Product<T>{a, b}; }
template <class T, int N> struct Dims { long v[N]; };
template <class T>
struct Patches {
  const T* in;
  int B, H, W, C, Kw, Kh, Sw, Sh;
  template <class D> Patches reshape(const D&) const { return *this; }
};
template <class T, int N> struct View;
template <class T, int N>
struct Assign {
  View<T, N>* v;
  cudaStream_t s;
  template <class F> void operator=(Gen<F> g) {
    long n = v->n();
    generate_kernel<<<blocks_for(n), 256, 0, s>>>((int*)v->p, n, g.f);
  }
  void operator=(Const<T> c) {
    long n = v->n();
    fill_kernel<<<blocks_for(n), 256, 0, s>>>(v->p, n, c.v);
  }
  void operator=(Product<T> m) {
    long n = v->n();
    product_kernel<<<blocks_for(n), 256, 0, s>>>(v->p, m.a.p, m.b.p, n);
  }
  void operator=(Patches<T> q) {
    int Nh = (q.H - q.Kh) / q.Sh + 1, Nw = (q.W - q.Kw) / q.Sw + 1;
    long n = (long)q.B * Nh * Nw * q.Kh * q.Kw * q.C;
    patches_kernel<<<blocks_for(n), 256, 0, s>>>(v->p, q.in, q.B, q.H, q.W, q.C, Nh, Nw, q.Kh, q.Kw, q.Sh, q.Sw);
  }
};
template <class T, int N>
struct View {
  T* p;
  Dims<T, N> dm;
  long n() const {
    long r = 1;
    for (int i = 0; i < N; i++) r *= dm.v[i];
    return r;
  }
  T* data() const { return p; }
  const Dims<T, N>& dimensions() const { return dm; }
  Assign<T, N> device(const Eigen::GpuDevice& d) { return Assign<T, N>{this, d.stream()}; }
  template <class F> Gen<F> generate(F f) const { return Gen<F>{f}; }
  Const<T> constant(T v) const { return Const<T>{v}; }
  // only slices along the leading dimension are used by the reference (rows [0,B) and [B,2B))
  Slice<typename std::remove_const<T>::type> slice(const Eigen::array<Eigen::Index, N>& off,
                                                   const Eigen::array<Eigen::Index, N>& ext) const {
    long stride = 1;
    for (int i = 1; i < N; i++) stride *= dm.v[i];
    long cnt = 1;
    for (int i = 0; i < N; i++) cnt *= ext[i];
    return {p + off[0] * stride, cnt};
  }
  Patches<typename std::remove_const<T>::type> extract_image_patches(int Kw, int Kh, int Sw, int Sh, int, int,
                                                                     Eigen::PaddingType) const {
    return {p, (int)dm.v[0], (int)dm.v[1], (int)dm.v[2], (int)dm.v[3], Kw, Kh, Sw, Sh};
  }
};
}  // namespace shim

template <class V>
V To32Bit(V v) { return v; }

struct Tensor {
  TensorShape s;
  void* dev = nullptr;   // device memory, except for `params` which the op keeps in host memory
  const TensorShape& shape() const { return s; }
  int64 NumElements() const { return s.num_elements(); }
  template <class T>
  shim::View<T, 1> flat() const {
    shim::View<T, 1> v;
    v.p = (T*)dev;
    v.dm.v[0] = s.num_elements();
    return v;
  }
  template <class T, int N>
  shim::View<T, N> shaped(std::initializer_list<long> l) const {
    shim::View<T, N> v;
    v.p = (T*)dev;
    int i = 0;
    for (auto x : l) v.dm.v[i++] = x;
    return v;
  }
  template <class T, int N>
  shim::View<T, N> shaped(std::initializer_list<int> l) const {
    shim::View<T, N> v;
    v.p = (T*)dev;
    int i = 0;
    for (auto x : l) v.dm.v[i++] = x;
    return v;
  }
};

struct OpKernelContext {
  Eigen::GpuDevice gpu;
  char* pool = nullptr;          // caller-provided device scratch
  size_t pool_bytes = 0, pool_used = 0;
  std::vector<void*> overflow;   // cudaMalloc'ed when the pool ran out; released by the wrapper
  Status allocate_temp(DataType dt, const TensorShape& sh, Tensor* t) {
    t->s = sh;
    size_t b = (size_t)sh.num_elements() * (dt == DT_INT8 ? 1 : 4);
    b = (b + 255) & ~(size_t)255;
    if (b == 0) b = 256;
    Status st;
    if (pool && pool_used + b <= pool_bytes) {
      t->dev = pool + pool_used;
      pool_used += b;
    } else {
      st.c = (int)cudaMalloc(&t->dev, b);
      if (st.c == 0) overflow.push_back(t->dev);
    }
    return st;
  }
  template <class D>
  const D& eigen_device() { return gpu; }
};

}  // namespace tensorflow
