// SNN-TC backward (SnnFcGrad / SnnCvGrad) for sm_100a: threshold-masked reductions on FP32 CUDA cores.
//
//   u[r,j]  = y[r,j] fired ? grad[r,j] * inv[r,j] : 0                       (snnfcgrad_kernels.cu.cc:171-172)
//   dX[r,i] = sum_j [x_ri <= y_rj] u_rj W[i,j]                              (snnfcgrad_kernels.cu.cc:56-65)
//   dW[i,j] = sum_r [x_ri <= y_rj] (x_ri - y_rj) u_rj, bias row uses x=biasvolt (snnfcgrad_kernels.cu.cc:100-120)
//
// u is formed once per call by a small kernel. Both reductions are register-tiled like an SGEMM
// (dX: 64x64 CTA tile, 4x4 per thread; dW: 128x64, 8x4 per thread) with the predicate applied per element. The same two kernels serve the convolution: dX is tiled by INPUT pixel and loops over
// the Kh*Kw taps, gathering the covering receptive fields, so no atomics are needed (the reference
// scatters with atomicAdd, snncvgrad_kernels.cu.cc:83); dW gathers its x tile straight from the
// NHWC image. dW splits the row dimension over CTAs and a second kernel adds the partial tiles in a
// fixed order, so results are reproducible run to run.
#include "snntc_common.cuh"

#include <math_constants.h>
#include <math.h>
#include <type_traits>

namespace snntc {

namespace {

constexpr int kBwdThreads = 256;
constexpr int kTile = 64;       // CTA tile edge (rows x columns of the output)
constexpr int kJT = 16;         // reduction chunk of the dX kernel (outputs j per shared-memory tile)
constexpr int kJTP = kJT + 4;   // padded row stride: keeps float4 alignment, spreads rows over banks
constexpr int kRT = 16;         // reduction chunk of the dW kernel (rows r per shared-memory tile)
constexpr int kTileI = 128;     // dW output tile: 128 fan-in rows x 64 outputs, 8x4 per thread

// u[r,j] = fired ? grad[r,j] * inv[r,j] : 0, once per backward call (the reference does the same with an
// Eigen expression, snnfcgrad_kernels.cu.cc:156-173); both gradient kernels then read (y, u).
// Besides u, this kernel decides whether the dW kernel may use its scaled, saturating inner loop (see
// snn_dw_kernel): *exact_flag is raised when some value lies outside the range in which scaling by a power
// of two is exact and (y - x) * scale stays below 1 -- an input below -MAX, a non-zero input or spike value
// smaller than 2^-60 in magnitude, or a u that is not below 2^100 in magnitude (NaN and inf included).
// `xin` is the whole input tensor (nx elements). The flag must be zero before the launch.
template <bool V4>   // V4: n and nx are multiples of 4 and all pointers 16-byte aligned: 16-byte loads and stores
__global__ void snn_u_kernel(const float* __restrict__ grad, const float* __restrict__ out, float* __restrict__ u,
                             size_t n, float maxcomp, const float* __restrict__ xin, size_t nx, float maxv,
                             int* __restrict__ exact_flag, unsigned* __restrict__ nz_count) {
  const float tiny = 8.67361737988e-19f;   // 2^-60
  const float big = 1.26765060023e30f;     // 2^100
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t t0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  bool odd = false;
  unsigned nz = 0;           // outputs of this thread that carry a gradient (u != 0)
  auto one = [&](float y, float g, float inv) {
    const float uu = (y > maxcomp) ? 0.f : g * inv;
    nz += uu != 0.f;
    const float ya = fabsf(y);
    odd |= (ya > 0.f && ya < tiny) || !(fabsf(uu) < big);
    return uu;
  };
  auto scan = [&](float xv) {
    const float xa = fabsf(xv);
    odd |= (xv < -maxv) || (xa > 0.f && xa < tiny);
  };
  if (V4) {
    const float4* y4 = reinterpret_cast<const float4*>(out);
    const float4* i4 = reinterpret_cast<const float4*>(out + n);
    const float4* g4 = reinterpret_cast<const float4*>(grad);
    float4* u4 = reinterpret_cast<float4*>(u);
    for (size_t e = t0; e < n / 4; e += stride) {
      const float4 y = __ldg(y4 + e), g = __ldg(g4 + e), iv = __ldg(i4 + e);
      u4[e] = make_float4(one(y.x, g.x, iv.x), one(y.y, g.y, iv.y), one(y.z, g.z, iv.z), one(y.w, g.w, iv.w));
    }
    const float4* x4 = reinterpret_cast<const float4*>(xin);
    for (size_t e = t0; e < nx / 4; e += stride) {
      const float4 xv = __ldg(x4 + e);
      scan(xv.x); scan(xv.y); scan(xv.z); scan(xv.w);
    }
  } else {
    for (size_t e = t0; e < n; e += stride) u[e] = one(__ldg(out + e), __ldg(grad + e), __ldg(out + n + e));
    for (size_t e = t0; e < nx; e += stride) scan(__ldg(xin + e));
  }
  if (odd) *exact_flag = 1;
  if (nz_count != nullptr) {   // one atomic per warp: *nz_count = number of outputs with a gradient (zero before the launch)
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) nz += __shfl_xor_sync(0xffffffffu, nz, d);
    if ((threadIdx.x & 31) == 0 && nz != 0u) atomicAdd(nz_count, nz);
  }
}

// acc += [x <= y] * u * w as one compare and one predicated FMA
__device__ __forceinline__ void masked_fma(float& acc, float x, float y, float u, float w) {
  asm("{\n\t.reg .pred p;\n\tsetp.le.f32 p, %1, %2;\n\t@p fma.rn.f32 %0, %3, %4, %0;\n\t}"
      : "+f"(acc) : "f"(x), "f"(y), "f"(u), "f"(w));
}

// Two-lane FP32 arithmetic of sm_100 (one issue slot for two IEEE single-precision results; each lane
// rounds exactly like the scalar instruction). A pair lives in one 64-bit register: low word = lane 0.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

// ------------------------------------------------------------------------------------------- dX
// "Points" p are dense samples (taps = 1, CH = I) or input pixels (taps = Kh*Kw, CH = C). The
// reduction runs over tiles t = (tap, block of 16 outputs); the loads of tile t+1 are issued before
// the arithmetic of tile t and parked in registers, shared memory is double buffered.
template <bool VEC>   // VEC: J % 4 == 0, tiles are fetched with 16-byte loads
__global__ void __launch_bounds__(kBwdThreads)
snn_dx_kernel(const DxGate gate, const Geometry g, const float* __restrict__ uv, const float* __restrict__ x,
              const float* __restrict__ w, const float* __restrict__ out, float* __restrict__ dx) {
  if (gate.nz != nullptr && __ldg(gate.nz) <= gate.threshold) return;   // the list-walking kernel takes this call
  __shared__ __align__(16) float Ys[2][kTile * kJTP];
  __shared__ __align__(16) float Us[2][kTile * kJTP];
  __shared__ __align__(16) float Ws[2][kTile * kJTP];
  __shared__ int s_pb[kTile], s_ph[kTile], s_pw[kTile];

  const int J = g.J;
  const int CH = g.is_conv ? g.C : g.I;
  const int P = g.is_conv ? g.B * g.H * g.W : g.R;
  const int taps = g.is_conv ? g.Kh * g.Kw : 1;
  const int njt = (J + kJT - 1) / kJT;
  const int ntiles = taps * njt;
  const float* __restrict__ yv = out;

  const int tid = threadIdx.x;
  const int tr = tid >> 4, ti = tid & 15;
  const int p0 = blockIdx.x * kTile, c0 = blockIdx.y * kTile;

  if (tid < kTile) {
    const int p = p0 + tid;
    int pb = -1, ph = 0, pw = 0;
    if (p < P) {
      if (!g.is_conv) {
        pb = p;
      } else {
        const int ww = p % g.W;
        const int t = p / g.W;
        pb = t / g.H;
        ph = t % g.H + g.pad_top;
        pw = ww + g.pad_left;
      }
    }
    s_pb[tid] = pb; s_ph[tid] = ph; s_pw[tid] = pw;
  }

  float xr[4][4], acc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int p = p0 + tr + 16 * a, c = c0 + ti + 16 * b;
      xr[a][b] = (p < P && c < CH) ? __ldg(x + (size_t)p * CH + c) : CUDART_INF_F;
      acc[a][b] = 0.f;
    }
  __syncthreads();

  // tile loaders. Scalar form: 16 consecutive j per row, rows ld_row + 16q. Vector form: one float4 of
  // row (tid >> 2) at columns 4*(tid & 3) for each of y, u, w. The values are parked in registers and
  // nothing may touch them before the arithmetic below, or the loads stop overlapping it.
  const int ld_jj = VEC ? (tid & 3) * 4 : (tid & 15);
  const int ld_row = VEC ? (tid >> 2) : (tid >> 4);
  float py[4], pu[4], pwv[4];

  auto out_row = [&](int row, int kh, int kw) -> int {
    int orow = s_pb[row];
    if (g.is_conv && orow >= 0) {
      const int hh = s_ph[row] - kh, wq = s_pw[row] - kw;
      int nh = hh, nw = wq;
      bool ok = hh >= 0 && wq >= 0;
      if (g.Sh != 1 || g.Sw != 1) {
        nh = hh / g.Sh; nw = wq / g.Sw;
        ok = ok && nh * g.Sh == hh && nw * g.Sw == wq;
      }
      ok = ok && nh < g.Nh && nw < g.Nw;
      orow = ok ? (orow * g.Nh + nh) * g.Nw + nw : -1;
    }
    return orow;
  };
  auto fetch = [&](int t) {
    const int tap = t / njt;
    const int j = (t - tap * njt) * kJT + ld_jj;
    int kh = 0, kw = 0;
    if (g.is_conv) { kh = tap / g.Kw; kw = tap - kh * g.Kw; }
    if (VEC) {
      const int orow = out_row(ld_row, kh, kw);
      float4 y4 = make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
      float4 u4 = make_float4(0.f, 0.f, 0.f, 0.f), w4 = u4;
      if (orow >= 0 && j < J) {
        const size_t o = (size_t)orow * J + j;
        y4 = __ldg(reinterpret_cast<const float4*>(yv + o));
        u4 = __ldg(reinterpret_cast<const float4*>(uv + o));
      }
      const int c = c0 + ld_row;
      if (c < CH && j < J) w4 = __ldg(reinterpret_cast<const float4*>(w + ((size_t)tap * CH + c) * J + j));
      py[0] = y4.x; py[1] = y4.y; py[2] = y4.z; py[3] = y4.w;
      pu[0] = u4.x; pu[1] = u4.y; pu[2] = u4.z; pu[3] = u4.w;
      pwv[0] = w4.x; pwv[1] = w4.y; pwv[2] = w4.z; pwv[3] = w4.w;
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int row = ld_row + 16 * q;
        const int orow = out_row(row, kh, kw);
        float y = -CUDART_INF_F, u = 0.f, wv = 0.f;
        if (orow >= 0 && j < J) {
          const size_t o = (size_t)orow * J + j;
          y = __ldg(yv + o);
          u = __ldg(uv + o);
        }
        const int c = c0 + row;
        if (c < CH && j < J) wv = __ldg(w + ((size_t)tap * CH + c) * J + j);
        py[q] = y; pu[q] = u; pwv[q] = wv;
      }
    }
  };
  auto park = [&](int buf) {
    if (VEC) {
      *reinterpret_cast<float4*>(&Ys[buf][ld_row * kJTP + ld_jj]) = make_float4(py[0], py[1], py[2], py[3]);
      *reinterpret_cast<float4*>(&Us[buf][ld_row * kJTP + ld_jj]) = make_float4(pu[0], pu[1], pu[2], pu[3]);
      *reinterpret_cast<float4*>(&Ws[buf][ld_row * kJTP + ld_jj]) = make_float4(pwv[0], pwv[1], pwv[2], pwv[3]);
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int row = ld_row + 16 * q;
        Ys[buf][row * kJTP + ld_jj] = py[q];
        Us[buf][row * kJTP + ld_jj] = pu[q];
        Ws[buf][row * kJTP + ld_jj] = pwv[q];
      }
    }
  };

  fetch(0);
  park(0);
  __syncthreads();

  for (int t = 0; t < ntiles; ++t) {
    const int buf = t & 1;
    if (t + 1 < ntiles) fetch(t + 1);

#pragma unroll
    for (int j4 = 0; j4 < kJT; j4 += 4) {
      float4 y4[4], u4[4], w4[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        y4[a] = *reinterpret_cast<const float4*>(&Ys[buf][(tr + 16 * a) * kJTP + j4]);
        u4[a] = *reinterpret_cast<const float4*>(&Us[buf][(tr + 16 * a) * kJTP + j4]);
      }
#pragma unroll
      for (int b = 0; b < 4; ++b) w4[b] = *reinterpret_cast<const float4*>(&Ws[buf][(ti + 16 * b) * kJTP + j4]);
      // one output column at a time across all 16 accumulators: no back-to-back dependent FMAs
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) masked_fma(acc[a][b], xr[a][b], y4[a].x, u4[a].x, w4[b].x);
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) masked_fma(acc[a][b], xr[a][b], y4[a].y, u4[a].y, w4[b].y);
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) masked_fma(acc[a][b], xr[a][b], y4[a].z, u4[a].z, w4[b].z);
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) masked_fma(acc[a][b], xr[a][b], y4[a].w, u4[a].w, w4[b].w);
    }

    if (t + 1 < ntiles) park(buf ^ 1);
    __syncthreads();
  }

#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int p = p0 + tr + 16 * a, c = c0 + ti + 16 * b;
      if (p < P && c < CH) dx[(size_t)p * CH + c] = acc[a][b];
    }
}

// ------------------------------------------------------------------------------------------- dX, wide tile
// Same computation as snn_dx_kernel for J % 4 == 0, with a 128-point x 64-channel CTA tile and 8x4
// outputs per thread: 32 independent compare/FMA pairs per output column instead of 16, which is what
// hides the compare -> predicated-FMA latency at two CTAs per SM. Shared-memory tiles are stored
// transposed ([j][point], [j][channel]) so that a thread reads its 8 points / 4 channels with 16-byte loads.
constexpr int kWideP = 128;
constexpr int kYStride = kWideP + 4;
constexpr int kWStride = kTile + 4;

__global__ void __launch_bounds__(kBwdThreads)
snn_dx_wide_kernel(const DxGate gate, const Geometry g, const float* __restrict__ uv, const float* __restrict__ x,
                   const float* __restrict__ w, const float* __restrict__ out, float* __restrict__ dx) {
  if (gate.nz != nullptr && __ldg(gate.nz) <= gate.threshold) return;   // the list-walking kernel takes this call
  __shared__ __align__(16) float Ys[2][kJT * kYStride];
  __shared__ __align__(16) float Us[2][kJT * kYStride];
  __shared__ __align__(16) float Ws[2][kJT * kWStride];
  __shared__ int s_pb[kWideP], s_ph[kWideP], s_pw[kWideP];

  const int J = g.J;
  const int CH = g.is_conv ? g.C : g.I;
  const int P = g.is_conv ? g.B * g.H * g.W : g.R;
  const int taps = g.is_conv ? g.Kh * g.Kw : 1;
  const int njt = (J + kJT - 1) / kJT;
  const int ntiles = taps * njt;
  const float* __restrict__ yv = out;

  const int tid = threadIdx.x;
  const int tp = tid >> 4, tc = tid & 15;
  const int p0 = blockIdx.x * kWideP, c0 = blockIdx.y * kTile;

  if (tid < kWideP) {
    const int p = p0 + tid;
    int pb = -1, ph = 0, pw = 0;
    if (p < P) {
      if (!g.is_conv) {
        pb = p;
      } else {
        const int ww = p % g.W;
        const int t = p / g.W;
        pb = t / g.H;
        ph = t % g.H + g.pad_top;
        pw = ww + g.pad_left;
      }
    }
    s_pb[tid] = pb; s_ph[tid] = ph; s_pw[tid] = pw;
  }

  float xr[8][4], acc[8][4];
#pragma unroll
  for (int a = 0; a < 8; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int p = p0 + 8 * tp + a, c = c0 + 4 * tc + b;
      xr[a][b] = (p < P && c < CH) ? __ldg(x + (size_t)p * CH + c) : CUDART_INF_F;
      acc[a][b] = 0.f;
    }
  __syncthreads();

  // loaders: y/u -> rows (tid >> 2) and (tid >> 2) + 64, columns 4*(tid & 3); w -> channel row (tid >> 2)
  const int ld_jj = (tid & 3) * 4, ld_row = tid >> 2;
  float4 py[2], pu[2], pwv;

  auto out_row = [&](int row, int kh, int kw) -> int {
    int orow = s_pb[row];
    if (g.is_conv && orow >= 0) {
      const int hh = s_ph[row] - kh, wq = s_pw[row] - kw;
      int nh = hh, nw = wq;
      bool ok = hh >= 0 && wq >= 0;
      if (g.Sh != 1 || g.Sw != 1) {
        nh = hh / g.Sh; nw = wq / g.Sw;
        ok = ok && nh * g.Sh == hh && nw * g.Sw == wq;
      }
      ok = ok && nh < g.Nh && nw < g.Nw;
      orow = ok ? (orow * g.Nh + nh) * g.Nw + nw : -1;
    }
    return orow;
  };
  auto fetch = [&](int t) {
    const int tap = t / njt;
    const int j = (t - tap * njt) * kJT + ld_jj;
    int kh = 0, kw = 0;
    if (g.is_conv) { kh = tap / g.Kw; kw = tap - kh * g.Kw; }
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int orow = out_row(ld_row + 64 * q, kh, kw);
      py[q] = make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
      pu[q] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (orow >= 0 && j < J) {
        const size_t o = (size_t)orow * J + j;
        py[q] = __ldg(reinterpret_cast<const float4*>(yv + o));
        pu[q] = __ldg(reinterpret_cast<const float4*>(uv + o));
      }
    }
    pwv = make_float4(0.f, 0.f, 0.f, 0.f);
    const int c = c0 + ld_row;
    if (c < CH && j < J) pwv = __ldg(reinterpret_cast<const float4*>(w + ((size_t)tap * CH + c) * J + j));
  };
  auto park = [&](int buf) {
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int row = ld_row + 64 * q;
      Ys[buf][(ld_jj + 0) * kYStride + row] = py[q].x; Us[buf][(ld_jj + 0) * kYStride + row] = pu[q].x;
      Ys[buf][(ld_jj + 1) * kYStride + row] = py[q].y; Us[buf][(ld_jj + 1) * kYStride + row] = pu[q].y;
      Ys[buf][(ld_jj + 2) * kYStride + row] = py[q].z; Us[buf][(ld_jj + 2) * kYStride + row] = pu[q].z;
      Ys[buf][(ld_jj + 3) * kYStride + row] = py[q].w; Us[buf][(ld_jj + 3) * kYStride + row] = pu[q].w;
    }
    Ws[buf][(ld_jj + 0) * kWStride + ld_row] = pwv.x;
    Ws[buf][(ld_jj + 1) * kWStride + ld_row] = pwv.y;
    Ws[buf][(ld_jj + 2) * kWStride + ld_row] = pwv.z;
    Ws[buf][(ld_jj + 3) * kWStride + ld_row] = pwv.w;
  };

  fetch(0);
  park(0);
  __syncthreads();

  for (int t = 0; t < ntiles; ++t) {
    const int buf = t & 1;
    if (t + 1 < ntiles) fetch(t + 1);

#pragma unroll
    for (int jj = 0; jj < kJT; ++jj) {
      const float4 ya = *reinterpret_cast<const float4*>(&Ys[buf][jj * kYStride + 8 * tp]);
      const float4 yb = *reinterpret_cast<const float4*>(&Ys[buf][jj * kYStride + 8 * tp + 4]);
      const float4 ua = *reinterpret_cast<const float4*>(&Us[buf][jj * kYStride + 8 * tp]);
      const float4 ub = *reinterpret_cast<const float4*>(&Us[buf][jj * kYStride + 8 * tp + 4]);
      const float4 w4 = *reinterpret_cast<const float4*>(&Ws[buf][jj * kWStride + 4 * tc]);
      const float y8[8] = {ya.x, ya.y, ya.z, ya.w, yb.x, yb.y, yb.z, yb.w};
      const float u8[8] = {ua.x, ua.y, ua.z, ua.w, ub.x, ub.y, ub.z, ub.w};
      const float wv[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
      for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) masked_fma(acc[a][b], xr[a][b], y8[a], u8[a], wv[b]);
    }

    if (t + 1 < ntiles) park(buf ^ 1);
    __syncthreads();
  }

#pragma unroll
  for (int a = 0; a < 8; ++a) {
    const int p = p0 + 8 * tp + a, c = c0 + 4 * tc;
    if (p < P) {
      if (c + 3 < CH && (CH & 3) == 0) {
        *reinterpret_cast<float4*>(dx + (size_t)p * CH + c) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
      } else {
#pragma unroll
        for (int b = 0; b < 4; ++b)
          if (c + b < CH) dx[(size_t)p * CH + c + b] = acc[a][b];
      }
    }
  }
}

// ------------------------------------------------------------------------------------------- dW
// Output tile 128 (fan-in rows i, bias row included) x 64 (outputs j), 8x4 per thread; blockIdx.z
// selects a slice of the rows r. partial = dw when gridDim.z == 1, else the slice's own [Itot,J] plane
// of the workspace. Same software pipeline as dX: the next 16 rows are loaded into registers while the
// current 16 are being reduced out of (double-buffered) shared memory.
//
// Per element the sum takes [x<=y]*(x-y)*u = relu(y-x)*(-u). With s a power of two such that (y-x)*s < 1
// for every pair that can occur, relu((y-x)*s) is ONE saturating add of the pre-scaled tiles, y*s + (-x*s)
// clamped to [0,1], and the product with -u/s is the same real number as before, so the fused multiply-add
// rounds to the same bits: one FADD.SAT per element plus one two-lane FMA per two elements, nothing on the
// half-rate compare/min pipe. Scaling by s is exact unless it underflows, and the bound on (y-x) needs
// x >= -MAX; snn_u_kernel checks the ranges of the call's tensors and raises *exact_flag otherwise, in
// which case the tiles stay unscaled (s = 1) and the clamp is an explicit max(., 0).
__device__ __forceinline__ float add_sat(float a, float b) {
  float r;
  asm("add.rn.sat.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

template <bool VEC>   // VEC: J % 4 == 0, the y/u tiles are fetched with 16-byte loads
__global__ void __launch_bounds__(kBwdThreads, 3)
snn_dw_kernel(const Geometry g, const float* __restrict__ uv, const float* __restrict__ x,
              const float* __restrict__ out, float* __restrict__ partial, int rows_per_split,
              float scale, const int* __restrict__ exact_flag) {
  // -x*s, y*s and -u/s as plain tiles. A two-lane FMA covers two neighbouring output columns of one fan-in row,
  // so its 64-bit operands are pairs of neighbouring columns straight out of a 16-byte read of the u tile.
  __shared__ __align__(16) float Xs[2][kRT * kTileI];
  __shared__ __align__(16) float Ys[2][kRT * kTile];
  __shared__ __align__(16) float Us[2][kRT * kTile];

  const int J = g.J, I = g.I, R = g.R;
  const int Itot = I + g.has_bias;
  const float* __restrict__ yv = out;
  const bool fast = scale != 1.0f && __ldg(exact_flag) == 0;
  const float sc = fast ? scale : 1.0f;     // s
  const float nsc = -sc;                    // -s
  const float nusc = fast ? -1.0f / scale : -1.0f;   // -1/s, exact: s is a power of two

  const int tid = threadIdx.x;
  const int ti = tid >> 4, tj = tid & 15;
  const int i0 = blockIdx.y * kTileI, j0 = blockIdx.x * kTile;
  const int r_begin = blockIdx.z * rows_per_split;
  const int r_end = min(R, r_begin + rows_per_split);

  // loader roles: x -> column (tid & 127), rows (tid >> 7) + 2q, q < 8; y/u -> column (tid & 63), rows (tid >> 6) + 4q, q < 4
  const int lx_c = tid & (kTileI - 1), lx_r = tid >> 7;
  const int ly_c = VEC ? (tid & 15) * 4 : (tid & (kTile - 1));
  const int ly_r = VEC ? (tid >> 4) : (tid >> 6);
  const int li = i0 + lx_c;   // fan-in index this thread loads
  const int lj = j0 + ly_c;   // output index this thread loads
  // conv: this loader's column is one tap (kh, kw, c) of the receptive field, the same for every row; where a
  // row's receptive field starts (element offset of its top-left input pixel, which may lie outside the image,
  // and that pixel's h, w) is worked out once per row by 16 threads, two tiles ahead, into rowinfo
  int l_kh = 0, l_kw = 0, l_off = 0;
  if (g.is_conv && li < I) {
    const int tap = li / g.C;
    const int c = li - tap * g.C;
    l_kh = tap / g.Kw;
    l_kw = tap - l_kh * g.Kw;
    l_off = (l_kh * g.W + l_kw) * g.C + c;
  }
  __shared__ int4 rowinfo[2][kRT];   // .x element offset of the top-left pixel, .y its h, .z its w
  auto fill_rowinfo = [&](int buf, int rb) {
    if (g.is_conv && tid < kRT) {
      const int r = rb + tid;
      int4 ri = make_int4(0, -(1 << 24), -(1 << 24), 0);   // rows past the slice: every tap reads as outside
      if (r < r_end) {
        const int nw = r % g.Nw;
        const int t = r / g.Nw;
        const int nh = t % g.Nh;
        const int b = t / g.Nh;
        ri.y = nh * g.Sh - g.pad_top;
        ri.z = nw * g.Sw - g.pad_left;
        ri.x = ((b * g.H + ri.y) * g.W + ri.z) * g.C;
      }
      rowinfo[buf][tid] = ri;
    }
  };

  float px[kRT / 2], py[kRT / 4], pu[kRT / 4];  // parked untouched until after the arithmetic, see dX
  auto fetch = [&](int rb, int ibuf) {
#pragma unroll
    for (int q = 0; q < kRT / 2; ++q) {
      const int rl = lx_r + 2 * q;
      const int r = rb + rl;
      // padding of the tile: x=+inf, y=0, u=0 gives relu(y-x) = 0 and a zero product (never inf-inf).
      // The loaded value must not be touched here (not even by a select): it is still in flight.
      float xv = (li == I && g.has_bias && r < r_end) ? g.biasvolt : CUDART_INF_F;
      if (!g.is_conv) {
        if (r < r_end && li < I) xv = __ldg(x + (size_t)r * I + li);
      } else {
        const int4 ri = rowinfo[ibuf][rl];
        const bool ok = li < I && (unsigned)(ri.y + l_kh) < (unsigned)g.H && (unsigned)(ri.z + l_kw) < (unsigned)g.W;
        if (ok) xv = __ldg(x + (ptrdiff_t)ri.x + l_off);
      }
      px[q] = xv;
    }
    if (VEC) {
      const int r = rb + ly_r;
      float4 y4 = make_float4(0.f, 0.f, 0.f, 0.f), u4 = y4;
      if (r < r_end && lj < J) {
        const size_t o = (size_t)r * J + lj;
        y4 = __ldg(reinterpret_cast<const float4*>(yv + o));
        u4 = __ldg(reinterpret_cast<const float4*>(uv + o));
      }
      py[0] = y4.x; py[1] = y4.y; py[2] = y4.z; py[3] = y4.w;
      pu[0] = u4.x; pu[1] = u4.y; pu[2] = u4.z; pu[3] = u4.w;
    } else {
#pragma unroll
      for (int q = 0; q < kRT / 4; ++q) {
        const int r = rb + ly_r + 4 * q;
        float y = 0.f, u = 0.f;
        if (r < r_end && lj < J) {
          const size_t o = (size_t)r * J + lj;
          y = __ldg(yv + o);
          u = __ldg(uv + o);
        }
        py[q] = y; pu[q] = u;
      }
    }
  };
  auto park = [&](int buf) {
#pragma unroll
    for (int q = 0; q < kRT / 2; ++q) Xs[buf][(lx_r + 2 * q) * kTileI + lx_c] = px[q] * nsc;
    if (VEC) {
      *reinterpret_cast<float4*>(&Ys[buf][ly_r * kTile + ly_c]) =
          make_float4(py[0] * sc, py[1] * sc, py[2] * sc, py[3] * sc);
      *reinterpret_cast<float4*>(&Us[buf][ly_r * kTile + ly_c]) =
          make_float4(pu[0] * nusc, pu[1] * nusc, pu[2] * nusc, pu[3] * nusc);
    } else {
#pragma unroll
      for (int q = 0; q < kRT / 4; ++q) {
        Ys[buf][(ly_r + 4 * q) * kTile + ly_c] = py[q] * sc;
        Us[buf][(ly_r + 4 * q) * kTile + ly_c] = pu[q] * nusc;
      }
    }
  };

  // acc[a][b2] holds the sums of fan-in row 8*ti + a and output columns 4*tj + 2*b2, +1 as one 64-bit pair
  uint64_t acc[8][2];
#pragma unroll
  for (int a = 0; a < 8; ++a)
#pragma unroll
    for (int b = 0; b < 2; ++b) acc[a][b] = pack2(0.f, 0.f);

  // 16 rows out of shared memory; FAST: the clamp is the saturation of the add
  auto reduce_tile = [&](int buf, auto fast_c) {
    constexpr bool FAST = decltype(fast_c)::value;
#pragma unroll
    for (int rr = 0; rr < kRT; ++rr) {
      const float4 xa4 = *reinterpret_cast<const float4*>(&Xs[buf][rr * kTileI + 8 * ti]);
      const float4 xb4 = *reinterpret_cast<const float4*>(&Xs[buf][rr * kTileI + 8 * ti + 4]);
      const float4 y4 = *reinterpret_cast<const float4*>(&Ys[buf][rr * kTile + 4 * tj]);
      const ulonglong2 u4 = *reinterpret_cast<const ulonglong2*>(&Us[buf][rr * kTile + 4 * tj]);
      const float nx[8] = {xa4.x, xa4.y, xa4.z, xa4.w, xb4.x, xb4.y, xb4.z, xb4.w};
      const float ys[4] = {y4.x, y4.y, y4.z, y4.w};
      const uint64_t nu2[2] = {u4.x, u4.y};
#pragma unroll
      for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          float t0, t1;
          if (FAST) {
            t0 = add_sat(ys[2 * b], nx[a]);
            t1 = add_sat(ys[2 * b + 1], nx[a]);
          } else {
            t0 = fmaxf(ys[2 * b] + nx[a], 0.f);
            t1 = fmaxf(ys[2 * b + 1] + nx[a], 0.f);
          }
          acc[a][b] = fma2(pack2(t0, t1), nu2[b], acc[a][b]);
        }
    }
  };

  fill_rowinfo(0, r_begin);
  fill_rowinfo(1, r_begin + kRT);
  __syncthreads();
  if (r_begin < r_end) {
    fetch(r_begin, 0);
    park(0);
  }
  __syncthreads();

  int it = 0;
  for (int rb = r_begin; rb < r_end; rb += kRT, ++it) {
    const int buf = it & 1;
    const bool more = rb + kRT < r_end;
    if (more) fetch(rb + kRT, buf ^ 1);
    if (fast) reduce_tile(buf, std::true_type{});
    else reduce_tile(buf, std::false_type{});
    if (more) park(buf ^ 1);
    fill_rowinfo(buf, rb + 2 * kRT);   // this tile's entry was last read one iteration ago
    __syncthreads();
  }

  float* __restrict__ dst = partial + (size_t)blockIdx.z * Itot * J;
#pragma unroll
  for (int a = 0; a < 8; ++a)
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      float lo, hi;
      unpack2(acc[a][b], lo, hi);
      const int i = i0 + 8 * ti + a, j = j0 + 4 * tj + 2 * b;
      if (i < Itot && j < J) dst[(size_t)i * J + j] = lo;
      if (i < Itot && j + 1 < J) dst[(size_t)i * J + j + 1] = hi;
    }
}

// ------------------------------------------------------------------------------------------- dW, small fan-in
// At most 32 weight rows (the first convolution of an image network: 3x3x3 + bias = 28): the 128-row tile of
// snn_dw_kernel would be three quarters padding. Here lane i of every warp owns weight row i and warp w the JB
// outputs w*JB .. w*JB+JB-1 (J = 8*JB), accumulators in registers; a CTA walks a slice of the rows r, a stage of
// 4096/J rows at a time through shared memory (u and y tiles copied whole, the inputs gathered a warp per row).
// Whether output (r,j) carries a gradient is the same question for all lanes, so rows without one are skipped by
// a warp-uniform branch. Same arithmetic per element as the other dW kernels (saturating FMA of the scaled difference, FMA with
// -u/s), same exactness rule.
__device__ __forceinline__ float fma_sat(float a, float b, float c) {
  float r;
  asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

template <int JB>
__global__ void __launch_bounds__(kBwdThreads)
snn_dw_small_kernel(const Geometry g, const float* __restrict__ uv, const float* __restrict__ x,
                    const float* __restrict__ out, float* __restrict__ partial, int rows_per_split,
                    float scale, const int* __restrict__ exact_flag) {
  constexpr int JJ = 8 * JB;              // fan-out
  constexpr int RS = 4096 / JJ < 64 ? 4096 / JJ : 64;   // rows r per stage: the u and y tiles are at most 16 KB each
  __shared__ __align__(16) float Us[RS * JJ];
  __shared__ __align__(16) float Ys[RS * JJ];
  __shared__ float Xs[RS * 32];
  __shared__ int4 rowinfo[RS];            // .x element offset of the row's top-left pixel, .y its h, .z its w, .w row valid
  const int I = g.I, R = g.R;
  const int Itot = I + g.has_bias;
  const bool fast = scale != 1.0f && __ldg(exact_flag) == 0;
  const float sc = fast ? scale : 1.0f;
  const float nsc = -sc;
  const float nusc = fast ? -1.0f / scale : -1.0f;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int j0 = warp * JB;
  const int r_begin = blockIdx.z * rows_per_split;
  const int r_end = min(R, r_begin + rows_per_split);
  // this lane's input: tap (kh, kw, c) of the receptive field, or the bias input, or nothing
  int l_kh = 0, l_kw = 0, l_off = 0;
  if (g.is_conv && lane < I) {
    const int tap = lane / g.C, c = lane - tap * g.C;
    l_kh = tap / g.Kw;
    l_kw = tap - l_kh * g.Kw;
    l_off = (l_kh * g.W + l_kw) * g.C + c;
  }
  float acc[JB];
#pragma unroll
  for (int q = 0; q < JB; ++q) acc[q] = 0.f;

  for (int rb = r_begin; rb < r_end; rb += RS) {
    // ---- tiles of this stage: u and y are RS whole rows, contiguous in memory; x is gathered
    const float4* u4g = reinterpret_cast<const float4*>(uv + (size_t)rb * JJ);
    const float4* y4g = reinterpret_cast<const float4*>(out + (size_t)rb * JJ);
    const int valid4 = min(RS, r_end - rb) * (JJ / 4);   // 16-byte chunks that belong to rows of this slice
#pragma unroll
    for (int n = 0; n < (RS * JJ / 4) / kBwdThreads; ++n) {
      const int e = tid + kBwdThreads * n;
      float4 u = make_float4(0.f, 0.f, 0.f, 0.f), y = u;
      if (e < valid4) { u = __ldg(u4g + e); y = __ldg(y4g + e); }
      reinterpret_cast<float4*>(Us)[e] = u;
      reinterpret_cast<float4*>(Ys)[e] = y;
    }
    if (g.is_conv && tid < RS) {
      const int r = rb + tid;
      int4 ri = make_int4(0, 0, 0, 0);
      if (r < r_end) {
        const int nw = r % g.Nw;
        const int t = r / g.Nw;
        const int nh = t % g.Nh;
        const int b = t / g.Nh;
        ri.y = nh * g.Sh - g.pad_top;
        ri.z = nw * g.Sw - g.pad_left;
        ri.x = ((b * g.H + ri.y) * g.W + ri.z) * g.C;
        ri.w = 1;
      }
      rowinfo[tid] = ri;
    }
    __syncthreads();
#pragma unroll
    for (int n = 0; n < (RS * 32) / kBwdThreads; ++n) {
      const int rl = warp + (kBwdThreads / 32) * n;    // a warp per row, lane = weight row
      const int r = rb + rl;
      float xv = g.maxv;    // a lane without an input, a row past the slice, a tap outside the image: never spikes
      if (r < r_end) {
        if (lane == I && g.has_bias) {
          xv = g.biasvolt;
        } else if (lane < I) {
          if (!g.is_conv) {
            xv = __ldg(x + (size_t)r * I + lane);
          } else {
            const int4 ri = rowinfo[rl];
            if ((unsigned)(ri.y + l_kh) < (unsigned)g.H && (unsigned)(ri.z + l_kw) < (unsigned)g.W)
              xv = __ldg(x + (ptrdiff_t)ri.x + l_off);
          }
        }
      }
      Xs[rl * 32 + lane] = xv;
    }
    __syncthreads();
    // ---- this warp's JB outputs against all rows of the stage
#pragma unroll 2
    for (int rl = 0; rl < RS; ++rl) {
      float4 u4[JB / 4];
      bool any = false;
#pragma unroll
      for (int q = 0; q < JB / 4; ++q) {
        u4[q] = *reinterpret_cast<const float4*>(Us + rl * JJ + j0 + 4 * q);
        any |= (u4[q].x != 0.f) | (u4[q].y != 0.f) | (u4[q].z != 0.f) | (u4[q].w != 0.f);
      }
      if (!any) continue;   // warp-uniform: every lane read the same values
      const float xv = Xs[rl * 32 + lane];
#pragma unroll
      for (int q = 0; q < JB / 4; ++q) {
        const float uu[4] = {u4[q].x, u4[q].y, u4[q].z, u4[q].w};
        if (uu[0] == 0.f && uu[1] == 0.f && uu[2] == 0.f && uu[3] == 0.f) continue;
        const float4 y4 = *reinterpret_cast<const float4*>(Ys + rl * JJ + j0 + 4 * q);
        const float yy[4] = {y4.x, y4.y, y4.z, y4.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          // (a zero u adds +-0: no need to branch inside a group of four)
          const float t = fast ? fma_sat(xv, nsc, yy[k] * sc) : fmaxf(yy[k] - xv, 0.f);
          acc[4 * q + k] = fmaf(t, uu[k] * nusc, acc[4 * q + k]);
        }
      }
    }
    __syncthreads();   // the tiles are overwritten by the next stage
  }
  if (lane < Itot) {
    float* dst = partial + (size_t)blockIdx.z * Itot * JJ + (size_t)lane * JJ + j0;
#pragma unroll
    for (int q = 0; q < JB; ++q) dst[q] = acc[q];
  }
}

static bool dw_small_ok(const Geometry& g, const float* uv, const float* out) {
  const int Itot = g.I + g.has_bias;
  if (Itot > 32 || g.R < 4096) return false;
  if (g.J != 32 && g.J != 64 && g.J != 128 && g.J != 256) return false;
  if (g.is_conv && (long long)g.B * g.H * g.W * g.C > 0x7fffffffLL) return false;
  return (((uintptr_t)uv | (uintptr_t)out) & 15) == 0;
}
static int dw_small_splits(const Geometry& g, const LaunchInfo& li, int* rows_per_split) {
  long want = 4L * li.num_sms;
  const long max_splits = ((long)g.R + 63) / 64;
  if (want > max_splits) want = max_splits;
  if (want < 1) want = 1;
  const long rps = ((long)g.R + want - 1) / want;
  *rows_per_split = (int)rps;
  return (int)(((long)g.R + rps - 1) / rps);
}

// Adds the partial planes of every element in a fixed order (four interleaved running sums, then their sum): the
// same bits every run, and eight independent loads in flight per thread -- a kernel with a few ten thousand
// threads and hundreds of planes is bound by load latency otherwise.
__global__ void snn_dw_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw, size_t n, int splits) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    int k = 0;
    for (; k + 8 <= splits; k += 8) {
      float v[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) v[q] = __ldcs(partial + (size_t)(k + q) * n + e);
      s0 += v[0]; s1 += v[1]; s2 += v[2]; s3 += v[3];
      s0 += v[4]; s1 += v[5]; s2 += v[6]; s3 += v[7];
    }
    for (; k < splits; ++k) s0 += __ldcs(partial + (size_t)k * n + e);
    dw[e] = (s0 + s1) + (s2 + s3);
  }
}

struct DwPlan { int splits; int rows_per_split; };

DwPlan plan_dw(const Geometry& g, const LaunchInfo& li) {
  const int Itot = g.I + g.has_bias;
  const long tiles = (long)((Itot + kTileI - 1) / kTileI) * ((g.J + kTile - 1) / kTile);
  long want = (3L * li.num_sms + tiles - 1) / tiles;
  long max_splits = ((long)g.R + 4 * kRT - 1) / (4 * kRT);
  if (want > max_splits) want = max_splits;
  if (want > 256) want = 256;
  if (want < 1) want = 1;
  long rps = ((long)g.R + want - 1) / want;
  rps = (rps + kRT - 1) / kRT * kRT;
  DwPlan p;
  p.rows_per_split = (int)rps;
  p.splits = (int)(((long)g.R + rps - 1) / rps);
  return p;
}

}  // namespace

static size_t u_bytes(const Geometry& g) { return (((size_t)g.R * g.J * sizeof(float)) + 255) & ~(size_t)255; }
constexpr size_t kFlagBytes = 256;

// The power of two s with 2*MAX*s <= 1/2 (so that (y - x)*s < 1 whenever y <= MAX and x >= -MAX), or 1 when
// MAX or the bias input are outside the range in which the scaled inner loop of the dW kernels is exact: with
// MAX <= 2^24, s >= 2^-27, so that -u/s stays finite for |u| < 2^100 and y*s, x*s stay normal numbers for
// magnitudes down to 2^-60 (the bounds snn_u_kernel checks on the tensors).
static float dw_scale(const Geometry& g) {
  if (!(g.maxv > 0.f) || !(g.maxv <= 16777216.0f)) return 1.0f;
  if (g.has_bias) {
    const float ba = fabsf(g.biasvolt);
    if (g.biasvolt < -g.maxv || (ba > 0.f && ba < 8.67361737988e-19f)) return 1.0f;
  }
  int e = 0;
  frexpf(g.maxv, &e);            // maxv = m * 2^e, m in [0.5, 1)  =>  maxv < 2^e
  return ldexpf(1.0f, -(e + 2));  // 2*maxv*s < 2^(e+1) * 2^-(e+2) = 1/2
}

// Where the row-skipping dW kernel is used: conv layers it supports with enough rows and fan-in to fill its tiles.
static bool want_dw_skip(const Geometry& g, const Options& opt) {
  if (opt.dw_kernel == 1) return false;
  if (!g.is_conv || (g.C & 3) != 0 || (g.J & 3) != 0) return false;
  if (opt.dw_kernel >= 2) return true;
  return g.R >= 2048 && g.I >= 128;
}

// Where the sparse dX kernel is used: conv layers it supports with enough receptive fields to be worth three launches.
static bool want_dx_sparse(const Geometry& g, const Options& opt) {
  if (opt.dx_kernel == 1 || !dx_sparse_shape_ok(g)) return false;
  if (opt.dx_kernel == 2) return true;
  return g.R >= 2048 && g.J >= 32;
}

// workspace = u[R,J] | 256 bytes with the range flag of snn_u_kernel | the partial dW planes (sized for whichever dW
// kernel needs more; none when neither splits the rows) | the scratch of the sparse dX kernel (conv layers it supports)
struct BackwardLayout { size_t flag, planes, dx_scratch, total; };
static BackwardLayout backward_layout(const Geometry& g, const LaunchInfo& li) {
  const size_t plane = (size_t)(g.I + g.has_bias) * (size_t)g.J * sizeof(float);
  const DwPlan p = plan_dw(g, li);
  size_t part = p.splits <= 1 ? 0 : (size_t)p.splits * plane;
  Options any;
  any.dw_kernel = 2;
  any.dx_kernel = 2;
  if (want_dw_skip(g, any)) {   // which dW kernel runs also depends on pointer alignment: sized for either
    int rps = 0;
    const size_t skip = (size_t)dw_skip_splits(g, li, &rps) * plane;
    if (skip > part) part = skip;
    if (dw_tma_shape_ok(g)) {
      const size_t tma = (size_t)dw_tma_splits(g, li, &rps) * plane;
      if (tma > part) part = tma;
    }
  }
  if (g.I + g.has_bias <= 32 && g.R >= 4096) {   // the small fan-in kernel
    int rps = 0;
    const size_t small = (size_t)dw_small_splits(g, li, &rps) * plane;
    if (small > part) part = small;
  }
  BackwardLayout l;
  l.flag = u_bytes(g);
  l.planes = l.flag + kFlagBytes;
  l.dx_scratch = l.planes + ((part + 255) & ~(size_t)255);
  l.total = l.dx_scratch + (want_dx_sparse(g, any) ? dx_sparse_bytes(g) : 0);
  return l;
}

size_t backward_workspace_bytes(const Geometry& g, const LaunchInfo& li) { return backward_layout(g, li).total; }

int launch_backward(const Geometry& g, const float* grad, const float* x, const float* w, const float* out,
                    float* dx, float* dw, void* ws, size_t ws_bytes, const LaunchInfo& li, const Options& opt,
                    cudaStream_t s) {
  const int Itot = g.I + g.has_bias;
  const int parts = opt.backward_parts;
  const BackwardLayout lay = backward_layout(g, li);
  if (!ws || ws_bytes < lay.total) return E_WORKSPACE;
  float* uv = static_cast<float*>(ws);
  int* exact_flag = reinterpret_cast<int*>(static_cast<unsigned char*>(ws) + lay.flag);
  unsigned* nz_count = reinterpret_cast<unsigned*>(exact_flag + 1);   // outputs with a gradient, counted by snn_u_kernel
  float* planes = reinterpret_cast<float*>(static_cast<unsigned char*>(ws) + lay.planes);
  void* dx_scratch = static_cast<unsigned char*>(ws) + lay.dx_scratch;
  // 16-byte tile loads need J % 4 == 0 and 16-byte aligned bases (rows then start aligned too)
  const bool vec = (g.J % 4 == 0) && (((uintptr_t)out | (uintptr_t)w | (uintptr_t)uv) & 15) == 0 &&
                   (((size_t)g.R * g.J) % 4 == 0);
  {
    const size_t n = (size_t)g.R * g.J;
    size_t blocks = (n + 255) / 256;
    if (blocks > (size_t)li.num_sms * 8) blocks = (size_t)li.num_sms * 8;
    if (cudaMemsetAsync(exact_flag, 0, 2 * sizeof(int), s) != cudaSuccess) return E_CUDA;   // the flag and the counter behind it
    const size_t nx = g.is_conv ? (size_t)g.B * g.H * g.W * g.C : (size_t)g.R * g.I;
    const bool v4 = (n % 4 == 0) && (nx % 4 == 0) &&
                    (((uintptr_t)grad | (uintptr_t)out | (uintptr_t)uv | (uintptr_t)x) & 15) == 0;
    if (v4) snn_u_kernel<true><<<(int)blocks, 256, 0, s>>>(grad, out, uv, n, g.maxv - 0.1f, x, nx, g.maxv, exact_flag, nz_count);
    else snn_u_kernel<false><<<(int)blocks, 256, 0, s>>>(grad, out, uv, n, g.maxv - 0.1f, x, nx, g.maxv, exact_flag, nz_count);
    count_launch();
    if (cudaGetLastError() != cudaSuccess) return E_CUDA;
  }
  // dX and dW only share read-only inputs: run dX on an auxiliary stream beside dW when both are wanted
  AuxSlot* aux = (dx && parts == 3 && (long)g.R * g.J >= 65536) ? aux_acquire(opt.overlap) : nullptr;
  cudaStream_t sdx = s;
  if (aux) {
    if (aux_fork(aux, s) != cudaSuccess) return E_CUDA;
    sdx = aux->stream;
  }
  int rc = OK;
  if (dx && (parts & 1)) {
    const int CH = g.is_conv ? g.C : g.I;
    const long P = g.is_conv ? (long)g.B * g.H * g.W : g.R;
    dim3 grid((unsigned)((P + kTile - 1) / kTile), (CH + kTile - 1) / kTile);
    // Conv layers the list-walking kernel supports: with dx_kernel 0 both kernels are queued and the device picks
    // (DxGate: the list-walking one up to 40 % of the outputs carrying a gradient -- its time grows with that share,
    // the dense tile's does not; they cross near 41 % on the benchmark layers); 1 / 2 name one.
    const bool sparse_ok = want_dx_sparse(g, opt) && dx_sparse_supported(g, x, dx);
    const bool both = sparse_ok && opt.dx_kernel == 0;
    DxGate gate = {nullptr, 0u};
    if (both) {
      gate.nz = nz_count;
      gate.threshold = (unsigned)(((size_t)g.R * g.J) / 5 * 2);
    }
    if (sparse_ok) rc = launch_dx_sparse(g, uv, x, w, out, dx, dx_scratch, gate, li, sdx);
    if (rc == OK && (!sparse_ok || both)) {
      if (vec && P >= 64 * kWideP && (reinterpret_cast<uintptr_t>(dx) & 15) == 0) {   // it stores dx 16 bytes at a time
        dim3 gridw((unsigned)((P + kWideP - 1) / kWideP), (CH + kTile - 1) / kTile);
        snn_dx_wide_kernel<<<gridw, kBwdThreads, 0, sdx>>>(gate, g, uv, x, w, out, dx);
      } else if (vec) {
        snn_dx_kernel<true><<<grid, kBwdThreads, 0, sdx>>>(gate, g, uv, x, w, out, dx);
      } else {
        snn_dx_kernel<false><<<grid, kBwdThreads, 0, sdx>>>(gate, g, uv, x, w, out, dx);
      }
      count_launch();
      if (cudaGetLastError() != cudaSuccess) rc = E_CUDA;
    }
  }
  if (rc == OK && (parts & 2)) {
    const float scale = dw_scale(g);
    const size_t n = (size_t)Itot * g.J;
    int splits = 1;
    float* partial = dw;
    if (want_dw_skip(g, opt) && dw_skip_supported(g, x, uv, out)) {
      int rps = 0;
      partial = planes;   // always reduced from the workspace: its tiles are stored 16 bytes at a time
      // tiles through tensor maps where the shape allows (dw_kernel 2: per-thread copies whatever the shape)
      if (opt.dw_kernel != 2 && dw_tma_supported(g, x, uv, out)) {
        splits = dw_tma_splits(g, li, &rps);
        rc = launch_dw_tma(g, uv, x, out, partial, splits, rps, scale, exact_flag, li, s);
      } else {
        splits = dw_skip_splits(g, li, &rps);
        rc = launch_dw_skip(g, uv, x, out, partial, splits, rps, scale, exact_flag, li, s);
      }
      splits = splits < 1 ? 1 : splits;
      if (rc == OK) {
        int blocks = (int)((n + 255) / 256);
        if (blocks > 4 * li.num_sms) blocks = 4 * li.num_sms;
        snn_dw_reduce_kernel<<<blocks, 256, 0, s>>>(partial, dw, n, splits);
        count_launch();
        if (cudaGetLastError() != cudaSuccess) rc = E_CUDA;
      }
    } else if (opt.dw_kernel != 1 && dw_small_ok(g, uv, out)) {
      int rps = 0;
      splits = dw_small_splits(g, li, &rps);
      partial = planes;
      dim3 grid(1, 1, splits);
      if (g.J == 32) snn_dw_small_kernel<4><<<grid, kBwdThreads, 0, s>>>(g, uv, x, out, partial, rps, scale, exact_flag);
      else if (g.J == 64) snn_dw_small_kernel<8><<<grid, kBwdThreads, 0, s>>>(g, uv, x, out, partial, rps, scale, exact_flag);
      else if (g.J == 128) snn_dw_small_kernel<16><<<grid, kBwdThreads, 0, s>>>(g, uv, x, out, partial, rps, scale, exact_flag);
      else snn_dw_small_kernel<32><<<grid, kBwdThreads, 0, s>>>(g, uv, x, out, partial, rps, scale, exact_flag);
      count_launch();
      if (cudaGetLastError() != cudaSuccess) rc = E_CUDA;
      if (rc == OK) {
        int blocks = (int)((n + 255) / 256);
        if (blocks > 4 * li.num_sms) blocks = 4 * li.num_sms;
        snn_dw_reduce_kernel<<<blocks, 256, 0, s>>>(partial, dw, n, splits);
        count_launch();
        if (cudaGetLastError() != cudaSuccess) rc = E_CUDA;
      }
    } else {
      const DwPlan p = plan_dw(g, li);
      if (p.splits > 1) partial = planes;
      dim3 grid((g.J + kTile - 1) / kTile, (Itot + kTileI - 1) / kTileI, p.splits);
      if (vec) snn_dw_kernel<true><<<grid, kBwdThreads, 0, s>>>(g, uv, x, out, partial, p.rows_per_split, scale, exact_flag);
      else snn_dw_kernel<false><<<grid, kBwdThreads, 0, s>>>(g, uv, x, out, partial, p.rows_per_split, scale, exact_flag);
      count_launch();
      if (cudaGetLastError() != cudaSuccess) rc = E_CUDA;
      if (rc == OK && p.splits > 1) {
        int blocks = (int)((n + 255) / 256);
        if (blocks > 4 * li.num_sms) blocks = 4 * li.num_sms;
        snn_dw_reduce_kernel<<<blocks, 256, 0, s>>>(partial, dw, n, p.splits);
        count_launch();
        if (cudaGetLastError() != cudaSuccess) rc = E_CUDA;
      }
    }
  }
  // the auxiliary stream is joined on every path, so that an error return never leaves it forked (a stream
  // capture in progress would otherwise be invalid)
  if (aux && aux_join(aux, s) != cudaSuccess && rc == OK) rc = E_CUDA;
  return rc;
}

}  // namespace snntc
