// Input gradient of SnnCvGrad (snntc/snncvgrad_kernels.cu.cc:15-84) over the outputs that carry a gradient only.
//
//   dX[p,c] = sum over taps t, outputs j of  [x_pc <= y_oj] u_oj W[(t,c),j],   o = the receptive field that sees
//             input pixel p through tap t,  u_oj = grad_oj / (sum w - theta), 0 wherever (o,j) did not fire.
//
// In a network u is sparse twice over: 50-65 % of the outputs of a layer do not fire, and a pooling layer behind
// the convolution sends the gradient to one input of each window only. On the layers in front of a 2x2 pooling
// nine of ten u are exactly zero. The dense register-tile kernel (snn_dx_wide_kernel) multiplies through all of
// them. Here
//   1. snn_act_lists_kernel compacts, per receptive field, the outputs with u != 0 into a list (y, u, j), j ascending;
//   2. snn_weight_transpose_kernel lays the weights out as Wt[tap][j][c], so that the C weights one list entry needs
//      for one tap are contiguous;
//   3. snn_dx_sparse_kernel keeps an input pixel's channels in registers (CPL per lane, C / CPL lanes per pixel),
//      gathers the lists of the receptive fields that cover the pixel, tap by tap, into shared memory and walks them:
//      per entry one broadcast shared-memory read, 16-byte weight reads and a compare + predicated FMA per channel.
//      Pixel-stationary as the dense kernel: no atomics (the reference scatters with atomicAdd,
//      snncvgrad_kernels.cu.cc:83).
// The terms of a sum are added in the same order as in the dense kernel (tap-major, j ascending; the skipped ones
// are +-0), so the two kernels give the same bits.
#include "snntc_common.cuh"

#include <math_constants.h>

namespace snntc {

namespace {

constexpr int kThreads = 256;

// One warp per receptive field r: list[r*J ..] receives (y bits, u bits, j, 0) for every output with u != 0, in
// ascending j; count[r] their number.
__global__ void __launch_bounds__(kThreads)
snn_act_lists_kernel(const float* __restrict__ out, const float* __restrict__ uv, int R, int J,
                     uint4* __restrict__ list, int* __restrict__ count, const DxGate gate) {
  if (gate.nz != nullptr && __ldg(gate.nz) > gate.threshold) return;   // the dense kernel takes this call
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < R; r += warps) {
    const float* yr = out + (size_t)r * J;
    const float* ur = uv + (size_t)r * J;
    uint4* dst = list + (size_t)r * J;
    int n = 0;
    for (int j0 = 0; j0 < J; j0 += 32) {
      const int j = j0 + lane;
      float y = 0.f, u = 0.f;
      if (j < J) { y = __ldg(yr + j); u = __ldg(ur + j); }
      const bool keep = u != 0.f;
      const unsigned m = __ballot_sync(0xffffffffu, keep);
      if (keep) dst[n + __popc(m & ((1u << lane) - 1u))] = make_uint4(__float_as_uint(y), __float_as_uint(u), (unsigned)j, 0u);
      n += __popc(m);
    }
    if (lane == 0) count[r] = n;
  }
}

// Wt[(tap*J + j)*C + c] = W[(tap*C + c)*J + j]  (the bias row is not part of dX)
__global__ void snn_weight_transpose_kernel(const float* __restrict__ w, float* __restrict__ wt, int taps, int C, int J,
                                            const DxGate gate) {
  if (gate.nz != nullptr && __ldg(gate.nz) > gate.threshold) return;
  const size_t n = (size_t)taps * C * J;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
    const int c = (int)(e % C);
    const size_t tj = e / C;
    const int j = (int)(tj % J);
    const int tap = (int)(tj / J);
    wt[e] = __ldg(w + ((size_t)tap * C + c) * J + j);
  }
}

// acc += [x <= y] * u * w as one compare and one predicated FMA
__device__ __forceinline__ void masked_fma(float& acc, float x, float y, float u, float w) {
  asm("{\n\t.reg .pred p;\n\tsetp.le.f32 p, %1, %2;\n\t@p fma.rn.f32 %0, %3, %4, %0;\n\t}"
      : "+f"(acc) : "f"(x), "f"(y), "f"(u), "f"(w));
}

// CPL channels per lane (4, 8 or 16), LPP lanes per pixel (a power of two, LPP * CPL >= C): a warp holds
// PPW = 32 / LPP input pixels at a time.
//
// The lists a pixel needs (one per tap that an output reads it through) are first copied into shared memory by
// the pixel's own lanes, back to back and with the tap folded into the entry (its third word becomes the element
// offset of weight row (tap, j) in Wt), kStage / PPW entries per pixel and round. The arithmetic then runs over
// that flat sequence: one broadcast shared-memory read per entry instead of a global read in front of every
// weight read, and one loop instead of one per tap.
constexpr int kStage = 256;   // staged list entries per warp and round

template <int CPL, int LPP>
__global__ void __launch_bounds__(kThreads)
snn_dx_sparse_kernel(const Geometry g, const float* __restrict__ x, const float* __restrict__ wt,
                     const uint4* __restrict__ list, const int* __restrict__ count, float* __restrict__ dx,
                     const DxGate gate) {
  if (gate.nz != nullptr && __ldg(gate.nz) > gate.threshold) return;
  constexpr int PPW = 32 / LPP;                       // pixels per warp
  constexpr int SB = kStage / PPW;                    // staged entries per pixel and round
  constexpr int UN = CPL <= 4 ? 4 : 2;                // entries whose weight reads are in flight together
  __shared__ uint4 stage_all[(kThreads / 32) * kStage];
  const int lane = threadIdx.x & 31;
  const int sub = lane / LPP;                         // which of the warp's pixels
  const int gl = lane % LPP;                          // lane within the pixel's group
  const int c0 = gl * CPL;                            // first channel of this lane
  uint4* stage = stage_all + (threadIdx.x >> 5) * kStage + sub * SB;
  const int C = g.C, J = g.J;
  const bool lane_has_channels = c0 < C;              // C % 4 == 0 and CPL % 4 == 0: a lane's float4s are all in or all out
  const int P = g.B * g.H * g.W;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int taps = g.Kh * g.Kw;
  const float* wlane = wt + c0;
  for (int pw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; pw * PPW < P; pw += warps) {
    const int p = pw * PPW + sub;
    const bool pix_ok = p < P;
    float xr[CPL], acc[CPL];
#pragma unroll
    for (int k = 0; k < CPL; ++k) { xr[k] = CUDART_INF_F; acc[k] = 0.f; }
    if (pix_ok && lane_has_channels) {
#pragma unroll
      for (int k4 = 0; k4 < CPL; k4 += 4) {
        if (c0 + k4 < C) {
          const float4 v = __ldg(reinterpret_cast<const float4*>(x + (size_t)p * C + c0 + k4));
          xr[k4] = v.x; xr[k4 + 1] = v.y; xr[k4 + 2] = v.z; xr[k4 + 3] = v.w;
        }
      }
    }
    int ph = 0, pwid = 0, pb = 0;
    if (pix_ok) {
      pwid = p % g.W;
      const int t = p / g.W;
      ph = t % g.H;
      pb = t / g.H;
    }
    // cursor of this pixel through its lists: tap, and the first entry of that tap's list not staged yet
    int tap = pix_ok ? 0 : taps, e0 = 0;
    for (;;) {
      // ---- stage up to SB entries of this pixel, tap after tap (the terms keep their order: tap-major, j ascending)
      int staged = 0;
      while (tap < taps && staged < SB) {
        const int kh = tap / g.Kw, kw = tap - kh * g.Kw;
        // the receptive field that reads this pixel through tap (kh, kw), if there is one
        const int hh = ph + g.pad_top - kh, ww = pwid + g.pad_left - kw;
        int nh = hh, nw = ww;
        bool ok = hh >= 0 && ww >= 0;
        if (g.Sh != 1 || g.Sw != 1) {
          nh = hh / g.Sh; nw = ww / g.Sw;
          ok = ok && nh * g.Sh == hh && nw * g.Sw == ww;
        }
        ok = ok && nh < g.Nh && nw < g.Nw;
        int n = 0;
        const uint4* src = list;
        if (ok) {
          const int r = (pb * g.Nh + nh) * g.Nw + nw;
          n = __ldg(count + r);
          src = list + (size_t)r * J;
        }
        const int take = min(n - e0, SB - staged);
        const unsigned tapoff = (unsigned)tap * (unsigned)J;
        for (int e = gl; e < take; e += LPP) {
          uint4 en = __ldg(src + e0 + e);
          en.z = (tapoff + en.z) * (unsigned)C;
          stage[staged + e] = en;
        }
        staged += take;
        e0 += take;
        if (e0 >= n) { ++tap; e0 = 0; }
      }
      __syncwarp();
      const int nmax = __reduce_max_sync(0xffffffffu, staged);
      if (nmax == 0) break;   // every pixel of the warp is through its lists
      // ---- the arithmetic over the staged entries. A slot past the end of this pixel's share holds
      // (y = -inf, u = 0, offset 0): its compare is false for every input and its weight read stays inside the table.
      for (int e = 0; e < nmax; e += UN) {
        uint4 en[UN];
#pragma unroll
        for (int q = 0; q < UN; ++q) {
          en[q] = make_uint4(0xff800000u, 0u, 0u, 0u);
          if (e + q < staged) en[q] = stage[e + q];
        }
        if (lane_has_channels) {
          float4 w4[UN][CPL / 4];
#pragma unroll
          for (int q = 0; q < UN; ++q) {
            const float* wrow = wlane + en[q].z;
#pragma unroll
            for (int k4 = 0; k4 < CPL; k4 += 4)
              w4[q][k4 / 4] = (c0 + k4 < C) ? __ldg(reinterpret_cast<const float4*>(wrow + k4)) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
#pragma unroll
          for (int q = 0; q < UN; ++q) {
            const float y = __uint_as_float(en[q].x), u = __uint_as_float(en[q].y);
#pragma unroll
            for (int k4 = 0; k4 < CPL; k4 += 4) {
              masked_fma(acc[k4], xr[k4], y, u, w4[q][k4 / 4].x);
              masked_fma(acc[k4 + 1], xr[k4 + 1], y, u, w4[q][k4 / 4].y);
              masked_fma(acc[k4 + 2], xr[k4 + 2], y, u, w4[q][k4 / 4].z);
              masked_fma(acc[k4 + 3], xr[k4 + 3], y, u, w4[q][k4 / 4].w);
            }
          }
        }
      }
      __syncwarp();   // the buffer is rewritten by the next round
    }
    if (pix_ok && lane_has_channels) {
#pragma unroll
      for (int k4 = 0; k4 < CPL; k4 += 4)
        if (c0 + k4 < C)
          *reinterpret_cast<float4*>(dx + (size_t)p * C + c0 + k4) = make_float4(acc[k4], acc[k4 + 1], acc[k4 + 2], acc[k4 + 3]);
    }
  }
}

size_t align256(size_t n) { return (n + 255) & ~(size_t)255; }

template <int CPL, int LPP>
int launch_one(const Geometry& g, const float* x, const float* wt, const uint4* list, const int* count, float* dx,
               DxGate gate, const LaunchInfo& li, cudaStream_t s) {
  const long P = (long)g.B * g.H * g.W;
  const long warps = (P + (32 / LPP) - 1) / (32 / LPP);
  long grid = (warps + (kThreads / 32) - 1) / (kThreads / 32);
  const long cap = (long)li.num_sms * 16;
  if (grid > cap) grid = cap;
  snn_dx_sparse_kernel<CPL, LPP><<<(int)grid, kThreads, 0, s>>>(g, x, wt, list, count, dx, gate);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? OK : E_CUDA;
}

}  // namespace

bool dx_sparse_shape_ok(const Geometry& g) {
  return g.is_conv && (g.C & 3) == 0 && g.C >= 16 && g.C <= 512;
}

bool dx_sparse_supported(const Geometry& g, const float* x, const float* dx) {
  if (!dx_sparse_shape_ok(g)) return false;
  return (((uintptr_t)x | (uintptr_t)dx) & 15) == 0;
}

// scratch: the lists (R*J entries of 16 bytes), their lengths, the transposed weights (fan-in x J; a workspace
// query knows the fan-in only as the number of weight rows, bias row included, which is an upper bound)
size_t dx_sparse_bytes(const Geometry& g) {
  return align256((size_t)g.R * g.J * sizeof(uint4)) + align256((size_t)g.R * sizeof(int)) +
         align256((size_t)g.I * g.J * sizeof(float));
}

int launch_dx_sparse(const Geometry& g, const float* uv, const float* x, const float* w, const float* out, float* dx,
                     void* scratch, DxGate gate, const LaunchInfo& li, cudaStream_t s) {
  unsigned char* base = static_cast<unsigned char*>(scratch);
  uint4* list = reinterpret_cast<uint4*>(base);
  int* count = reinterpret_cast<int*>(base + align256((size_t)g.R * g.J * sizeof(uint4)));
  float* wt = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(count) + align256((size_t)g.R * sizeof(int)));

  long grid = ((long)g.R + (kThreads / 32) - 1) / (kThreads / 32);
  if (grid > (long)li.num_sms * 16) grid = (long)li.num_sms * 16;
  snn_act_lists_kernel<<<(int)grid, kThreads, 0, s>>>(out, uv, g.R, g.J, list, count, gate);
  count_launch();
  if (cudaGetLastError() != cudaSuccess) return E_CUDA;
  const size_t nw = (size_t)g.Kh * g.Kw * g.C * g.J;
  long tg = (long)((nw + 255) / 256);
  if (tg > (long)li.num_sms * 8) tg = (long)li.num_sms * 8;
  snn_weight_transpose_kernel<<<(int)tg, 256, 0, s>>>(w, wt, g.Kh * g.Kw, g.C, g.J, gate);
  count_launch();
  if (cudaGetLastError() != cudaSuccess) return E_CUDA;

  const int C = g.C;
  if (C <= 16) return launch_one<4, 4>(g, x, wt, list, count, dx, gate, li, s);
  if (C <= 32) return launch_one<4, 8>(g, x, wt, list, count, dx, gate, li, s);
  if (C <= 64) return launch_one<4, 16>(g, x, wt, list, count, dx, gate, li, s);
  if (C <= 128) return launch_one<4, 32>(g, x, wt, list, count, dx, gate, li, s);
  if (C <= 256) return launch_one<8, 32>(g, x, wt, list, count, dx, gate, li, s);
  return launch_one<16, 32>(g, x, wt, list, count, dx, gate, li, s);
}

}  // namespace snntc
