// Weight gradient of SnnCvGrad (snntc/snncvgrad_kernels.cu.cc:87-161) that skips the outputs that did not fire.
//
//   dW[i,j] = sum_r [x_ri <= y_rj] (x_ri - y_rj) u_rj,   u_rj = 0 wherever output (r,j) did not fire.
//
// In the networks this library is built for, 50-65 % of the outputs of a layer do not fire, and an output
// channel that rarely fires does so for almost every receptive field. The dense register-tile kernel
// (snn_dw_kernel) multiplies through all of them. Here a warp owns FOUR output channels and every lane 4*QL
// fan-in rows, so "did (r,j) fire" is the same question for all 32 lanes: a warp-uniform branch skips the
// whole row of the tile for that channel, and the inputs of row r are not even read from shared memory when
// none of the warp's four channels fired. What is left costs what the dense kernel costs per element: one
// saturating FMA (the clamp [x<=y](y-x) as the saturation of (y-x)*s, s a power of two, see snn_dw_kernel)
// and half a two-lane FMA.
//
// CTA: 256 threads = 8 warps = 32 output channels; 128*QL fan-in rows; blockIdx.z takes a slice of the rows r.
// The x tile (16 rows of r at a time, double buffered) is gathered straight from the NHWC image with 16-byte
// asynchronous copies (four channels of one tap are contiguous), never passing through registers; taps outside
// the image, rows past the slice and the bias row are plain 16-byte stores of constants (NOT copies from a
// constant in global memory: every CTA fetching the same 16 bytes makes one L2 line the bottleneck of the kernel).
#include "snntc_common.cuh"

#include <math_constants.h>
#include <type_traits>

namespace snntc {

namespace {

constexpr int kThreads = 256;
constexpr int kRS = 16;          // rows r per stage
constexpr int kJT = 32;          // output channels per CTA (4 per warp)

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
__device__ __forceinline__ float fma_sat(float a, float b, float c) {
  float r;
  asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int QL>
__global__ void __launch_bounds__(kThreads, 2)
snn_dw_skip_kernel(const Geometry g, const float* __restrict__ uv, const float* __restrict__ x,
                   const float* __restrict__ out, float* __restrict__ partial, int rows_per_split,
                   float scale, const int* __restrict__ exact_flag) {
  constexpr int kTI = 128 * QL;        // fan-in rows per CTA
  constexpr int kCh = 32 * QL;         // 16-byte chunks per row of the x tile
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* Xs = reinterpret_cast<float*>(smem_raw);                 // [2][kRS][kTI]
  float* Ys = Xs + 2 * kRS * kTI;                                 // [2][kRS][kJT]
  float* Us = Ys + 2 * kRS * kJT;                                 // [2][kRS][kJT]
  int4* rowinfo = reinterpret_cast<int4*>(Us + 2 * kRS * kJT);    // [2][kRS]: .x element offset of the top-left pixel, .y its h, .z its w, .w row valid

  const int J = g.J, I = g.I, R = g.R;
  const int Itot = I + g.has_bias;
  const bool fast = scale != 1.0f && __ldg(exact_flag) == 0;
  const float sc = fast ? scale : 1.0f;                 // s
  const float nsc = -sc;
  const float nusc = fast ? -1.0f / scale : -1.0f;      // -1/s, exact: s is a power of two

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int i0 = blockIdx.y * kTI, j0 = blockIdx.x * kJT;
  const int r_begin = blockIdx.z * rows_per_split;
  const int r_end = min(R, r_begin + rows_per_split);
  // what stands in for inputs that are not there: an input that never spikes; the bias input and the padding beside it
  const float4 v_never = make_float4(g.maxv, g.maxv, g.maxv, g.maxv);
  const float4 v_bias = make_float4(g.biasvolt, g.maxv, g.maxv, g.maxv);

  // this thread's column chunk of the x tile (threads below kCh): .x element offset of its tap from a row's top-left
  // pixel, .y kh, .z kw, .w 1 = image tap, 2 = bias chunk, 0 = padding behind the last weight row
  int4 tapinfo_reg = make_int4(0, 0, 0, 0);
  if (tid < kCh) {
    const int i = i0 + 4 * tid;
    if (i < I) {
      const int tap = i / g.C, c = i - tap * g.C;
      const int kh = tap / g.Kw, kw = tap - kh * g.Kw;
      tapinfo_reg = make_int4((kh * g.W + kw) * g.C + c, kh, kw, 1);
    } else if (i == I && g.has_bias) {
      tapinfo_reg.w = 2;
    }
  }
  auto fill_rowinfo = [&](int buf, int rb) {
    if (tid < kRS) {
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
      rowinfo[buf * kRS + tid] = ri;
    }
  };
  // Queues the asynchronous copies of the 16 rows starting at rb into buffer `buf` (rowinfo[buf] describes them).
  // Thread t < kCh owns column chunk t of the x tile -- its tap is the same for every row and stays in registers --
  // and walks the 16 rows; the other threads fetch the y and u tiles (16 rows x 8 chunks each).
  static_assert(kCh < kThreads, "some threads must be left for the y and u tiles");
  const int4 my_tap = tapinfo_reg;
  auto issue = [&](int buf, int rb) {
    if (tid < kCh) {
      float* dst = Xs + buf * kRS * kTI + 4 * tid;
#pragma unroll
      for (int rl = 0; rl < kRS; ++rl) {
        const int4 ri = rowinfo[buf * kRS + rl];   // the same word for the whole warp: a broadcast
        const bool in_image = ri.w != 0 && my_tap.w == 1 && (unsigned)(ri.y + my_tap.y) < (unsigned)g.H &&
                              (unsigned)(ri.z + my_tap.z) < (unsigned)g.W;
        if (in_image) cp_async16(dst + rl * kTI, x + ((ptrdiff_t)ri.x + my_tap.x));
        else *reinterpret_cast<float4*>(dst + rl * kTI) = (ri.w != 0 && my_tap.w == 2) ? v_bias : v_never;
      }
    } else {
      for (int e = tid - kCh; e < 2 * kRS * (kJT / 4); e += kThreads - kCh) {
        const int which = e / (kRS * (kJT / 4));            // 0: y, 1: u
        const int h = e - which * (kRS * (kJT / 4));
        const int rl = h / (kJT / 4), cq = h - rl * (kJT / 4);
        const int r = rb + rl, j = j0 + 4 * cq;
        const float* base = which == 0 ? out : uv;
        float* dst = (which == 0 ? Ys : Us) + (buf * kRS + rl) * kJT + 4 * cq;
        if (r < r_end && j < J) cp_async16(dst, base + (size_t)r * J + j);
        else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);   // no spike value, no gradient
      }
    }
    cp_async_commit();
  };

  // acc[c][jj][h]: fan-in rows i0 + 4*(lane + 32c) + 2h, +1 (one 64-bit pair), output channel j0 + 4*warp + jj
  uint64_t acc[QL][4][2];
#pragma unroll
  for (int c = 0; c < QL; ++c)
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) acc[c][jj][0] = acc[c][jj][1] = pack2(0.f, 0.f);

  auto reduce_stage = [&](int buf, auto fast_c) {
    constexpr bool FAST = decltype(fast_c)::value;
    const float* xs = Xs + buf * kRS * kTI;
    // which of the 16 rows carry a gradient for one of this warp's four channels: lane rl looks at row rl, one vote
    unsigned todo;
    {
      const float4 uq = *reinterpret_cast<const float4*>(Us + (buf * kRS + (lane & (kRS - 1))) * kJT + 4 * warp);
      todo = __ballot_sync(0xffffffffu, (uq.x != 0.f) | (uq.y != 0.f) | (uq.z != 0.f) | (uq.w != 0.f)) & ((1u << kRS) - 1u);
    }
#pragma unroll 1
    while (todo != 0u) {
      const int rl = __ffs((int)todo) - 1;
      todo &= todo - 1u;
      const float4 y4 = *reinterpret_cast<const float4*>(Ys + (buf * kRS + rl) * kJT + 4 * warp);
      const float4 u4 = *reinterpret_cast<const float4*>(Us + (buf * kRS + rl) * kJT + 4 * warp);
      float xr[QL][4];
#pragma unroll
      for (int c = 0; c < QL; ++c) {
        const float4 v = *reinterpret_cast<const float4*>(xs + rl * kTI + 4 * (lane + 32 * c));
        xr[c][0] = v.x; xr[c][1] = v.y; xr[c][2] = v.z; xr[c][3] = v.w;
      }
      const float yv[4] = {y4.x, y4.y, y4.z, y4.w};
      const float uu[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        if (uu[jj] == 0.f) continue;              // warp-uniform
        const float ys = yv[jj] * sc;
        const float nu = uu[jj] * nusc;
        const uint64_t nu2 = pack2(nu, nu);
#pragma unroll
        for (int c = 0; c < QL; ++c) {
          float t[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) t[k] = FAST ? fma_sat(xr[c][k], nsc, ys) : fmaxf(ys - xr[c][k], 0.f);
          acc[c][jj][0] = fma2(pack2(t[0], t[1]), nu2, acc[c][jj][0]);
          acc[c][jj][1] = fma2(pack2(t[2], t[3]), nu2, acc[c][jj][1]);
        }
      }
    }
  };

  fill_rowinfo(0, r_begin);
  fill_rowinfo(1, r_begin + kRS);
  __syncthreads();
  if (r_begin < r_end) issue(0, r_begin);
  __syncthreads();   // rowinfo[0] is rewritten inside the loop: every thread must have queued its copies first

  int it = 0;
  for (int rb = r_begin; rb < r_end; rb += kRS, ++it) {
    const int buf = it & 1;
    const bool more = rb + kRS < r_end;
    if (more) issue(buf ^ 1, rb + kRS);
    fill_rowinfo(buf, rb + 2 * kRS);   // this stage's entries were last read when its copies were queued
    if (more) cp_async_wait<1>(); else cp_async_wait<0>();
    __syncthreads();
    if (fast) reduce_stage(buf, std::true_type{});
    else reduce_stage(buf, std::false_type{});
    __syncthreads();
  }

  float* __restrict__ dst = partial + (size_t)blockIdx.z * Itot * J;
  const int j = j0 + 4 * warp;
  if (j < J) {
#pragma unroll
    for (int c = 0; c < QL; ++c)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float v[2][4];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) unpack2(acc[c][jj][h], v[0][jj], v[1][jj]);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int i = i0 + 4 * (lane + 32 * c) + 2 * h + e;
          if (i < Itot)
            *reinterpret_cast<float4*>(dst + (size_t)i * J + j) = make_float4(v[e][0], v[e][1], v[e][2], v[e][3]);
        }
      }
  }
}

size_t smem_bytes(int QL) {
  const size_t kTI = 128 * (size_t)QL;
  return (2 * kRS * kTI + 4 * kRS * kJT) * sizeof(float) + 2 * kRS * sizeof(int4);
}

// fan-in tiles: as few as possible with at most 640 rows each, then the narrowest tile that covers the share
void plan_tiles(int Itot, int* ntiles, int* ql) {
  int n = (Itot + 639) / 640;
  int per = (Itot + n - 1) / n;
  int q = (per + 127) / 128;
  if (q < 1) q = 1;
  if (q > 5) q = 5;
  *ql = q;
  *ntiles = (Itot + 128 * q - 1) / (128 * q);
}

template <int QL>
int launch_ql(const Geometry& g, const float* uv, const float* x, const float* out, float* partial, dim3 grid,
              int rows_per_split, float scale, const int* exact_flag, cudaStream_t s) {
  const size_t smem = smem_bytes(QL);
  if (cudaFuncSetAttribute(snn_dw_skip_kernel<QL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return E_CUDA;
  snn_dw_skip_kernel<QL><<<grid, kThreads, smem, s>>>(g, uv, x, out, partial, rows_per_split, scale, exact_flag);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? OK : E_CUDA;
}

}  // namespace

bool dw_skip_supported(const Geometry& g, const float* x, const float* uv, const float* out) {
  if (!g.is_conv || (g.C & 3) != 0 || (g.J & 3) != 0) return false;
  if (((uintptr_t)x | (uintptr_t)uv | (uintptr_t)out) & 15) return false;
  if ((long long)g.B * g.H * g.W * g.C > 0x7fffffffLL) return false;   // element offsets are 32-bit
  return true;
}

int dw_skip_splits(const Geometry& g, const LaunchInfo& li, int* rows_per_split) {
  int ntiles = 1, ql = 1;
  plan_tiles(g.I + g.has_bias, &ntiles, &ql);
  const long tiles = (long)ntiles * ((g.J + kJT - 1) / kJT);
  // several waves of CTAs: the work of a CTA depends on how often ITS channels fired, small slices even that out
  long want = (8L * li.num_sms + tiles - 1) / tiles;
  const long max_splits = ((long)g.R + 4 * kRS - 1) / (4 * kRS);
  if (want > max_splits) want = max_splits;
  if (want > 1024) want = 1024;
  if (want < 1) want = 1;
  long rps = ((long)g.R + want - 1) / want;
  rps = (rps + kRS - 1) / kRS * kRS;
  *rows_per_split = (int)rps;
  return (int)(((long)g.R + rps - 1) / rps);
}

int launch_dw_skip(const Geometry& g, const float* uv, const float* x, const float* out, float* partial,
                   int splits, int rows_per_split, float scale, const int* exact_flag,
                   const LaunchInfo& li, cudaStream_t s) {
  (void)li;
  int ntiles = 1, ql = 1;
  plan_tiles(g.I + g.has_bias, &ntiles, &ql);
  dim3 grid((g.J + kJT - 1) / kJT, ntiles, splits);
  switch (ql) {
    case 1: return launch_ql<1>(g, uv, x, out, partial, grid, rows_per_split, scale, exact_flag, s);
    case 2: return launch_ql<2>(g, uv, x, out, partial, grid, rows_per_split, scale, exact_flag, s);
    case 3: return launch_ql<3>(g, uv, x, out, partial, grid, rows_per_split, scale, exact_flag, s);
    case 4: return launch_ql<4>(g, uv, x, out, partial, grid, rows_per_split, scale, exact_flag, s);
    default: return launch_ql<5>(g, uv, x, out, partial, grid, rows_per_split, scale, exact_flag, s);
  }
}

}  // namespace snntc
