// Weight gradient of SnnCvGrad (snntc/snncvgrad_kernels.cu.cc:87-161) for stride-1 convolutions on a power-of-two
// number of channels: the row-skipping kernel of snntc_dw_skip.cu with its tiles brought in by the tensor memory
// accelerator instead of per-thread copies.
//
//   dW[i,j] = sum_r [x_ri <= y_rj] (x_ri - y_rj) u_rj,   u_rj = 0 wherever output (r,j) carries no gradient.
//
// As there, a warp owns FOUR output channels and every lane 4*QL fan-in rows, a CTA 32 channels, a slice of the
// rows r (blockIdx.z) and a tile of the fan-in (blockIdx.y), and the rows of a stage of 16 whose four channels
// carry no gradient are skipped by a warp-uniform branch. What differs is how a stage gets into shared memory. In
// snn_dw_skip_kernel 160 threads issue sixteen 16-byte copies each per stage, with the tap arithmetic and the
// image-border tests in front of every copy -- a third of the instructions of the warps that also do the
// arithmetic. Here one thread issues one tiled bulk copy per tap of the kernel window. A stage is a block of
// hseg x wseg = 16 receptive fields of one image (16 columns of one row of the output map, or 8 columns of two rows,
// ... where the map is narrower than 16): through tap (kh, kw) they read a box of [rows][columns][channels] of the
// NHWC image, which is exactly what a 4-D tensor map describes. Coordinates outside the image are legal for a load
// and read as the fill value -- NaN here, which behaves like an input that never spikes: the saturating FMA of the
// inner loop flushes a NaN to +0 (PTX .sat), and fmaxf(NaN, 0) of the unscaled loop is 0. The y and u tiles are two
// more boxes, of the outputs seen as [image][row][column][channel]; where the map's width or height is no multiple
// of the block, the fields past its edge read as u = 0 (zero fill) and are skipped like any field without a
// gradient. Every copy completes on the mbarrier of its buffer; the warps wait for it (with a time limit) and meet
// once per stage, after the arithmetic, before the buffer is refilled.
//
// The x tile of a stage is laid out [tap][row][channel] (one box after the other), so a fan-in tile is made of
// whole taps, taps_per_tile = 640 / C of them; the bias row (x = biasvolt for every r) is a sum per output channel
// that the CTAs of the last fan-in tile keep beside their tile.
#include "snntc_common.cuh"

#include <cuda.h>
#include <math_constants.h>
#include <mutex>
#include <type_traits>

namespace snntc {

namespace {

constexpr int kThreads = 256;
constexpr int kRS = 16;          // rows r per stage
constexpr int kJT = 32;          // output channels per CTA (4 per warp)
constexpr int kMaxTileFloats = 640;
constexpr long long kWaitClocks = 2000000000LL;   // SM clocks a thread waits for a stage's copies (about a second)
__device__ unsigned g_dw_copy_timeouts = 0u;        // CTAs that gave up waiting since the library was loaded

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
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

// x box: coordinates (channel, column, row, image); the channel coordinate is always 0 (16-byte aligned)
__device__ __forceinline__ void tma_load_4d(unsigned dst, const CUtensorMap* map, unsigned bar, int c, int w, int h, int b) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(b) : "memory");
}
// (the y / u boxes use the same instruction: coordinates (output channel, column, row, image), the channel
// coordinate a multiple of 32)

template <int QL, bool C256>   // C256: 256 channels (a chunk column is half a tap), else a power of two up to 128
__global__ void __launch_bounds__(kThreads, 2)
snn_dw_tma_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                  const __grid_constant__ CUtensorMap map_u, const Geometry g, float* __restrict__ partial,
                  int stages_per_split, float scale, const int* __restrict__ exact_flag, int taps_per_tile,
                  int wseg_log2) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bars[2];
  unsigned char* base = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);   // boxes land on 128-byte boundaries
  const int C = g.C, J = g.J, I = g.I;
  const int Itot = I + g.has_bias;
  const int taps = g.Kh * g.Kw;
  const int tap0 = blockIdx.y * taps_per_tile;
  const int ntap = max(0, min(taps_per_tile, taps - tap0));
  const bool bias_here = g.has_bias && blockIdx.y == gridDim.y - 1;
  const int xfloats = taps_per_tile * kRS * C;                     // floats of one x buffer
  float* Xs = reinterpret_cast<float*>(base);                      // [2][taps_per_tile][kRS][C]
  float* Ys = Xs + 2 * xfloats;                                    // [2][kRS][kJT]
  float* Us = Ys + 2 * kRS * kJT;                                  // [2][kRS][kJT]

  const bool fast = scale != 1.0f && __ldg(exact_flag) == 0;
  const float sc = fast ? scale : 1.0f;                 // s
  const float nsc = -sc;
  const float nusc = fast ? -1.0f / scale : -1.0f;      // -1/s, exact: s is a power of two

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int j0 = blockIdx.x * kJT;
  // stages: blocks of hseg x wseg fields, column blocks fastest, then row blocks, then images
  const int wseg = 1 << wseg_log2, hseg = kRS >> wseg_log2;
  const int WB = (g.Nw + wseg - 1) >> wseg_log2, HB = (g.Nh + hseg - 1) / hseg;
  const int total_stages = g.B * HB * WB;
  const int s_begin = blockIdx.z * stages_per_split;
  const int nstages = max(0, min(total_stages, s_begin + stages_per_split) - s_begin);

  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bars[0])) : "memory");
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bars[1])) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  // Thread 0 queues the copies of stage `st` into buffer `buf`: one box per tap, the y box and the u box.
  auto issue = [&](int st, int buf) {
    const int sg = s_begin + st;
    const int nw0 = (sg % WB) << wseg_log2;
    const int t = sg / WB;
    const int nh0 = (t % HB) * hseg;
    const int b = t / HB;
    const unsigned bar = smem_u32(&bars[buf]);
    const unsigned bytes = (unsigned)(ntap * kRS * C + 2 * kRS * kJT) * 4u;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    for (int tl = 0; tl < ntap; ++tl) {
      const int tap = tap0 + tl;
      const int kh = tap / g.Kw, kw = tap - kh * g.Kw;
      tma_load_4d(smem_u32(Xs + buf * xfloats + tl * kRS * C), &map_x, bar, 0, nw0 - g.pad_left + kw,
                  nh0 - g.pad_top + kh, b);
    }
    tma_load_4d(smem_u32(Ys + buf * kRS * kJT), &map_y, bar, j0, nw0, nh0, b);
    tma_load_4d(smem_u32(Us + buf * kRS * kJT), &map_u, bar, j0, nw0, nh0, b);
  };
  // try_wait suspends the thread until the phase completes or a hardware time limit passes, so a waiting warp does
  // not take issue slots from the SM's other CTA; the clock bounds the number of attempts
  auto copies_arrived = [&](int buf, unsigned parity) {
    const unsigned bar = smem_u32(&bars[buf]);
    auto attempt = [&]() {
      unsigned ok;
      asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                   : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
      return ok != 0u;
    };
    bool arrived = attempt();
    if (!arrived) {
      const long long t0 = clock64();
      do arrived = attempt(); while (!arrived && clock64() - t0 < kWaitClocks);
    }
    return arrived;
  };

  // This lane's 16-byte chunks of the fan-in tile: chunk q = lane + 32c holds fan-in floats f = 4*lane + 128c of the
  // tile, i.e. channel f % C of tap f / C, at float (f / C)*16*C + f % C of row 0 of an x buffer. C is a power of two:
  // for C <= 128 a step of c is 128 / C whole taps (2048 floats), for C = 256 it is half a tap, so the offset is a
  // part that depends on the lane plus a compile-time constant per c. A chunk behind the tile's taps is read all
  // the same (what it reads lies inside the CTA's shared memory: the other x buffer or the y/u tiles) and its sums
  // are dropped at the end.
  const int lane_part = C256 ? 4 * lane : ((4 * lane) / C) * kRS * C + (4 * lane) % C;
  int irow[QL];              // weight row of the chunk's first float; -1: the chunk lies behind the tile's taps
#pragma unroll
  for (int c = 0; c < QL; ++c) {
    const int f = 4 * lane + 128 * c;
    irow[c] = f < ntap * C ? tap0 * C + f : -1;
  }
  // the bias row: x = biasvolt for every r, one sum per output channel, kept by every lane alike (it takes two
  // instructions per row and channel beside the thirty of a fan-in chunk)
  float accb[4] = {0.f, 0.f, 0.f, 0.f};

  // acc[c][jj][h]: fan-in rows irow[c] + 2h, +1 (one 64-bit pair), output channel j0 + 4*warp + jj
  uint64_t acc[QL][4][2];
#pragma unroll
  for (int c = 0; c < QL; ++c)
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) acc[c][jj][0] = acc[c][jj][1] = pack2(0.f, 0.f);

  auto reduce_stage = [&](int buf, auto fast_c) {
    constexpr bool FAST = decltype(fast_c)::value;
    const float* xb = Xs + buf * xfloats + lane_part;
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
      const float* xrow = xb + rl * C;
#pragma unroll
      for (int c = 0; c < QL; ++c) {
        const float4 v = *reinterpret_cast<const float4*>(xrow + (C256 ? (c >> 1) * kRS * 256 + (c & 1) * 128 : 2048 * c));
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
        if (bias_here) accb[jj] = fmaf(FAST ? fma_sat(g.biasvolt, nsc, ys) : fmaxf(ys - g.biasvolt, 0.f), nu, accb[jj]);
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

  if (tid == 0) {
    if (nstages > 0) issue(0, 0);
    if (nstages > 1) issue(1, 1);
  }
  bool failed = false;
  for (int it = 0; it < nstages; ++it) {
    const int buf = it & 1;
    if (!failed) failed = !copies_arrived(buf, (unsigned)(it >> 1) & 1u);
    if (!failed) {
      if (fast) reduce_stage(buf, std::true_type{});
      else reduce_stage(buf, std::false_type{});
    }
    // everyone is through with this buffer (or some thread's copies never came: the CTA stops)
    if (__syncthreads_or(failed)) { failed = true; break; }
    if (tid == 0 && it + 2 < nstages) issue(it + 2, buf);
  }
  if (failed) {
    // give the copies that may still be in flight the same time once more before the shared memory is handed on
    if (tid == 0) atomicAdd(&g_dw_copy_timeouts, 1u);
    const long long t0 = clock64();
    while (clock64() - t0 < kWaitClocks) {}
    __syncthreads();
  }

  float* __restrict__ dst = partial + (size_t)blockIdx.z * Itot * J;
  const int j = j0 + 4 * warp;
  if (j < J) {
#pragma unroll
    for (int c = 0; c < QL; ++c) {
      if (irow[c] < 0) continue;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float v[2][4];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) unpack2(acc[c][jj][h], v[0][jj], v[1][jj]);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int i = irow[c] + 2 * h + e;
          *reinterpret_cast<float4*>(dst + (size_t)i * J + j) = make_float4(v[e][0], v[e][1], v[e][2], v[e][3]);
        }
      }
    }
    if (bias_here && lane == 0)
      *reinterpret_cast<float4*>(dst + (size_t)I * J + j) = make_float4(accb[0], accb[1], accb[2], accb[3]);
  }
}

struct TmaPlan { int taps_per_tile, ntiles, ql; size_t smem; };

TmaPlan plan(const Geometry& g) {
  TmaPlan p;
  const int taps = g.I / g.C > 0 ? g.I / g.C : 1;      // (a workspace query knows the fan-in, not the kernel window)
  int tpt = kMaxTileFloats / g.C;
  if (tpt < 1) tpt = 1;
  if (tpt > taps) tpt = taps;
  p.taps_per_tile = tpt;
  p.ntiles = (taps + tpt - 1) / tpt;                   // the bias row rides in the last tile
  p.ql = (tpt * g.C + 127) / 128;
  p.smem = (size_t)2 * tpt * kRS * g.C * sizeof(float) + (size_t)4 * kRS * kJT * sizeof(float) + 128;
  return p;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// the driver's cuTensorMapEncodeTiled, looked up once through the runtime (the library does not link libcuda)
EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      (void)cudaGetLastError();
  });
  return fn;
}

// how the 16 fields of a stage are laid over the output map: wseg columns (a power of two, at most 16) x 16/wseg rows
int stage_wseg_log2(const Geometry& g) {
  int lg = 0;
  while (lg < 4 && (1 << lg) < g.Nw) ++lg;
  return lg;
}
long stage_count(const Geometry& g) {
  const int lg = stage_wseg_log2(g);
  const int wseg = 1 << lg, hseg = kRS >> lg;
  return (long)g.B * ((g.Nh + hseg - 1) / hseg) * ((g.Nw + wseg - 1) / wseg);
}

template <int QL, bool C256>
int launch_ql(const CUtensorMap& mx, const CUtensorMap& my, const CUtensorMap& mu, const Geometry& g, float* partial,
              dim3 grid, int stages_per_split, float scale, const int* exact_flag, const TmaPlan& p, cudaStream_t s) {
  if (cudaFuncSetAttribute(snn_dw_tma_kernel<QL, C256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem) != cudaSuccess)
    return E_CUDA;
  snn_dw_tma_kernel<QL, C256><<<grid, kThreads, p.smem, s>>>(mx, my, mu, g, partial, stages_per_split, scale, exact_flag,
                                                             p.taps_per_tile, stage_wseg_log2(g));
  count_launch();
  return cudaGetLastError() == cudaSuccess ? OK : E_CUDA;
}

}  // namespace

bool dw_tma_shape_ok(const Geometry& g) {
  if (!g.is_conv || g.Sh != 1 || g.Sw != 1) return false;
  if (g.C < 4 || g.C > 256 || (g.C & (g.C - 1)) != 0 || (g.J & 3) != 0) return false;   // channels: a power of two
  if (g.Nh < 1 || g.Nw < 1 || g.B < 1) return false;
  if ((long long)g.B * g.H * g.W * g.C > 0x7fffffffLL) return false;
  if (stage_count(g) > 0x7fffffffL) return false;
  return true;
}

bool dw_tma_supported(const Geometry& g, const float* x, const float* uv, const float* out) {
  if (!dw_tma_shape_ok(g)) return false;
  if (((uintptr_t)x | (uintptr_t)uv | (uintptr_t)out) & 15) return false;
  return encode_tiled() != nullptr;
}

// The stages are cut into `return value` slices of *stages_per_split stages each (blockIdx.z).
int dw_tma_splits(const Geometry& g, const LaunchInfo& li, int* stages_per_split) {
  const TmaPlan p = plan(g);
  const long tiles = (long)p.ntiles * ((g.J + kJT - 1) / kJT);
  const long stages = stage_count(g);
  // several waves of CTAs: the work of a CTA depends on how often ITS channels carry a gradient
  long want = (8L * li.num_sms + tiles - 1) / tiles;
  const long max_splits = (stages + 3) / 4;
  if (want > max_splits) want = max_splits;
  if (want > 1024) want = 1024;
  if (want < 1) want = 1;
  const long sps = (stages + want - 1) / want;
  *stages_per_split = (int)sps;
  return (int)((stages + sps - 1) / sps);
}

int launch_dw_tma(const Geometry& g, const float* uv, const float* x, const float* out, float* partial, int splits,
                  int stages_per_split, float scale, const int* exact_flag, const LaunchInfo& li, cudaStream_t s) {
  (void)li;
  EncodeTiledFn enc = encode_tiled();
  if (!enc) return E_UNSUPPORTED;
  const TmaPlan p = plan(g);
  const int lg = stage_wseg_log2(g);
  const cuuint32_t wseg = 1u << lg, hseg = (cuuint32_t)kRS >> lg;
  const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  CUtensorMap mx, my, mu;
  {
    const cuuint64_t dims[4] = {(cuuint64_t)g.C, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)g.B};
    const cuuint64_t strides[3] = {(cuuint64_t)g.C * 4, (cuuint64_t)g.W * g.C * 4, (cuuint64_t)g.H * g.W * g.C * 4};
    const cuuint32_t box[4] = {(cuuint32_t)g.C, wseg, hseg, 1u};
    if (enc(&mx, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(x), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NAN_REQUEST_ZERO_FMA) != CUDA_SUCCESS)
      return E_UNSUPPORTED;
  }
  {
    // the outputs as [image][row][column][channel]: fields past the edge of the map read as zero
    const cuuint64_t dims[4] = {(cuuint64_t)g.J, (cuuint64_t)g.Nw, (cuuint64_t)g.Nh, (cuuint64_t)g.B};
    const cuuint64_t strides[3] = {(cuuint64_t)g.J * 4, (cuuint64_t)g.Nw * g.J * 4, (cuuint64_t)g.Nh * g.Nw * g.J * 4};
    const cuuint32_t box[4] = {(cuuint32_t)kJT, wseg, hseg, 1u};
    if (enc(&my, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(out), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return E_UNSUPPORTED;
    if (enc(&mu, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(uv), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return E_UNSUPPORTED;
  }
  dim3 grid((g.J + kJT - 1) / kJT, p.ntiles, splits);
  if (g.C == 256) {   // tiles of one or two taps: 2 or 4 chunk columns
    if (p.ql <= 2) return launch_ql<2, true>(mx, my, mu, g, partial, grid, stages_per_split, scale, exact_flag, p, s);
    return launch_ql<4, true>(mx, my, mu, g, partial, grid, stages_per_split, scale, exact_flag, p, s);
  }
  switch (p.ql) {
    case 1: return launch_ql<1, false>(mx, my, mu, g, partial, grid, stages_per_split, scale, exact_flag, p, s);
    case 2: return launch_ql<2, false>(mx, my, mu, g, partial, grid, stages_per_split, scale, exact_flag, p, s);
    case 3: return launch_ql<3, false>(mx, my, mu, g, partial, grid, stages_per_split, scale, exact_flag, p, s);
    case 4: return launch_ql<4, false>(mx, my, mu, g, partial, grid, stages_per_split, scale, exact_flag, p, s);
    default: return launch_ql<5, false>(mx, my, mu, g, partial, grid, stages_per_split, scale, exact_flag, p, s);
  }
}

unsigned long long dw_copy_timeouts() {
  unsigned n = 0;
  if (cudaMemcpyFromSymbol(&n, g_dw_copy_timeouts, sizeof(n)) != cudaSuccess) note_cuda_error(cudaGetLastError());
  return n;
}

}  // namespace snntc
